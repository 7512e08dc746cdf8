"""Parity at the full sizes of the benchmark configurations, where the CPU oracle cannot run the whole problem.

Two kinds of checks: (1) the oracle on single heads / head groups of the full-size problem (heads are
independent, so a head of the big run must equal the oracle's run on that head alone), and (2) size-independent
properties of the operator: linearity of (o, final_state) in (v, h0), of the gradients in (do, dht), equality
of one pass with two half passes chained through the state, context parallel on/off.
Inputs are generated on the device (seeded); tolerances are the ones of the small-size tests.
"""
import os

import pytest
import torch

from conftest import check_close
from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu
os.environ.setdefault("FLASHQLA_CHECK_STATUS", "1")

TOL_BF16 = 1e-2
TOL_FP32 = 5e-3
TOL_LIN = 1.5e-2  # sums of two bf16-rounded results against one bf16-rounded result


def _l2(x):
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def _inputs(seed, B, T, Hq, Hv, n_seq=None):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=gen)
    N = B if n_seq is None else n_seq
    q = _l2(rn(B, T, Hq, 128)).bfloat16()
    k = _l2(rn(B, T, Hq, 128)).bfloat16()
    v = rn(B, T, Hv, 128).bfloat16()
    g = torch.nn.functional.logsigmoid(rn(B, T, Hv))
    beta = rn(B, T, Hv).sigmoid()
    h0 = 0.1 * rn(N, Hv, 128, 128)
    return q, k, v, g, beta, h0


def _rel(x, ref):
    den = ref.double().abs().max().item()
    return (x.double() - ref.double()).abs().max().item() / max(den, 1e-30)


def test_config2_forward_full_size():
    """B=1, T=32768, Hq=Hv=64 (forward prefill)."""
    from flashqla_b200 import ops
    B, T, H = 1, 32768, 64
    q, k, v, g, beta, h0 = _inputs(2, B, T, H, H)
    scale = 128 ** -0.5
    _, _, o, _, fs = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, True, False, True)
    # (1) two heads against the oracle
    for h in (0, 63):
        sl = slice(h, h + 1)
        _, _, o_ref, _, fs_ref = orc.gdr_fwd(q[:, :, sl].float().cpu(), k[:, :, sl].float().cpu(), v[:, :, sl].float().cpu(),
                                             g[:, :, sl].cpu(), beta[:, :, sl].cpu(), scale, h0[:, sl].cpu(), None)
        assert orc.rel_to_max(o[:, :, sl].float().cpu(), o_ref) < TOL_BF16, f"o head {h}"
        assert orc.rel_to_max(fs[:, sl].cpu(), fs_ref) < TOL_FP32, f"final_state head {h}"
    # (2a) context parallel off gives the same result
    _, _, o_ser, _, fs_ser = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, True, False, False)
    assert _rel(o.float(), o_ser.float()) < TOL_BF16
    assert _rel(fs, fs_ser) < TOL_FP32
    # (2b) two half passes chained through the state
    Th = T // 2
    _, _, o1, _, s1 = ops.chunk_gated_delta_rule_fwd(q[:, :Th].contiguous(), k[:, :Th].contiguous(), v[:, :Th].contiguous(),
                                                     g[:, :Th].contiguous(), beta[:, :Th].contiguous(), scale, h0, None, True, False, True)
    _, _, o2, _, s2 = ops.chunk_gated_delta_rule_fwd(q[:, Th:].contiguous(), k[:, Th:].contiguous(), v[:, Th:].contiguous(),
                                                     g[:, Th:].contiguous(), beta[:, Th:].contiguous(), scale, s1, None, True, False, True)
    assert _rel(torch.cat([o1, o2], 1).float(), o.float()) < TOL_BF16
    assert _rel(s2, fs) < TOL_FP32
    # (2c) linearity in (v, h0)
    q2, k2, v2, g2, beta2, h02 = _inputs(3, B, T, H, H)
    _, _, oa, _, fa = ops.chunk_gated_delta_rule_fwd(q, k, v2, g, beta, scale, h02, None, True, False, True)
    vs = (v.float() + v2.float()).bfloat16()
    # the sum is rounded to bf16 once more: compare against the operator on the rounded sum's components
    _, _, osum, _, fsum = ops.chunk_gated_delta_rule_fwd(q, k, vs, g, beta, scale, h0 + h02, None, True, False, True)
    assert _rel(o.float() + oa.float(), osum.float()) < TOL_LIN
    assert _rel(fs + fa, fsum) < TOL_LIN


def test_config3_backward_full_size():
    """B=4, T=8192, Hq=16, Hv=32 (training forward + backward)."""
    from flashqla_b200 import ops
    B, T, Hq, Hv = 4, 8192, 16, 32
    q, k, v, g, beta, h0 = _inputs(4, B, T, Hq, Hv)
    gen = torch.Generator(device="cuda").manual_seed(5)
    do = torch.randn(B, T, Hv, 128, device="cuda", generator=gen).bfloat16()
    dht = 0.01 * torch.randn(B, Hv, 128, 128, device="cuda", generator=gen)
    scale = 128 ** -0.5
    gc, A, o, _, fs = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, True, False, True)
    got = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, do, dht, scale, h0, None)
    names = ("dq", "dk", "dv", "db", "dg", "dh0")
    # (1) one batch row and one QK-head group (its two V-heads) against the oracle
    b, hq = 2, 5
    hv = slice(2 * hq, 2 * hq + 2)
    cpu = lambda x: x.float().cpu()
    gcs = orc.chunk_local_cumsum(g[b:b + 1, :, hv].cpu(), None)
    ref = orc.gdr_bwd(cpu(q[b:b + 1, :, hq:hq + 1]), cpu(k[b:b + 1, :, hq:hq + 1]), cpu(v[b:b + 1, :, hv]), gcs,
                      beta[b:b + 1, :, hv].cpu(), cpu(do[b:b + 1, :, hv]), dht[b:b + 1, hv].cpu(), scale, h0[b:b + 1, hv].cpu(), None)
    mine = (got[0][b:b + 1, :, hq:hq + 1], got[1][b:b + 1, :, hq:hq + 1], got[2][b:b + 1, :, hv], got[3][b:b + 1, :, hv],
            got[4][b:b + 1, :, hv], got[5][b:b + 1, hv])
    for n, x, r in zip(names, mine, ref):
        assert orc.rel_to_max(x.float().cpu(), r) < TOL_BF16, n
    # (2) linearity of all gradients in (do, dht)
    do2 = torch.randn(B, T, Hv, 128, device="cuda", generator=gen).bfloat16()
    dht2 = 0.01 * torch.randn(B, Hv, 128, 128, device="cuda", generator=gen)
    got2 = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, do2, dht2, scale, h0, None)
    dos = (do.float() + do2.float()).bfloat16()
    gots = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, dos, dht + dht2, scale, h0, None)
    for n, x1, x2, xs in zip(names, got, got2, gots):
        assert _rel(x1.float() + x2.float(), xs.float()) < TOL_LIN, n


def test_config4_packed_varlen_full_size():
    """24 sequences with lengths uniform in [256, 16384] packed into B=1 (about 200k tokens), Hq=Hv=16."""
    from flashqla_b200 import ops
    gen = torch.Generator().manual_seed(6)
    lens = torch.randint(256, 16385, (24,), generator=gen)
    cu = torch.zeros(25, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0).to(torch.int32)
    T, H = int(cu[-1]), 16
    q, k, v, g, beta, h0 = _inputs(7, 1, T, H, H, n_seq=24)
    gd = torch.Generator(device="cuda").manual_seed(8)
    do = torch.randn(1, T, H, 128, device="cuda", generator=gd).bfloat16()
    scale = 128 ** -0.5
    cud = cu.cuda()
    gc, A, o, _, fs = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, cud, True, False, True)
    got = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, do, None, scale, h0, cud)
    # one head against the oracle, forward over all sequences, backward over the three shortest ones
    h = 9
    sl = slice(h, h + 1)
    cpu = lambda x: x.float().cpu()
    gcr, _, o_ref, _, fs_ref = orc.gdr_fwd(cpu(q[:, :, sl]), cpu(k[:, :, sl]), cpu(v[:, :, sl]), g[:, :, sl].cpu(),
                                           beta[:, :, sl].cpu(), scale, h0[:, sl].cpu(), cu)
    assert orc.rel_to_max(o[:, :, sl].float().cpu(), o_ref) < TOL_BF16
    assert orc.rel_to_max(fs[:, sl].cpu(), fs_ref) < TOL_FP32
    for si in torch.argsort(lens)[:3].tolist():
        a, e = int(cu[si]), int(cu[si + 1])
        ref = orc.gdr_bwd(cpu(q[:, a:e, sl]), cpu(k[:, a:e, sl]), cpu(v[:, a:e, sl]), gcr[:, a:e], beta[:, a:e, sl].cpu(),
                          cpu(do[:, a:e, sl]), None, scale, h0[si:si + 1, sl].cpu(), None)
        mine = (got[0][:, a:e, sl], got[1][:, a:e, sl], got[2][:, a:e, sl], got[3][:, a:e, sl], got[4][:, a:e, sl],
                got[5][si:si + 1, sl])
        for n, x, r in zip(("dq", "dk", "dv", "db", "dg", "dh0"), mine, ref):
            assert orc.rel_to_max(x.float().cpu(), r) < TOL_BF16, f"{n} of sequence {si}"


def _c5_inputs(T, H, seed):
    q, k, v, g, beta, h0 = _inputs(seed, 1, T, H, H)
    gen = torch.Generator(device="cuda").manual_seed(seed + 1000)
    do = torch.randn(1, T, H, 128, device="cuda", generator=gen).bfloat16()
    dht = 0.01 * torch.randn(1, H, 128, 128, device="cuda", generator=gen)
    return q, k, v, g, beta, h0, do, dht


def test_config5_one_rank_share():
    """B=1, T=131072, Hq=Hv=8: the share of one rank when the 1M-token sequence of the long-context configuration
    is split over 8 GPUs.  Forward and backward of the whole problem; one head against the oracle run on that head
    alone (forward and backward in full)."""
    from flashqla_b200 import ops
    T, H = 131072, 8
    q, k, v, g, beta, h0, do, dht = _c5_inputs(T, H, 21)
    scale = 128 ** -0.5
    gc, A, o, _, fs = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, True, False, True)
    got = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, do, dht, scale, h0, None)
    torch.cuda.synchronize()
    h = 5
    sl = slice(h, h + 1)
    cpu = lambda x: x.float().cpu()
    gcr, _, o_ref, _, fs_ref = orc.gdr_fwd(cpu(q[:, :, sl]), cpu(k[:, :, sl]), cpu(v[:, :, sl]), g[:, :, sl].cpu(),
                                           beta[:, :, sl].cpu(), scale, h0[:, sl].cpu(), None)
    check_close([o[:, :, sl], fs[:, sl]], [o_ref, fs_ref], {"o": TOL_BF16, "final_state": TOL_FP32}, ["o", "final_state"])
    ref = orc.gdr_bwd(cpu(q[:, :, sl]), cpu(k[:, :, sl]), cpu(v[:, :, sl]), gcr, beta[:, :, sl].cpu(), cpu(do[:, :, sl]),
                      dht[:, sl].cpu(), scale, h0[:, sl].cpu(), None)
    mine = [got[0][:, :, sl], got[1][:, :, sl], got[2][:, :, sl], got[3][:, :, sl], got[4][:, :, sl], got[5][:, sl]]
    check_close(mine, ref, TOL_BF16, ["dq", "dk", "dv", "db", "dg", "dh0"])


def test_config5_full_length():
    """B=1, T=1048576, Hq=Hv=8 on one GPU (16384 chunks per head, 131072 units): one head of the forward against the
    oracle's forward AND backward on that head in full; context parallel on = off; and the backward as a whole through
    size-independent properties: linearity in (do, dht), one pass = two half passes chained through the state and
    its gradient."""
    from flashqla_b200 import ops
    T, H = 1 << 20, 8
    q, k, v, g, beta, h0, do, dht = _c5_inputs(T, H, 23)
    scale = 128 ** -0.5
    gc, A, o, _, fs = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, True, False, True)
    torch.cuda.synchronize()
    # (1) one head against the oracle
    h = 2
    sl = slice(h, h + 1)
    cpu = lambda x: x.float().cpu()
    _, _, o_ref, _, fs_ref = orc.gdr_fwd(cpu(q[:, :, sl]), cpu(k[:, :, sl]), cpu(v[:, :, sl]), g[:, :, sl].cpu(),
                                         beta[:, :, sl].cpu(), scale, h0[:, sl].cpu(), None)
    check_close([o[:, :, sl], fs[:, sl]], [o_ref, fs_ref], {"o": TOL_BF16, "final_state": TOL_FP32}, ["o", "final_state"])
    del o_ref
    # (2) context parallel off gives the same result
    _, _, o_ser, _, fs_ser = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, True, False, False)
    check_close([o, fs], [o_ser, fs_ser], {"o": TOL_BF16, "final_state": TOL_FP32}, ["o", "final_state"], "cp on/off: ")
    del o_ser
    # (3) backward: linearity in (do, dht)
    names = ("dq", "dk", "dv", "db", "dg", "dh0")
    got = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, do, dht, scale, h0, None)
    gen = torch.Generator(device="cuda").manual_seed(77)
    do2 = torch.randn(1, T, H, 128, device="cuda", generator=gen).bfloat16()
    dht2 = 0.01 * torch.randn(1, H, 128, 128, device="cuda", generator=gen)
    got2 = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, do2, dht2, scale, h0, None)
    dos = (do.float() + do2.float()).bfloat16()
    gots = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, dos, dht + dht2, scale, h0, None)
    check_close([a.float() + b.float() for a, b in zip(got, got2)], gots, TOL_LIN, names, "linearity: ")
    # (3b) the same head's six gradients against the oracle's backward on that head in full (16384 chunk steps)
    gcr = orc.chunk_local_cumsum(g[:, :, sl].cpu(), None)
    ref = orc.gdr_bwd(cpu(q[:, :, sl]), cpu(k[:, :, sl]), cpu(v[:, :, sl]), gcr, beta[:, :, sl].cpu(), cpu(do[:, :, sl]),
                      dht[:, sl].cpu(), scale, h0[:, sl].cpu(), None)
    mine = [got[0][:, :, sl], got[1][:, :, sl], got[2][:, :, sl], got[3][:, :, sl], got[4][:, :, sl], got[5][:, sl]]
    check_close(mine, ref, TOL_BF16, names, "head vs oracle: ")
    del ref
    del got2, gots, do2, dos
    # (4) backward: two half passes chained through the state (forward) and its gradient (backward)
    Th = T // 2
    first = lambda x: x[:, :Th].contiguous()
    second = lambda x: x[:, Th:].contiguous()
    gc1, A1, _, _, s1 = ops.chunk_gated_delta_rule_fwd(first(q), first(k), first(v), first(g), first(beta), scale, h0, None,
                                                       True, False, True)
    gc2, A2, _, _, _ = ops.chunk_gated_delta_rule_fwd(second(q), second(k), second(v), second(g), second(beta), scale, s1, None,
                                                      True, False, True)
    b2 = ops.chunk_gated_delta_rule_bwd(second(q), second(k), second(v), gc2, second(beta), A2, second(do), dht, scale, s1, None)
    b1 = ops.chunk_gated_delta_rule_bwd(first(q), first(k), first(v), gc1, first(beta), A1, first(do), b2[5], scale, h0, None)
    chained = [torch.cat([x1, x2], 1) for x1, x2 in zip(b1[:5], b2[:5])] + [b1[5]]
    check_close(chained, got, TOL_BF16, names, "two half passes: ")
