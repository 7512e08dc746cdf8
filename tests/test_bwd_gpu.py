"""GPU parity of the backward path against the CPU oracle and the golden fixtures.

Tolerance (stated): max|x - ref| <= 1e-2 * max|ref| for every gradient (dq, dk, dv bf16; dbeta, dg,
dh0 fp32) against the fp32 oracle on the same bf16-rounded inputs.  The reference's own acceptance
bound is 2e-2 (tests/test_gdr.py:362-420 of the reference).
"""
import os

import pytest
import torch

from conftest import check_close, load_golden
from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu
os.environ.setdefault("FLASHQLA_CHECK_STATUS", "1")

TOL = 1e-2
NAMES = ["dq", "dk", "dv", "db", "dg", "dh0"]


def make_inputs(seed, B, T, Hq, Hv, dist="baseline", n_seq=None):
    torch.manual_seed(seed)
    N = B if n_seq is None else n_seq
    q = orc.l2norm(torch.randn(B, T, Hq, 128)).bfloat16()
    k = orc.l2norm(torch.randn(B, T, Hq, 128)).bfloat16()
    v = torch.randn(B, T, Hv, 128).bfloat16()
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, Hv))
    beta = torch.randn(B, T, Hv).sigmoid()
    do = torch.randn(B, T, Hv, 128).bfloat16()
    if dist == "baseline":
        h0, dht = 0.1 * torch.randn(N, Hv, 128, 128), 0.01 * torch.randn(N, Hv, 128, 128)
    else:
        g = g / 16
        g[:, :, -1] = 0.0
        h0, dht = torch.randn(N, Hv, 128, 128), torch.randn(N, Hv, 128, 128) / 8
    return q, k, v, g, beta, h0, do, dht


def run_bwd(q, k, v, g, beta, h0, do, dht, cu):
    from flashqla_b200 import ops
    dev = "cuda"
    c = lambda x: None if x is None else x.to(dev)
    gc, A, o, _, fs = ops.chunk_gated_delta_rule_fwd(c(q), c(k), c(v), c(g), c(beta), None, c(h0), c(cu), True, False, False)
    outs = ops.chunk_gated_delta_rule_bwd(c(q), c(k), c(v), gc, c(beta), A, c(do), c(dht), None, c(h0), c(cu))
    torch.cuda.synchronize()
    return [None if x is None else x.float().cpu() for x in outs]


BWD_CASES = [
    (1, 64, 1, 1, None, "baseline"),
    (1, 256, 2, 2, None, "baseline"),
    (2, 200, 2, 4, None, "baseline"),
    (1, 33, 2, 2, None, "reftest"),
    (1, 1000, 2, 4, [0, 1, 64, 65, 300, 300, 777, 1000], "reftest"),
    (1, 1024, 2, 2, None, "reftest"),
]


@pytest.mark.parametrize("B,T,Hq,Hv,cu,dist", BWD_CASES)
def test_backward_vs_oracle(B, T, Hq, Hv, cu, dist):
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    q, k, v, g, beta, h0, do, dht = make_inputs(11, B, T, Hq, Hv, dist, None if cu is None else len(cu) - 1)
    gc = orc.chunk_local_cumsum(g, cu_t)
    ref = orc.gdr_bwd(q.float(), k.float(), v.float(), gc, beta, do.float(), dht, None, h0, cu_t)
    got = run_bwd(q, k, v, g, beta, h0, do, dht, cu_t)
    check_close(got, ref, TOL, NAMES)


@pytest.mark.parametrize("name", ["dense_tail_bf16", "varlen_gva_reftest_bf16"])
def test_backward_vs_reference_fixture(name):
    z = load_golden(name)
    got = run_bwd(z["q"], z["k"], z["v"], z["g"], z["beta"], z["h0"], z["do"], z["dht"], z.get("cu_seqlens"))
    check_close(got, [z[n] for n in NAMES], TOL, NAMES)


@pytest.mark.parametrize("recompute_tiles", [False, True])
def test_autograd_entry(recompute_tiles, monkeypatch):
    """Public differentiable entry; with and without keeping the gated tiles A_g / P_g for the backward."""
    import flash_qla
    from flashqla_b200 import ops
    monkeypatch.setattr(ops, "_RECOMPUTE_TILES", recompute_tiles)
    q, k, v, g, beta, h0, do, dht = make_inputs(5, 2, 192, 2, 4)
    dev = "cuda"
    leaves = [x.to(dev).requires_grad_() for x in (q, k, v, g, beta, h0)]
    o, fs = flash_qla.chunk_gated_delta_rule(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4],
                                             initial_state=leaves[5], output_final_state=True)
    ((o.float() * do.to(dev).float()).sum() + (fs * dht.to(dev)).sum()).backward()
    gc = orc.chunk_local_cumsum(g, None)
    ref = orc.gdr_bwd(q.float(), k.float(), v.float(), gc, beta, do.float(), dht, None, h0, None)
    got = [leaves[0].grad, leaves[1].grad, leaves[2].grad, leaves[4].grad, leaves[3].grad, leaves[5].grad]
    check_close(got, ref, TOL, NAMES)


@pytest.mark.parametrize("with_h0,with_final", [(False, True), (True, False), (False, False)])
def test_autograd_optional_states(with_h0, with_final):
    """initial_state=None and / or output_final_state=False through the differentiable entry: the first segment of
    a truncated back-propagation (no initial state, final state handed on) must not return a gradient for the
    missing input, and a missing final state means a zero state gradient at the end."""
    import flash_qla
    q, k, v, g, beta, h0, do, dht = make_inputs(7, 2, 200, 2, 4)
    dev = "cuda"
    leaves = [x.to(dev).requires_grad_() for x in (q, k, v, g, beta)]
    h0_leaf = h0.to(dev).requires_grad_() if with_h0 else None
    o, fs = flash_qla.chunk_gated_delta_rule(*leaves, initial_state=h0_leaf, output_final_state=with_final)
    assert (fs is not None) == with_final
    loss = (o.float() * do.to(dev).float()).sum()
    if with_final:
        loss = loss + (fs * dht.to(dev)).sum()
    loss.backward()
    gc = orc.chunk_local_cumsum(g, None)
    ref = orc.gdr_bwd(q.float(), k.float(), v.float(), gc, beta, do.float(), dht if with_final else None, None,
                      h0 if with_h0 else None, None)
    got = [leaves[0].grad, leaves[1].grad, leaves[2].grad, leaves[4].grad, leaves[3].grad]
    check_close(got, ref[:5], TOL, NAMES[:5])
    if with_h0:
        check_close([h0_leaf.grad], [ref[5]], TOL, ["dh0"])


CP_CASES = [
    (1, 1024, 2, 2, None, "baseline", 4),
    (1, 1024, 2, 2, None, "reftest", 4),   # the g = 0 head replays to the sequence end / start: exact
    (2, 520, 1, 2, None, "baseline", 2),
    (1, 1500, 2, 4, [0, 1, 64, 65, 700, 700, 1500], "reftest", 3),
    # piece length chosen by the planner; the g = 0 head and (with short pieces) the slowly decaying heads take the
    # transition-matrix route: state pass, chain of piece states, final pass
    (1, 4096, 2, 4, None, "reftest", None),
    (1, 6000, 1, 2, [0, 3000, 3100, 6000], "reftest", 5),
]


@pytest.mark.parametrize("B,T,Hq,Hv,cu,dist,pc", CP_CASES)
def test_backward_context_parallel(B, T, Hq, Hv, cu, dist, pc, monkeypatch):
    """State recompute and the dS recurrence split into pieces (forward and reverse gate-driven warm-up)."""
    from flashqla_b200 import ops
    monkeypatch.setattr(ops, "_FORCE_PIECE_CHUNKS", pc)
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    q, k, v, g, beta, h0, do, dht = make_inputs(13, B, T, Hq, Hv, dist, None if cu is None else len(cu) - 1)
    gc = orc.chunk_local_cumsum(g, cu_t)
    ref = orc.gdr_bwd(q.float(), k.float(), v.float(), gc, beta, do.float(), dht, None, h0, cu_t)
    got = run_bwd(q, k, v, g, beta, h0, do, dht, cu_t)
    check_close(got, ref, TOL, NAMES)


def test_backward_is_reproducible():
    """dq, dk, dv and dh0 are bitwise the same from run to run (every accumulator is fed by one issuing thread, in a
    fixed order); dg and dbeta are summed with shared-memory atomics and may differ in the last bits."""
    q, k, v, g, beta, h0, do, dht = make_inputs(31, 2, 1536, 2, 4, "baseline", None)
    ref = run_bwd(q, k, v, g, beta, h0, do, dht, None)   # (dq, dk, dv, db, dg, dh0)
    for _ in range(8):
        got = run_bwd(q, k, v, g, beta, h0, do, dht, None)
        for i in (0, 1, 2, 5):
            assert torch.equal(got[i], ref[i]), NAMES[i]
        for i in (3, 4):
            assert (got[i] - ref[i]).abs().max() <= 1e-5 * ref[i].abs().max()


def test_repeated_forward_backward_is_race_free():
    """200 forward + backward passes of one packed, grouped-head batch that runs context parallel (pieces of three
    chunks; the zero-gate head takes the transition-matrix route): every pass must leave the status word at zero and
    reproduce o, final_state, dq, dk, dv and dh0 bit for bit (dg and dbeta, summed with atomics, to 1e-5).  The
    reference guards its kernels the same way with 1000 repetitions (tests/test_gdr.py:203,362 of FlashQLA)."""
    from flashqla_b200 import kernels, ops
    old = ops._FORCE_PIECE_CHUNKS
    ops._FORCE_PIECE_CHUNKS = 3
    try:
        cu = [0, 1, 64, 65, 700, 700, 1500, 2900]
        cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
        q, k, v, g, beta, h0, do, dht = (x.cuda() for x in make_inputs(17, 1, cu[-1], 2, 4, "reftest", len(cu) - 1))

        def one_pass():
            gc, A, o, _, fs = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, None, h0, cu_t, True, False, True)
            outs = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, do, dht, None, h0, cu_t)
            return [o, fs] + list(outs)

        names = ["o", "final_state"] + NAMES
        ref = one_pass()   # FLASHQLA_CHECK_STATUS=1: every pass reads the status word and raises if it is not zero
        for rep in range(200):
            got = one_pass()
            for n, x, r in zip(names, got, ref):
                if n in ("db", "dg"):
                    assert (x - r).abs().max() <= 1e-5 * r.abs().max(), f"{n} differs in repetition {rep}"
                else:
                    assert torch.equal(x, r), f"{n} differs in repetition {rep}"
    finally:
        ops._FORCE_PIECE_CHUNKS = old


@pytest.mark.parametrize("gate_mode,beta_sigmoid,cu", [(1, True, None), (2, True, None), (2, False, [0, 100, 101, 470]), (1, False, None)])
def test_gate_activations_in_kernel(gate_mode, beta_sigmoid, cu):
    """use_gate_in_kernel / use_beta_sigmoid_in_kernel: raw gate and beta inputs, activations applied inside the tile
    kernel, their derivatives inside the backward.  Reference: the oracle on torch-activated inputs, with torch.autograd
    carrying the oracle's dg / dbeta through the activations (fp32).  Tolerance 1e-2 rel-to-max as elsewhere."""
    import flash_qla
    torch.manual_seed(23)
    B, T, Hq, Hv = (2, 200, 2, 4) if cu is None else (1, cu[-1], 2, 4)
    N = B if cu is None else len(cu) - 1
    q = orc.l2norm(torch.randn(B, T, Hq, 128)).bfloat16()
    k = orc.l2norm(torch.randn(B, T, Hq, 128)).bfloat16()
    v = torch.randn(B, T, Hv, 128).bfloat16()
    g_raw = torch.randn(B, T, Hv)
    b_raw = torch.randn(B, T, Hv)
    A_log = torch.log(torch.empty(Hv).uniform_(0.5, 4.0))
    dt_bias = 0.5 * torch.randn(Hv)
    h0, dht = 0.1 * torch.randn(N, Hv, 128, 128), 0.01 * torch.randn(N, Hv, 128, 128)
    do = torch.randn(B, T, Hv, 128).bfloat16()
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    # reference: activations in torch (differentiable), operator maths in the oracle
    leaves = [x.clone().requires_grad_() for x in (g_raw, b_raw, A_log, dt_bias)]
    g_act = torch.nn.functional.logsigmoid(leaves[0]) if gate_mode == 1 else \
        -leaves[2].exp() * torch.nn.functional.softplus(leaves[0] + leaves[3])
    b_act = leaves[1].sigmoid() if beta_sigmoid else leaves[1]
    gcr, _, o_ref, _, fs_ref = orc.gdr_fwd(q.float(), k.float(), v.float(), g_act.detach(), b_act.detach(), None, h0, cu_t)
    ref = orc.gdr_bwd(q.float(), k.float(), v.float(), gcr, b_act.detach(), do.float(), dht, None, h0, cu_t)
    torch.autograd.backward([g_act, b_act], [ref[4], ref[3]])
    # operator with raw inputs
    dev = "cuda"
    kw = {}
    ins = [x.to(dev).requires_grad_() for x in (q, k, v, g_raw, b_raw, h0)]
    if gate_mode == 2:
        kw = dict(A_log=A_log.to(dev).requires_grad_(), dt_bias=dt_bias.to(dev).requires_grad_())
    o, fs = flash_qla.chunk_gated_delta_rule(ins[0], ins[1], ins[2], ins[3], ins[4], initial_state=ins[5],
                                             output_final_state=True, cu_seqlens=None if cu is None else cu_t.to(dev),
                                             use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=beta_sigmoid, **kw)
    check_close([o, fs], [o_ref, fs_ref], {"o": 1e-2, "final_state": 5e-3}, ["o", "final_state"])
    ((o.float() * do.to(dev).float()).sum() + (fs * dht.to(dev)).sum()).backward()
    got = [ins[0].grad, ins[1].grad, ins[2].grad, ins[4].grad, ins[3].grad, ins[5].grad]
    want = [ref[0], ref[1], ref[2], leaves[1].grad, leaves[0].grad, ref[5]]
    check_close(got, want, TOL, ["dq", "dk", "dv", "db_raw", "dg_raw", "dh0"])
    if gate_mode == 2:
        check_close([kw["A_log"].grad, kw["dt_bias"].grad], [leaves[2].grad, leaves[3].grad], TOL, ["dA_log", "ddt_bias"])
