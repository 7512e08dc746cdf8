"""The CPU oracle against the outputs of the unmodified reference (tests/golden/*.npz)."""
import pytest
import torch

from conftest import load_golden
from oracle import gdr_oracle as orc


def _decay(gc_chunked):
    return orc._decay_mask(gc_chunked)


@pytest.mark.parametrize("name", ["c1_fwd_fp32", "dense_tail_bf16", "varlen_gva_reftest_bf16"])
def test_forward_matches_reference(name):
    z = load_golden(name)
    q, k, v = z["q"].float(), z["k"].float(), z["v"].float()
    cu = z.get("cu_seqlens")
    gc, A, o, h, fs = orc.gdr_fwd(q, k, v, z["g"], z["beta"], z["scale"], z["h0"], cu,
                                  output_h="h" in z)
    assert orc.rel_to_max(gc, z["g_cumsum"]) < 1e-6
    assert orc.rel_to_max(o, z["o"]) < 2e-5
    assert orc.rel_to_max(fs, z["final_state"]) < 2e-5
    if "h" in z:
        assert orc.rel_to_max(h, z["h"]) < 2e-5


@pytest.mark.parametrize("name", ["dense_tail_bf16", "varlen_gva_reftest_bf16"])
def test_backward_matches_reference(name):
    z = load_golden(name)
    q, k, v, do = z["q"].float(), z["k"].float(), z["v"].float(), z["do"].float()
    cu = z.get("cu_seqlens")
    outs = orc.gdr_bwd(q, k, v, z["g_cumsum"], z["beta"], do, z["dht"], z["scale"], z["h0"], cu)
    for nm, x in zip(["dq", "dk", "dv", "db", "dg", "dh0"], outs):
        assert x.shape == z[nm].shape, nm
        assert orc.rel_to_max(x, z[nm]) < 5e-5, nm


def test_gated_inverse_relation():
    """The reference's torch A is the gated inverse: A_ref = A_gate_free o exp(g_i - g_j)."""
    z = load_golden("dense_tail_bf16")
    gc, A, *_ = orc.gdr_fwd(z["q"].float(), z["k"].float(), z["v"].float(), z["g"], z["beta"],
                            z["scale"], z["h0"], None)
    B, T, H, C = A.shape
    for b in range(B):
        for c0 in range(0, T, 64):
            n = min(64, T - c0)
            g_ = gc[b, c0:c0 + n]                       # [n,H]
            G = (g_[:, None, :] - g_[None, :, :]).permute(0, 2, 1)  # [i,H,j]
            lower = torch.ones(n, n).tril().bool()[:, None, :]
            Gm = torch.where(lower, G, torch.tensor(-float("inf"))).exp()
            got = A[b, c0:c0 + n, :, :n] * Gm
            assert orc.rel_to_max(got, z["A_gated"][b, c0:c0 + n, :, :n]) < 2e-5


def test_backward_equals_autograd_of_recurrence():
    torch.manual_seed(3)
    B, T, Hq, Hv, K = 1, 100, 1, 2, 128
    dt = torch.float64
    q = orc.l2norm(torch.randn(B, T, Hq, K, dtype=dt)); k = orc.l2norm(torch.randn(B, T, Hq, K, dtype=dt))
    v = torch.randn(B, T, Hv, K, dtype=dt); g = torch.nn.functional.logsigmoid(torch.randn(B, T, Hv, dtype=dt)) / 4
    beta = torch.randn(B, T, Hv, dtype=dt).sigmoid(); cu = torch.tensor([0, 37, 100], dtype=torch.int32)
    h0 = torch.randn(2, Hv, K, K, dtype=dt); do = torch.randn(B, T, Hv, K, dtype=dt); dht = torch.randn(2, Hv, K, K, dtype=dt)
    leaves = [x.clone().requires_grad_() for x in (q, k, v, beta, g, h0)]
    o, fs = orc.gdr_recurrent(leaves[0], leaves[1], leaves[2], leaves[4], leaves[3], None, leaves[5], cu, dtype=dt)
    ((o * do).sum() + (fs * dht).sum()).backward()
    gc = orc.chunk_local_cumsum(g, cu, dtype=dt)
    outs = orc.gdr_bwd(q, k, v, gc, beta, do, dht, None, h0, cu, dtype=dt)
    _, _, o2, _, fs2 = orc.gdr_fwd(q, k, v, g, beta, None, h0, cu, dtype=dt)
    assert orc.rel_to_max(o2, o.detach()) < 1e-11 and orc.rel_to_max(fs2, fs.detach()) < 1e-11
    for nm, x, leaf in zip(["dq", "dk", "dv", "db", "dg", "dh0"], outs, leaves):
        assert orc.rel_to_max(x, leaf.grad) < 1e-10, nm
