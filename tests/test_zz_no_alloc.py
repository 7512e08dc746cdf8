"""The allocation-free backward entry point against the regular one.

fq_gdr_bwd_chunk_gva_noalloc serves callers that may not allocate device memory where the backward
runs (a pre-planned step with a frozen allocator, or a host that would otherwise pay a
device-synchronising cudaMalloc per call): it keeps the per-V-head dq / dk partial results in an
array inside the library instead of in two caller-allocated buffers.  The test drives both entry
points through the C ABI on the same inputs, twice in a row (the second call reuses the array with the
first call's contents still in it): dq, dk and dv must agree bitwise, dg and dbeta to 1e-5 of their maximum (they
are summed with shared-memory atomics, whose order is not fixed).

This file is named so that pytest collects it last.
"""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-5  # dg and dbeta only (sums by shared-memory atomics); dq, dk and dv are compared bitwise


def _inputs(seed, B, T, Hq, Hv, cu):
    torch.manual_seed(seed)
    dev = "cuda"
    n_seq = B if cu is None else len(cu) - 1
    q = orc.l2norm(torch.randn(B, T, Hq, 128)).bfloat16().to(dev)
    k = orc.l2norm(torch.randn(B, T, Hq, 128)).bfloat16().to(dev)
    v = torch.randn(B, T, Hv, 128).bfloat16().to(dev)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, Hv)).to(dev)
    beta = torch.randn(B, T, Hv).sigmoid().to(dev)
    do = torch.randn(B, T, Hv, 128).bfloat16().to(dev)
    h0 = (0.1 * torch.randn(n_seq, Hv, 128, 128)).to(dev)
    dht = (0.01 * torch.randn(n_seq, Hv, 128, 128)).to(dev)
    return q, k, v, g, beta, do, h0, dht


# the third case sits exactly on the size limit B*T*H = 65536; the fourth follows it with a small packed batch, so the
# array then still holds the big case's rows
@pytest.mark.parametrize("B,T,Hq,Hv,cu", [(2, 200, 2, 4, None), (1, 500, 1, 4, [0, 130, 131, 500]), (1, 8192, 2, 8, None),
                                          (1, 300, 2, 4, [0, 7, 71, 300])])
def test_noalloc_matches_regular_entry_point(B, T, Hq, Hv, cu):
    from flashqla_b200 import _lib, kernels, ops
    lib = _lib.load()
    q, k, v, g, beta, do, h0, dht = _inputs(21, B, T, Hq, Hv, cu)
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device="cuda")
    plan = kernels.make_plan(B, T, cu_t, q.device)
    scale = 128 ** -0.5
    gc, A, _, _, _ = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, cu_t, True, False, False)
    _, Ag, Pg = kernels.kkt_solve_gated(k, q, beta, gc, scale, plan, A=A)
    _, h, _ = kernels.fused_gdr_fwd(q, k, v, Ag, None, gc, beta, scale, initial_state=h0, output_final_state=False,
                                    output_h=True, output_o=False, plan=plan)
    dh = torch.empty_like(h)
    cu_p, off_p = plan.ptrs()
    st = kernels._stream()
    rc = lib.fq_gdr_bwd_dh(q.data_ptr(), k.data_ptr(), Ag.data_ptr(), Pg.data_ptr(), do.data_ptr(), gc.data_ptr(), beta.data_ptr(),
                           dht.data_ptr(), None, dh.data_ptr(), B, T, Hv, Hq, cu_p, off_p,
                           plan.n_seq, plan.total_chunks, scale, None, st)
    _lib.check(rc, "fq_gdr_bwd_dh")

    def common_args(dq, dk, dv, dg, db):
        return (q.data_ptr(), k.data_ptr(), v.data_ptr(), A.data_ptr(), Ag.data_ptr(), Pg.data_ptr(), do.data_ptr(),
                h.data_ptr(), dh.data_ptr(), gc.data_ptr(), beta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                dg.data_ptr(), db.data_ptr(), B, T, Hv, Hq, cu_p, off_p, plan.n_seq, plan.total_chunks, scale, None, st)

    # regular path: caller-allocated per-V-head buffers + head sum
    dq_h = torch.empty(B, T, Hv, 128, dtype=torch.bfloat16, device="cuda")
    dk_h = torch.empty_like(dq_h)
    dg_ref = torch.empty(B, T, Hv, device="cuda")
    db_ref = torch.empty_like(dg_ref)
    dv_ref = torch.empty_like(v)
    _lib.check(lib.fq_gdr_bwd_chunk(*common_args(dq_h, dk_h, dv_ref, dg_ref, db_ref)), "fq_gdr_bwd_chunk")
    dq_ref = torch.empty(B, T, Hq, 128, dtype=torch.bfloat16, device="cuda")
    dk_ref = torch.empty_like(dq_ref)
    _lib.check(lib.fq_group_reduce(dq_h.data_ptr(), dq_ref.data_ptr(), B * T, Hv, Hq, st), "fq_group_reduce")
    _lib.check(lib.fq_group_reduce(dk_h.data_ptr(), dk_ref.data_ptr(), B * T, Hv, Hq, st), "fq_group_reduce")

    for call in range(2):
        dq = torch.full((B, T, Hq, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        dk = torch.full_like(dq, float("nan"))
        dg = torch.full((B, T, Hv), float("nan"), device="cuda")
        db = torch.full_like(dg, float("nan"))
        dv = torch.full_like(v, float("nan"))
        _lib.check(lib.fq_gdr_bwd_chunk_gva_noalloc(*common_args(dq, dk, dv, dg, db)), "fq_gdr_bwd_chunk_gva_noalloc")
        torch.cuda.synchronize()
        # the same kernel computes dq, dk and dv in the same order on both paths: every bit must agree
        for name, got, ref in (("dq", dq, dq_ref), ("dk", dk, dk_ref), ("dv", dv, dv_ref)):
            assert torch.isfinite(got.float()).all(), f"{name} (call {call})"
            assert torch.equal(got, ref), f"{name} (call {call}): not bitwise equal to the regular entry point"
        for name, got, ref in (("dg", dg, dg_ref), ("db", db, db_ref)):
            assert torch.isfinite(got).all(), f"{name} (call {call})"
            err = orc.rel_to_max(got.cpu(), ref.cpu())
            assert err < TOL, f"{name} (call {call}): rel-to-max {err:.2e}, max-abs {(got - ref).abs().max().item():.3e}"


def test_noalloc_rejects_oversized_problem():
    from flashqla_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(16, device="cuda")
    p = x.data_ptr()
    rc = lib.fq_gdr_bwd_chunk_gva_noalloc(p, p, p, p, p, p, p, p, p, p, p, p, p, p, p, p, 1, 65536, 2, 1, None, None, 1, 1024,
                                          0.1, None, None)
    assert rc == -4 and b"exceeds the built-in scratch" in lib.fq_last_error()
