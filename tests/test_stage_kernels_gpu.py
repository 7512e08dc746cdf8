"""GPU parity of the chunk-parallel stage kernels and of the tensor-core plumbing."""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4, 5, 6])
def test_umma_selftest(mode):
    from flashqla_b200 import kernels
    torch.manual_seed(mode)
    a = torch.randn(128, 128, device="cuda").bfloat16()
    b = torch.randn(128, 128, device="cuda").bfloat16()
    d = kernels.selftest_umma(a, b, mode)
    af, bf = a.float(), b.float()
    if mode in (0, 2, 4, 6):
        ref = af @ bf.T
    elif mode == 1:
        ref = af[:, :64] @ bf[:64, :]
    elif mode == 3:
        ref = torch.zeros(128, 128, device="cuda")
        ref[:64] = af[:64] @ bf.T
    else:
        ref = af[:64, :].T @ bf[:, :64].T
    err = (d - ref).abs().max().item()
    assert err < 1e-2 * ref.abs().max().item(), f"mode {mode}: max err {err}"


CASES = [
    # B, T, Hq, Hv, cu_seqlens
    (2, 256, 2, 2, None),
    (3, 200, 1, 4, None),
    (1, 33, 2, 2, None),
    (1, 1000, 2, 4, [0, 1, 64, 65, 300, 300, 777, 1000]),
    (1, 4096, 8, 8, None),
]


@pytest.mark.parametrize("B,T,Hq,Hv,cu", CASES)
@pytest.mark.parametrize("reverse", [False, True])
def test_chunk_cumsum(B, T, Hq, Hv, cu, reverse):
    from flashqla_b200 import kernels
    torch.manual_seed(0)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, Hv))
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    ref = orc.chunk_local_cumsum(g, cu_t, reverse=reverse)
    got = kernels.chunk_local_cumsum(g.cuda(), reverse=reverse, cu_seqlens=None if cu is None else cu_t.cuda())
    assert torch.allclose(got.cpu(), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("B,T,Hq,Hv,cu", CASES)
def test_kkt_solve(B, T, Hq, Hv, cu):
    from flashqla_b200 import kernels
    torch.manual_seed(1)
    k = orc.l2norm(torch.randn(B, T, Hq, 128)).bfloat16()
    beta = torch.randn(B, T, Hv).sigmoid()
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    q = torch.zeros_like(k)
    v = torch.zeros(B, T, Hv, 128)
    g = torch.zeros(B, T, Hv)
    _, A_ref, *_ = orc.gdr_fwd(q.float(), k.float(), v, g, beta, None, None, cu_t)
    A = kernels.kkt_solve(k.cuda(), beta.cuda(), cu_seqlens=None if cu is None else cu_t.cuda()).float().cpu()
    # bf16 output: half an ulp of the largest entry (1.0 on the diagonal) is 2^-9
    assert (A - A_ref).abs().max().item() < 6e-3
    assert orc.rel_to_max(A, A_ref) < 6e-3


def test_bounded_wait_expires_and_the_context_survives():
    """A wait that nothing satisfies gives up after its limit, reports (kernel id << 12) + site through the status
    word, releases the other waits of the CTA, frees the tensor memory and lets the kernel end; the next ordinary
    call on the device works.  The limit is passed in (1e6 cycles, about half a millisecond): nothing traps, faults
    or spins without a bound."""
    from flashqla_b200 import _lib, kernels
    lib = _lib.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.fq_selftest_wait_expiry(status.data_ptr(), done.data_ptr(), 1_000_000, kernels._stream())
    _lib.check(rc, "fq_selftest_wait_expiry")
    torch.cuda.synchronize()
    assert int(done.item()) == 1
    assert int(status.item()) == (14 << 12) + 5
    # limits outside the accepted range are refused on the host
    assert lib.fq_selftest_wait_expiry(status.data_ptr(), done.data_ptr(), 0, kernels._stream()) == -1
    assert lib.fq_selftest_wait_expiry(status.data_ptr(), done.data_ptr(), 10 ** 10, kernels._stream()) == -1
    # the device is fine afterwards: a tensor-core self-test (fresh tensor-memory allocation) passes
    a = torch.randn(128, 128, device="cuda").bfloat16()
    b = torch.randn(128, 128, device="cuda").bfloat16()
    d = kernels.selftest_umma(a, b, 0)
    ref = a.float() @ b.float().t()
    assert (d - ref).abs().max().item() < 1e-2 * ref.abs().max().item()


@pytest.mark.parametrize("B,T,Hq,Hv,cu", [(2, 256, 2, 4, None), (1, 500, 1, 2, [0, 130, 131, 500]), (1, 2048, 2, 8, None),
                                          (1, 300, 1, 3, [0, 7, 71, 300])])
def test_bwd_chunk_grouped_sums_the_value_heads_in_the_kernel(B, T, Hq, Hv, cu):
    """fq_gdr_bwd_chunk_grouped (dq, dk summed over the V-heads of a QK head inside the kernel: TMA reduce for whole
    chunks, row by row for tails) against fq_gdr_bwd_chunk + fq_group_reduce_pair.  Two V-heads per QK head: bitwise
    equal (one rounding of an exact two-term sum on both paths); more: the partial sums are rounded to bf16 one
    more time per head, so 2^-7 of the maximum is allowed."""
    from oracle import gdr_oracle as orc
    from flashqla_b200 import _lib, kernels, ops
    lib = _lib.load()
    torch.manual_seed(33)
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
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=dev)
    plan = kernels.make_plan(B, T, cu_t, q.device)
    scale = 128 ** -0.5
    gc, A, _, _, _ = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, cu_t, True, False, False)
    _, Ag, Pg = kernels.kkt_solve_gated(k, q, beta, gc, scale, plan, A=A)
    _, h, _ = kernels.fused_gdr_fwd(q, k, v, Ag, None, gc, beta, scale, initial_state=h0, output_final_state=False,
                                    output_h=True, output_o=False, plan=plan)
    dh = torch.empty_like(h)
    cu_p, off_p = plan.ptrs()
    st = kernels._stream()
    _lib.check(lib.fq_gdr_bwd_dh(q.data_ptr(), k.data_ptr(), Ag.data_ptr(), Pg.data_ptr(), do.data_ptr(), gc.data_ptr(),
                                 beta.data_ptr(), dht.data_ptr(), None, dh.data_ptr(), B, T, Hv, Hq, cu_p, off_p, plan.n_seq,
                                 plan.total_chunks, scale, None, st), "fq_gdr_bwd_dh")

    def args(dq, dk, dv, dg, db):
        return (q.data_ptr(), k.data_ptr(), v.data_ptr(), A.data_ptr(), Ag.data_ptr(), Pg.data_ptr(), do.data_ptr(),
                h.data_ptr(), dh.data_ptr(), gc.data_ptr(), beta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                dg.data_ptr(), db.data_ptr(), B, T, Hv, Hq, cu_p, off_p, plan.n_seq, plan.total_chunks, scale, None, st)

    dq_h = torch.empty(B, T, Hv, 128, dtype=torch.bfloat16, device=dev)
    dk_h = torch.empty_like(dq_h)
    dg_r, db_r, dv_r = torch.empty(B, T, Hv, device=dev), torch.empty(B, T, Hv, device=dev), torch.empty_like(v)
    _lib.check(lib.fq_gdr_bwd_chunk(*args(dq_h, dk_h, dv_r, dg_r, db_r)), "fq_gdr_bwd_chunk")
    dq_r = torch.empty(B, T, Hq, 128, dtype=torch.bfloat16, device=dev)
    dk_r = torch.empty_like(dq_r)
    _lib.check(lib.fq_group_reduce_pair(dq_h.data_ptr(), dq_r.data_ptr(), dk_h.data_ptr(), dk_r.data_ptr(), B * T, Hv, Hq, st),
               "fq_group_reduce_pair")
    dq = torch.full((B, T, Hq, 128), float("nan"), dtype=torch.bfloat16, device=dev)
    dk = torch.full_like(dq, float("nan"))
    dg, db, dv = torch.empty(B, T, Hv, device=dev), torch.empty(B, T, Hv, device=dev), torch.full_like(v, float("nan"))
    _lib.check(lib.fq_gdr_bwd_chunk_grouped(*args(dq, dk, dv, dg, db)), "fq_gdr_bwd_chunk_grouped")
    torch.cuda.synchronize()
    valid = torch.zeros(B, T, dtype=torch.bool, device=dev)
    if cu is None:
        valid[:] = True
    else:
        valid[0, :cu[-1]] = True
    assert torch.equal(dv[valid], dv_r[valid]), "dv"
    for name, got, ref in (("dq", dq, dq_r), ("dk", dk, dk_r)):
        got, ref = got[valid], ref[valid]
        assert torch.isfinite(got.float()).all(), name
        if Hv // Hq == 2:
            assert torch.equal(got, ref), f"{name}: not bitwise equal to the two-kernel path"
        else:
            err = (got.float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
            assert err < 2 ** -7, f"{name}: rel-to-max {err:.2e}"
    for name, got, ref in (("dg", dg, dg_r), ("db", db, db_r)):
        err = orc.rel_to_max(got[valid].cpu(), ref[valid].cpu())
        assert err < 1e-5, f"{name}: rel-to-max {err:.2e}"
