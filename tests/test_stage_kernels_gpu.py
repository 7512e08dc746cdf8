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
