"""The public operator without host synchronisation: variable-length batches planned from a host copy of
``cu_seqlens``, capture of forward + backward into a CUDA graph, and the float16 entry (computed as bfloat16).

Device-side / sync-free planning is the open TODO at flash_qla/utils/index.py:76 and
flash_qla/ops/gated_delta_rule/chunk/cp_context.py:38 of the reference (its planner reads the device tensor back).
"""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _no_status_readback(monkeypatch):
    """Other test modules switch on the debug read-back of the kernels' status word (a synchronisation by design);
    these tests run the operator as a user does, without it."""
    from flashqla_b200 import ops
    monkeypatch.setenv("FLASHQLA_CHECK_STATUS", "0")
    monkeypatch.setattr(ops, "_DEBUG_STATUS", False)


def _inputs(seed, B, T, Hq, Hv, n_seq=None, dtype=torch.bfloat16):
    torch.manual_seed(seed)
    N = B if n_seq is None else n_seq
    dev = "cuda"
    q = orc.l2norm(torch.randn(B, T, Hq, 128)).to(dtype).to(dev)
    k = orc.l2norm(torch.randn(B, T, Hq, 128)).to(dtype).to(dev)
    v = torch.randn(B, T, Hv, 128).to(dtype).to(dev)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, Hv)).to(dev)
    beta = torch.randn(B, T, Hv).sigmoid().to(dev)
    h0 = (0.1 * torch.randn(N, Hv, 128, 128)).to(dev)
    return q, k, v, g, beta, h0


def _same(got, want):
    """(o, final_state, dq, dk, dv, dg, dbeta, dh0): everything bitwise except dg and dbeta, which the backward sums
    with shared-memory atomics whose order varies from run to run (those to 1e-4 of their maximum)."""
    for i, (a, b) in enumerate(zip(got, want)):
        if i in (5, 6):
            assert (a.float() - b.float()).abs().max() <= 1e-4 * b.float().abs().max()
        else:
            assert torch.equal(a, b), i


def _fwd_bwd(q, k, v, g, beta, h0, do, dht, **kw):
    from flashqla_b200 import chunk_gated_delta_rule
    leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v, g, beta, h0)]
    o, ht = chunk_gated_delta_rule(*leaves[:5], initial_state=leaves[5], output_final_state=True, **kw)
    torch.autograd.backward([o, ht], [do, dht])
    return [o.detach(), ht.detach()] + [t.grad for t in leaves]


def test_varlen_from_host_copy_does_not_synchronise():
    """First use of a new cu_seqlens pair under torch's sync detector: planning, forward and backward must not
    synchronise; results equal the call that reads the device tensor back."""
    lens = [0, 70, 64, 1, 1300, 5000, 129]
    cu_list = [0]
    for n in lens:
        cu_list.append(cu_list[-1] + n)
    T = cu_list[-1]
    q, k, v, g, beta, h0 = _inputs(5, 1, T, 2, 4, n_seq=len(lens))
    do = torch.randn_like(v)
    dht = 0.01 * torch.randn_like(h0)
    cu_dev = torch.tensor(cu_list, dtype=torch.int32, device="cuda")
    ref = _fwd_bwd(q, k, v, g, beta, h0, do, dht, cu_seqlens=cu_dev)  # also warms up one-time kernel attributes
    torch.cuda.synchronize()
    cu_dev2 = cu_dev.clone()                      # a tensor object the plan cache has not seen
    cu_cpu = torch.tensor(cu_list, dtype=torch.int32)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        got = _fwd_bwd(q, k, v, g, beta, h0, do, dht, cu_seqlens=cu_dev2, cu_seqlens_cpu=cu_cpu)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    _same(got, ref)


@pytest.mark.parametrize("varlen", [False, True])
def test_forward_backward_in_a_cuda_graph(varlen):
    """Capture forward + backward once, replay on new data in the static buffers, compare with eager calls."""
    from flashqla_b200 import chunk_gated_delta_rule
    if varlen:
        cu_list = [0, 100, 1124, 1124, 3000]
        B, T, n_seq = 1, cu_list[-1], len(cu_list) - 1
        kw = dict(cu_seqlens=torch.tensor(cu_list, dtype=torch.int32, device="cuda"),
                  cu_seqlens_cpu=torch.tensor(cu_list, dtype=torch.int32))
    else:
        B, T, n_seq = 2, 1536, 2
        kw = {}
    Hq, Hv = 2, 4
    static = [t.clone().requires_grad_(True) for t in _inputs(11, B, T, Hq, Hv, n_seq=n_seq)]
    do = torch.randn(B, T, Hv, 128, device="cuda").bfloat16()
    dht = 0.01 * torch.randn(n_seq, Hv, 128, 128, device="cuda")

    def step():
        o, ht = chunk_gated_delta_rule(*static[:5], initial_state=static[5], output_final_state=True, **kw)
        grads = torch.autograd.grad([o, ht], static, [do, dht])
        return (o, ht) + tuple(grads)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):  # warm-up outside capture: plan cache, kernel attributes, allocator pools
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    for seed in (21, 22):
        fresh = _inputs(seed, B, T, Hq, Hv, n_seq=n_seq)
        with torch.no_grad():
            for dst, src in zip(static, fresh):
                dst.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        got = [t.clone() for t in outs]
        want = _fwd_bwd(*fresh, do, dht, **kw)
        torch.cuda.synchronize()
        _same(got, want)


def test_float16_inputs_are_computed_as_bfloat16():
    """float16 q/k/v: outputs and gradients come back as float16 and agree with the fp32 oracle on the same
    (bfloat16-rounded) inputs within the bf16 tolerance max|x - ref| <= 1e-2 * max|ref|."""
    from flashqla_b200 import chunk_gated_delta_rule
    B, T, Hq, Hv = 1, 300, 2, 2
    q, k, v, g, beta, h0 = _inputs(3, B, T, Hq, Hv, dtype=torch.float16)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    o, ht = chunk_gated_delta_rule(*leaves, g, beta, initial_state=h0, output_final_state=True)
    assert o.dtype == torch.float16 and ht.dtype == torch.float32
    do = torch.randn_like(o)
    o.backward(do)
    assert all(t.grad.dtype == torch.float16 for t in leaves)
    qb, kb, vb = (t.detach().bfloat16().float().cpu() for t in (q, k, v))
    _, _, o_ref, _, ht_ref = orc.gdr_fwd(qb, kb, vb, g.cpu(), beta.cpu(), scale=128 ** -0.5, initial_state=h0.cpu())
    assert (o.float().cpu() - o_ref).abs().max() <= 1e-2 * o_ref.abs().max()
    assert (ht.cpu() - ht_ref).abs().max() <= 5e-3 * ht_ref.abs().max()
