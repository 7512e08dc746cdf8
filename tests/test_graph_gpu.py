"""The differentiable operator inside a CUDA graph: one captured forward + backward step, replayed, must give the same
bits as the eager step (dense with the context-parallel split engaged; packed with a host copy of cu_seqlens)."""
import pytest
import torch

import flashqla_b200 as fq

pytestmark = pytest.mark.gpu


def _inputs(B, T, Hq, Hv, n_state, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=gen)
    q = torch.nn.functional.normalize(r(B, T, Hq, 128), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(r(B, T, Hq, 128), dim=-1).bfloat16()
    v = r(B, T, Hv, 128).bfloat16()
    g = torch.nn.functional.logsigmoid(r(B, T, Hv))
    beta = r(B, T, Hv).sigmoid()
    h0 = 0.1 * r(n_state, Hv, 128, 128)
    do = r(B, T, Hv, 128).bfloat16()
    dht = 0.1 * r(n_state, Hv, 128, 128)
    return [x.requires_grad_() for x in (q, k, v, g, beta, h0)], do, dht


@pytest.mark.parametrize("packed", [False, True])
def test_captured_step_equals_eager(packed):
    if packed:
        cu_host = torch.tensor([0, 700, 1900, 4096], dtype=torch.int32)
        cu = cu_host.cuda()
        leaves, do, dht = _inputs(1, 4096, 2, 4, 3, 11)
        kw = dict(cu_seqlens=cu, cu_seqlens_cpu=cu_host)
    else:
        leaves, do, dht = _inputs(1, 8192, 2, 4, 1, 12)
        kw = {}
    out = {}

    def step():
        for x in leaves:
            x.grad = None
        o, fs = fq.chunk_gated_delta_rule(*leaves[:5], initial_state=leaves[5], output_final_state=True, **kw)
        torch.autograd.backward([o, fs], [do, dht])
        out["o"], out["fs"] = o, fs

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    eager = [out["o"].clone(), out["fs"].clone()] + [x.grad.clone() for x in leaves]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    held = [out["o"], out["fs"]] + [x.grad for x in leaves]   # the graph's own output tensors
    for t in held:
        t.zero_()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    names = ["o", "final_state", "dq", "dk", "dv", "dg", "dbeta", "dh0"]
    for n, a, b in zip(names, eager, held):
        if n in ("dg", "dbeta"):  # row sums gathered with shared-memory atomics: equal up to the order of those sums
            assert torch.allclose(a, b, rtol=1e-4, atol=1e-4 * a.abs().max().item()), \
                f"{n}: max abs {(a - b).abs().max().item():.3e} of {a.abs().max().item():.3e}"
            continue
        assert torch.equal(a, b), f"{n}: the replayed step differs from the eager one (max abs {(a.float() - b.float()).abs().max().item():.3e})"
