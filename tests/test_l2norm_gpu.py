"""Fused q/k L2 normalisation (the operator's use_qk_l2norm_in_kernel flag) against plain torch in fp32."""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu


def _ref(x, eps=1e-6):
    xf = x.float()
    return xf * torch.rsqrt((xf * xf).sum(-1, keepdim=True) + eps)


@pytest.mark.parametrize("shape", [(1, 7, 3, 128), (2, 513, 4, 128), (1, 1, 1, 128)])
def test_l2norm_forward_backward(shape):
    from flashqla_b200 import ops
    torch.manual_seed(0)
    x = (3.0 * torch.randn(*shape)).bfloat16().cuda().requires_grad_()
    dy = torch.randn(*shape).bfloat16().cuda()
    y = ops.l2norm(x)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = _ref(xr)
    yr.backward(dy.float())
    # bf16 outputs: half an ulp of values up to 1 is 2^-9
    assert (y.float() - yr).abs().max().item() <= 4e-3
    assert orc.rel_to_max(x.grad.float().cpu(), xr.grad.cpu()) < 1e-2


def test_operator_flag_equals_prenormalised_inputs():
    import flash_qla
    torch.manual_seed(1)
    B, T, Hq, Hv = 2, 200, 2, 4
    dev = "cuda"
    q = torch.randn(B, T, Hq, 128).bfloat16().to(dev)
    k = torch.randn(B, T, Hq, 128).bfloat16().to(dev)
    v = torch.randn(B, T, Hv, 128).bfloat16().to(dev)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, Hv)).to(dev)
    beta = torch.randn(B, T, Hv).sigmoid().to(dev)
    do = torch.randn(B, T, Hv, 128).bfloat16().to(dev)
    # with the flag
    q1, k1 = q.clone().requires_grad_(), k.clone().requires_grad_()
    o1, _ = flash_qla.chunk_gated_delta_rule(q1, k1, v, g, beta, use_qk_l2norm_in_kernel=True)
    (o1.float() * do.float()).sum().backward()
    # reference: normalise in fp32 torch (rounded to bf16 like the kernel's output), differentiate through it
    q2, k2 = q.clone().float().requires_grad_(), k.clone().float().requires_grad_()
    o2, _ = flash_qla.chunk_gated_delta_rule(_ref(q2).bfloat16(), _ref(k2).bfloat16(), v, g, beta)
    (o2.float() * do.float()).sum().backward()
    assert orc.rel_to_max(o1.float().cpu(), o2.float().cpu()) < 1e-2
    assert orc.rel_to_max(q1.grad.float().cpu(), q2.grad.cpu()) < 1.5e-2
    assert orc.rel_to_max(k1.grad.float().cpu(), k2.grad.cpu()) < 1.5e-2
