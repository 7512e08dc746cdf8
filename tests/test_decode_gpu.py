"""Token-by-token recurrence kernel (decode step) against the fp64 token-level oracle, and its hand-over with the
chunked operator: prefill + continuation must equal one chunked pass over the whole sequence."""
import pytest
import torch

from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-2   # rel-to-max on o (bf16 outputs), same bound as the forward tests
TOL_S = 5e-3  # final state (fp32)


def _inputs(seed, N, T, Hq, Hv):
    torch.manual_seed(seed)
    q = orc.l2norm(torch.randn(N, T, Hq, 128)).bfloat16()
    k = orc.l2norm(torch.randn(N, T, Hq, 128)).bfloat16()
    v = torch.randn(N, T, Hv, 128).bfloat16()
    g = torch.nn.functional.logsigmoid(torch.randn(N, T, Hv))
    beta = torch.randn(N, T, Hv).sigmoid()
    h0 = 0.1 * torch.randn(N, Hv, 128, 128)
    return q, k, v, g, beta, h0


@pytest.mark.parametrize("N,T,Hq,Hv,with_h0", [(3, 1, 2, 2, True), (2, 5, 1, 4, True), (1, 3, 2, 2, False), (5, 2, 4, 8, True)])
def test_recurrent_vs_token_oracle(N, T, Hq, Hv, with_h0):
    from flashqla_b200 import fused_recurrent_gated_delta_rule
    q, k, v, g, beta, h0 = _inputs(3, N, T, Hq, Hv)
    h0 = h0 if with_h0 else None
    o_ref, s_ref = orc.gdr_recurrent(q.float(), k.float(), v.float(), g, beta, None, h0)
    dev = "cuda"
    o, s = fused_recurrent_gated_delta_rule(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev),
                                            initial_state=None if h0 is None else h0.to(dev))
    assert orc.rel_to_max(o.float().cpu(), o_ref) < TOL
    assert orc.rel_to_max(s.cpu(), s_ref) < TOL_S


def test_inplace_state_and_errors():
    from flashqla_b200 import _lib, fused_recurrent_gated_delta_rule
    q, k, v, g, beta, h0 = _inputs(4, 2, 1, 2, 2)
    dev = "cuda"
    st = h0.to(dev).clone()
    o1, s1 = fused_recurrent_gated_delta_rule(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), initial_state=h0.to(dev))
    o2, s2 = fused_recurrent_gated_delta_rule(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev), initial_state=st,
                                              inplace_state=True)
    assert s2.data_ptr() == st.data_ptr()
    assert torch.equal(o1, o2) and torch.equal(s1, st)
    with pytest.raises(_lib.FlashQLAError):
        fused_recurrent_gated_delta_rule(q.to(dev).half(), k.to(dev).half(), v.to(dev).half(), g.to(dev), beta.to(dev))
    with pytest.raises(ValueError):
        fused_recurrent_gated_delta_rule(q.to(dev), k.to(dev), v.to(dev), g.to(dev), beta.to(dev),
                                         initial_state=h0.to(dev)[:, :1])


def test_prefill_then_decode_equals_one_chunked_pass():
    import flash_qla
    from flashqla_b200 import fused_recurrent_gated_delta_rule
    N, T, Td, Hq, Hv = 2, 200, 3, 2, 4
    q, k, v, g, beta, h0 = _inputs(5, N, T + Td, Hq, Hv)
    dev = "cuda"
    qd, kd, vd, gd, bd, hd = (x.to(dev) for x in (q, k, v, g, beta, h0))
    o_all, s_all = flash_qla.chunk_gated_delta_rule(qd, kd, vd, gd, bd, initial_state=hd, output_final_state=True)
    o_pre, s_pre = flash_qla.chunk_gated_delta_rule(qd[:, :T].contiguous(), kd[:, :T].contiguous(), vd[:, :T].contiguous(),
                                                    gd[:, :T].contiguous(), bd[:, :T].contiguous(), initial_state=hd,
                                                    output_final_state=True)
    o_dec, s_dec = fused_recurrent_gated_delta_rule(qd[:, T:].contiguous(), kd[:, T:].contiguous(), vd[:, T:].contiguous(),
                                                    gd[:, T:].contiguous(), bd[:, T:].contiguous(), initial_state=s_pre)
    assert orc.rel_to_max(o_dec.float().cpu(), o_all[:, T:].float().cpu()) < TOL
    assert orc.rel_to_max(s_dec.cpu(), s_all.cpu()) < TOL_S
