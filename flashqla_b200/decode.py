"""Token-by-token gated delta rule (decode / short continuations after a chunked prefill).

The reference library covers prefill and training only; its forward hands a ``final_state`` to the caller
(``flash_qla/ops/gated_delta_rule/chunk/hopper/fused_fwd.py:214-221``) and takes it back as ``initial_state``
(``:173-179``).  This module is the step on the other side of that hand-over: it advances the state by the new
tokens of every sequence with one HBM-bound kernel (``csrc/decode.cu``).
"""
from __future__ import annotations

import torch

from . import _lib, kernels


def fused_recurrent_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=True,
                                     inplace_state=False):
    """``q, k [N,T,Hg,128]``, ``v [N,T,H,128]`` bf16; ``g`` (log gate per token, not cumulated) and ``beta``
    ``[N,T,H]``; ``initial_state [N,H,128,128]`` fp32 or None.  Returns ``(o [N,T,H,128] bf16, final_state)``.

    With ``inplace_state`` the new state overwrites ``initial_state`` (no second 64 KiB per head is allocated).
    Same arithmetic as the chunked operator: ``chunk_gated_delta_rule`` on the prefix followed by this function on
    the continuation equals ``chunk_gated_delta_rule`` on the whole sequence up to bf16 rounding."""
    kernels._require_cuda(q, k, v, g, beta)
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise _lib.FlashQLAError("fused_recurrent_gated_delta_rule: q, k, v must be bfloat16")
    N, T, Hg, K = k.shape
    H, V = v.shape[2], v.shape[3]
    if K != 128 or V != 128:
        raise _lib.FlashQLAError("fused_recurrent_gated_delta_rule: head dims must be 128")
    if H % Hg != 0:
        raise _lib.FlashQLAError("fused_recurrent_gated_delta_rule: H must be a multiple of Hg")
    if scale is None:
        scale = K ** -0.5
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    g = g.contiguous() if g.dtype == torch.float32 else g.float().contiguous()
    bt = beta.contiguous() if beta.dtype == torch.float32 else beta.float().contiguous()
    st_in = None
    if initial_state is not None:
        if tuple(initial_state.shape) != (N, H, K, V):
            raise ValueError(f"initial_state must be [{N}, {H}, {K}, {V}], got {tuple(initial_state.shape)}")
        if inplace_state and not (initial_state.dtype == torch.float32 and initial_state.is_contiguous()):
            raise _lib.FlashQLAError("inplace_state needs a contiguous float32 initial_state")
        st_in = initial_state if inplace_state else initial_state.float().contiguous()
    if inplace_state and st_in is None:
        raise _lib.FlashQLAError("inplace_state needs an initial_state")
    st_out = None
    if output_final_state or inplace_state:
        st_out = st_in if inplace_state else torch.empty(N, H, K, V, dtype=torch.float32, device=q.device)
    o = torch.empty_like(v)
    pp = lambda t: None if t is None else t.data_ptr()
    rc = _lib.load().fq_gdr_recurrent(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), bt.data_ptr(), pp(st_in),
                                      pp(st_out), o.data_ptr(), N, T, H, Hg, float(scale), kernels._stream())
    _lib.check(rc, "fq_gdr_recurrent")
    return o, (st_out if output_final_state else None)
