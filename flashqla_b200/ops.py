"""Operator interface: same names, argument meaning and return tuples as
``flash_qla/ops/gated_delta_rule/chunk/__init__.py`` of the reference (lines cited per function).
"""
from __future__ import annotations

import os

import torch

from . import _lib, kernels
from .kernels import make_plan

_DEBUG_STATUS = os.environ.get("FLASHQLA_CHECK_STATUS", "0") == "1"


def l2norm(x: torch.Tensor, dim: int = -1, eps: float = 1e-6) -> torch.Tensor:
    """x * rsqrt(sum(x^2) + eps) over the last dim (flash_qla/utils/math.py:7-21)."""
    assert dim == -1
    xf = x.float()
    return (xf * torch.rsqrt((xf * xf).sum(-1, keepdim=True) + eps)).to(x.dtype)


def chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None,
                               output_final_state=True, output_h=False, auto_cp=True):
    """Forward pipeline (chunk/__init__.py:17-67): cumsum -> K K^T + solve -> fused recurrence.

    Returns ``(g_cumsum, A, o, h, final_state)``; ``A`` is the gate-free inverse (opaque, only
    meant to be passed back to ``chunk_gated_delta_rule_bwd``)."""
    B, T, Hg, K = k.shape
    H = v.shape[2]
    if scale is None:
        scale = K ** -0.5
    plan = make_plan(B, T, cu_seqlens, q.device)
    g_cum = kernels.chunk_local_cumsum(g, cu_seqlens=cu_seqlens, plan=plan)
    A = kernels.kkt_solve(k, beta, plan=plan)
    status = kernels._status_tensor(q.device) if _DEBUG_STATUS else None
    o, h, final_state = kernels.fused_gdr_fwd(q, k, v, A, g_cum, beta, scale, initial_state=initial_state,
                                              output_final_state=output_final_state, output_h=output_h,
                                              plan=plan, status=status)
    if status is not None:
        kernels.check_status(status, "fq_gdr_fwd")
    return g_cum, A, o, h, final_state
