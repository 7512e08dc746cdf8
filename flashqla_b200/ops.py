"""Operator interface: same names, argument meaning and return tuples as
``flash_qla/ops/gated_delta_rule/chunk/__init__.py`` of the reference (lines cited per function).
"""
from __future__ import annotations

import os

import torch

from . import _lib, kernels
from .kernels import make_plan
from .planner import plan_cp

_DEBUG_STATUS = os.environ.get("FLASHQLA_CHECK_STATUS", "0") == "1"
# testing hook: force a piece length (in chunks) for the context-parallel split
_FORCE_PIECE_CHUNKS = int(os.environ["FLASHQLA_PIECE_CHUNKS"]) if "FLASHQLA_PIECE_CHUNKS" in os.environ else None
# The autograd function keeps the gated operand tiles A_g and P_g (2 x [B,T,H,64] bf16) for the backward, which then
# skips the pass that rebuilds them; set FLASHQLA_RECOMPUTE_TILES=1 to keep only A, like the reference does.
_RECOMPUTE_TILES = os.environ.get("FLASHQLA_RECOMPUTE_TILES", "0") == "1"
# It also keeps the bf16 state before every chunk (32 KiB per chunk and V-head, written by the forward kernel on its way)
# when that tensor stays below this budget, so that the backward need not recompute it with a second state pass; larger
# problems (and FLASHQLA_KEEP_STATES_MB=0) recompute like the reference does.
_KEEP_STATES_BYTES = int(float(os.environ.get("FLASHQLA_KEEP_STATES_MB", "8192")) * (1 << 20))


class _L2NormFunction(torch.autograd.Function):
    """x * rsqrt(sum(x^2) + eps) over the last dim (128) with the fused kernels of csrc/l2norm.cu."""

    @staticmethod
    def forward(ctx, x, eps):
        x = x.contiguous()
        y = torch.empty_like(x)
        rc = _lib.load().fq_l2norm_fwd(x.data_ptr(), y.data_ptr(), x.numel() // x.shape[-1], float(eps), kernels._stream())
        _lib.check(rc, "fq_l2norm_fwd")
        ctx.save_for_backward(x)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy.contiguous().to(x.dtype)
        dx = torch.empty_like(x)
        rc = _lib.load().fq_l2norm_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel() // x.shape[-1],
                                       float(ctx.eps), kernels._stream())
        _lib.check(rc, "fq_l2norm_bwd")
        return dx, None


def l2norm(x: torch.Tensor, dim: int = -1, eps: float = 1e-6) -> torch.Tensor:
    """x * rsqrt(sum(x^2) + eps) over the last dim (flash_qla/utils/math.py:7-21), differentiable.
    One fused pass over HBM per direction; bf16 CUDA tensors with a last dim of 128 only."""
    assert dim == -1
    kernels._require_cuda(x)
    if x.dtype != torch.bfloat16 or x.shape[-1] != 128:
        raise _lib.FlashQLAError("l2norm: bfloat16 tensors with a last dimension of 128 only")
    return _L2NormFunction.apply(x, eps)


def chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None,
                               output_final_state=True, output_h=False, auto_cp=True, _return_tiles=None, _plan=None,
                               _want_A=True, _act=None, _keep_h=False):
    """Forward pipeline (chunk/__init__.py:17-67): [cumsum + K K^T + solve + gated tiles] -> fused recurrence.

    Returns ``(g_cumsum, A, o, h, final_state)``; ``A`` is the gate-free inverse (opaque, only
    meant to be passed back to ``chunk_gated_delta_rule_bwd``).  With ``auto_cp`` long sequences are
    split into pieces that run as independent CTAs (context parallel inside the GPU)."""
    B, T, Hg, K = k.shape
    H = v.shape[2]
    if scale is None:
        scale = K ** -0.5
    plan = _plan if _plan is not None else make_plan(B, T, cu_seqlens, q.device)
    # the cumsum of g is formed in the same launch; A is only stored if a backward may follow.  The second gated tile
    # P_g is formed inside the recurrence kernel, which also stores it when the caller keeps the tiles for a backward.
    if _act is None:
        g_cum, A, Ag, _ = kernels.kkt_solve_fused(k, q, beta, g, scale, plan, want_A=_want_A)
    else:
        # g / beta are RAW inputs: the tile kernel applies the activations; from here on `beta` is the activated one
        gate_mode, beta_mode, A_log, dt_bias = _act
        g_cum, beta, A, Ag = kernels.kkt_solve_fused_act(k, beta, g, scale, plan, gate_mode, beta_mode, A_log, dt_bias,
                                                         want_A=_want_A)
    Pg = kernels._tile_alloc(plan, B, T)(B, T, H, kernels.CHUNK, dtype=k.dtype, device=k.device) if _return_tiles else None
    status = kernels._status_tensor(q.device) if _DEBUG_STATUS else None
    cp = warm = None
    if auto_cp:
        cp = plan_cp(plan, B, T, H, kernels.sm_count(q.device), q.device, piece_chunks=_FORCE_PIECE_CHUNKS)
        if cp is not None:
            warm = kernels.cp_warmup(g_cum, cp, H)
    keep_h = _keep_h and plan.total_chunks * H * K * v.shape[-1] * 2 <= _KEEP_STATES_BYTES
    o, h, final_state = kernels.fused_gdr_fwd(q, k, v, Ag, Pg, g_cum, beta, scale, initial_state=initial_state,
                                              output_final_state=output_final_state, output_h=output_h or keep_h,
                                              plan=plan, cp=cp, warmup=warm, status=status)
    if status is not None:
        kernels.check_status(status, "fq_gdr_fwd")
    h_kernel = h if keep_h else None  # [.., V, K] as the kernels store and read it
    if h is not None:
        h = h.transpose(-1, -2) if output_h else None  # the interface is [.., K, V]
    if _return_tiles is not None:
        return g_cum, A, o, h, final_state, ((Ag, Pg, h_kernel) if _return_tiles else None), beta
    return g_cum, A, o, h, final_state


def chunk_gated_delta_rule_bwd(q, k, v, g, beta, A, do, dht=None, scale=None, initial_state=None, cu_seqlens=None,
                               _gated_tiles=None, _plan=None, _want_dh0=None, _h_saved=None):
    """Backward pipeline (chunk/__init__.py:70-113).  ``g`` is the cumsum returned by the forward,
    ``A`` the tensor returned by the forward.  Returns ``(dq, dk, dv, db, dg, dh0)``; ``dh0`` is None when
    neither ``dht`` nor ``initial_state`` is given (``_want_dh0`` overrides that rule)."""
    from . import bwd  # the backward kernels live in their own module
    return bwd.chunk_gated_delta_rule_bwd(q, k, v, g, beta, A, do, dht, scale, initial_state, cu_seqlens,
                                          gated_tiles=_gated_tiles, plan=_plan, want_dh0=_want_dh0, h_saved=_h_saved)


class ChunkGatedDeltaRuleFunction(torch.autograd.Function):
    """Autograd glue (chunk/__init__.py:116-180): saves (q, k, v, g_cumsum, beta, A, h0, cu_seqlens) and, unless
    FLASHQLA_RECOMPUTE_TILES=1, the gated tiles A_g and P_g; neither o nor the per-chunk states are kept.
    With ``gate_mode`` / ``beta_mode`` != 0 the inputs g / beta are raw pre-activations (see ``chunk_gated_delta_rule``):
    the activations run inside the tile kernel and their derivatives inside one elementwise backward kernel."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
                plan=None, A_log=None, dt_bias=None, gate_mode=0, beta_mode=0):
        # without a gradient to come (inference / prefill) neither A nor anything else is kept
        needs_bwd = any(ctx.needs_input_grad)
        act = (gate_mode, beta_mode, A_log, dt_bias) if (gate_mode or beta_mode) else None
        g_cum, A, o, _, final_state, tiles, beta_act = chunk_gated_delta_rule_fwd(
            q=q, k=k, v=v, g=g, beta=beta, scale=scale, initial_state=initial_state,
            output_final_state=output_final_state, output_h=False, cu_seqlens=cu_seqlens,
            _return_tiles=needs_bwd and not _RECOMPUTE_TILES, _plan=plan, _want_A=needs_bwd, _act=act,
            _keep_h=needs_bwd and not _RECOMPUTE_TILES)
        if not needs_bwd:
            return o.to(q.dtype), final_state
        ctx.plan = plan  # the backward reuses the forward's sequence plan (no second look at cu_seqlens)
        ctx.keep_tiles = not _RECOMPUTE_TILES
        ctx.act = act is not None
        ctx.modes = (gate_mode, beta_mode)
        extra = (g, beta, A_log, dt_bias) if act is not None else ()
        ctx.keep_h = False
        if ctx.keep_tiles:
            Ag, Pg, h_kernel = tiles
            ctx.keep_h = h_kernel is not None
            kept = (Ag, Pg, h_kernel) if ctx.keep_h else (Ag, Pg)
            ctx.save_for_backward(q, k, v, g_cum, beta_act, A, initial_state, cu_seqlens, *kept, *extra)
        else:
            ctx.save_for_backward(q, k, v, g_cum, beta_act, A, initial_state, cu_seqlens, *extra)
        ctx.scale = scale
        ctx.g_dtype = g.dtype
        ctx.beta_dtype = beta.dtype
        return o.to(q.dtype), final_state

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, do, dht):
        q, k, v, g_cum, beta, A, initial_state, cu_seqlens = ctx.saved_tensors[:8]
        n = 8
        tiles = None
        h_saved = None
        if ctx.keep_tiles:
            tiles = tuple(ctx.saved_tensors[8:10])
            n = 10
            if ctx.keep_h:
                h_saved = ctx.saved_tensors[10]
                n = 11
        # a gradient for the initial state is formed only if one was passed in and asks for it: returning a tensor
        # for an input that was None (initial_state=None with output_final_state=True, the first segment of a
        # truncated back-propagation) is an autograd error
        need_dh0 = initial_state is not None and ctx.needs_input_grad[6]
        dq, dk, dv, db, dg, dh0 = chunk_gated_delta_rule_bwd(
            q=q, k=k, v=v, g=g_cum, beta=beta, A=A, do=do, dht=dht, scale=ctx.scale,
            initial_state=initial_state, cu_seqlens=cu_seqlens, _gated_tiles=tiles, _plan=ctx.plan,
            _want_dh0=need_dh0, _h_saved=h_saved)
        dA_log = ddt_bias = None
        if ctx.act:
            g_raw, b_raw, A_log, dt_bias = ctx.saved_tensors[n:n + 4]
            dg, db, dA_log, ddt_bias = kernels.gate_act_bwd(dg, db, g_raw, b_raw, ctx.modes[0], ctx.modes[1], A_log, dt_bias)
            if dA_log is not None:
                dA_log = dA_log.to(A_log.dtype)
            if ddt_bias is not None:
                ddt_bias = ddt_bias.to(dt_bias.dtype)
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dg.to(ctx.g_dtype), db.to(ctx.beta_dtype),
                None, dh0, None, None, None, dA_log, ddt_bias, None, None)


@torch.compiler.disable
def chunk_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, cu_seqlens=None, head_first=False, cu_seqlens_cpu=None,
                           use_gate_in_kernel=False, A_log=None, dt_bias=None, use_beta_sigmoid_in_kernel=False):
    """Public, differentiable entry (chunk/__init__.py:183-237).  Returns ``(o, final_state)``.

    Not in the reference:
    ``cu_seqlens_cpu`` is an optional host copy of ``cu_seqlens``; with it the variable-length schedule is made
    without reading the device tensor back, so the call neither synchronises nor blocks capture into a CUDA graph.
    ``use_gate_in_kernel``: ``g`` is the RAW gate input and the activation runs inside the tile kernel:
    ``g = logsigmoid(g)`` or, when ``A_log`` ([H]) is given, ``g = -exp(A_log) * softplus(g + dt_bias)`` (``dt_bias`` [H]
    optional); ``use_beta_sigmoid_in_kernel``: ``beta`` is raw and ``sigmoid`` runs in the kernel.  Gradients flow to
    the raw inputs (and to ``A_log`` / ``dt_bias``)."""
    assert q.dtype == k.dtype == v.dtype
    assert q.dtype != torch.float32, (
        "ChunkGatedDeltaRuleFunction does not support float32. Please use bfloat16 or float16.")
    assert not head_first, "head_first=True is not supported."
    assert v.shape[2] % k.shape[2] == 0, "num_qk_heads must be divisible to num_v_heads."
    if q.dtype == torch.float16:
        # The kernels are built for bfloat16 operands only.  float16 inputs are cast in and the output cast back (one
        # extra elementwise pass per tensor; autograd casts the gradients the same way), so the arithmetic is bfloat16.
        o, final_state = chunk_gated_delta_rule(q.bfloat16(), k.bfloat16(), v.bfloat16(), g, beta, scale, initial_state,
                                                output_final_state, use_qk_l2norm_in_kernel, cu_seqlens, head_first,
                                                cu_seqlens_cpu, use_gate_in_kernel, A_log, dt_bias,
                                                use_beta_sigmoid_in_kernel)
        return o.to(torch.float16), final_state
    if q.dtype != torch.bfloat16:
        raise _lib.FlashQLAError("the sm_100a kernels take bfloat16 (or float16, computed as bfloat16) q/k/v")
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
                f"Please flatten variable-length inputs before processing.")
        if initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input sequences, "
                f"i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}.")
    if A_log is not None and not use_gate_in_kernel:
        raise ValueError("A_log / dt_bias are only used with use_gate_in_kernel=True")
    if scale is None:
        scale = k.shape[-1] ** -0.5
    if use_qk_l2norm_in_kernel:
        q = l2norm(q)
        k = l2norm(k)
    gate_mode = (2 if A_log is not None else 1) if use_gate_in_kernel else 0
    beta_mode = 1 if use_beta_sigmoid_in_kernel else 0
    plan = make_plan(q.shape[0], q.shape[1], cu_seqlens, q.device, host=cu_seqlens_cpu)
    return ChunkGatedDeltaRuleFunction.apply(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                                             plan, A_log, dt_bias, gate_mode, beta_mode)
