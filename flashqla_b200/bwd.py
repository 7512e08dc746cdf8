"""Backward orchestration (flash_qla/ops/gated_delta_rule/chunk/__init__.py:70-113 of the reference):
state recompute -> reverse dS recurrence -> chunk-parallel gradients -> GVA head sum -> reverse cumsum."""
from __future__ import annotations

import os

import torch

from . import _lib, kernels
from .kernels import make_plan
from .planner import plan_cp


def chunk_gated_delta_rule_bwd(q, k, v, g, beta, A, do, dht=None, scale=None, initial_state=None, cu_seqlens=None,
                               gated_tiles=None, plan=None, want_dh0=None, h_saved=None):
    """``gated_tiles`` = (A_g, P_g) as produced by the forward for the same inputs; when given, the pass that
    rebuilds them from ``A`` is skipped (the autograd function keeps them unless FLASHQLA_RECOMPUTE_TILES=1).
    ``h_saved``: the bf16 state before every chunk as the forward kernel stored it ([.., V, K]); when given, the state
    pass that recomputes it is skipped."""
    kernels._require_cuda(q, k, v, g, beta, A, do)
    if q.dtype != torch.bfloat16:
        raise _lib.FlashQLAError("chunk_gated_delta_rule_bwd: only bfloat16 q/k/v are supported")
    B, T, Hg, K = k.shape
    H, V = v.shape[2], v.shape[3]
    if scale is None:
        scale = K ** -0.5
    dev = q.device
    plan = plan if plan is not None else make_plan(B, T, cu_seqlens, dev)
    check = os.environ.get("FLASHQLA_CHECK_STATUS", "0") == "1"
    status = kernels._status_tensor(dev) if check else None
    st_p = None if status is None else status.data_ptr()
    q, k, v, A, do = q.contiguous(), k.contiguous(), v.contiguous(), A.contiguous(), do.contiguous()
    if do.dtype != q.dtype:
        do = do.to(q.dtype)
    g = g.contiguous() if g.dtype == torch.float32 else g.float().contiguous()
    bt = beta.contiguous() if beta.dtype == torch.float32 else beta.float().contiguous()
    h0 = None
    if initial_state is not None:
        h0 = initial_state.contiguous() if initial_state.dtype == torch.float32 else initial_state.float().contiguous()
    dht_c = None
    if dht is not None:
        dht_c = dht.contiguous() if dht.dtype == torch.float32 else dht.float().contiguous()

    # 1. gated tiles from the given A, then the state before every chunk (bf16) with the forward
    #    recurrence kernel in state-only mode (context parallel like the forward)
    if gated_tiles is not None:
        Ag, Pg = gated_tiles
    else:
        _, Ag, Pg = kernels.kkt_solve_gated(k, q, bt, g, scale, plan, A=A)
    from . import ops as _ops
    cp = plan_cp(plan, B, T, H, kernels.sm_count(dev), dev, piece_chunks=_ops._FORCE_PIECE_CHUNKS)
    warm = h0_piece = tmats = None
    if cp is not None:
        # gate scans in both directions; pairs that would replay too far start from corrected states / gradients
        warm = kernels.cp_warmup(g, cp, H, with_reverse=True)
        h0_piece, tmats = kernels.cp_correct_states(q, k, v, Ag, g, bt, scale, h0, cp, warm, status, return_bt=True)
    if h_saved is not None:
        h = h_saved
    else:
        _, h, _ = kernels.fused_gdr_fwd(q, k, v, Ag, None, g, bt, scale, initial_state=h0, output_final_state=False,
                                        output_h=True, output_o=False, plan=plan, cp=cp, warmup=warm, status=status,
                                        h0_piece=h0_piece)
    # 2. reverse recurrence of the state gradient
    dh = torch.empty_like(h)
    if want_dh0 is None:
        want_dh0 = (dht is not None) or (initial_state is not None)
    dh0 = torch.empty(plan.n_seq, H, K, V, dtype=torch.float32, device=dev) if want_dh0 else None
    cu_p, off_p = plan.ptrs()
    lib = _lib.load()
    pp = lambda t: None if t is None else t.data_ptr()
    if cp is None:
        rc = lib.fq_gdr_bwd_dh(q.data_ptr(), k.data_ptr(), Ag.data_ptr(), Pg.data_ptr(), do.data_ptr(), g.data_ptr(),
                               bt.data_ptr(), pp(dht_c), pp(dh0), dh.data_ptr(), B, T, H, Hg,
                               cu_p, off_p, plan.n_seq, plan.total_chunks, float(scale), st_p, kernels._stream())
    else:
        P = cp.n_pieces
        args = (q.data_ptr(), k.data_ptr(), Ag.data_ptr(), Pg.data_ptr(), do.data_ptr(), g.data_ptr(), bt.data_ptr(),
                pp(dht_c))
        tail = (1, B * T, H, Hg, cp.cu_seqlens.data_ptr(), cp.chunk_offsets.data_ptr(), P, cp.total_chunks,
                float(scale), st_p, kernels._stream())
        # gradient pass of the flagged pairs: left-edge gradient C_r of every piece but the first (from zero; the last
        # piece from dht), then e_{r-1} = T_r^T e_r + C_r down the pieces; dh is overwritten by the final pass
        c_out = torch.empty(P, H, K, V, dtype=torch.float32, device=dev)
        dht_piece = torch.empty(P, H, K, V, dtype=torch.float32, device=dev)
        rc = lib.fq_gdr_bwd_dh_cp_ex(*args, c_out.data_ptr(), dh.data_ptr(), cp.seq_index.data_ptr(),
                                     cp.entry_slot.data_ptr(), cp.seq_end.data_ptr(), warm.pass1_rev.data_ptr(), None,
                                     *tail)
        _lib.check(rc, "fq_gdr_bwd_dh")
        rc = lib.fq_cp_chain_reverse(c_out.data_ptr(), tmats[P:].data_ptr(), dht_piece.data_ptr(), warm.flags.data_ptr(),
                                     cp.seq_piece_offsets.data_ptr(), P, cp.n_seq, H, kernels._stream())
        _lib.check(rc, "fq_cp_chain_reverse")
        rc = lib.fq_gdr_bwd_dh_cp_ex(*args, pp(dh0), dh.data_ptr(), cp.seq_index.data_ptr(),
                                     cp.out_index_bwd.data_ptr(), cp.seq_end.data_ptr(), warm.codes_rev.data_ptr(),
                                     dht_piece.data_ptr(), *tail)
    _lib.check(rc, "fq_gdr_bwd_dh")
    # 3. chunk-parallel gradients; with grouped value heads the kernel sums dq / dk over the V-heads of every QK head itself
    #    (flash_qla/ops/gated_delta_rule/chunk/__init__.py:107-110 does it with a separate kernel)
    dq = torch.empty(B, T, Hg, K, dtype=q.dtype, device=dev)
    dk = torch.empty(B, T, Hg, K, dtype=q.dtype, device=dev)
    dg_c = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    db = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    dv = torch.empty_like(v)
    entry = lib.fq_gdr_bwd_chunk_grouped if Hg < H else lib.fq_gdr_bwd_chunk
    rc = entry(q.data_ptr(), k.data_ptr(), v.data_ptr(), A.data_ptr(), Ag.data_ptr(), Pg.data_ptr(),
               do.data_ptr(), h.data_ptr(), dh.data_ptr(), g.data_ptr(), bt.data_ptr(), dq.data_ptr(),
               dk.data_ptr(), dv.data_ptr(), dg_c.data_ptr(), db.data_ptr(), B, T, H, Hg, cu_p, off_p, plan.n_seq,
               plan.total_chunks, float(scale), st_p, kernels._stream())
    _lib.check(rc, "fq_gdr_bwd_chunk")
    # 3b. the whole-state dot product in dg of a sequence's first / last chunk, corrected with the fp32 initial state /
    #     final-state gradient (the chunk kernel used their bf16 copies)
    if h0 is not None or dht_c is not None:
        rc = lib.fq_dg_boundary_fix(pp(h0), pp(dht_c), h.data_ptr(), dh.data_ptr(), g.data_ptr(), dg_c.data_ptr(), B, T, H,
                                    cu_p, off_p, plan.n_seq, plan.total_chunks, kernels._stream())
        _lib.check(rc, "fq_dg_boundary_fix")
    # 4. d/d(cumsum) -> d/d(raw gate)
    dg = kernels.chunk_local_cumsum(dg_c, reverse=True, plan=plan)
    if status is not None:
        kernels.check_status(status, "backward kernels")
    return dq, dk, dv, db, dg, dh0
