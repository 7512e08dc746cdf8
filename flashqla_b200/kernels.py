"""Thin torch-tensor wrappers over the C ABI (one function per entry point).

All tensors must live on the current CUDA device; work is enqueued on the current stream.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from .planner import SeqPlan, plan_dense, plan_packed

CHUNK = 64


try:  # the raw handle of the current stream without building a torch.cuda.Stream object (15 us -> under 1 us per launch)
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:  # pragma: no cover - a torch without that binding
    _raw_stream = None


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.FlashQLAError("flashqla_b200 kernels need CUDA tensors (there is no CPU path)")


def make_plan(B: int, T: int, cu_seqlens, device, host=None) -> SeqPlan:
    if cu_seqlens is None:
        return plan_dense(B, T)
    if B != 1:
        raise ValueError(
            f"The batch size is expected to be 1 rather than {B} when using `cu_seqlens`."
            f"Please flatten variable-length inputs before processing.")
    plan = plan_packed(cu_seqlens, device, host=host)
    if plan.total_tokens > T:
        # the tail-chunk stores of the kernels are plain pointer writes: a sequence that ends past the tensors would
        # write out of bounds
        raise ValueError(f"cu_seqlens[-1] = {plan.total_tokens} exceeds the {T} tokens of the packed tensors")
    return plan


def chunk_local_cumsum(g: torch.Tensor, chunk_size: int = CHUNK, reverse: bool = False, cu_seqlens=None,
                       plan: SeqPlan | None = None) -> torch.Tensor:
    """Chunk-local cumulative sum of g [B,T,H] (fp32 result)."""
    assert chunk_size == CHUNK, "chunk size is fixed at 64"
    _require_cuda(g)
    B, T, H = g.shape
    plan = plan or make_plan(B, T, cu_seqlens, g.device)
    gin = g.contiguous() if g.dtype == torch.float32 else g.float().contiguous()
    out = torch.empty_like(gin)
    cu_p, off_p = plan.ptrs()
    rc = _lib.load().fq_chunk_cumsum(gin.data_ptr(), out.data_ptr(), B, T, H, cu_p, off_p, plan.n_seq,
                                     plan.total_chunks, int(reverse), _stream())
    _lib.check(rc, "fq_chunk_cumsum")
    return out


def kkt_solve(k: torch.Tensor, b: torch.Tensor, cu_seqlens=None, plan: SeqPlan | None = None) -> torch.Tensor:
    """A = (I + tril(diag(b) K K^T, -1))^-1, bf16 [B,T,H,64] (gate-free)."""
    _require_cuda(k, b)
    if k.dtype != torch.bfloat16:
        raise _lib.FlashQLAError("kkt_solve: only bfloat16 keys are supported")
    B, T, Hg, K = k.shape
    H = b.shape[-1]
    assert K == 128, "head dim must be 128"
    plan = plan or make_plan(B, T, cu_seqlens, k.device)
    k = k.contiguous()
    bf = b.contiguous() if b.dtype == torch.float32 else b.float().contiguous()
    # rows of partial tail chunks are never written by the kernel -> start from zeros
    A = torch.zeros(B, T, H, CHUNK, dtype=k.dtype, device=k.device) if T % CHUNK or plan.packed else \
        torch.empty(B, T, H, CHUNK, dtype=k.dtype, device=k.device)
    cu_p, off_p = plan.ptrs()
    rc = _lib.load().fq_kkt_solve(k.data_ptr(), bf.data_ptr(), A.data_ptr(), B, T, H, Hg, cu_p, off_p, plan.n_seq,
                                  plan.total_chunks, _stream())
    _lib.check(rc, "fq_kkt_solve")
    return A


def selftest_umma(a: torch.Tensor, b: torch.Tensor, mode: int) -> torch.Tensor:
    _require_cuda(a, b)
    d = torch.zeros(128, 128, dtype=torch.float32, device=a.device)
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    rc = _lib.load().fq_selftest_umma(a.data_ptr(), b.data_ptr(), d.data_ptr(), mode, status.data_ptr(), _stream())
    _lib.check(rc, "fq_selftest_umma")
    st = int(status.item())
    if st != 0:
        raise _lib.FlashQLAError(f"fq_selftest_umma: device wait timed out (code {st:#x})")
    return d


def _status_tensor(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor, what: str) -> None:
    """Raise if a kernel's bounded wait expired (costs a device sync; used by tests and debug mode)."""
    st = int(status.item())
    if st != 0:
        raise _lib.FlashQLAError(f"{what}: device-side wait timed out (code {st:#x})")


def _tile_alloc(plan: SeqPlan, B: int, T: int):
    """Allocator of the [B,T,H,64] tile tensors.  Rows past the last sequence (packed tensors longer than
    cu_seqlens[-1]) are never written by the tile kernel, but the last tail tile of the recurrence kernels covers them
    and masks them by multiplication: they must hold finite values, so such batches start from zeros."""
    return torch.zeros if plan.total_tokens < B * T else torch.empty


def kkt_solve_gated(k, q, b, g_cum, scale, plan: SeqPlan, A=None, want_pg=True):
    """A (gate-free inverse, computed unless given), A_g and P_g tiles, bf16 [B,T,H,64] each."""
    _require_cuda(k, q, b, g_cum)
    if k.dtype != torch.bfloat16:
        raise _lib.FlashQLAError("kkt_solve_gated: only bfloat16 keys are supported")
    B, T, Hg, K = k.shape
    H = b.shape[-1]
    assert K == 128, "head dim must be 128"
    k, q = k.contiguous(), q.contiguous()
    bf = b.contiguous() if b.dtype == torch.float32 else b.float().contiguous()
    a_is_input = A is not None
    if A is None:
        A = torch.empty(B, T, H, CHUNK, dtype=k.dtype, device=k.device)
    else:
        A = A.contiguous()
    alloc = _tile_alloc(plan, B, T)
    Ag = alloc(B, T, H, CHUNK, dtype=k.dtype, device=k.device)
    Pg = alloc(B, T, H, CHUNK, dtype=k.dtype, device=k.device) if want_pg else None
    cu_p, off_p = plan.ptrs()
    rc = _lib.load().fq_kkt_solve_gated(k.data_ptr(), q.data_ptr(), bf.data_ptr(), g_cum.data_ptr(), A.data_ptr(),
                                        Ag.data_ptr(), None if Pg is None else Pg.data_ptr(), int(a_is_input), B, T, H,
                                        Hg, cu_p, off_p, plan.n_seq, plan.total_chunks, float(scale), _stream())
    _lib.check(rc, "fq_kkt_solve_gated")
    return A, Ag, Pg


def kkt_solve_fused(k, q, b, g, scale, plan: SeqPlan, want_A=True, want_pg=False):
    """Chunk-local cumsum of the raw log gate `g`, A and A_g in one launch.  Returns (g_cumsum, A, A_g, P_g).
    `want_A=False` (A is None then) skips the store of the gate-free inverse, which only the backward reads.  P_g is
    None unless `want_pg`: the forward recurrence forms that tile itself (and stores it for a backward)."""
    _require_cuda(k, q, b, g)
    if k.dtype != torch.bfloat16:
        raise _lib.FlashQLAError("kkt_solve_fused: only bfloat16 keys are supported")
    B, T, Hg, K = k.shape
    H = b.shape[-1]
    assert K == 128, "head dim must be 128"
    assert g.stride(-1) == 1, "g must be contiguous in its last dimension"
    k, q = k.contiguous(), q.contiguous()
    bf = b.contiguous() if b.dtype == torch.float32 else b.float().contiguous()
    gf = g.contiguous() if g.dtype == torch.float32 else g.float().contiguous()
    g_cum = torch.empty_like(gf)
    alloc = _tile_alloc(plan, B, T)
    Ag = alloc(B, T, H, CHUNK, dtype=k.dtype, device=k.device)
    Pg = alloc(B, T, H, CHUNK, dtype=k.dtype, device=k.device) if want_pg else None
    A = alloc(B, T, H, CHUNK, dtype=k.dtype, device=k.device) if want_A else None
    cu_p, off_p = plan.ptrs()
    rc = _lib.load().fq_kkt_solve_fused(k.data_ptr(), q.data_ptr(), bf.data_ptr(), gf.data_ptr(), g_cum.data_ptr(),
                                        None if A is None else A.data_ptr(), Ag.data_ptr(),
                                        None if Pg is None else Pg.data_ptr(), B, T, H, Hg, cu_p, off_p, plan.n_seq,
                                        plan.total_chunks, float(scale), _stream())
    _lib.check(rc, "fq_kkt_solve_fused")
    return g_cum, A, Ag, Pg


def kkt_solve_fused_act(k, b_raw, g_raw, scale, plan: SeqPlan, gate_mode: int, beta_mode: int, A_log=None, dt_bias=None,
                        want_A=True):
    """kkt_solve_fused with the gate / beta activations applied inside the kernel (modes as in include/flashqla.h).
    Returns (g_cumsum of the activated gate, activated beta (the input itself for beta_mode 0), A, A_g)."""
    _require_cuda(k, b_raw, g_raw)
    if k.dtype != torch.bfloat16:
        raise _lib.FlashQLAError("kkt_solve_fused_act: only bfloat16 keys are supported")
    B, T, Hg, K = k.shape
    H = b_raw.shape[-1]
    k = k.contiguous()
    bf = b_raw.contiguous() if b_raw.dtype == torch.float32 else b_raw.float().contiguous()
    gf = g_raw.contiguous() if g_raw.dtype == torch.float32 else g_raw.float().contiguous()
    p = lambda t: None if t is None else t.float().contiguous().data_ptr()
    al = None if A_log is None else A_log.float().contiguous()
    db_ = None if dt_bias is None else dt_bias.float().contiguous()
    g_cum = torch.empty_like(gf)
    beta_act = (torch.zeros_like(bf) if plan.total_tokens < B * T else torch.empty_like(bf)) if beta_mode else bf
    alloc = _tile_alloc(plan, B, T)
    Ag = alloc(B, T, H, CHUNK, dtype=k.dtype, device=k.device)
    A = alloc(B, T, H, CHUNK, dtype=k.dtype, device=k.device) if want_A else None
    cu_p, off_p = plan.ptrs()
    rc = _lib.load().fq_kkt_solve_fused_act(k.data_ptr(), bf.data_ptr(), gf.data_ptr(), None if al is None else al.data_ptr(),
                                            None if db_ is None else db_.data_ptr(), int(gate_mode), int(beta_mode),
                                            g_cum.data_ptr(), beta_act.data_ptr() if beta_mode else None,
                                            None if A is None else A.data_ptr(), Ag.data_ptr(), B, T, H, Hg, cu_p, off_p,
                                            plan.n_seq, plan.total_chunks, float(scale), _stream())
    _lib.check(rc, "fq_kkt_solve_fused_act")
    return g_cum, beta_act, A, Ag


def gate_act_bwd(dg, db, g_raw, b_raw, gate_mode: int, beta_mode: int, A_log=None, dt_bias=None):
    """Backward of the in-kernel activations.  Returns (dg_raw, db_raw, dA_log or None, ddt_bias or None)."""
    H = dg.shape[-1]
    rows = dg.numel() // H
    gf = g_raw.contiguous() if g_raw.dtype == torch.float32 else g_raw.float().contiguous()
    bf = b_raw.contiguous() if b_raw.dtype == torch.float32 else b_raw.float().contiguous()
    dg, db = dg.contiguous(), db.contiguous()
    dg_raw, db_raw = torch.empty_like(dg), torch.empty_like(db)
    al = None if A_log is None else A_log.float().contiguous()
    bi = None if dt_bias is None else dt_bias.float().contiguous()
    dA = torch.zeros(H, dtype=torch.float32, device=dg.device) if gate_mode == 2 else None
    dB = torch.zeros(H, dtype=torch.float32, device=dg.device) if (gate_mode == 2 and dt_bias is not None) else None
    p = lambda t: None if t is None else t.data_ptr()
    rc = _lib.load().fq_gate_act_bwd(dg.data_ptr(), db.data_ptr(), gf.data_ptr(), bf.data_ptr(), p(al), p(bi), int(gate_mode),
                                     int(beta_mode), dg_raw.data_ptr(), db_raw.data_ptr(), p(dA), p(dB), rows, H, _stream())
    _lib.check(rc, "fq_gate_act_bwd")
    return dg_raw, db_raw, dA, dB


def sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


@dataclass
class CpWarm:
    """Start-up codes of a context-parallel run (csrc/cp.cu): `codes` [P,H] for the final forward pass, `pass1`
    [2P,H] for the state pass of the transition-matrix fallback, `flags` [n_seq,H] = which (sequence, head) pairs
    use that fallback; with the reverse direction also `codes_rev` / `pass1_rev` [P,H] for the state-gradient
    recurrence."""
    codes: torch.Tensor
    pass1: torch.Tensor
    flags: torch.Tensor
    codes_rev: torch.Tensor | None = None
    pass1_rev: torch.Tensor | None = None


def cp_warmup(g_cum, cp, H, threshold=-16.0, with_reverse=False) -> CpWarm:
    """Gate scans and start-up codes for a context-parallel run.  A pair whose replay would exceed one piece length
    (in either direction when `with_reverse`) is switched to corrected start states."""
    dev = g_cum.device
    P = cp.n_pieces
    cap = int(cp.piece_chunks)
    codes = torch.empty(P, H, dtype=torch.int32, device=dev)
    pass1 = torch.empty(2 * P, H, dtype=torch.int32, device=dev)
    flags = torch.empty(cp.n_seq, H, dtype=torch.int32, device=dev)
    warm = CpWarm(codes, pass1, flags)
    if with_reverse:
        warm.codes_rev = torch.empty_like(codes)
        warm.pass1_rev = torch.empty_like(codes)
    # scans, flag and codes of every (sequence, head) in one launch
    rc = _lib.load().fq_cp_plan(g_cum.data_ptr(), cp.piece_start.data_ptr(), cp.piece_end.data_ptr(),
                                cp.chunks_before.data_ptr(), cp.chunks_after.data_ptr(), cp.last_chunk_len.data_ptr(),
                                cp.seq_piece_offsets.data_ptr(), flags.data_ptr(), codes.data_ptr(), pass1.data_ptr(),
                                None if not with_reverse else warm.codes_rev.data_ptr(),
                                None if not with_reverse else warm.pass1_rev.data_ptr(), P, cp.n_seq, H,
                                float(threshold), cap, _stream())
    _lib.check(rc, "fq_cp_plan")
    return warm


def cp_correct_states(q, k, v, ag, g, b, scale, h0, cp, warm: CpWarm, status=None, return_bt=False):
    """Corrected start state of every piece for the (sequence, head) pairs flagged in `warm` (other slots are left
    unwritten): one state-only launch over 2P entries (end state from zero, transition matrix) and the chain
    h0[r+1] = T_r h0[r] + B_r.  All inputs contiguous, as prepared by fused_gdr_fwd.  `return_bt` also returns the
    [2P,H,128,128] scratch whose second half holds the transition matrices (the backward reuses them)."""
    B, T, Hg, K = k.shape
    H = v.shape[2]
    dev = q.device
    P = cp.n_pieces
    bt = torch.empty(2 * P, H, K, K, dtype=torch.float32, device=dev)
    h0_piece = torch.empty(P, H, K, K, dtype=torch.float32, device=dev)
    p = lambda t: None if t is None else t.data_ptr()
    lib = _lib.load()
    rc = lib.fq_gdr_fwd_cp_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), ag.data_ptr(), None, g.data_ptr(), b.data_ptr(),
                              p(h0), bt.data_ptr(), cp.entry_slot.data_ptr(), cp.seq_index.data_ptr(),
                              warm.pass1.data_ptr(), cp.entry_piece.data_ptr(), 2 * P, None, None, None, 1, B * T, H, Hg,
                              cp.cu_seqlens.data_ptr(), cp.chunk_offsets.data_ptr(), P, cp.total_chunks, float(scale),
                              p(status), _stream())
    _lib.check(rc, "fq_gdr_fwd_cp_ex")
    rc = lib.fq_cp_chain(bt.data_ptr(), h0_piece.data_ptr(), warm.flags.data_ptr(), cp.seq_piece_offsets.data_ptr(), P,
                         cp.n_seq, H, _stream())
    _lib.check(rc, "fq_cp_chain")
    return (h0_piece, bt) if return_bt else h0_piece


def fused_gdr_fwd(q, k, v, ag, pg, g, b, scale, initial_state=None, output_final_state=True, output_h=False,
                  output_o=True, plan: SeqPlan | None = None, cp=None, warmup=None, status=None, h0_piece=None):
    """Fused forward recurrence.  g is the chunk-local cumsum, ag the gated tile A_g from kkt_solve_fused / _gated.
    `pg`: None, or a [B,T,H,64] bf16 tensor that RECEIVES the P_g tiles the kernel forms (kept for the backward;
    only written when o is produced).  With a CpPlan `cp` (and its `warmup` table) every piece of a sequence runs as
    its own CTA.

    Returns (o or None, hT or None, final_state or None).  hT holds the state before every chunk
    TRANSPOSED ([..., H, V, K]): the kernel stores it by TMA straight from its bf16 operand buffer and the
    backward kernels consume it in that layout; ``hT.transpose(-1, -2)`` is the [K, V] view."""
    _require_cuda(q, k, v, ag, g, b)
    if q.dtype != torch.bfloat16:
        raise _lib.FlashQLAError("fused_gdr_fwd: only bfloat16 q/k/v are supported")
    B, T, Hg, K = k.shape
    H, V = v.shape[2], v.shape[3]
    assert K == 128 and V == 128, "head dims must be 128"
    plan = plan or plan_dense(B, T)
    dev = q.device
    q, k, v, ag = q.contiguous(), k.contiguous(), v.contiguous(), ag.contiguous()
    g = g.contiguous() if g.dtype == torch.float32 else g.float().contiguous()
    b = b.contiguous() if b.dtype == torch.float32 else b.float().contiguous()
    h0 = None
    if initial_state is not None:
        h0 = initial_state.contiguous() if initial_state.dtype == torch.float32 else initial_state.float().contiguous()
        assert h0.shape == (plan.n_seq, H, K, V), f"initial_state shape {tuple(h0.shape)} != {(plan.n_seq, H, K, V)}"
    o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev) if output_o else None
    h = torch.empty(1 if plan.packed else B, plan.total_chunks // (1 if plan.packed else B), H, K, V, dtype=q.dtype,
                    device=dev) if output_h else None
    ht = torch.empty(plan.n_seq, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
    p = lambda t: None if t is None else t.data_ptr()
    if cp is None:
        cu_p, off_p = plan.ptrs()
        rc = _lib.load().fq_gdr_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), ag.data_ptr(), p(pg), g.data_ptr(),
                                    b.data_ptr(), p(h0), p(ht), None, p(o), p(h), B, T, H, Hg, cu_p, off_p, plan.n_seq,
                                    plan.total_chunks, float(scale), p(status), _stream())
    else:
        if isinstance(warmup, CpWarm):
            if h0_piece is None:
                h0_piece = cp_correct_states(q, k, v, ag, g, b, scale, h0, cp, warmup, status)
            codes = warmup.codes
        else:
            codes = warmup
        rc = _lib.load().fq_gdr_fwd_cp_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), ag.data_ptr(), p(pg), g.data_ptr(),
                                          b.data_ptr(), p(h0), p(ht), cp.out_index_fwd.data_ptr(),
                                          cp.seq_index.data_ptr(), codes.data_ptr(), None, cp.n_pieces, p(h0_piece),
                                          p(o), p(h), 1, B * T, H, Hg, cp.cu_seqlens.data_ptr(),
                                          cp.chunk_offsets.data_ptr(), cp.n_pieces, cp.total_chunks, float(scale),
                                          p(status), _stream())
    _lib.check(rc, "fq_gdr_fwd")
    return o, h, ht
