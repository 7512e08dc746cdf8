"""Host-side scheduling for variable-length batches: per-sequence chunk tables.

Mirrors flash_qla/utils/index.py:71-138 (prepare_chunk_indices / prepare_chunk_offsets and the
identity-keyed cache) of the reference.  The reference computes the chunk prefix sums in a tiny
GPU kernel followed by an ``.item()`` sync; here they are computed on the host from one copy of
``cu_seqlens`` and cached per tensor, so a ``cu_seqlens`` object costs one sync the first time
it is seen and none afterwards.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass

import torch

CHUNK = 64


@dataclass
class SeqPlan:
    """Sequence layout of one batch.

    dense : n_seq == B sequences of T tokens, ``cu_seqlens``/``chunk_offsets`` are None.
    packed: B == 1; ``cu_seqlens`` int32 device [n_seq+1]; ``chunk_offsets`` int32 device [n_seq+1].
    """
    n_seq: int
    total_chunks: int
    total_tokens: int
    max_chunks: int
    cu_seqlens: torch.Tensor | None
    chunk_offsets: torch.Tensor | None
    cu_host: list | None
    offsets_host: list | None

    @property
    def packed(self) -> bool:
        return self.cu_seqlens is not None

    def ptrs(self):
        if self.cu_seqlens is None:
            return None, None
        return self.cu_seqlens.data_ptr(), self.chunk_offsets.data_ptr()


def chunk_offsets_from_lengths(cu: list) -> list:
    off = [0]
    for i in range(len(cu) - 1):
        off.append(off[-1] + (cu[i + 1] - cu[i] + CHUNK - 1) // CHUNK)
    return off


_CACHE: "OrderedDict[tuple, tuple]" = OrderedDict()
_CACHE_SIZE = 256


_DENSE_CACHE: dict = {}


def plan_dense(B: int, T: int) -> SeqPlan:
    """Plan of a dense batch; one object per (B, T) so that plans derived from it can be cached by identity."""
    plan = _DENSE_CACHE.get((B, T))
    if plan is None:
        nc = (T + CHUNK - 1) // CHUNK
        plan = SeqPlan(B, B * nc, B * T, nc, None, None, None, None)
        if len(_DENSE_CACHE) > _CACHE_SIZE:
            _DENSE_CACHE.clear()
        _DENSE_CACHE[(B, T)] = plan
    return plan


def _to_device_i32(values, device) -> torch.Tensor:
    """int32 device tensor from a host list / host tensor without a stream synchronisation (pinned staging buffer,
    asynchronous copy on the current stream)."""
    host = values if isinstance(values, torch.Tensor) else torch.tensor(values, dtype=torch.int32)
    host = host.to(torch.int32).contiguous()
    device = torch.device(device)
    if device.type != "cuda":
        return host.to(device)
    return host.pin_memory().to(device, non_blocking=True)


def plan_packed(cu_seqlens: torch.Tensor, device=None, host: torch.Tensor | None = None) -> SeqPlan:
    """Plan for a packed batch.  ``cu_seqlens`` may live on the host or on the device; ``host`` is an optional host
    copy of a device ``cu_seqlens``: with it the plan is made without reading the device tensor back, i.e. without a
    synchronisation (the counterpart of the device-side TODO at flash_qla/utils/index.py:76 of the reference)."""
    if cu_seqlens.dim() != 1 or cu_seqlens.numel() < 2:
        raise ValueError("cu_seqlens must be a 1-D tensor with at least two entries")
    device = torch.device(device) if device is not None else cu_seqlens.device
    key = (id(cu_seqlens), cu_seqlens._version, cu_seqlens.data_ptr(), str(device))
    hit = _CACHE.get(key)
    if hit is not None and hit[0] is cu_seqlens:
        _CACHE.move_to_end(key)
        return hit[1]
    if host is not None:
        if host.is_cuda or host.shape != cu_seqlens.shape:
            raise ValueError("the host copy of cu_seqlens must be a CPU tensor of the same shape")
        cu = [int(x) for x in host.tolist()]
    else:
        cu = [int(x) for x in cu_seqlens.tolist()]
    if cu[0] != 0 or any(cu[i + 1] < cu[i] for i in range(len(cu) - 1)):
        raise ValueError("cu_seqlens must start at 0 and be non-decreasing")
    off = chunk_offsets_from_lengths(cu)
    if cu_seqlens.device == device and cu_seqlens.dtype == torch.int32 and cu_seqlens.is_contiguous():
        cu_dev = cu_seqlens
    elif cu_seqlens.is_cuda:
        cu_dev = cu_seqlens.to(device=device, dtype=torch.int32).contiguous()
    else:
        cu_dev = _to_device_i32(cu_seqlens, device)
    off_dev = _to_device_i32(off, device)
    plan = SeqPlan(len(cu) - 1, off[-1], cu[-1], max((off[i + 1] - off[i]) for i in range(len(cu) - 1)),
                   cu_dev, off_dev, cu, off)
    _CACHE[key] = (cu_seqlens, plan)
    if len(_CACHE) > _CACHE_SIZE:
        _CACHE.popitem(last=False)
    return plan


def prepare_chunk_indices(cu_seqlens: torch.Tensor, chunk_size: int = CHUNK) -> torch.Tensor:
    """[(sequence, chunk-in-sequence)] for every chunk, in order (index.py:71-83 of the reference)."""
    assert chunk_size == CHUNK
    plan = plan_packed(cu_seqlens)
    rows = [(s, c) for s in range(plan.n_seq) for c in range(plan.offsets_host[s + 1] - plan.offsets_host[s])]
    return torch.tensor(rows, dtype=cu_seqlens.dtype, device=cu_seqlens.device).reshape(-1, 2)


def prepare_chunk_offsets(cu_seqlens: torch.Tensor, chunk_size: int = CHUNK):
    """(prefix sums of per-sequence chunk counts, total) (index.py:126-138 of the reference)."""
    assert chunk_size == CHUNK
    plan = plan_packed(cu_seqlens)
    return plan.chunk_offsets.to(cu_seqlens.dtype), plan.total_chunks


# --------------------------------------------------------------------------- context parallel
@dataclass
class CpPlan:
    """Split of the sequences of a batch into pieces that run as independent CTAs.

    Counterpart of `_calc_cp_seqs` (flash_qla/ops/gated_delta_rule/chunk/cp_context.py:32-103).  Pieces
    of one sequence are contiguous, every piece but the last of a sequence holds `piece_chunks`
    whole chunks, so chunk boundaries (and with them the cumsum, A and h tensors) are the same with
    and without the split.  All tensors are int32 on the device.
    """
    n_pieces: int
    piece_chunks: int
    total_chunks: int
    cu_seqlens: torch.Tensor        # [P+1] piece token boundaries in the flattened [B*T] token axis
    chunk_offsets: torch.Tensor     # [P+1] prefix sums of chunks per piece
    seq_index: torch.Tensor         # [P] raw sequence of each piece (slot of h0 / dht)
    out_index_fwd: torch.Tensor     # [P] raw sequence for the LAST piece of a sequence, else -1 (slot of ht)
    out_index_bwd: torch.Tensor     # [P] raw sequence for the FIRST piece of a sequence, else -1 (slot of dh0)
    piece_start: torch.Tensor       # [P] first token of the piece
    piece_end: torch.Tensor         # [P] first token after the piece
    chunks_before: torch.Tensor     # [P] chunks of the sequence that precede the piece
    chunks_after: torch.Tensor      # [P] chunks of the sequence that follow the piece
    last_chunk_len: torch.Tensor    # [P] tokens in the last chunk of the piece's sequence
    seq_end: torch.Tensor           # [P] first token after the piece's sequence
    seq_piece_offsets: torch.Tensor = None  # [n_seq+1] first piece of every sequence
    entry_piece: torch.Tensor = None        # [2P] piece of every entry of the two-run state pass (0..P-1 twice)
    entry_slot: torch.Tensor = None         # [2P] 0..2P-1: where each entry's end state goes
    n_seq: int = 0


def _makespan(pieces: list, H: int, n_sm: int, overhead: int) -> float:
    """Finish time of list scheduling: CTAs (one per piece and head, in launch order) go to the SM that frees up first."""
    import heapq
    if not pieces:
        return 0.0
    free = [0.0] * n_sm
    heapq.heapify(free)
    end = 0.0
    for x in pieces:
        if x <= 0:
            continue
        for _ in range(H):
            t = heapq.heappop(free) + x + overhead
            end = max(end, t)
            heapq.heappush(free, t)
    return end


def choose_piece_chunks(n_chunks: list, H: int, n_sm: int, overhead: int = 8) -> int | None:
    """Chunks per piece, or None to run un-split.

    Cost model in units of one chunk step of one CTA: a CTA costs (chunks + overhead), the overhead
    standing for the replayed chunks and the CTA start-up; the kernels keep one CTA per SM, so the
    run time is the makespan of scheduling the CTAs, in launch order, on n_sm machines.  The
    reference's rule (cp_context.py:52-57, 86-87) was fitted to 132 SMs with up to two CTAs each;
    this one follows from the one-CTA-per-SM kernels and was checked against sweeps of the piece length on the
    reference's benchmark grid.
    """
    longest = max(n_chunks) if n_chunks else 0
    if longest <= 8:
        return None

    def cost(L):
        if L >= longest:
            return _makespan(list(n_chunks), H, n_sm, overhead)
        pieces = [min(L, c - i) for c in n_chunks for i in range(0, c, L)]
        # Splitting has a price beyond the replayed chunks: a handful of extra launches (about twelve chunk steps),
        # and - for heads whose gate decays too slowly, which only the device knows - a state pass (L chunk steps, or
        # half the final pass once the SMs are saturated: two runs per piece for about a quarter of the heads) plus one
        # chain step per piece of the longest sequence; that part is weighted three quarters.
        span = _makespan(pieces, H, n_sm, overhead)
        return span + 12 + 0.75 * max(L + -(-longest // L), 0.5 * span)

    base = cost(longest)
    best_L, best = None, base
    cands = set()
    L = 1 << (longest - 1).bit_length()
    while L >= 8:
        cands.update((L, (3 * L) // 4))
        L //= 2
    for parts in range(2, 65):  # equal splits of the longest sequence
        cands.add(-(-longest // parts))
    for cand in sorted(cands, reverse=True):
        if 8 <= cand < longest:
            c = cost(cand)
            if c < best * 0.999:
                best_L, best = cand, c
    if best_L is None or best > 0.9 * base:
        return None
    return best_L


_CP_CACHE: "OrderedDict[tuple, CpPlan | None]" = OrderedDict()


def plan_cp(plan: SeqPlan, B: int, T: int, H: int, n_sm: int, device, piece_chunks: int | None = None):
    """CpPlan for a batch, or None when splitting does not pay.  Dense batches are treated as packed
    ones over the flattened token axis (row b*T + t)."""
    key = (id(plan), B, T, H, n_sm, str(device), piece_chunks)
    hit = _CP_CACHE.get(key)
    if hit is not None and hit[0] is plan:
        return hit[1]
    cu = plan.cu_host if plan.packed else [b * T for b in range(B + 1)]
    n_chunks = [(cu[i + 1] - cu[i] + CHUNK - 1) // CHUNK for i in range(len(cu) - 1)]
    L = piece_chunks if piece_chunks is not None else choose_piece_chunks(n_chunks, H, n_sm)
    result = None
    if L is not None and L >= 1 and max(n_chunks, default=0) > L:
        starts, ends, seq_idx, before, after, lastlen, out_f, out_b, send = [], [], [], [], [], [], [], [], []
        for i, nc in enumerate(n_chunks):
            s, e = cu[i], cu[i + 1]
            if nc == 0:  # empty sequence: one empty piece so that its final state / dh0 still gets written
                starts.append(s); ends.append(e); seq_idx.append(i); before.append(0); after.append(0)
                lastlen.append(0); out_f.append(i); out_b.append(i); send.append(e)
                continue
            ll = (e - s) - (nc - 1) * CHUNK
            for c0 in range(0, nc, L):
                c1 = min(nc, c0 + L)
                starts.append(s + c0 * CHUNK)
                ends.append(min(e, s + c1 * CHUNK))
                seq_idx.append(i); before.append(c0); after.append(nc - c1); lastlen.append(ll)
                out_f.append(i if c1 == nc else -1)
                out_b.append(i if c0 == 0 else -1)
                send.append(e)
        bounds = starts + [cu[-1]]
        offs = [0]
        for a_, b_ in zip(starts, ends):
            offs.append(offs[-1] + (b_ - a_ + CHUNK - 1) // CHUNK)

        def t(x):
            return _to_device_i32(x, device)

        P = len(starts)
        seq_off = [0]
        for i in range(len(n_chunks)):
            seq_off.append(seq_off[-1] + sum(1 for s_ in seq_idx if s_ == i))
        result = CpPlan(P, L, offs[-1], t(bounds), t(offs), t(seq_idx), t(out_f), t(out_b), t(starts), t(ends),
                        t(before), t(after), t(lastlen), t(send), t(seq_off), t(list(range(P)) * 2), t(list(range(2 * P))),
                        len(n_chunks))
    _CP_CACHE[key] = (plan, result)
    if len(_CP_CACHE) > _CACHE_SIZE:
        _CP_CACHE.popitem(last=False)
    return result
