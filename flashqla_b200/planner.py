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


def plan_dense(B: int, T: int) -> SeqPlan:
    nc = (T + CHUNK - 1) // CHUNK
    return SeqPlan(B, B * nc, B * T, nc, None, None, None, None)


def plan_packed(cu_seqlens: torch.Tensor, device=None) -> SeqPlan:
    """Plan for a packed batch.  ``cu_seqlens`` may live on the host or on the device."""
    if cu_seqlens.dim() != 1 or cu_seqlens.numel() < 2:
        raise ValueError("cu_seqlens must be a 1-D tensor with at least two entries")
    device = torch.device(device) if device is not None else cu_seqlens.device
    key = (id(cu_seqlens), cu_seqlens._version, cu_seqlens.data_ptr(), str(device))
    hit = _CACHE.get(key)
    if hit is not None and hit[0] is cu_seqlens:
        _CACHE.move_to_end(key)
        return hit[1]
    cu = [int(x) for x in cu_seqlens.tolist()]
    if cu[0] != 0 or any(cu[i + 1] < cu[i] for i in range(len(cu) - 1)):
        raise ValueError("cu_seqlens must start at 0 and be non-decreasing")
    off = chunk_offsets_from_lengths(cu)
    cu_dev = cu_seqlens.to(device=device, dtype=torch.int32).contiguous()
    off_dev = torch.tensor(off, dtype=torch.int32, device=device)
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
