// Sequence / chunk lookup shared by the chunk-parallel kernels.
#pragma once
#include "common.cuh"

namespace fq {

struct SeqArgs {
  int T;                     // tokens per batch row (dense) or total tokens (packed, B == 1)
  const int* cu_seqlens;     // [n_seq+1] or nullptr
  const int* chunk_offsets;  // [n_seq+1] or nullptr
  int n_seq;
  int nc_dense;              // chunks per sequence for dense batches
};

struct ChunkPos {
  int seq;    // sequence index
  int cin;    // chunk index inside the sequence
  int tok0;   // row of the chunk's first token in the flattened [B*T] token axis
  int len;    // valid tokens in the chunk (1..64)
};

// Maps a global chunk number to its sequence.  Packed batches: binary search over the chunk
// prefix sums (the last sequence whose first chunk is <= c, which skips empty sequences).
__device__ __forceinline__ ChunkPos chunk_lookup(const SeqArgs& s, int c) {
  ChunkPos p;
  if (s.cu_seqlens == nullptr) {
    p.seq = c / s.nc_dense;
    p.cin = c - p.seq * s.nc_dense;
    p.tok0 = p.seq * s.T + p.cin * kChunk;
    p.len = min(kChunk, s.T - p.cin * kChunk);
  } else {
    int lo = 0, hi = s.n_seq;
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (__ldg(s.chunk_offsets + mid) <= c) lo = mid; else hi = mid;
    }
    p.seq = lo;
    p.cin = c - __ldg(s.chunk_offsets + lo);
    const int b = __ldg(s.cu_seqlens + lo), e = __ldg(s.cu_seqlens + lo + 1);
    p.tok0 = b + p.cin * kChunk;
    p.len = min(kChunk, e - p.tok0);
  }
  return p;
}

}  // namespace fq
