// Gate scan for context-parallel pieces: how many whole chunks before a piece have to be replayed
// so that everything older has decayed below `threshold` (a log-decay, e.g. -16 -> 1e-7).
// One thread per (piece, head) walks the chunks backwards and sums each chunk's total log-decay
// (the chunk-local cumsum at the chunk's last token).  If the sequence start is reached first, the
// replay starts there and is exact (bit 30 of the result tells the recurrence kernel to load the
// initial state).  Counterpart of get_warmup_chunks,
// flash_qla/ops/gated_delta_rule/chunk/hopper/cp_fwd.py:69-101 (which scans inside the previous piece
// and falls back to a transition matrix; here the replay may simply run further back).
#include "flashqla.h"
#include "host.cuh"

namespace fq {

__global__ void __launch_bounds__(128) cp_warmup_kernel(const float* __restrict__ g_cum,
                                                       const int* __restrict__ piece_start,
                                                       const int* __restrict__ piece_first_chunk,
                                                       int* __restrict__ warmup, int n_pieces, int H, float threshold,
                                                       int reverse, const int* __restrict__ piece_chunks_after) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_pieces * H) return;
  const int piece = idx / H, h = idx - piece * H;
  if (!reverse) {
    const int avail = __ldg(piece_first_chunk + piece);
    const long long start = __ldg(piece_start + piece);
    float acc = 0.f;
    int w = 0;
    bool decayed = false;
    while (w < avail) {
      acc += __ldg(g_cum + (start - static_cast<long long>(w) * kChunk - 1) * H + h);
      ++w;
      if (acc < threshold) { decayed = true; break; }
    }
    warmup[idx] = decayed ? w : (avail | (1 << 30));
  } else {
    // reverse direction (state gradient): replay the chunks AFTER the piece; piece_start holds the
    // first token after the piece, piece_chunks_after the number of chunks that follow it in the
    // sequence and piece_first_chunk the length in tokens of the sequence's last chunk.
    const int avail = __ldg(piece_chunks_after + piece);
    const long long end = __ldg(piece_start + piece);
    const int last_len = __ldg(piece_first_chunk + piece);
    float acc = 0.f;
    int w = 0;
    bool decayed = false;
    while (w < avail) {
      const int len = (w == avail - 1) ? last_len : kChunk;
      acc += __ldg(g_cum + (end + static_cast<long long>(w) * kChunk + len - 1) * H + h);
      ++w;
      if (acc < threshold) { decayed = true; break; }
    }
    warmup[idx] = decayed ? w : (avail | (1 << 30));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Transition-matrix fallback.  A replay of more than `w_max` chunks costs more than it saves (a head whose gate
// never decays would replay its whole prefix in every piece).  Such a (sequence, head) is flagged, and all of its
// pieces then start from corrected states instead:
//   pass 1  every piece r but the last runs state-only from zero (from h0 for the first piece): end state B_r; and,
//           for r > first, once more with S = I and V = 0: end state T_r (the piece's transition matrix, K x K);
//   chain   h0_{r+1} = T_r h0_r + B_r along the pieces of the sequence (cp_chain_kernel, fp32);
//   pass 2  the normal kernel, every piece starting from its h0_r with no replay.
// Counterpart of the (ht, mt) scheme of flash_qla/ops/gated_delta_rule/chunk/hopper/cp_fwd.py:256-309.
// Codes (per piece or pass-1 entry, and head), on top of the replay length in bits 0-23 and bit 30 (start from the
// sequence's initial state): bit 29 = start from the piece's corrected state, bit 28 = transition run (S = I, V = 0),
// bit 27 = nothing to do.

__global__ void __launch_bounds__(128) cp_flag_kernel(const int* __restrict__ warmup, const int* __restrict__ piece_seq,
                                                     int* __restrict__ flags, int n_pieces, int H, int w_max) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_pieces * H) return;
  const int piece = idx / H, h = idx - piece * H;
  if ((__ldg(warmup + idx) & 0xFFFFFF) > w_max) atomicOr(flags + __ldg(piece_seq + piece) * H + h, 1);
}

__global__ void __launch_bounds__(128) cp_resolve_kernel(const int* __restrict__ warmup_in,
                                                        const int* __restrict__ piece_seq,
                                                        const int* __restrict__ chunks_before,
                                                        const int* __restrict__ chunks_after,
                                                        const int* __restrict__ flags, int* __restrict__ warmup_out,
                                                        int* __restrict__ pass1, int n_pieces, int H) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_pieces * H) return;
  const int piece = idx / H, h = idx - piece * H;
  const bool flagged = __ldg(flags + __ldg(piece_seq + piece) * H + h) != 0;
  const bool first = __ldg(chunks_before + piece) == 0, last = __ldg(chunks_after + piece) == 0;
  const int code = __ldg(warmup_in + idx);
  warmup_out[idx] = (flagged && !first) ? (1 << 29) : code;
  constexpr int kSkip = 1 << 27;
  pass1[idx] = (flagged && !last) ? (first ? (1 << 30) : 0) : kSkip;               // B_r
  pass1[n_pieces * H + idx] = (flagged && !last && !first) ? (1 << 28) : kSkip;    // T_r
}

// h0_{r+1} = T_r h0_r + B_r for the pieces of one flagged (sequence, head); a CTA owns 16 of the 128 state columns.
// bt: [2 * n_pieces, H, 128, 128] fp32 (B_r in slot r, T_r in slot n_pieces + r); h0_piece: [n_pieces, H, 128, 128].
__global__ void __launch_bounds__(256) cp_chain_kernel(const float* __restrict__ bt, float* __restrict__ h0_piece,
                                                      const int* __restrict__ flags,
                                                      const int* __restrict__ seq_piece_offsets, int n_pieces, int H) {
  constexpr int kCols = 16;
  __shared__ float sx[kDim][kCols];       // current state slice
  __shared__ float st[kDim][kDim / 4 + 1];  // a 128 x 32 tile of T_r
  const int seq = blockIdx.x / H, h = blockIdx.x - seq * H, c0 = blockIdx.y * kCols;
  if (__ldg(flags + seq * H + h) == 0) return;
  const int p0 = __ldg(seq_piece_offsets + seq), p1 = __ldg(seq_piece_offsets + seq + 1);
  const int tid = threadIdx.x;
  const int i = tid >> 1, cb = (tid & 1) * 8;  // this thread's output row and its 8 columns
  const size_t mat = static_cast<size_t>(kDim) * kDim;
  for (int r = p0; r + 1 < p1; ++r) {
    const float* B = bt + (static_cast<size_t>(r) * H + h) * mat;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = __ldg(B + static_cast<size_t>(i) * kDim + c0 + cb + e);
    if (r > p0) {
      const float* Tm = bt + (static_cast<size_t>(n_pieces + r) * H + h) * mat;
      for (int k0 = 0; k0 < kDim; k0 += 32) {
        __syncthreads();  // the previous tile (and, for k0 == 0, the previous state) has been consumed
        for (int idx = tid; idx < kDim * 32; idx += 256) st[idx >> 5][idx & 31] = __ldg(Tm + static_cast<size_t>(idx >> 5) * kDim + k0 + (idx & 31));
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
          const float t = st[i][kk];
          const float4 x0 = *reinterpret_cast<const float4*>(&sx[k0 + kk][cb]);
          const float4 x1 = *reinterpret_cast<const float4*>(&sx[k0 + kk][cb + 4]);
          acc[0] += t * x0.x; acc[1] += t * x0.y; acc[2] += t * x0.z; acc[3] += t * x0.w;
          acc[4] += t * x1.x; acc[5] += t * x1.y; acc[6] += t * x1.z; acc[7] += t * x1.w;
        }
      }
    }
    __syncthreads();  // every thread has read the old state
    float* dst = h0_piece + (static_cast<size_t>(r + 1) * H + h) * mat + static_cast<size_t>(i) * kDim + c0 + cb;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      sx[i][cb + e] = acc[e];
      dst[e] = acc[e];
    }
    __syncthreads();
  }
}

}  // namespace fq

extern "C" FQ_API int fq_cp_warmup(const float* g_cumsum, const int32_t* piece_edge, const int32_t* piece_aux,
                                   const int32_t* piece_chunks_after, int32_t* warmup, int n_pieces, int H,
                                   float threshold, int reverse, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(g_cumsum && piece_edge && piece_aux && warmup, "fq_cp_warmup: null tensor");
  FQ_CHECK_ARG(!reverse || piece_chunks_after, "fq_cp_warmup: the reverse scan needs piece_chunks_after");
  FQ_CHECK_ARG(n_pieces > 0 && H > 0 && threshold < 0.f, "fq_cp_warmup: bad arguments");
  const int total = n_pieces * H;
  cp_warmup_kernel<<<(total + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      g_cumsum, piece_edge, piece_aux, warmup, n_pieces, H, threshold, reverse, piece_chunks_after);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_cp_transition_plan(const int32_t* warmup_in, const int32_t* piece_seq,
                                            const int32_t* chunks_before, const int32_t* chunks_after, int32_t* flags,
                                            int32_t* warmup_out, int32_t* pass1_codes, int n_pieces, int n_seq, int H,
                                            int w_max, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(warmup_in && piece_seq && chunks_before && chunks_after && flags && warmup_out && pass1_codes,
               "fq_cp_transition_plan: null tensor");
  FQ_CHECK_ARG(n_pieces > 0 && n_seq > 0 && H > 0 && w_max >= 0, "fq_cp_transition_plan: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FQ_CHECK_CUDA(cudaMemsetAsync(flags, 0, sizeof(int32_t) * static_cast<size_t>(n_seq) * H, st));
  const int total = n_pieces * H;
  cp_flag_kernel<<<(total + 127) / 128, 128, 0, st>>>(warmup_in, piece_seq, flags, n_pieces, H, w_max);
  cp_resolve_kernel<<<(total + 127) / 128, 128, 0, st>>>(warmup_in, piece_seq, chunks_before, chunks_after, flags,
                                                         warmup_out, pass1_codes, n_pieces, H);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_cp_chain(const float* bt, float* h0_piece, const int32_t* flags,
                                  const int32_t* seq_piece_offsets, int n_pieces, int n_seq, int H, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(bt && h0_piece && flags && seq_piece_offsets, "fq_cp_chain: null tensor");
  FQ_CHECK_ARG(n_pieces > 0 && n_seq > 0 && H > 0, "fq_cp_chain: bad arguments");
  dim3 grid(static_cast<unsigned>(n_seq) * H, kDim / 16);
  cp_chain_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(bt, h0_piece, flags, seq_piece_offsets, n_pieces, H);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}
