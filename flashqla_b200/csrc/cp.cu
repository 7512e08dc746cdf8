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
