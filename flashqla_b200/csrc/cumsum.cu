// Chunk-local prefix / suffix sum of the log-gate.  HBM-bound: 8 bytes per (token, head).
// One thread owns one (chunk, head) column of 64 tokens; consecutive threads own consecutive
// heads, so every load and store of a warp covers contiguous head runs of the [tokens, H] rows.
#include "flashqla.h"
#include "host.cuh"
#include "seq.cuh"

namespace fq {

__global__ void __launch_bounds__(256) chunk_cumsum_kernel(const float* __restrict__ g, float* __restrict__ out,
                                                          int H, SeqArgs sa, long long total, int reverse) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int c = static_cast<int>(idx / H);
  const int h = static_cast<int>(idx - static_cast<long long>(c) * H);
  const ChunkPos p = chunk_lookup(sa, c);
  const size_t base = static_cast<size_t>(p.tok0) * H + h;
  const float* src = g + base;
  float* dst = out + base;
  float v[kChunk];
#pragma unroll
  for (int i = 0; i < kChunk; ++i) v[i] = (i < p.len) ? src[static_cast<size_t>(i) * H] : 0.f;
  float acc = 0.f;
  if (!reverse) {
#pragma unroll
    for (int i = 0; i < kChunk; ++i) {
      acc += v[i];
      if (i < p.len) dst[static_cast<size_t>(i) * H] = acc;
    }
  } else {
#pragma unroll
    for (int i = kChunk - 1; i >= 0; --i) {
      acc += v[i];
      if (i < p.len) dst[static_cast<size_t>(i) * H] = acc;
    }
  }
}

}  // namespace fq

extern "C" FQ_API int fq_chunk_cumsum(const float* g, float* out, int B, int T, int H, const int32_t* cu_seqlens,
                                      const int32_t* chunk_offsets, int n_seq, int total_chunks, int reverse,
                                      void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(g && out, "fq_chunk_cumsum: null tensor");
  FQ_CHECK_ARG(B > 0 && T >= 0 && H > 0 && n_seq > 0 && total_chunks >= 0, "fq_chunk_cumsum: bad sizes");
  FQ_CHECK_ARG((cu_seqlens == nullptr) == (chunk_offsets == nullptr),
               "fq_chunk_cumsum: cu_seqlens and chunk_offsets must be given together");
  FQ_CHECK_ARG(cu_seqlens == nullptr || B == 1, "fq_chunk_cumsum: packed batches need B == 1");
  FQ_CHECK_ARG(cu_seqlens != nullptr || n_seq == B, "fq_chunk_cumsum: dense batches need n_seq == B");
  if (total_chunks == 0) return FQ_OK;
  SeqArgs sa{T, cu_seqlens, chunk_offsets, n_seq, (T + kChunk - 1) / kChunk};
  FQ_CHECK_ARG(cu_seqlens != nullptr || total_chunks == B * sa.nc_dense, "fq_chunk_cumsum: total_chunks mismatch");
  const long long total = static_cast<long long>(total_chunks) * H;
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  chunk_cumsum_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      g, out, H, sa, total, reverse);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}
