// Chunk-local prefix / suffix sum of the log-gate.  HBM-bound: 8 bytes per (token, head).
// One thread owns one (chunk, head) column of 64 tokens; consecutive threads own consecutive
// heads, so every load and store of a warp covers contiguous head runs of the [tokens, H] rows (whole 32-byte
// sectors from H = 8 on).
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
  // Sixteen rows at a time: the sixteen loads are independent (in flight together), the running sum is carried across the
  // four blocks.  A thread then needs about forty registers, so the SM holds its full complement of warps - with all 64
  // rows in registers (143 registers) it held an eighth of them and the kernel ran at the latency of its own loads.
  float acc = 0.f;
#pragma unroll 1
  for (int blk = 0; blk < kChunk / 16; ++blk) {
    const int r0 = reverse ? kChunk - 16 * (blk + 1) : 16 * blk;
    if (!reverse && r0 >= p.len) break;
    if (reverse && r0 >= p.len) continue;
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = (r0 + i < p.len) ? __ldg(src + static_cast<size_t>(r0 + i) * H) : 0.f;
    if (!reverse) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        acc += v[i];
        v[i] = acc;
      }
    } else {
#pragma unroll
      for (int i = 15; i >= 0; --i) {
        acc += v[i];
        v[i] = acc;
      }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (r0 + i < p.len) dst[static_cast<size_t>(r0 + i) * H] = v[i];
  }
}

// ---------------------------------------------------------------------------------------------------------------
// fp32 correction of the gate gradient at the two ends of every sequence.
//
// dg of a chunk's last token contains gamma_last * sum(dS o S0) over the whole 128 x 128 state (S0: state before the
// chunk, dS: gradient w.r.t. the state after it).  The chunk-parallel backward evaluates that sum from the bf16 copies
// of both states that travel between the kernels.  The sum cancels heavily (16384 products of either sign), so for a
// sequence's FIRST chunk (S0 = the caller's fp32 initial state, e.g. ~ randn) and LAST chunk (dS = the caller's fp32
// final-state gradient) the rounding of those copies can show in dg of a short sequence.  Both fp32 tensors are at
// hand, so the difference between the exact products and the rounded ones is added here:
//   first chunk:  gamma_last * sum( bf16(dS) o (h0 - bf16(h0)) )
//   last chunk:   gamma_last * sum( (dht - bf16(dht)) o S0x ),  S0x = h0 (fp32) if the sequence has one chunk, else
//                 the bf16 state copy before the last chunk
// Eight CTAs per (sequence, head): (first | last chunk) x four blocks of 32 state columns.  h, dh: [total_chunks, H, 128(v), 128(k)] bf16 (transposed, as the recurrences store
// them); h0, dht: [n_seq, H, 128(k), 128(v)] fp32 or nullptr; dg_cum: [rows, H] gradient w.r.t. the gate cumsum, updated
// in place at the last valid token of the chunk concerned.
__global__ void __launch_bounds__(256) dg_boundary_fix_kernel(const float* __restrict__ h0, const float* __restrict__ dht,
                                                             const __nv_bfloat16* __restrict__ h,
                                                             const __nv_bfloat16* __restrict__ dh,
                                                             const float* __restrict__ g_cum, float* __restrict__ dg_cum,
                                                             int H, SeqArgs sa) {
  __shared__ float tile[32][kDim + 1];
  __shared__ float red[8];
  const int seq = blockIdx.x / H, hd = blockIdx.x - seq * H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int tok_begin, seq_len, chunk_off;
  if (sa.cu_seqlens == nullptr) {
    tok_begin = seq * sa.T; seq_len = sa.T; chunk_off = seq * sa.nc_dense;
  } else {
    tok_begin = __ldg(sa.cu_seqlens + seq);
    seq_len = __ldg(sa.cu_seqlens + seq + 1) - tok_begin;
    chunk_off = __ldg(sa.chunk_offsets + seq);
  }
  if (seq_len <= 0) return;
  const int nchunks = (seq_len + kChunk - 1) / kChunk;
  const size_t mat = static_cast<size_t>(kDim) * kDim;
  const float* h0m = h0 ? h0 + (static_cast<size_t>(seq) * H + hd) * mat : nullptr;
  const float* dhtm = dht ? dht + (static_cast<size_t>(seq) * H + hd) * mat : nullptr;
  // blockIdx.y = 4 * part + (block of 32 v): part 0 = first chunk (needs h0), part 1 = last chunk (needs dht); the
  // partial sums of a pair's CTAs meet in dg_cum by atomic adds
  const int part = blockIdx.y >> 2, vb = (blockIdx.y & 3) * 32;
  const float* fp = part == 0 ? h0m : dhtm;  // the fp32 tensor whose rounding is corrected, [k][v]
  if (fp == nullptr) return;
  const int c = part == 0 ? 0 : nchunks - 1;
  // the other factor: part 0 -> bf16 dS of chunk 0; part 1 -> fp32 h0 for a one-chunk sequence, else bf16 S0 of chunk c
  const bool other_fp32 = (part == 1 && nchunks == 1 && h0m != nullptr);
  const __nv_bfloat16* ot = (part == 0 ? dh : h) + (static_cast<size_t>(chunk_off + c) * H + hd) * mat;  // [v][k]
  if (!other_fp32) {
    // rows vb .. vb+31 of the transposed tile: 32 x 128 bf16 = 512 pieces of 16 bytes, two per thread
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int i = tid + 256 * it, r = i >> 4, piece = i & 15;
      const uint4 x = __ldg(reinterpret_cast<const uint4*>(ot + static_cast<size_t>(vb + r) * kDim) + piece);
      const uint32_t* xw = reinterpret_cast<const uint32_t*>(&x);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        tile[r][piece * 8 + 2 * e] = bf16_lo(xw[e]);
        tile[r][piece * 8 + 2 * e + 1] = bf16_hi(xw[e]);
      }
    }
    __syncthreads();
  }
  float x[16], o[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {  // sixteen independent loads in flight per thread
    const int k = warp + 8 * i;
    x[i] = __ldg(fp + static_cast<size_t>(k) * kDim + vb + lane);
    o[i] = other_fp32 ? __ldg(h0m + static_cast<size_t>(k) * kDim + vb + lane) : tile[lane][k];
  }
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) acc += (x[i] - __bfloat162float(__float2bfloat16_rn(x[i]))) * o[i];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (tid == 0) {
    float sum = 0.f;
    for (int w = 0; w < 8; ++w) sum += red[w];
    const int len = min(kChunk, seq_len - c * kChunk);
    const size_t off = (static_cast<size_t>(tok_begin) + c * kChunk + len - 1) * H + hd;
    atomicAdd(dg_cum + off, sum * __expf(g_cum[off]));
  }
}

}  // namespace fq

extern "C" FQ_API int fq_dg_boundary_fix(const float* h0, const float* dht, const void* h, const void* dh,
                                         const float* g_cumsum, float* dg_cum, int B, int T, int H,
                                         const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                                         int total_chunks, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(h && dh && g_cumsum && dg_cum, "fq_dg_boundary_fix: null tensor");
  FQ_CHECK_ARG(B > 0 && T >= 0 && H > 0 && n_seq > 0 && total_chunks >= 0, "fq_dg_boundary_fix: bad sizes");
  FQ_CHECK_ARG((cu_seqlens == nullptr) == (chunk_offsets == nullptr),
               "fq_dg_boundary_fix: cu_seqlens and chunk_offsets must be given together");
  FQ_CHECK_ARG(cu_seqlens != nullptr || n_seq == B, "fq_dg_boundary_fix: dense batches need n_seq == B");
  if (total_chunks == 0 || (h0 == nullptr && dht == nullptr)) return FQ_OK;
  SeqArgs sa{T, cu_seqlens, chunk_offsets, n_seq, (T + kChunk - 1) / kChunk};
  const long long ctas = static_cast<long long>(n_seq) * H;
  FQ_CHECK_ARG(ctas < (1ll << 31), "fq_dg_boundary_fix: too many (sequence, head) pairs");
  dg_boundary_fix_kernel<<<dim3(static_cast<unsigned>(ctas), 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      h0, dht, static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(dh), g_cumsum, dg_cum, H, sa);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

namespace fq {
// Backward of the gate / beta activations that fq_kkt_solve_fused_act applies (same modes): dg, db are the gradients
// w.r.t. the ACTIVATED log gate and beta, the outputs those w.r.t. the raw inputs; for gate mode 2 also the per-head
// sums dA_log[h] += sum dg * g and ddt_bias[h] += sum dg * dg/dz (shared-memory partial sums, one atomic per head and CTA).
__global__ void __launch_bounds__(256) gate_act_bwd_kernel(const float* __restrict__ dg, const float* __restrict__ db,
                                                          const float* __restrict__ g_raw, const float* __restrict__ beta_raw,
                                                          const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                          int gate_mode, int beta_mode, float* __restrict__ dg_raw,
                                                          float* __restrict__ db_raw, float* __restrict__ dA_log,
                                                          float* __restrict__ ddt_bias, long long total, int H) {
  extern __shared__ float part[];  // [2 * H]
  const bool sums = gate_mode == 2 && (dA_log != nullptr || ddt_bias != nullptr);
  if (sums) {
    for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) part[i] = 0.f;
    __syncthreads();
  }
  // when the grid stride is a multiple of H every thread stays on one head: its two sums then live in registers and
  // reach shared memory once, instead of two shared-memory atomics per element
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const bool one_head = sums && (stride % H) == 0;
  float acc_a = 0.f, acc_b = 0.f;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int h = static_cast<int>(idx % H);
    const float d = dg[idx];
    float out = d;
    if (gate_mode == 1) {
      out = d / (1.f + __expf(g_raw[idx]));  // d logsigmoid(x) / dx = sigmoid(-x)
    } else if (gate_mode == 2) {
      const float ea = __expf(__ldg(A_log + h));
      const float z = g_raw[idx] + (dt_bias ? __ldg(dt_bias + h) : 0.f);
      const float sp = z > 20.f ? z : log1pf(__expf(z));
      const float dz = -ea / (1.f + __expf(-z));          // d g / d z
      out = d * dz;
      if (one_head) {
        acc_a += d * (-ea * sp);                          // d g / d A_log = g
        acc_b += out;
      } else if (sums) {
        atomicAdd(&part[h], d * (-ea * sp));
        atomicAdd(&part[H + h], out);
      }
    }
    dg_raw[idx] = out;
    if (db_raw != nullptr) {
      float o2 = db[idx];
      if (beta_mode == 1) {
        const float sg = 1.f / (1.f + __expf(-beta_raw[idx]));
        o2 *= sg * (1.f - sg);
      }
      db_raw[idx] = o2;
    }
  }
  if (one_head) {
    const int h = static_cast<int>((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) % H);
    atomicAdd(&part[h], acc_a);
    atomicAdd(&part[H + h], acc_b);
  }
  if (sums) {
    __syncthreads();
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      if (dA_log) atomicAdd(dA_log + i, part[i]);
      if (ddt_bias) atomicAdd(ddt_bias + i, part[H + i]);
    }
  }
}
}  // namespace fq

extern "C" FQ_API int fq_gate_act_bwd(const float* dg, const float* db, const float* g_raw, const float* beta_raw,
                                      const float* A_log, const float* dt_bias, int gate_mode, int beta_mode, float* dg_raw,
                                      float* db_raw, float* dA_log, float* ddt_bias, long long rows, int H, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(dg && g_raw && dg_raw && rows >= 0 && H > 0 && H <= 4096, "fq_gate_act_bwd: bad arguments");
  FQ_CHECK_ARG(db_raw == nullptr || (db != nullptr && beta_raw != nullptr), "fq_gate_act_bwd: dbeta needs db and beta_raw");
  FQ_CHECK_ARG(gate_mode >= 0 && gate_mode <= 2 && beta_mode >= 0 && beta_mode <= 1, "fq_gate_act_bwd: bad mode");
  FQ_CHECK_ARG(gate_mode != 2 || A_log != nullptr, "fq_gate_act_bwd: gate mode 2 needs A_log");
  if (rows == 0) return FQ_OK;
  const long long total = rows * H;
  const long long blocks = (total + 255) / 256;
  const long long cap = 8LL * sm_count();
  gate_act_bwd_kernel<<<static_cast<unsigned>(blocks < cap ? blocks : cap), 256, 2 * H * sizeof(float),
                        static_cast<cudaStream_t>(stream)>>>(dg, db, g_raw, beta_raw, A_log, dt_bias, gate_mode, beta_mode,
                                                             dg_raw, db_raw, dA_log, ddt_bias, total, H);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

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
