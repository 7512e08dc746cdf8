// A = (I + strictly_lower(diag(beta) K K^T))^-1 for every (chunk, V-head).
//
// One CTA (4 warps) owns one (chunk, QK-head): it loads the 64x128 K tile once, forms K K^T once
// with warp-level bf16 MMA and then, for each of the G V-heads that share the QK head, inverts the
// unit lower-triangular 64x64 matrix:
//   1. the four 16x16 diagonal blocks by column-parallel forward substitution in fp32,
//   2. the two 16x16 blocks next to the diagonal:  X10 = -D1 (L10 D0),  X32 = -D3 (L32 D2),
//   3. the 32x32 block below:  X_lo_hi = -X_hi (L_hl X_lo),
// steps 2 and 3 on tensor cores with TF32 operands and fp32 accumulation.  TF32 rounding (2^-11) of
// these products changes A by at most 2.4e-4 (rms 9e-6) on unit-norm keys, below the 1e-3 rounding of
// the bf16 result.  The unit costs 24 KB of HBM traffic for ~1.4 MFLOP, i.e. it is HBM-bound by
// arithmetic intensity, which is why the legacy warp-level MMA path is enough here.
//
// Optionally (Ag / Pg given) the same CTA also emits the two gated, chunk-parallel operand tiles
// of the recurrences, so that the serial kernels carry only serial work:
//   A_g[i][j] = A[i][j] * exp(g_i - g_j) * beta_j   (j <= i)
//   P_g[i][j] = scale * exp(g_i - g_j) * (q_i . k_j) (j <= i)
// with g the chunk-local cumsum of the log gate (padded rows use the last valid value).
#include "flashqla.h"
#include "host.cuh"
#include "seq.cuh"

namespace fq {

constexpr int kKLd = 136;  // bf16 elements per K-tile row in shared memory (pad: conflict-free fragments)
constexpr int kFLd = 68;   // fp32 elements per row of the 64x64 work matrices

struct KktSmem {
  union {  // the Q tile is only read while Q K^T is formed; K K^T (fp32) then takes its place
    __nv_bfloat16 q[kChunk * kKLd];
    float kk[kChunk * kFLd];
  };
  union {  // the K tile is dead once K K^T and Q K^T are formed; the inverse X (fp32) then takes its place
    __nv_bfloat16 k[kChunk * kKLd];
    float x[kChunk * kFLd];
  };
  float beta[kChunk];
  float g[kChunk];
};
// Only the lower block triangle of K K^T is formed, so rows 0-31 x columns 32-63 of `kk` are free: the 32x32
// scratch of the block products lives there (row stride kFLd).
constexpr int kTLd = kFLd;
constexpr int kTOff = 32;

// 16-byte asynchronous copy global -> shared; `bytes` = 0 writes zeros instead (rows past the sequence end).
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma_tf32_1688(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// Four 8x8 bf16 matrices from shared memory in MMA fragment layout; lane l supplies the address of row (l & 7) of
// matrix (l >> 3).
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}
// c += a * b with a, b given in fp32 and rounded to TF32.
__device__ __forceinline__ void mma_tf32(float (&c)[4], const float (&a)[4], const float (&b)[2]) {
  uint32_t ah[4], bh[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(ah[i]) : "f"(a[i]));
#pragma unroll
  for (int i = 0; i < 2; ++i) asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bh[i]) : "f"(b[i]));
  mma_tf32_1688(c, ah, bh);
}

// acc[j] (16 rows m0.. of `a_tile` times the 8 rows 8j.. of `b_tile`, both [64][kKLd] bf16) for the lower block
// triangle j < ntiles.  Fragment loads with ldmatrix: lane l addresses row (l & 7) + 8 * ((l >> 3) & 1) of a 16-row
// block and the 8-column half (l >> 4) for the A operand; for the B operand one x4 load covers two 8-row tiles.
__device__ __forceinline__ void gram_pass(float (&acc)[8][4], const __nv_bfloat16* a_tile, const __nv_bfloat16* b_tile,
                                          int m0, int ntiles, int lane) {
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const int a_row = m0 + (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
  const int b_row = (lane & 7) + 8 * (lane >> 4), b_col = 8 * ((lane >> 3) & 1);
#pragma unroll
  for (int k0 = 0; k0 < kDim; k0 += 16) {
    uint32_t a[4];
    ldmatrix_x4(a, &a_tile[a_row * kKLd + k0 + a_col]);
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      if (j < ntiles) {  // ntiles is even
        uint32_t b4[4];
        ldmatrix_x4(b4, &b_tile[(j * 8 + b_row) * kKLd + k0 + b_col]);
        const uint32_t b0[2] = {b4[0], b4[1]}, b1[2] = {b4[2], b4[3]};
        mma_bf16_16816(acc[j], a, b0);
        mma_bf16_16816(acc[j + 1], a, b1);
      }
    }
  }
}

// P_g straight from the Q K^T fragments (rows m0+g and m0+g+8, column pairs 8j+2t); g2 = gate cumsum * log2(e).
// `stage`: this warp's own 16 rows of a dead [64][kKLd] bf16 tile, or nullptr.  With it the values are first laid down
// in shared memory and leave as 16-byte pieces (eight lanes per 128-byte row) instead of 4-byte stores.
__device__ __forceinline__ void store_pg(const float (&qk)[8][4], const float* g2, __nv_bfloat16* dstp, size_t row_stride,
                                         int warp, int lane, int len, float scale, __nv_bfloat16* stage = nullptr) {
  const int m0 = warp * 16, g = lane >> 2, t = lane & 3;
  const float log2_scale = log2f(scale);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = m0 + g + 8 * half;
    if (row < len) {
      const float gi = g2[row] + log2_scale;  // scale * 2^(g_i - g_j) = 2^(g_i + log2(scale) - g_j)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c0 = j * 8 + 2 * t;
        float y0 = 0.f, y1 = 0.f;
        if (j < 2 * warp + 2) {
          const float2 gj = *reinterpret_cast<const float2*>(&g2[c0]);
          if (c0 <= row) y0 = exp2f(gi - gj.x) * qk[j][2 * half];
          if (c0 + 1 <= row) y1 = exp2f(gi - gj.y) * qk[j][2 * half + 1];
        }
        if (stage) *reinterpret_cast<uint32_t*>(stage + (g + 8 * half) * kKLd + c0) = pack_bf16(y0, y1);
        else *reinterpret_cast<uint32_t*>(dstp + static_cast<size_t>(row) * row_stride + c0) = pack_bf16(y0, y1);
      }
    }
  }
  if (stage) {
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int i = it * 32 + lane, r = i >> 3, piece = i & 7;
      if (m0 + r < len)
        *(reinterpret_cast<uint4*>(dstp + static_cast<size_t>(m0 + r) * row_stride) + piece) =
            *reinterpret_cast<const uint4*>(stage + r * kKLd + piece * 8);
    }
  }
}

// Optional activations of the caller's raw gate / beta inputs, applied while the values are loaded (the elementwise
// passes a caller otherwise runs before the operator):
//   gate_mode 0: g is the log gate          1: g = logsigmoid(x)          2: g = -exp(A_log[h]) * softplus(x + dt_bias[h])
//   beta_mode 0: beta as given              1: beta = sigmoid(x); the activated values are also written to beta_out
//                                              ([rows, H] fp32), which the recurrence kernels read
struct GateAct {
  int gate_mode;
  int beta_mode;
  const float* A_log;    // [H], mode 2
  const float* dt_bias;  // [H] or nullptr, mode 2
  float* beta_out;       // [rows, H], beta_mode 1
};
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(__expf(z)); }
__device__ __forceinline__ float act_gate(const GateAct& a, float x, int h) {
  if (a.gate_mode == 1) return fminf(x, 0.f) - log1pf(__expf(-fabsf(x)));
  if (a.gate_mode == 2) return -__expf(__ldg(a.A_log + h)) * softplus_f(x + (a.dt_bias ? __ldg(a.dt_bias + h) : 0.f));
  return x;
}
__device__ __forceinline__ float act_beta(const GateAct& a, float x) { return a.beta_mode == 1 ? 1.f / (1.f + __expf(-x)) : x; }

// Gate values of one (chunk, head) into shared memory, times log2(e): exp(g_i - g_j) = exp2(g2_i - g2_j).  Called by
// warps 0 and 1.  With `g_cum_out` the input is the RAW log gate: warp 0 forms the chunk-local inclusive sum (two tokens
// per lane, shuffle scan) and also stores it, so that no separate prefix-sum pass over g is needed
// (chunk_local_cumsum, flash_qla/ops/utils/cumsum.py:131-165, folded into this kernel).  Rows past the sequence end
// get the last valid sum.
__device__ __forceinline__ void load_gates(float* sg, const float* __restrict__ g_in, float* __restrict__ g_cum_out,
                                           size_t base, int H, int len, int tid, const GateAct& act = GateAct{0, 0, nullptr, nullptr, nullptr},
                                           int head = 0) {
  constexpr float kLog2e = 1.4426950408889634f;
  if (g_cum_out == nullptr) {
    sg[tid] = kLog2e * __ldg(g_in + base + static_cast<size_t>(min(tid, len - 1)) * H);
    return;
  }
  if (tid >= 32) return;
  float a = (tid < len) ? act_gate(act, __ldg(g_in + base + static_cast<size_t>(tid) * H), head) : 0.f;
  float b = (tid + 32 < len) ? act_gate(act, __ldg(g_in + base + static_cast<size_t>(tid + 32) * H), head) : 0.f;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float ya = __shfl_up_sync(0xffffffffu, a, d), yb = __shfl_up_sync(0xffffffffu, b, d);
    if (tid >= d) { a += ya; b += yb; }
  }
  b += __shfl_sync(0xffffffffu, a, 31);
  if (tid < len) g_cum_out[base + static_cast<size_t>(tid) * H] = a;
  if (tid + 32 < len) g_cum_out[base + static_cast<size_t>(tid + 32) * H] = b;
  sg[tid] = kLog2e * a;
  sg[tid + 32] = kLog2e * b;
}

// The per-V-head part shared by both kernels: with K K^T (raw, lower block triangle) in s.kk, for each of the G V-heads of
// the QK head - gates and beta into shared memory, the block inverse X in s.x (or A fetched when it is an input), then A
// and / or A_g stored, and P_g from the Q K^T fragments `qk` when asked for.  kSingle: G == 1 and the caller has already
// loaded beta and the gates.
template <bool kSingle, class Smem>
__device__ __forceinline__ void solve_heads(Smem& s, const ChunkPos& p, const float (&qk)[8][4], const float* __restrict__ beta,
                                            __nv_bfloat16* __restrict__ A, int H, int Hg, int hg,
                                            const float* __restrict__ g_cum, __nv_bfloat16* __restrict__ Ag,
                                            __nv_bfloat16* __restrict__ Pg, float scale,
                                            const __nv_bfloat16* __restrict__ A_in, float* __restrict__ g_cum_out,
                                            const GateAct& act = GateAct{0, 0, nullptr, nullptr, nullptr}) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = H / Hg;
  for (int hi = 0; hi < G; ++hi) {
    const int hv = hg * G + hi;
    __syncthreads();  // kk complete, tiles read (first pass) / previous head's stores done
    if (!kSingle) {
      if (tid < kChunk) {
        float bv = 0.f;
        if (tid < p.len) {
          bv = act_beta(act, __ldg(beta + static_cast<size_t>(p.tok0 + tid) * H + hv));
          if (act.beta_out) act.beta_out[static_cast<size_t>(p.tok0 + tid) * H + hv] = bv;
        }
        s.beta[tid] = bv;
        if (Ag || Pg) load_gates(s.g, g_cum, g_cum_out, static_cast<size_t>(p.tok0) * H + hv, H, p.len, tid, act, hv);
      }
      __syncthreads();
    }

    if (A_in != nullptr) {
      // A was computed earlier (backward pass): fetch it instead of solving again
      const __nv_bfloat16* asrc = A_in + (static_cast<size_t>(p.tok0) * H + hv) * kChunk;
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int row = it * 16 + (tid >> 3), piece = tid & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < p.len) v = __ldg(reinterpret_cast<const uint4*>(asrc + static_cast<size_t>(row) * H * kChunk) + piece);
        const uint32_t* vw = reinterpret_cast<const uint32_t*>(&v);
        float* xr = &s.x[row * kFLd + piece * 8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          xr[2 * e] = bf16_lo(vw[e]);
          xr[2 * e + 1] = bf16_hi(vw[e]);
        }
      }
      __syncthreads();
    } else {
    // ---- step 1: inverse of the four 16x16 diagonal blocks, one column per thread
    if (tid < kChunk) {
      const int b0 = (tid >> 4) * 16, j = tid & 15;
      float xcol[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int m = 0; m < i; ++m) acc += s.kk[(b0 + i) * kFLd + b0 + m] * xcol[m];
        xcol[i] = (i == j) ? 1.f : -s.beta[b0 + i] * acc;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) s.x[(b0 + i) * kFLd + b0 + j] = xcol[i];
    }
    __syncthreads();

    // ---- step 2: X10 = -D1 (L10 D0) and X32 = -D3 (L32 D2); warp = (block pair, 8-column half)
    {
      const int blk = warp >> 1, nt = warp & 1;
      const int r0 = 16 * (2 * blk + 1), c0 = 16 * (2 * blk);
      float* ts = &s.kk[(16 * (warp >> 1)) * kTLd + kTOff + 16 * (warp & 1)];  // private 16 x 8 scratch
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k0 = 0; k0 < 16; k0 += 8) {
        float a[4], b[2];
        const float bg = s.beta[r0 + g], bg8 = s.beta[r0 + g + 8];
        a[0] = bg * s.kk[(r0 + g) * kFLd + c0 + k0 + t];
        a[1] = bg8 * s.kk[(r0 + g + 8) * kFLd + c0 + k0 + t];
        a[2] = bg * s.kk[(r0 + g) * kFLd + c0 + k0 + t + 4];
        a[3] = bg8 * s.kk[(r0 + g + 8) * kFLd + c0 + k0 + t + 4];
        b[0] = s.x[(c0 + k0 + t) * kFLd + c0 + 8 * nt + g];
        b[1] = s.x[(c0 + k0 + t + 4) * kFLd + c0 + 8 * nt + g];
        mma_tf32(c, a, b);
      }
      ts[g * kTLd + 2 * t] = c[0];
      ts[g * kTLd + 2 * t + 1] = c[1];
      ts[(g + 8) * kTLd + 2 * t] = c[2];
      ts[(g + 8) * kTLd + 2 * t + 1] = c[3];
      __syncwarp();
      float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k0 = 0; k0 < 16; k0 += 8) {
        float a[4], b[2];
        a[0] = s.x[(r0 + g) * kFLd + r0 + k0 + t];
        a[1] = s.x[(r0 + g + 8) * kFLd + r0 + k0 + t];
        a[2] = s.x[(r0 + g) * kFLd + r0 + k0 + t + 4];
        a[3] = s.x[(r0 + g + 8) * kFLd + r0 + k0 + t + 4];
        b[0] = ts[(k0 + t) * kTLd + g];
        b[1] = ts[(k0 + t + 4) * kTLd + g];
        mma_tf32(d, a, b);
      }
      __syncthreads();  // every warp has read its diagonal blocks; the scratch is free again
      *reinterpret_cast<float2*>(&s.x[(r0 + g) * kFLd + c0 + 8 * nt + 2 * t]) = make_float2(-d[0], -d[1]);
      *reinterpret_cast<float2*>(&s.x[(r0 + g + 8) * kFLd + c0 + 8 * nt + 2 * t]) = make_float2(-d[2], -d[3]);
    }
    __syncthreads();

    // ---- step 3: X[32:64, 0:32] = -X_hi (L_hl X_lo); warp = 16x16 quadrant
    {
      const int wr = warp >> 1, wc = warp & 1;
      float c[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
      const float bg = s.beta[32 + 16 * wr + g], bg8 = s.beta[32 + 16 * wr + g + 8];
#pragma unroll
      for (int k0 = 0; k0 < 32; k0 += 8) {
        float a[4];
        a[0] = bg * s.kk[(32 + 16 * wr + g) * kFLd + k0 + t];
        a[1] = bg8 * s.kk[(32 + 16 * wr + g + 8) * kFLd + k0 + t];
        a[2] = bg * s.kk[(32 + 16 * wr + g) * kFLd + k0 + t + 4];
        a[3] = bg8 * s.kk[(32 + 16 * wr + g + 8) * kFLd + k0 + t + 4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          float b[2];
          b[0] = s.x[(k0 + t) * kFLd + 16 * wc + 8 * n + g];
          b[1] = s.x[(k0 + t + 4) * kFLd + 16 * wc + 8 * n + g];
          mma_tf32(c[n], a, b);
        }
      }
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        *reinterpret_cast<float2*>(&s.kk[kTOff + (16 * wr + g) * kTLd + 16 * wc + 8 * n + 2 * t]) = make_float2(c[n][0], c[n][1]);
        *reinterpret_cast<float2*>(&s.kk[kTOff + (16 * wr + g + 8) * kTLd + 16 * wc + 8 * n + 2 * t]) =
            make_float2(c[n][2], c[n][3]);
      }
      __syncthreads();
      float d[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) d[n][0] = d[n][1] = d[n][2] = d[n][3] = 0.f;
#pragma unroll
      for (int k0 = 0; k0 < 32; k0 += 8) {
        float a[4];
        a[0] = s.x[(32 + 16 * wr + g) * kFLd + 32 + k0 + t];
        a[1] = s.x[(32 + 16 * wr + g + 8) * kFLd + 32 + k0 + t];
        a[2] = s.x[(32 + 16 * wr + g) * kFLd + 32 + k0 + t + 4];
        a[3] = s.x[(32 + 16 * wr + g + 8) * kFLd + 32 + k0 + t + 4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          float b[2];
          b[0] = s.kk[kTOff + (k0 + t) * kTLd + 16 * wc + 8 * n + g];
          b[1] = s.kk[kTOff + (k0 + t + 4) * kTLd + 16 * wc + 8 * n + g];
          mma_tf32(d[n], a, b);
        }
      }
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        *reinterpret_cast<float2*>(&s.x[(32 + 16 * wr + g) * kFLd + 16 * wc + 8 * n + 2 * t]) =
            make_float2(-d[n][0], -d[n][1]);
        *reinterpret_cast<float2*>(&s.x[(32 + 16 * wr + g + 8) * kFLd + 16 * wc + 8 * n + 2 * t]) =
            make_float2(-d[n][2], -d[n][3]);
      }
    }
    __syncthreads();

    }
    // ---- store A (bf16) and, if asked, A_g, in 16-byte pieces (8 columns of one token row).  Only the 320 pieces of
    //      the lower block triangle carry values; they are spread evenly over the threads (2.5 per thread), the 192
    //      pieces above it are written as zeros without touching the work matrix.
    {
      // A itself is only read by the backward: a forward that will not be differentiated passes A == nullptr
      __nv_bfloat16* dst = (A_in == nullptr && A != nullptr) ? A + (static_cast<size_t>(p.tok0) * H + hv) * kChunk : nullptr;
      __nv_bfloat16* dstg = Ag ? Ag + (static_cast<size_t>(p.tok0) * H + hv) * kChunk : nullptr;
      const size_t rs = static_cast<size_t>(H) * kChunk;
      auto emit = [&](int row, int piece) {
        if (row >= p.len) return;
        const float4 x0 = *reinterpret_cast<const float4*>(&s.x[row * kFLd + piece * 8]);
        const float4 x1 = *reinterpret_cast<const float4*>(&s.x[row * kFLd + piece * 8 + 4]);
        const float xr[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        uint4 v;
        if (dst) {
          v.x = pack_bf16(xr[0], xr[1]);
          v.y = pack_bf16(xr[2], xr[3]);
          v.z = pack_bf16(xr[4], xr[5]);
          v.w = pack_bf16(xr[6], xr[7]);
          *(reinterpret_cast<uint4*>(dst + row * rs) + piece) = v;
        }
        if (dstg) {
          const float gi = s.g[row];
          const float4 g0 = *reinterpret_cast<const float4*>(&s.g[piece * 8]);
          const float4 g1 = *reinterpret_cast<const float4*>(&s.g[piece * 8 + 4]);
          const float4 b0 = *reinterpret_cast<const float4*>(&s.beta[piece * 8]);
          const float4 b1 = *reinterpret_cast<const float4*>(&s.beta[piece * 8 + 4]);
          const float gj[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
          const float bj[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
          float y[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] = (piece * 8 + e <= row) ? xr[e] * exp2f(gi - gj[e]) * bj[e] : 0.f;
          v.x = pack_bf16(y[0], y[1]);
          v.y = pack_bf16(y[2], y[3]);
          v.z = pack_bf16(y[4], y[5]);
          v.w = pack_bf16(y[6], y[7]);
          *(reinterpret_cast<uint4*>(dstg + row * rs) + piece) = v;
        }
      };
      auto emit_zero = [&](int row, int piece) {
        if (row >= p.len) return;
        if (dst) *(reinterpret_cast<uint4*>(dst + row * rs) + piece) = make_uint4(0, 0, 0, 0);
        if (dstg) *(reinterpret_cast<uint4*>(dstg + row * rs) + piece) = make_uint4(0, 0, 0, 0);
      };
      emit(48 + (tid >> 3), tid & 7);  // rows 48-63: all 8 pieces
      if (warp < 3) {                  // rows 32-47: pieces 0-5
        const int r = tid / 6;
        emit(32 + r, tid - 6 * r);
      } else {                         // rows 0-15: pieces 0-1
        emit((tid - 96) >> 1, tid & 1);
      }
      if (warp < 2) {                  // rows 16-31: pieces 0-3
        emit(16 + (tid >> 2), tid & 3);
      } else {                         // the 192 zero pieces
        const int i = tid - 64;
        emit_zero(i >> 2, 4 + (i & 3));
        emit_zero(16 + (i >> 2), 4 + (i & 3));
        if (i < 32) emit_zero(i >> 1, 2 + (i & 1));
        else emit_zero(32 + ((i - 32) >> 1), 6 + (i & 1));
      }
    }
    if (!kSingle && Pg)
      store_pg(qk, s.g, Pg + (static_cast<size_t>(p.tok0) * H + hv) * kChunk, static_cast<size_t>(H) * kChunk, warp, lane,
               p.len, scale);
  }
}

// kSingle: every QK head has one V head (G == 1); the gates are then loaded with the tiles and P_g leaves before
// the solve, so that the Q K^T fragments are dead while K K^T is formed and inverted.
template <bool kSingle>
__global__ void __launch_bounds__(128, 6) kkt_solve_kernel(const __nv_bfloat16* __restrict__ k,
                                                       const float* __restrict__ beta,
                                                       __nv_bfloat16* __restrict__ A, int H, int Hg, SeqArgs sa,
                                                       const __nv_bfloat16* __restrict__ q,
                                                       const float* __restrict__ g_cum,
                                                       __nv_bfloat16* __restrict__ Ag, __nv_bfloat16* __restrict__ Pg,
                                                       float scale, const __nv_bfloat16* __restrict__ A_in,
                                                       float* __restrict__ g_cum_out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  KktSmem& s = *reinterpret_cast<KktSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int hg = blockIdx.y;
  const int G = H / Hg;
  const ChunkPos p = chunk_lookup(sa, blockIdx.x);

  // ---- K and Q tiles -> shared by asynchronous 16-byte copies (rows past the sequence end are zero-filled)
  {
    const __nv_bfloat16* src = k + (static_cast<size_t>(p.tok0) * Hg + hg) * kDim;
    const __nv_bfloat16* qsrc = Pg ? q + (static_cast<size_t>(p.tok0) * Hg + hg) * kDim : nullptr;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int idx = it * 128 + tid;  // 16-byte piece index: 16 per row
      const int row = idx >> 4, piece = idx & 15;
      const int ok = row < p.len;
      const size_t off = static_cast<size_t>(ok ? row : 0) * Hg * kDim + piece * 8;
      cp_async16(&s.k[row * kKLd + piece * 8], src + off, ok ? 16 : 0);
      if (Pg) cp_async16(&s.q[row * kKLd + piece * 8], qsrc + off, ok ? 16 : 0);
    }
    if (kSingle && tid < kChunk) {
      s.beta[tid] = (tid < p.len) ? __ldg(beta + static_cast<size_t>(p.tok0 + tid) * H + hg) : 0.f;
      if (Ag || Pg) load_gates(s.g, g_cum, g_cum_out, static_cast<size_t>(p.tok0) * H + hg, H, p.len, tid);
    }
    cp_async_wait_all();
  }
  __syncthreads();

  // ---- Q K^T (registers) and K K^T (fp32, to shared), lower block triangle only, one pass each
  float qk[8][4];
  {
    const int m0 = warp * 16;
    const int ntiles = 2 * warp + 2;
    if (Pg) {
      gram_pass(qk, s.q, s.k, m0, ntiles, lane);
      if (kSingle)
        // the warp's own rows of the Q tile are dead once its Q K^T fragments are formed: staging for P_g
        store_pg(qk, s.g, Pg + (static_cast<size_t>(p.tok0) * H + hg) * kChunk, static_cast<size_t>(H) * kChunk, warp, lane,
                 p.len, scale, &s.q[m0 * kKLd]);
    }
    if (A_in == nullptr) {
      float acc[8][4];
      gram_pass(acc, s.k, s.k, m0, ntiles, lane);
      __syncthreads();  // every warp is done reading the Q and K tiles, whose storage kk and x reuse
      {  // the two 16x16 blocks above the diagonal that the 32x32 block products read must be zero
        const int blk = tid >> 6, idx = tid & 63;
        *reinterpret_cast<float4*>(&s.x[(32 * blk + (idx >> 2)) * kFLd + 32 * blk + 16 + 4 * (idx & 3)]) =
            make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < ntiles) {
          *reinterpret_cast<float2*>(&s.kk[(m0 + g) * kFLd + j * 8 + 2 * t]) = make_float2(acc[j][0], acc[j][1]);
          *reinterpret_cast<float2*>(&s.kk[(m0 + g + 8) * kFLd + j * 8 + 2 * t]) = make_float2(acc[j][2], acc[j][3]);
        }
      }
    }
  }

  solve_heads<kSingle>(s, p, qk, beta, A, H, Hg, hg, g_cum, Ag, Pg, scale, A_in, g_cum_out);
}

// ---------------------------------------------------------------------------------------------------------------
// The forward's tile kernel on the Blackwell path (neither P_g nor a given A: only k is read).  Persistent CTAs of four
// warps walk the (chunk, QK-head) units; per unit
//   - the K tile [64 x 128] arrives by TMA (two 128-byte-swizzled halves, no padding, no per-thread copies),
//   - K K^T [64 x 64] is ONE group of eight tcgen05 products (M = 64, N = 64, K = 16 each) into 64 columns of tensor
//     memory that the CTA holds for its whole life,
//   - the accumulator rows come back with tcgen05.ld (row r in lane r & 15 of warp r >> 4) and are laid down in
//     shared memory for the block inverse; rows past the sequence end are written as zeros, so whatever the tile
//     held there (the next sequence's tokens) never enters the arithmetic,
//   - solve_heads() does the rest (the 16 x 16 substitutions and the small block products stay on CUDA cores / the
//     warp-level tensor path: they are 16-wide, far below a tcgen05 tile).
// The gates and beta of the unit are fetched while the tile is in flight.
struct KktTcSmem {
  union {  // the K tile is dead once K K^T is formed; the inverse X (fp32) then takes its place
    unsigned char ktile[16384];  // two 64-row x 128-byte regions (d 0-63 | d 64-127), 128-byte swizzle
    float x[kChunk * kFLd];
  };
  float kk[kChunk * kFLd];
  float beta[kChunk];
  float g[kChunk];
  uint64_t bar_tma, bar_mma, drain_bar;
  uint32_t tmem_base;
  int abort_flag;
};

template <bool kSingle>
__global__ void __launch_bounds__(128, 6)
kkt_solve_tc_kernel(const __grid_constant__ CUtensorMap map_k, const float* __restrict__ beta,
                    __nv_bfloat16* __restrict__ A, int H, int Hg, SeqArgs sa, const float* __restrict__ g_cum,
                    __nv_bfloat16* __restrict__ Ag, float scale, float* __restrict__ g_cum_out, int total_chunks,
                    int* status_dev, const GateAct act) {
  extern __shared__ unsigned char smem_dyn[];
  KktTcSmem& s = *reinterpret_cast<KktTcSmem*>(
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023)));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wc{&s.abort_flag, status_dev, 4, kWaitLimitCycles};
  if (tid == 0) {
    s.abort_flag = 0;
    mbar_init(&s.bar_tma, 1);
    mbar_init(&s.bar_mma, 1);
    mbar_init(&s.drain_bar, 1);
    fence_mbar_init();
    tma_prefetch_desc(&map_k);
  }
  if (warp == 0) {
    tmem_alloc(&s.tmem_base, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;
  constexpr uint32_t idesc = umma_idesc(64, 64, false, false, true);
  const uint32_t sk = smem_u32(s.ktile);
  const long long units = static_cast<long long>(total_chunks) * Hg;
  uint32_t phase = 0;
  float qk_unused[8][4];  // solve_heads' P_g input; never read here (no P_g)
#pragma unroll 1
  for (long long u = blockIdx.x; u < units; u += gridDim.x) {
    if (s.abort_flag) break;  // read by every thread after the barrier that ended the previous unit
    const int chunk = static_cast<int>(u / Hg), hg = static_cast<int>(u - static_cast<long long>(chunk) * Hg);
    const ChunkPos p = chunk_lookup(sa, chunk);
    if (tid == 0) {
      mbar_arrive_expect_tx(&s.bar_tma, 16384);
      tma_load_3d(s.ktile, &map_k, &s.bar_tma, 0, hg, p.tok0);
      tma_load_3d(s.ktile + 8192, &map_k, &s.bar_tma, 64, hg, p.tok0);
    }
    if (kSingle && tid < kChunk) {  // beta and the gates while the tile is in flight
      float bv = 0.f;
      if (tid < p.len) {
        bv = act_beta(act, __ldg(beta + static_cast<size_t>(p.tok0 + tid) * H + hg));
        if (act.beta_out) act.beta_out[static_cast<size_t>(p.tok0 + tid) * H + hg] = bv;
      }
      s.beta[tid] = bv;
      if (Ag) load_gates(s.g, g_cum, g_cum_out, static_cast<size_t>(p.tok0) * H + hg, H, p.len, tid, act, hg);
    }
    mbar_wait(wc, &s.bar_tma, phase, 1);
    if (warp == 0) {
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // K K^T: A and B are the same K-major tile
          const uint64_t d = umma_desc_sw128(sk + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024);
          umma_ss(tm, d, d, idesc, kk > 0);
        }
        umma_commit(&s.bar_mma);
      }
      __syncwarp();
    }
    mbar_wait(wc, &s.bar_mma, phase, 2);
    phase ^= 1;
    tc_fence_after();
    {
      // accumulator row r = 16 warp + lane (lanes 0-15) -> s.kk; only the lower block triangle is read later
      uint32_t r0[32], r1[32];
      tmem_ld32(tmem_addr(tm, warp * 32, 0), r0);
      tmem_ld32(tmem_addr(tm, warp * 32, 32), r1);
      tmem_wait_ld();
      tc_fence_before();
      __syncthreads();  // every warp is past its reads of tensor memory and nobody reads the K tile any more: x may be written
      if (lane < 16) {
        const int r = 16 * warp + lane;
        const bool live = r < p.len;
        float* dst = &s.kk[r * kFLd];
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          if (c4 < 4 * (warp + 1)) {
            float4 v0 = make_float4(__uint_as_float(r0[4 * c4]), __uint_as_float(r0[4 * c4 + 1]), __uint_as_float(r0[4 * c4 + 2]),
                                    __uint_as_float(r0[4 * c4 + 3]));
            if (!live) v0 = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(dst + 4 * c4) = v0;
          }
        }
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          if (8 + c4 < 4 * (warp + 1)) {
            float4 v1 = make_float4(__uint_as_float(r1[4 * c4]), __uint_as_float(r1[4 * c4 + 1]), __uint_as_float(r1[4 * c4 + 2]),
                                    __uint_as_float(r1[4 * c4 + 3]));
            if (!live) v1 = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(dst + 32 + 4 * c4) = v1;
          }
        }
      }
      {  // the two 16x16 blocks above the diagonal that the 32x32 block products read must be zero
        const int blk = tid >> 6, idx = tid & 63;
        *reinterpret_cast<float4*>(&s.x[(32 * blk + (idx >> 2)) * kFLd + 32 * blk + 16 + 4 * (idx & 3)]) =
            make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    solve_heads<kSingle>(s, p, qk_unused, beta, A, H, Hg, hg, g_cum, Ag, nullptr, scale, nullptr, g_cum_out, act);
    __syncthreads();  // the unit's reads of x are done: the next tile may land there
  }
  tc_fence_before();
  __syncthreads();
  if (s.abort_flag) {
    drain_after_abort(warp == 0 && elect_one(), &s.drain_bar);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tm, 64);
}

}  // namespace fq

static int kkt_launch(const void* k, const void* q, const float* beta, const float* g_cumsum, float* g_cum_out, void* A,
                      void* Ag, void* Pg, int a_is_input, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                      const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale, void* stream,
                      fq::GateAct act = fq::GateAct{0, 0, nullptr, nullptr, nullptr}) {
  using namespace fq;
  FQ_CHECK_ARG(k && beta && (A || (Ag && !a_is_input)), "fq_kkt_solve: null tensor");
  FQ_CHECK_ARG((Ag == nullptr && Pg == nullptr) || (g_cumsum != nullptr), "fq_kkt_solve: A_g / P_g need the gate cumsum");
  FQ_CHECK_ARG(Pg == nullptr || q != nullptr, "fq_kkt_solve: P_g needs q");
  FQ_CHECK_ARG(B > 0 && T >= 0 && H > 0 && Hg > 0 && H % Hg == 0 && n_seq > 0 && total_chunks >= 0,
               "fq_kkt_solve: bad sizes");
  FQ_CHECK_ARG(Hg <= 65535, "fq_kkt_solve: too many QK heads");
  FQ_CHECK_ARG((cu_seqlens == nullptr) == (chunk_offsets == nullptr),
               "fq_kkt_solve: cu_seqlens and chunk_offsets must be given together");
  FQ_CHECK_ARG(cu_seqlens == nullptr || B == 1, "fq_kkt_solve: packed batches need B == 1");
  FQ_CHECK_ARG(cu_seqlens != nullptr || n_seq == B, "fq_kkt_solve: dense batches need n_seq == B");
  if (total_chunks == 0) return FQ_OK;
  SeqArgs sa{T, cu_seqlens, chunk_offsets, n_seq, (T + kChunk - 1) / kChunk};
  {
    static std::atomic<unsigned long long> done0{0};
    const int rc_attr = set_smem_limit_once(reinterpret_cast<const void*>(kkt_solve_kernel<true>), static_cast<int>(sizeof(KktSmem)), &done0);
    if (rc_attr != FQ_OK) return rc_attr;
  }
  {
    static std::atomic<unsigned long long> done1{0};
    const int rc_attr = set_smem_limit_once(reinterpret_cast<const void*>(kkt_solve_kernel<false>), static_cast<int>(sizeof(KktSmem)), &done1);
    if (rc_attr != FQ_OK) return rc_attr;
  }
  if (!a_is_input && Pg == nullptr) {
    // the forward's case (only k is read): TMA + tcgen05 front end, persistent CTAs
    CUtensorMap mk;
    const uint64_t rows = static_cast<uint64_t>(B) * static_cast<uint64_t>(T);
    FQ_CHECK_ARG(rows > 0 && rows < (1ull << 31), "fq_kkt_solve: token count out of range");
    int rc = make_tmap_rows_heads_dim(&mk, k, rows, Hg, kDim, kChunk, 64);
    if (rc != FQ_OK) return rc;
    const int smem = static_cast<int>(sizeof(KktTcSmem) + 1024);
    {
      static std::atomic<unsigned long long> done0{0}, done1{0};
      if ((rc = set_smem_limit_once(reinterpret_cast<const void*>(kkt_solve_tc_kernel<true>), smem, &done0)) != FQ_OK) return rc;
      if ((rc = set_smem_limit_once(reinterpret_cast<const void*>(kkt_solve_tc_kernel<false>), smem, &done1)) != FQ_OK) return rc;
    }
    const long long units = static_cast<long long>(total_chunks) * Hg;
    const long long cap = 6LL * sm_count();
    const unsigned grid_tc = static_cast<unsigned>(units < cap ? units : cap);
    auto kern_tc = (H == Hg) ? kkt_solve_tc_kernel<true> : kkt_solve_tc_kernel<false>;
    kern_tc<<<grid_tc, 128, smem, static_cast<cudaStream_t>(stream)>>>(mk, beta, static_cast<__nv_bfloat16*>(A), H, Hg, sa, g_cumsum,
                                                                      static_cast<__nv_bfloat16*>(Ag), scale, g_cum_out,
                                                                      total_chunks, nullptr, act);
    FQ_CHECK_CUDA(cudaGetLastError());
    return FQ_OK;
  }
  dim3 grid(total_chunks, Hg);
  auto kern = (H == Hg) ? kkt_solve_kernel<true> : kkt_solve_kernel<false>;
  kern<<<grid, 128, sizeof(KktSmem), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(k), beta, static_cast<__nv_bfloat16*>(A), H, Hg, sa,
      static_cast<const __nv_bfloat16*>(q), g_cumsum, static_cast<__nv_bfloat16*>(Ag), static_cast<__nv_bfloat16*>(Pg),
      scale, a_is_input ? static_cast<const __nv_bfloat16*>(A) : nullptr, g_cum_out);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_kkt_solve_gated(const void* k, const void* q, const float* beta, const float* g_cumsum, void* A,
                                         void* Ag, void* Pg, int a_is_input, int B, int T, int H, int Hg,
                                         const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                                         int total_chunks, float scale, void* stream) {
  return kkt_launch(k, q, beta, g_cumsum, nullptr, A, Ag, Pg, a_is_input, B, T, H, Hg, cu_seqlens, chunk_offsets, n_seq,
                    total_chunks, scale, stream);
}

extern "C" FQ_API int fq_kkt_solve_fused(const void* k, const void* q, const float* beta, const float* g, float* g_cumsum,
                                         void* A, void* Ag, void* Pg, int B, int T, int H, int Hg,
                                         const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                                         int total_chunks, float scale, void* stream) {
  FQ_CHECK_ARG(g && g_cumsum && Ag, "fq_kkt_solve_fused: null tensor");
  FQ_CHECK_ARG(Pg == nullptr || q != nullptr, "fq_kkt_solve_fused: P_g needs q");
  return kkt_launch(k, q, beta, g, g_cumsum, A, Ag, Pg, 0, B, T, H, Hg, cu_seqlens, chunk_offsets, n_seq, total_chunks,
                    scale, stream);
}

extern "C" FQ_API int fq_kkt_solve(const void* k, const float* beta, void* A, int B, int T, int H, int Hg,
                                   const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                                   int total_chunks, void* stream) {
  return fq_kkt_solve_gated(k, nullptr, beta, nullptr, A, nullptr, nullptr, 0, B, T, H, Hg, cu_seqlens, chunk_offsets, n_seq,
                            total_chunks, 0.f, stream);
}

extern "C" FQ_API int fq_kkt_solve_fused_act(const void* k, const float* beta_raw, const float* g_raw, const float* A_log,
                                             const float* dt_bias, int gate_mode, int beta_mode, float* g_cumsum,
                                             float* beta_out, void* A, void* Ag, int B, int T, int H, int Hg,
                                             const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                                             int total_chunks, float scale, void* stream) {
  FQ_CHECK_ARG(g_raw && g_cumsum && Ag && beta_raw, "fq_kkt_solve_fused_act: null tensor");
  FQ_CHECK_ARG(gate_mode >= 0 && gate_mode <= 2 && beta_mode >= 0 && beta_mode <= 1, "fq_kkt_solve_fused_act: bad mode");
  FQ_CHECK_ARG(gate_mode != 2 || A_log != nullptr, "fq_kkt_solve_fused_act: gate mode 2 needs A_log");
  FQ_CHECK_ARG(beta_mode == 0 || beta_out != nullptr, "fq_kkt_solve_fused_act: an activated beta needs beta_out");
  fq::GateAct act{gate_mode, beta_mode, A_log, dt_bias, beta_mode ? beta_out : nullptr};
  return kkt_launch(k, nullptr, beta_raw, g_raw, g_cumsum, A, Ag, nullptr, 0, B, T, H, Hg, cu_seqlens, chunk_offsets, n_seq,
                    total_chunks, scale, stream, act);
}
