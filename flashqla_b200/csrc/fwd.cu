// Fused GDN forward: inter-chunk state recurrence + chunk outputs, one persistent CTA per
// (sequence, V-head).  All contractions run on tcgen05 with the state kept TRANSPOSED in tensor
// memory (S^T: lane = v, column = k), so that every product has M = 128:
//
//   PK   [128 x 64]  = [K;Q] K^T            rows 64..127 give Q K^T            (state independent)
//   UQ   [128 x 128] = S^T_bf16 [K;Q]^T     cols 0..63 = U^T, cols 64..127 = (Q S)^T
//   VD   [128 x 64]  = W^T A_g^T            W = V - gamma o U                  (aliases U^T)
//   OX   [128 x 64]  = V_d^T P_g^T
//   S   += V'^T K                           V' = rho o V_d; S was pre-scaled by gamma_last
//
// Per chunk:  o = scale*gamma o (Q S) + P_g V_d,   S <- gamma_last S + K^T V'.
// Warp roles (16 warps): 0 TMA producer, 1 UMMA issuer, 2-3 gate loader, 4-7 W / V_d / V'
// (critical chain), 8-11 state (TMEM -> bf16 operand, decay), 12-15 A_g / P_g and output.
// Every wait on an mbarrier is bounded; on expiry the CTA drains and reports through status_dev.
#include "flashqla.h"
#include "host.cuh"
#include "seq.cuh"

namespace fq {

constexpr int kFwdThreads = 512;
constexpr int kGateStages = 4;
constexpr uint32_t kStageBytes = 32768 + 16384 + 8192;

// TMEM column map (512 columns allocated)
constexpr uint32_t kColS = 0;     // fp32 state S^T, 128 columns
constexpr uint32_t kColUQ = 128;  // U^T | (QS)^T, 128 columns; V_d^T reuses the first 64
constexpr uint32_t kColPK = 256;  // [K;Q] K^T, 64 columns
constexpr uint32_t kColOX = 320;  // (P_g V_d)^T, 64 columns

struct FwdSmem {
  unsigned char kq[2][32768];  // per stage, two 128-row x 128-byte regions (d 0-63 | d 64-127); rows 0-63 k, 64-127 q
  unsigned char v[2][16384];   // per stage, two 64-row x 128-byte regions (v 0-63 | v 64-127)
  unsigned char a[2][8192];    // per stage, A tile [64 i][64 j]; rewritten in place as A_g
  unsigned char sbf[32768];    // bf16 S^T [128 v][128 k] as two 128-row regions
  unsigned char w[16384];      // W^T, later V'^T   [128 v][64 c]
  unsigned char vd[16384];     // V_d^T             [128 v][64 i]
  unsigned char pg[8192];      // P_g               [64 i][64 j]
  float gate[kGateStages][4][kChunk];  // g, exp(g), exp(g_last - g), beta
  uint64_t full[2], empty[2], gate_full[kGateStages], gate_empty[kGateStages];
  uint64_t pk_done, uq_done, vd_done, s_done;
  uint64_t s_ready, s_scaled, w_ready, vp_ready, ag_ready, pg_ready, o_free;
  uint32_t tmem_base;
  int abort_flag;
};

struct FwdParams {
  const float* g_cum;   // [rows, H] chunk-local cumsum of the log gate
  const float* beta;    // [rows, H]
  const float* h0;      // [n_seq, H, 128, 128] or nullptr
  float* ht;            // [n_out, H, 128, 128] or nullptr
  const int* ht_index;  // [n_seq] slot in ht per sequence (negative: do not write) or nullptr (= sequence index)
  __nv_bfloat16* o;     // [rows, H, 128] or nullptr
  __nv_bfloat16* h_out; // [total_chunks, H, 128, 128] state before each chunk, or nullptr
  int H, Hg;
  float scale;
  SeqArgs sa;
  int* status_dev;
};

__device__ __forceinline__ uint32_t kq_off(int kk) { return (kk >> 2) * 16384 + (kk & 3) * 32; }

__global__ void __launch_bounds__(kFwdThreads, 1)
gdr_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_a, const FwdParams p) {
  extern __shared__ unsigned char smem_dyn[];
  FwdSmem& s = *reinterpret_cast<FwdSmem*>(
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023)));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq = blockIdx.x / p.H, h = blockIdx.x - seq * p.H;
  const int hg = h / (p.H / p.Hg);
  int tok_begin, seq_len, chunk_off;
  if (p.sa.cu_seqlens == nullptr) {
    tok_begin = seq * p.sa.T;
    seq_len = p.sa.T;
    chunk_off = seq * p.sa.nc_dense;
  } else {
    tok_begin = __ldg(p.sa.cu_seqlens + seq);
    seq_len = __ldg(p.sa.cu_seqlens + seq + 1) - tok_begin;
    chunk_off = __ldg(p.sa.chunk_offsets + seq);
  }
  const int nchunks = (seq_len + kChunk - 1) / kChunk;
  WaitCtx wc{&s.abort_flag, p.status_dev, 1};

  if (tid == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < 2; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 5); }
    for (int i = 0; i < kGateStages; ++i) { mbar_init(&s.gate_full[i], 64); mbar_init(&s.gate_empty[i], 12); }
    mbar_init(&s.pk_done, 1); mbar_init(&s.uq_done, 1); mbar_init(&s.vd_done, 1); mbar_init(&s.s_done, 1);
    mbar_init(&s.s_ready, 4); mbar_init(&s.s_scaled, 4); mbar_init(&s.w_ready, 4); mbar_init(&s.vp_ready, 4);
    mbar_init(&s.o_free, 4); mbar_init(&s.ag_ready, 2); mbar_init(&s.pg_ready, 2);
    fence_mbar_init();
    tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v); tma_prefetch_desc(&map_a);
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int n = 0; n < nchunks; ++n) {
        const int st = n & 1;
        if (n >= 2 && !mbar_wait(wc, &s.empty[st], ((n >> 1) + 1) & 1, 1)) break;
        mbar_arrive_expect_tx(&s.full[st], kStageBytes);
        const int row = tok_begin + n * kChunk;
        tma_load_3d(s.kq[st], &map_k, &s.full[st], 0, hg, row);
        tma_load_3d(s.kq[st] + 16384, &map_k, &s.full[st], 64, hg, row);
        tma_load_3d(s.kq[st] + 8192, &map_q, &s.full[st], 0, hg, row);
        tma_load_3d(s.kq[st] + 24576, &map_q, &s.full[st], 64, hg, row);
        tma_load_3d(s.v[st], &map_v, &s.full[st], 0, h, row);
        tma_load_3d(s.v[st] + 8192, &map_v, &s.full[st], 64, h, row);
        tma_load_3d(s.a[st], &map_a, &s.full[st], 0, h, row);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      constexpr uint32_t id128 = umma_idesc(128, 128, false, false, true);
      constexpr uint32_t id64 = umma_idesc(128, 64, false, false, true);
      constexpr uint32_t id128_bmn = umma_idesc(128, 128, false, true, true);
      const uint32_t sbf = smem_u32(s.sbf), sw = smem_u32(s.w), svd = smem_u32(s.vd), spg = smem_u32(s.pg);
      for (int n = 0; n < nchunks; ++n) {
        const int st = n & 1;
        const uint32_t ph = n & 1;
        const uint32_t skq = smem_u32(s.kq[st]), sa = smem_u32(s.a[st]);
        if (!mbar_wait(wc, &s.full[st], (n >> 1) & 1, 2)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tm + kColPK, umma_desc_sw128(skq + kq_off(kk), 16, 1024), umma_desc_sw128(skq + kq_off(kk), 16, 1024),
                  id64, kk > 0);
        umma_commit(&s.pk_done);
        if (!mbar_wait(wc, &s.s_ready, ph, 3)) break;
        if (n > 0 && !mbar_wait(wc, &s.o_free, (n - 1) & 1, 4)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tm + kColUQ, umma_desc_sw128(sbf + kq_off(kk), 16, 1024), umma_desc_sw128(skq + kq_off(kk), 16, 1024),
                  id128, kk > 0);
        umma_commit(&s.uq_done);
        if (!mbar_wait(wc, &s.w_ready, ph, 5)) break;
        if (!mbar_wait(wc, &s.ag_ready, ph, 6)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kColUQ, umma_desc_sw128(sw + kk * 32, 16, 1024), umma_desc_sw128(sa + kk * 32, 16, 1024), id64,
                  kk > 0);
        umma_commit(&s.vd_done);
        if (!mbar_wait(wc, &s.vp_ready, ph, 7)) break;
        if (!mbar_wait(wc, &s.pg_ready, ph, 8)) break;
        if (!mbar_wait(wc, &s.s_scaled, ph, 9)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kColOX, umma_desc_sw128(svd + kk * 32, 16, 1024), umma_desc_sw128(spg + kk * 32, 16, 1024), id64,
                  kk > 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kColS, umma_desc_sw128(sw + kk * 32, 16, 1024), umma_desc_sw128(skq + kk * 2048, 16384, 1024),
                  id128_bmn, 1);
        umma_commit(&s.s_done);
        umma_commit(&s.empty[st]);
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ gate loader
    const int t = tid - 64;
    for (int n = 0; n < nchunks; ++n) {
      const int gs = n & (kGateStages - 1);
      if (n >= kGateStages && !mbar_wait(wc, &s.gate_empty[gs], ((n >> 2) + 1) & 1, 10)) break;
      const int len = min(kChunk, seq_len - n * kChunk);
      const size_t row = static_cast<size_t>(tok_begin) + n * kChunk;
      const float gl = __ldg(p.g_cum + (row + len - 1) * p.H + h);
      float gi = gl, bi = 0.f;
      if (t < len) {
        gi = __ldg(p.g_cum + (row + t) * p.H + h);
        bi = __ldg(p.beta + (row + t) * p.H + h);
      }
      s.gate[gs][0][t] = gi;
      s.gate[gs][1][t] = fast_exp(gi);
      s.gate[gs][2][t] = (t < len) ? fast_exp(gl - gi) : 0.f;
      s.gate[gs][3][t] = bi;
      mbar_arrive(&s.gate_full[gs]);
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ W, V_d, V' (critical chain)
    const int v = tid - 128;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32;
    for (int n = 0; n < nchunks; ++n) {
      const int st = n & 1, gs = n & (kGateStages - 1);
      const uint32_t ph = n & 1;
      if (!mbar_wait(wc, &s.full[st], (n >> 1) & 1, 11)) break;
      if (!mbar_wait(wc, &s.gate_full[gs], (n >> 2) & 1, 12)) break;
      if (!mbar_wait(wc, &s.uq_done, ph, 13)) break;
      tc_fence_after();
      const unsigned char* vt = s.v[st] + (v >> 6) * 8192;
      const uint32_t vb = (v & 63) * 2;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t u[32];
        tmem_ld32(tmem_addr(tm, lane_base, kColUQ + half * 32), u);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int c = half * 32 + i;
          const float v0 = __uint_as_float(static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(vt + sw128(c, vb))) << 16);
          const float v1 = __uint_as_float(static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(vt + sw128(c + 1, vb))) << 16);
          const float w0 = v0 - s.gate[gs][1][c] * __uint_as_float(u[i]);
          const float w1 = v1 - s.gate[gs][1][c + 1] * __uint_as_float(u[i + 1]);
          pk[i >> 1] = pack_bf16(w0, w1);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(s.w + sw128(v, half * 64 + j * 16)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
      }
      tc_fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s.w_ready); mbar_arrive(&s.empty[st]); }
      if (!mbar_wait(wc, &s.vd_done, ph, 14)) break;
      tc_fence_after();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t d[32];
        tmem_ld32(tmem_addr(tm, lane_base, kColUQ + half * 32), d);
        tmem_wait_ld();
        uint32_t pd[16], pp[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int c = half * 32 + i;
          const float d0 = __uint_as_float(d[i]), d1 = __uint_as_float(d[i + 1]);
          pd[i >> 1] = pack_bf16(d0, d1);
          pp[i >> 1] = pack_bf16(s.gate[gs][2][c] * d0, s.gate[gs][2][c + 1] * d1);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          *reinterpret_cast<uint4*>(s.vd + sw128(v, half * 64 + j * 16)) = make_uint4(pd[4 * j], pd[4 * j + 1], pd[4 * j + 2], pd[4 * j + 3]);
          *reinterpret_cast<uint4*>(s.w + sw128(v, half * 64 + j * 16)) = make_uint4(pp[4 * j], pp[4 * j + 1], pp[4 * j + 2], pp[4 * j + 3]);
        }
      }
      tc_fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s.vp_ready); mbar_arrive(&s.gate_empty[gs]); }
    }
  } else if (warp < 12) {
    // ------------------------------------------------------------------ state: TMEM <-> bf16 operand, decay, h / final state
    const int v = tid - 256;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32;
    {
      const float* src = p.h0 ? p.h0 + (static_cast<size_t>(seq) * p.H + h) * kDim * kDim + v : nullptr;
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = src ? __float_as_uint(__ldg(src + static_cast<size_t>(cb * 32 + i) * kDim)) : 0u;
        tmem_st32(tmem_addr(tm, lane_base, kColS + cb * 32), r);
      }
      tmem_wait_st();
    }
    bool alive = true;
    for (int n = 0; n < nchunks && alive; ++n) {
      const int gs = n & (kGateStages - 1);
      if (n > 0) {
        if (!mbar_wait(wc, &s.s_done, (n - 1) & 1, 15)) { alive = false; break; }
        tc_fence_after();
      }
      if (!mbar_wait(wc, &s.gate_full[gs], (n >> 2) & 1, 16)) { alive = false; break; }
      const float gL = s.gate[gs][1][kChunk - 1];
      __nv_bfloat16* hdst = p.h_out ? p.h_out + (static_cast<size_t>(chunk_off + n) * p.H + h) * kDim * kDim + v : nullptr;
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, lane_base, kColS + cb * 32), r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 q4;
          q4.x = pack_bf16(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
          q4.y = pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
          q4.z = pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
          q4.w = pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
          *reinterpret_cast<uint4*>(s.sbf + (cb >> 1) * 16384 + sw128(v, (cb & 1) * 64 + j * 16)) = q4;
        }
        if (hdst) {
#pragma unroll
          for (int i = 0; i < 32; ++i) hdst[static_cast<size_t>(cb * 32 + i) * kDim] = __float2bfloat16(__uint_as_float(r[i]));
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * gL);
        tmem_st32(tmem_addr(tm, lane_base, kColS + cb * 32), r);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.s_ready);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s.s_scaled); mbar_arrive(&s.gate_empty[gs]); }
    }
    if (alive && nchunks > 0) {
      alive = mbar_wait(wc, &s.s_done, (nchunks - 1) & 1, 17);
      tc_fence_after();
    }
    const int slot = p.ht_index ? __ldg(p.ht_index + seq) : seq;
    if (alive && p.ht && slot >= 0) {
      float* dst = p.ht + (static_cast<size_t>(slot) * p.H + h) * kDim * kDim + v;
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, lane_base, kColS + cb * 32), r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[static_cast<size_t>(cb * 32 + i) * kDim] = __uint_as_float(r[i]);
      }
    }
  } else {
    // ------------------------------------------------------------------ A_g, P_g and the output tile
    const int wid = warp - 12;
    const int v = tid - 384;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32;
    for (int n = 0; n < nchunks; ++n) {
      const int st = n & 1, gs = n & (kGateStages - 1);
      const uint32_t ph = n & 1;
      if (!mbar_wait(wc, &s.gate_full[gs], (n >> 2) & 1, 18)) break;
      if (wid < 2) {
        if (!mbar_wait(wc, &s.full[st], (n >> 1) & 1, 19)) break;
        const int i = wid * 32 + lane;
        const float gi = s.gate[gs][0][i];
#pragma unroll
        for (int j8 = 0; j8 < 8; ++j8) {
          uint4* ptr = reinterpret_cast<uint4*>(s.a[st] + sw128(i, j8 * 16));
          uint4 a4 = *ptr;
          uint32_t* aw = reinterpret_cast<uint32_t*>(&a4);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = j8 * 8 + 2 * e;
            const float x0 = (j <= i) ? bf16_lo(aw[e]) * fast_exp(gi - s.gate[gs][0][j]) * s.gate[gs][3][j] : 0.f;
            const float x1 = (j + 1 <= i) ? bf16_hi(aw[e]) * fast_exp(gi - s.gate[gs][0][j + 1]) * s.gate[gs][3][j + 1] : 0.f;
            aw[e] = pack_bf16(x0, x1);
          }
          *ptr = a4;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.ag_ready);
      } else {
        if (!mbar_wait(wc, &s.pk_done, ph, 20)) break;
        tc_fence_after();
        const int i = (wid - 2) * 32 + lane;
        const float gi = s.gate[gs][0][i];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld32(tmem_addr(tm, lane_base, kColPK + half * 32), r);
          tmem_wait_ld();
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const int j = half * 32 + e;
            const float x0 = (j <= i) ? p.scale * fast_exp(gi - s.gate[gs][0][j]) * __uint_as_float(r[e]) : 0.f;
            const float x1 = (j + 1 <= i) ? p.scale * fast_exp(gi - s.gate[gs][0][j + 1]) * __uint_as_float(r[e + 1]) : 0.f;
            pk[e >> 1] = pack_bf16(x0, x1);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(s.pg + sw128(i, half * 64 + j * 16)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        }
        tc_fence_before();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.pg_ready);
      }
      // output tile: o[c][v] = scale * gamma_c * (Q S)[c][v] + (P_g V_d)[c][v]
      if (!mbar_wait(wc, &s.s_done, ph, 21)) break;
      tc_fence_after();
      uint32_t packed[32];
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t oi[16], ox[16];
        tmem_ld16(tmem_addr(tm, lane_base, kColUQ + 64 + qd * 16), oi);
        tmem_ld16(tmem_addr(tm, lane_base, kColOX + qd * 16), ox);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const int c = qd * 16 + e;
          const float o0 = p.scale * s.gate[gs][1][c] * __uint_as_float(oi[e]) + __uint_as_float(ox[e]);
          const float o1 = p.scale * s.gate[gs][1][c + 1] * __uint_as_float(oi[e + 1]) + __uint_as_float(ox[e + 1]);
          packed[c >> 1] = pack_bf16(o0, o1);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s.o_free); mbar_arrive(&s.gate_empty[gs]); }
      if (p.o) {
        const int len = min(kChunk, seq_len - n * kChunk);
        unsigned short* dst = reinterpret_cast<unsigned short*>(p.o) +
                              (static_cast<size_t>(tok_begin) + n * kChunk) * p.H * kDim + static_cast<size_t>(h) * kDim + v;
        const size_t rs = static_cast<size_t>(p.H) * kDim;
#pragma unroll
        for (int c = 0; c < kChunk; c += 2) {
          if (c < len) dst[c * rs] = static_cast<unsigned short>(packed[c >> 1] & 0xFFFFu);
          if (c + 1 < len) dst[(c + 1) * rs] = static_cast<unsigned short>(packed[c >> 1] >> 16);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tm, 512);
}

}  // namespace fq

extern "C" FQ_API int fq_gdr_fwd(const void* q, const void* k, const void* v, const void* A, const float* g_cumsum,
                                 const float* beta, const float* h0, float* ht, const int32_t* ht_index, void* o,
                                 void* h_out, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                                 const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale,
                                 int32_t* status_dev, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(q && k && v && A && g_cumsum && beta, "fq_gdr_fwd: null input tensor");
  FQ_CHECK_ARG(B > 0 && T >= 0 && H > 0 && Hg > 0 && H % Hg == 0 && n_seq > 0 && total_chunks >= 0, "fq_gdr_fwd: bad sizes");
  FQ_CHECK_ARG((cu_seqlens == nullptr) == (chunk_offsets == nullptr),
               "fq_gdr_fwd: cu_seqlens and chunk_offsets must be given together");
  FQ_CHECK_ARG(cu_seqlens == nullptr || B == 1, "fq_gdr_fwd: packed batches need B == 1");
  FQ_CHECK_ARG(cu_seqlens != nullptr || n_seq == B, "fq_gdr_fwd: dense batches need n_seq == B");
  const uint64_t rows = static_cast<uint64_t>(B) * static_cast<uint64_t>(T);
  FQ_CHECK_ARG(rows > 0 && rows < (1ull << 31), "fq_gdr_fwd: token count out of range");
  CUtensorMap mq, mk, mv, ma;
  int rc;
  if ((rc = make_tmap_rows_heads_dim(&mq, q, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mk, k, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mv, v, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&ma, A, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  FwdParams p;
  p.g_cum = g_cumsum; p.beta = beta; p.h0 = h0; p.ht = ht; p.ht_index = ht_index;
  p.o = static_cast<__nv_bfloat16*>(o); p.h_out = static_cast<__nv_bfloat16*>(h_out);
  p.H = H; p.Hg = Hg; p.scale = scale;
  p.sa = SeqArgs{T, cu_seqlens, chunk_offsets, n_seq, (T + kChunk - 1) / kChunk};
  p.status_dev = status_dev;
  const size_t smem = sizeof(FwdSmem) + 1024;
  static bool attr_set[64] = {false};
  int dev = 0;
  FQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    FQ_CHECK_CUDA(cudaFuncSetAttribute(gdr_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr_set[dev] = true;
  }
  const long long ctas = static_cast<long long>(n_seq) * H;
  FQ_CHECK_ARG(ctas < (1ll << 31), "fq_gdr_fwd: too many (sequence, head) pairs");
  gdr_fwd_kernel<<<static_cast<unsigned>(ctas), kFwdThreads, smem, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, ma, p);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}
