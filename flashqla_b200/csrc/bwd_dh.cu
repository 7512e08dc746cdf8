// Backward, serial part: the reverse recurrence of the state gradient dS, one persistent CTA per
// (sequence, V-head), chunks visited last to first.  Same transposed-state layout as the forward
// (dS^T in tensor memory: lane = v, column = k), so every product has M = 128:
//
//   D2   [128 x 64]  = dO^T P_g                   (state independent; A_g and P_g come from kkt_solve.cu)
//   D1   [128 x 64]  = dS^T_bf16 K^T
//        dV'^T = rho o D1 + D2
//   DW   [128 x 64]  = dV'^T A_g                  (aliases D1)
//        dVg^T = -gamma o DW
//   dS  <- gamma_last dS + dVg^T K + (scale*gamma o dO)^T Q
//
// The state BEFORE each update (the gradient w.r.t. the state after the chunk) is written as bf16
// (transposed, by TMA from a shared-memory tile) to dh [chunks, H, 128, 128]; the chunk-parallel kernel
// (bwd_chunk.cu) consumes it and forms dv, dq, dk, dg, dbeta.  Nothing else is stored here.
//
// The operands that the CUDA cores produce on the chain (dS^T, dV'^T, dVg^T as bf16) reach the tensor core as A
// operands in TENSOR memory (bf16 pairs, written over / beside the accumulators they come from): no shared-memory
// round trip and no operand fetch from shared memory for them.  The issuing warp runs its loop with all lanes and
// issues through one elected lane (see elect_one in common.cuh).
#include "flashqla.h"
#include "host.cuh"
#include "seq.cuh"

namespace fq {

constexpr int kDhThreads = 512;
constexpr int kDhGateStages = 4;
constexpr uint32_t kDhStageBytes = 32768 + 16384 + 8192 + 8192;

constexpr uint32_t kDhColS = 0;     // fp32 dS^T
constexpr uint32_t kDhColD1 = 128;  // D1, later DW
constexpr uint32_t kDhColD2 = 192;
constexpr uint32_t kDhColSB = 256;  // bf16 pairs of dS^T (64 columns): the A operand of D1 = dS^T K^T
constexpr uint32_t kDhColDOS = 320; // bf16 pairs of (scale*gamma o dO)^T (32 columns): an A operand of the dS update

struct BwdDhSmem {
  unsigned char kq[2][32768];    // k rows 0-63 | q rows 64-127, two 128-row regions (d 0-63 | 64-127)
  unsigned char dout[2][16384];  // dO tile [64 c][128 v] as two 64-row regions
  unsigned char a[2][8192];      // A_g tile [64 i][64 j]
  unsigned char pg[2][8192];     // P_g tile [64 i][64 j]
  unsigned char dsbf[32768];     // bf16 dS^T [128 v][128 k]
  float gate[kDhGateStages][4][kChunk];
  uint64_t full[2], empty[2], gate_full[kDhGateStages], gate_empty[kDhGateStages];
  uint64_t d2_done, d1_done, dw_done, ds_done;
  uint64_t ds_ready, ds_scaled, dvp_ready, dvg_ready, dos_ready;
  uint64_t drain_bar;    // only used by drain_after_abort
  uint64_t pg_ready[2];  // per stage: the aux warps may run one iteration ahead of the UMMA issuer
  uint32_t tmem_base;
  int abort_flag;
};

struct BwdDhParams {
  const float* g_cum;
  const float* beta;
  const float* dht;        // [n_seq, H, 128, 128] or nullptr
  float* dh0;              // [n_seq, H, 128, 128] or nullptr
  __nv_bfloat16* dh_out;   // [total_chunks, H, 128(v), 128(k)] TRANSPOSED, written by TMA from the operand buffer
  // context parallel (all nullptr for whole sequences): per piece the slot of dht / dh0 and the first
  // token after the piece's sequence; per (piece, head) the chunks to replay AFTER the piece
  // (bit 30: the replay starts at the sequence end, i.e. from dht).
  const int* dht_index;
  const int* dh0_index;
  const int* seq_end;
  const int* warmup;
  // further bits of warmup: bit 29 = start from dht_piece[piece] ([n_pieces, H, 128, 128] fp32, the corrected
  // gradient at the piece's end) with no replay; bit 27 = nothing to do for this (piece, head)
  const float* dht_piece;
  int H, Hg;
  float scale;
  SeqArgs sa;
  int* status_dev;
};

__device__ __forceinline__ uint32_t dh_koff(int kk) { return (kk >> 2) * 16384 + (kk & 3) * 32; }

__global__ void __launch_bounds__(kDhThreads, 1)
gdr_bwd_dh_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_a,
                  const __grid_constant__ CUtensorMap map_pg, const __grid_constant__ CUtensorMap map_dh,
                  const BwdDhParams p) {
  extern __shared__ unsigned char smem_dyn[];
  BwdDhSmem& s = *reinterpret_cast<BwdDhSmem*>(
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
  const int warm_code = p.warmup ? __ldg(p.warmup + static_cast<size_t>(seq) * p.H + h) : (1 << 30);
  const int warm = warm_code & 0xFFFFFF;
  const bool use_dht = (warm_code >> 30) & 1, use_piece_dht = (warm_code >> 29) & 1;
  if ((warm_code >> 27) & 1) return;  // nothing to do: leave before any barrier or tensor memory is set up
  // iteration `it` handles chunk n = total - 1 - it of the piece.  An EMPTY piece with a replay (warm > 0) only walks
  // the chunks behind it: its dh0 slot receives the state gradient at that point of the sequence.
  const int total = (nchunks > 0 || warm > 0) ? nchunks + warm : 0;
  // tokens available from the piece start to the end of its sequence (bounds the length of replayed chunks)
  const int avail = p.seq_end ? __ldg(p.seq_end + seq) - tok_begin : seq_len;
  WaitCtx wc{&s.abort_flag, p.status_dev, 2, kWaitLimitCycles};

  if (tid == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < 2; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 5); }
    for (int i = 0; i < kDhGateStages; ++i) { mbar_init(&s.gate_full[i], 64); mbar_init(&s.gate_empty[i], 12); }
    mbar_init(&s.d2_done, 1); mbar_init(&s.d1_done, 1); mbar_init(&s.dw_done, 1);
    mbar_init(&s.ds_done, 1);
    mbar_init(&s.ds_ready, 4); mbar_init(&s.ds_scaled, 4); mbar_init(&s.dvp_ready, 4); mbar_init(&s.dvg_ready, 4);
    mbar_init(&s.dos_ready, 4); mbar_init(&s.pg_ready[0], 4); mbar_init(&s.pg_ready[1], 4);
    mbar_init(&s.drain_bar, 1);
    fence_mbar_init();
    tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_do); tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_pg); tma_prefetch_desc(&map_dh);
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
      #pragma unroll 1
      for (int it = 0; it < total; ++it) {
        const int n = total - 1 - it, st = it & 1;
        if (it >= 2) mbar_wait(wc, &s.empty[st], ((it >> 1) + 1) & 1, 1);
        // after an expiry the other roles run through without waiting; no further tiles are requested then
        if (s.abort_flag) break;
        mbar_arrive_expect_tx(&s.full[st], kDhStageBytes);
        const int row = tok_begin + n * kChunk;
        tma_load_3d(s.kq[st], &map_k, &s.full[st], 0, hg, row);
        tma_load_3d(s.kq[st] + 16384, &map_k, &s.full[st], 64, hg, row);
        tma_load_3d(s.kq[st] + 8192, &map_q, &s.full[st], 0, hg, row);
        tma_load_3d(s.kq[st] + 24576, &map_q, &s.full[st], 64, hg, row);
        tma_load_3d(s.dout[st], &map_do, &s.full[st], 0, h, row);
        tma_load_3d(s.dout[st] + 8192, &map_do, &s.full[st], 64, h, row);
        tma_load_3d(s.a[st], &map_a, &s.full[st], 0, h, row);
        tma_load_3d(s.pg[st], &map_pg, &s.full[st], 0, h, row);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer: the whole warp runs the loop,
    // one elected lane issues (see elect_one)
    {
      constexpr uint32_t id64 = umma_idesc(128, 64, false, false, true);
      constexpr uint32_t id64_bmn = umma_idesc(128, 64, false, true, true);
      constexpr uint32_t id64_abmn = umma_idesc(128, 64, true, true, true);
      constexpr uint32_t id128_bmn = umma_idesc(128, 128, false, true, true);
      #pragma unroll 1
      for (int it = 0; it < total; ++it) {
        const int st = it & 1;
        const uint32_t ph = it & 1;
        const uint32_t skq = smem_u32(s.kq[st]), sa = smem_u32(s.a[st]), sdo = smem_u32(s.dout[st]), spg = smem_u32(s.pg[st]);
        mbar_wait(wc, &s.full[st], (it >> 1) & 1, 2);
        tc_fence_after();
        mbar_wait(wc, &s.pg_ready[st], (it >> 1) & 1, 3);
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tm + kDhColD2, umma_desc_sw128(sdo + kk * 2048, 8192, 1024), umma_desc_sw128(spg + kk * 2048, 8192, 1024),
                    id64_abmn, kk > 0);
          umma_commit(&s.d2_done);
        }
        __syncwarp();
        mbar_wait(wc, &s.ds_ready, ph, 4);
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ts(tm + kDhColD1, tm + kDhColSB + 8 * kk, umma_desc_sw128(skq + dh_koff(kk), 16, 1024),
                    id64, kk > 0);
          umma_commit(&s.d1_done);
        }
        __syncwarp();
        mbar_wait(wc, &s.dvp_ready, ph, 5);
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts(tm + kDhColD1, tm + kDhColD2 + 8 * kk, umma_desc_sw128(sa + kk * 2048, 8192, 1024),
                    id64_bmn, kk > 0);
          umma_commit(&s.dw_done);
        }
        __syncwarp();
        mbar_wait(wc, &s.dvg_ready, ph, 7);
        mbar_wait(wc, &s.dos_ready, ph, 8);
        mbar_wait(wc, &s.ds_scaled, ph, 9);
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts(tm + kDhColS, tm + kDhColD1 + 8 * kk, umma_desc_sw128(skq + kk * 2048, 16384, 1024),
                    id128_bmn, 1);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts(tm + kDhColS, tm + kDhColDOS + 8 * kk,
                    umma_desc_sw128(skq + 8192 + kk * 2048, 16384, 1024), id128_bmn, 1);
          umma_commit(&s.ds_done);
          umma_commit(&s.empty[st]);
        }
        __syncwarp();
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ gate loader
    const int t = tid - 64;
    #pragma unroll 1
    for (int it = 0; it < total; ++it) {
      const int n = total - 1 - it, gs = it & (kDhGateStages - 1);
      if (it >= kDhGateStages) mbar_wait(wc, &s.gate_empty[gs], ((it >> 2) + 1) & 1, 10);
      const int len = min(kChunk, avail - n * kChunk);
      const size_t row = static_cast<size_t>(tok_begin) + n * kChunk;
      const float gl = __ldg(p.g_cum + (row + len - 1) * p.H + h);
      // (beta is folded into the A_g tile by the pre-kernel: this kernel never reads it)
      const float gi = (t < len) ? __ldg(p.g_cum + (row + t) * p.H + h) : gl;
      s.gate[gs][0][t] = gi;
      s.gate[gs][1][t] = fast_exp(gi);
      s.gate[gs][2][t] = (t < len) ? fast_exp(gl - gi) : 0.f;
      mbar_arrive(&s.gate_full[gs]);
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ dV', dv, dVg (critical chain)
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32;
    #pragma unroll 1
    for (int it = 0; it < total; ++it) {
      const int n = total - 1 - it, gs = it & (kDhGateStages - 1);
      const uint32_t ph = it & 1;
      mbar_wait(wc, &s.gate_full[gs], (it >> 2) & 1, 11);
      mbar_wait(wc, &s.d2_done, ph, 12);
      mbar_wait(wc, &s.d1_done, ph, 13);
      tc_fence_after();
      uint32_t packed[32];
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t d1[16], d2[16];
        tmem_ld16(tmem_addr(tm, lane_base, kDhColD1 + qd * 16), d1);
        tmem_ld16(tmem_addr(tm, lane_base, kDhColD2 + qd * 16), d2);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const int c = qd * 16 + e;
          const float x0 = s.gate[gs][2][c] * __uint_as_float(d1[e]) + __uint_as_float(d2[e]);
          const float x1 = s.gate[gs][2][c + 1] * __uint_as_float(d1[e + 1]) + __uint_as_float(d2[e + 1]);
          packed[c >> 1] = pack_bf16(x0, x1);
        }
      }
      // dV'^T goes to the tensor core as an A operand in tensor memory (bf16 pairs: 32 columns), written over the
      // D2 accumulator that this thread has just read; likewise dVg^T below over the dW accumulator
      tmem_st32(tmem_addr(tm, lane_base, kDhColD2), packed);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.dvp_ready);
      mbar_wait(wc, &s.dw_done, ph, 14);
      tc_fence_after();
      uint32_t pg2[32];
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t dw[16];
        tmem_ld16(tmem_addr(tm, lane_base, kDhColD1 + qd * 16), dw);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const int c = qd * 16 + e;
          const float w0 = __uint_as_float(dw[e]), w1 = __uint_as_float(dw[e + 1]);
          pg2[c >> 1] = pack_bf16(-s.gate[gs][1][c] * w0, -s.gate[gs][1][c + 1] * w1);
        }
      }
      tmem_st32(tmem_addr(tm, lane_base, kDhColD1), pg2);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s.dvg_ready); mbar_arrive(&s.gate_empty[gs]); }
    }
  } else if (warp < 12) {
    // ------------------------------------------------------------------ state gradient: TMEM <-> bf16 operand, decay, dh
    const int v = tid - 256;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32;
    {
      const int in_slot = p.dht_index ? __ldg(p.dht_index + seq) : seq;
      const float* src = (p.dht && use_dht) ? p.dht + (static_cast<size_t>(in_slot) * p.H + h) * kDim * kDim + v : nullptr;
      if (use_piece_dht) src = p.dht_piece + (static_cast<size_t>(seq) * p.H + h) * kDim * kDim + v;
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = src ? __float_as_uint(__ldg(src + static_cast<size_t>(cb * 32 + i) * kDim)) : 0u;
        tmem_st32(tmem_addr(tm, lane_base, kDhColS + cb * 32), r);
      }
      tmem_wait_st();
    }
    #pragma unroll 1
    for (int it = 0; it < total; ++it) {
      const int n = total - 1 - it, gs = it & (kDhGateStages - 1);
      if (it > 0) {
        mbar_wait(wc, &s.ds_done, (it - 1) & 1, 15);
        tc_fence_after();
      }
      mbar_wait(wc, &s.gate_full[gs], (it >> 2) & 1, 16);
      const float gL = s.gate[gs][1][kChunk - 1];
      const bool store_dh = n < nchunks;
      // chain part: a bf16 copy of dS^T in tensor memory, the A operand of D1 = dS^T K^T (two column blocks per
      // round trip)
#pragma unroll 1
      for (int cb = 0; cb < 4; cb += 2) {
        uint32_t r0[32], r1[32];
        tmem_ld32(tmem_addr(tm, lane_base, kDhColS + cb * 32), r0);
        tmem_ld32(tmem_addr(tm, lane_base, kDhColS + cb * 32 + 32), r1);
        tmem_wait_ld();
        uint32_t pk[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          pk[j] = pack_bf16(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
          pk[16 + j] = pack_bf16(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
        }
        tmem_st32(tmem_addr(tm, lane_base, kDhColSB + cb * 16), pk);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.ds_ready);
      // trailing part: the same values as a shared-memory tile for the TMA store of dh, and the decay in place
      if (tid == 256) tma_store_wait_read<0>();  // the previous chunk's TMA store has read the tile
      asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, lane_base, kDhColS + cb * 32), r);
        tmem_wait_ld();
        if (p.dh_out != nullptr) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 q4;
            q4.x = pack_bf16(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
            q4.y = pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            q4.z = pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            q4.w = pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            *reinterpret_cast<uint4*>(s.dsbf + (cb >> 1) * 16384 + sw128(v, (cb & 1) * 64 + j * 16)) = q4;
          }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * gL);
        tmem_st32(tmem_addr(tm, lane_base, kDhColS + cb * 32), r);
      }
      fence_async_smem();
      asm volatile("bar.sync 2, 128;" ::: "memory");  // all four warps have written (and fenced) their rows
      if (store_dh && tid == 256) {
        const int hr = static_cast<int>((static_cast<long long>(chunk_off + n) * p.H + h) * kDim);
        tma_store_3d(&map_dh, s.dsbf, 0, 0, hr);
        tma_store_3d(&map_dh, s.dsbf + 16384, 64, 0, hr);
        tma_store_commit();
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s.ds_scaled); mbar_arrive(&s.gate_empty[gs]); }
    }
    if (tid == 256) tma_store_wait_all<0>();
    if (total > 0) {
      mbar_wait(wc, &s.ds_done, (total - 1) & 1, 17);
      tc_fence_after();
    }
    const int out_slot = p.dh0_index ? __ldg(p.dh0_index + seq) : seq;
    if (p.dh0 && out_slot >= 0) {
      float* dst = p.dh0 + (static_cast<size_t>(out_slot) * p.H + h) * kDim * kDim + v;
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, lane_base, kDhColS + cb * 32), r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[static_cast<size_t>(cb * 32 + i) * kDim] = __uint_as_float(r[i]);
      }
    }
  } else {
    // ------------------------------------------------------------------ tail fix of P_g, scaled dO^T
    const int v = tid - 384;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32;
    #pragma unroll 1
    for (int it = 0; it < total; ++it) {
      const int n = total - 1 - it, st = it & 1, gs = it & (kDhGateStages - 1);
      const uint32_t ph = it & 1;
      const int len = min(kChunk, avail - n * kChunk);
      mbar_wait(wc, &s.gate_full[gs], (it >> 2) & 1, 18);
      mbar_wait(wc, &s.full[st], (it >> 1) & 1, 19);
      // P_g rows past the sequence end were produced for the NEXT sequence's tokens: clear them
      if (len < kChunk) {
        for (int idx = v; idx < (kChunk - len) * 8; idx += 128) {
          const int r = len + (idx >> 3), pc = idx & 7;
          *reinterpret_cast<uint4*>(s.pg[st] + r * 128 + pc * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.pg_ready[st]);
      // (scale * gamma_c * dO[c][v])^T as bf16 pairs, formed before the wait below so that only the store remains
      // once the previous iteration's state update has consumed the columns
      uint32_t pk[32];
      {
        const unsigned char* dt = s.dout[st] + (v >> 6) * 8192;
        const uint32_t vb = (v & 63) * 2;
#pragma unroll
        for (int c = 0; c < kChunk; c += 2) {
          const float x0 = __uint_as_float(static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(dt + sw128(c, vb))) << 16);
          const float x1 = __uint_as_float(static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(dt + sw128(c + 1, vb))) << 16);
          const float s0 = (c < len) ? p.scale * s.gate[gs][1][c] * x0 : 0.f;
          const float s1 = (c + 1 < len) ? p.scale * s.gate[gs][1][c + 1] * x1 : 0.f;
          pk[c >> 1] = pack_bf16(s0, s1);
        }
      }
      if (it > 0) mbar_wait(wc, &s.ds_done, (it - 1) & 1, 21);
      tc_fence_after();
      tmem_st32(tmem_addr(tm, lane_base, kDhColDOS), pk);  // A operand in tensor memory, like dV' and dVg
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s.dos_ready); mbar_arrive(&s.empty[st]); mbar_arrive(&s.gate_empty[gs]); }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (s.abort_flag) {  // a wait expired somewhere in the CTA (the same value for every thread: all roles are done)
    drain_after_abort(warp == 1 && elect_one(), &s.drain_bar);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tm, 512);
}

}  // namespace fq

extern "C" FQ_API int fq_gdr_bwd_dh(const void* q, const void* k, const void* Ag, const void* Pg, const void* dout,
                                    const float* g_cumsum, const float* beta, const float* dht, float* dh0,
                                    void* dh_out, int B, int T, int H, int Hg,
                                    const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                                    int total_chunks, float scale, int32_t* status_dev, void* stream) {
  return fq_gdr_bwd_dh_cp(q, k, Ag, Pg, dout, g_cumsum, beta, dht, dh0, dh_out, nullptr, nullptr, nullptr,
                          nullptr, B, T, H, Hg, cu_seqlens, chunk_offsets, n_seq, total_chunks, scale, status_dev, stream);
}

extern "C" FQ_API int fq_gdr_bwd_dh_cp(const void* q, const void* k, const void* Ag, const void* Pg, const void* dout,
                                       const float* g_cumsum, const float* beta, const float* dht, float* dh0,
                                       void* dh_out, const int32_t* dht_index,
                                       const int32_t* dh0_index, const int32_t* seq_end, const int32_t* warmup, int B,
                                       int T, int H, int Hg, const int32_t* cu_seqlens, const int32_t* chunk_offsets,
                                       int n_seq, int total_chunks, float scale, int32_t* status_dev, void* stream) {
  return fq_gdr_bwd_dh_cp_ex(q, k, Ag, Pg, dout, g_cumsum, beta, dht, dh0, dh_out, dht_index, dh0_index, seq_end, warmup,
                             nullptr, B, T, H, Hg, cu_seqlens, chunk_offsets, n_seq, total_chunks, scale, status_dev,
                             stream);
}

extern "C" FQ_API int fq_gdr_bwd_dh_cp_ex(const void* q, const void* k, const void* Ag, const void* Pg,
                                          const void* dout, const float* g_cumsum, const float* beta, const float* dht,
                                          float* dh0, void* dh_out, const int32_t* dht_index, const int32_t* dh0_index,
                                          const int32_t* seq_end, const int32_t* warmup, const float* dht_piece, int B,
                                          int T, int H, int Hg, const int32_t* cu_seqlens,
                                          const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale,
                                          int32_t* status_dev, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(q && k && Ag && Pg && dout && g_cumsum && beta && dh_out, "fq_gdr_bwd_dh: null tensor");
  FQ_CHECK_ARG(B > 0 && T >= 0 && H > 0 && Hg > 0 && H % Hg == 0 && n_seq > 0 && total_chunks >= 0,
               "fq_gdr_bwd_dh: bad sizes");
  FQ_CHECK_ARG((cu_seqlens == nullptr) == (chunk_offsets == nullptr),
               "fq_gdr_bwd_dh: cu_seqlens and chunk_offsets must be given together");
  FQ_CHECK_ARG(cu_seqlens == nullptr || B == 1, "fq_gdr_bwd_dh: packed batches need B == 1");
  FQ_CHECK_ARG(cu_seqlens != nullptr || n_seq == B, "fq_gdr_bwd_dh: dense batches need n_seq == B");
  const uint64_t rows = static_cast<uint64_t>(B) * static_cast<uint64_t>(T);
  FQ_CHECK_ARG(rows > 0 && rows < (1ull << 31), "fq_gdr_bwd_dh: token count out of range");
  CUtensorMap mq, mk, mdo, ma, mpg, mdh;
  int rc;
  if ((rc = make_tmap_rows_heads_dim(&mq, q, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mk, k, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdo, dout, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&ma, Ag, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mpg, Pg, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  {
    const uint64_t hrows = static_cast<uint64_t>(total_chunks) * H * kDim;
    FQ_CHECK_ARG(hrows > 0 && hrows < (1ull << 31), "fq_gdr_bwd_dh: chunk count out of range");
    if ((rc = make_tmap_rows_heads_dim(&mdh, dh_out, hrows, 1, kDim, kDim, 64)) != FQ_OK) return rc;
  }
  BwdDhParams p;
  p.g_cum = g_cumsum; p.beta = beta; p.dht = dht; p.dh0 = dh0;
  p.dh_out = static_cast<__nv_bfloat16*>(dh_out);
  p.dht_index = dht_index; p.dh0_index = dh0_index; p.seq_end = seq_end; p.warmup = warmup;
  p.dht_piece = dht_piece;
  p.H = H; p.Hg = Hg; p.scale = scale;
  p.sa = SeqArgs{T, cu_seqlens, chunk_offsets, n_seq, (T + kChunk - 1) / kChunk};
  p.status_dev = status_dev;
  const size_t smem = sizeof(BwdDhSmem) + 1024;
  {
    static std::atomic<unsigned long long> done0{0};
    const int rc_attr = set_smem_limit_once(reinterpret_cast<const void*>(gdr_bwd_dh_kernel), static_cast<int>(smem), &done0);
    if (rc_attr != FQ_OK) return rc_attr;
  }
  const long long ctas = static_cast<long long>(n_seq) * H;
  FQ_CHECK_ARG(ctas < (1ll << 31), "fq_gdr_bwd_dh: too many (sequence, head) pairs");
  gdr_bwd_dh_kernel<<<static_cast<unsigned>(ctas), kDhThreads, smem, static_cast<cudaStream_t>(stream)>>>(mq, mk, mdo, ma, mpg, mdh, p);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}
