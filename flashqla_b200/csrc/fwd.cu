// Fused GDN forward: inter-chunk state recurrence + chunk outputs, one persistent CTA per
// (sequence piece, V-head).  The chunk-parallel operand tile A_g = A o G o beta_col comes from the
// pre-kernel (kkt_solve.cu); this kernel carries what is serial and forms the second gated tile
// P_g = scale * G o (Q K^T) itself: the tensor core has the room, the tile never touches HBM unless a backward asks for
// it, and the pre-kernel neither reads q nor pays for the tile.  The state is kept TRANSPOSED in tensor memory
// (S^T: lane = v, column = k), so the products on the critical chain have M = 128:
//
//   U    [128 x 64]  = S^T_bf16 K^T
//   VD   [128 x 64]  = V^T A_g^T - (gamma o U)^T A_g^T = V_d^T     (the V term is state independent:
//                                                                  its A operand is the V tile as loaded)
//   S   += V'^T K                                                  V' = rho o V_d; S pre-scaled by gamma_last
//   OI   [64 x 128]  = Q S,   OX [64 x 128] = P_g V_d              natural orientation (row = token)
//   QK   [128 x 64]  = [K; Q] K^T of the NEXT chunk                rows 64-127 = Q K^T -> P_g.  It is parked in the
//                                                                  columns of U between this chunk's V_d products and
//                                                                  the next chunk's U
//
// Per chunk:  o = scale*gamma o OI + OX,   S <- gamma_last S + K^T V'.
// W^T = -(gamma o U)^T and V'^T are handed to the tensor core as A operands in TENSOR memory (bf16 pairs written over
// the accumulators they come from); the bf16 state and V_d^T stay in shared memory (they are B operands, and the
// state leaves by TMA).  The issuing warp runs its loop with all lanes and issues through one elected lane.
// Warp roles (16 warps): 0 TMA producer, 1 UMMA issuer, 2-3 gate loader, 4-11 chain group
// (TMEM state -> bf16 operand + decay, then -gamma o U, then V_d / V'), 12-15 output group: warps 14-15 (the two that
// can read TMEM lanes 64-127) turn Q K^T of the chunk ahead into its P_g tile, then all four lay the finished chunk's o
// rows down in a staging tile that leaves by TMA.
//
// Context parallel: a CTA may own a piece of a sequence.  It then first replays `w` whole chunks
// that precede the piece (state only, nothing stored) starting from a zero state - or from the
// sequence's initial state when the replay reaches the sequence start.  `w` comes from the gate
// scan (cp.cu): the decay accumulated over the replayed chunks makes older history negligible.
//
// Every wait on an mbarrier is bounded; on expiry the CTA reports through status_dev and runs through without
// blocking again (WaitCtx in common.cuh).
#include "flashqla.h"
#include "host.cuh"
#include "seq.cuh"
#include "fwd_params.cuh"

namespace fq {


constexpr int kFwdThreads = 512;
constexpr int kGateStages = 4;
constexpr uint32_t kStageBytes = 32768 + 16384 + 8192;  // k | q, v, A_g

// TMEM column map (512 columns allocated)
constexpr uint32_t kColS = 0;     // fp32 state S^T, 128 columns
constexpr uint32_t kColUQ = 128;  // U^T, 64 columns; between two chunks' use: [K; Q] K^T of the chunk ahead
constexpr uint32_t kColVD = 192;  // V_d^T, 64 columns
constexpr uint32_t kColOI = 256;  // Q S      [64 x 128] (M = 64: rows in lanes 0-15 of every 32-lane quarter)
constexpr uint32_t kColOX = 384;  // P_g V_d  [64 x 128]

struct FwdSmem {
  unsigned char kq[2][32768];  // per stage, two 128-row x 128-byte regions (d 0-63 | d 64-127); rows 0-63 k, 64-127 q
  unsigned char v[2][16384];   // per stage, two 64-row x 128-byte regions (v 0-63 | v 64-127)
  unsigned char a[2][8192];    // per stage, A_g tile [64 i][64 j]
  unsigned char pg[2][8192];   // P_g tile [64 i][64 j] of chunk c in buffer c & 1, written by the output warps
  unsigned char sbf[32768];    // bf16 S^T [128 v][128 k] as two 128-row regions
  unsigned char vd[16384];     // V_d^T             [128 v][64 i]
  unsigned char ostage[16384]; // o tile of a whole chunk [64 c][128 v] as two 64-row regions (v 0-63 | 64-127): TMA store
  float gate[kGateStages][4][kChunk];  // g, exp(g), exp(g_last - g), (unused)
  uint64_t full[2], empty[2], gate_full[kGateStages], gate_empty[kGateStages];
  uint64_t uq_done, vd_done, s_done, o_done, qk_done;
  uint64_t pq_ready;
  uint64_t s_ready, s_scaled, w_ready, vp_ready, o_free;
  uint64_t drain_bar;  // only used by drain_after_abort
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t kq_off(int kk) { return (kk >> 2) * 16384 + (kk & 3) * 32; }
// The chain group hands W^T = -(gamma o U)^T and V'^T to the tensor core as A operands in TENSOR memory, written over
// the accumulator they were computed from: the warp that owns the fp32 columns [32 hf, 32 hf + 32) of U^T (V_d^T)
// stores its 32 values as 16 bf16 pairs into columns [32 hf, 32 hf + 16).  K step kk (16 tokens = 8 pair columns):
__device__ __forceinline__ uint32_t a_col(int kk) { return 32 * (kk >> 1) + 8 * (kk & 1); }

// kStateOnly: no output is asked for (state recompute for the backward, state pass of the context-parallel fallback).
// The two instantiations keep each other's code out of the instruction cache; the state-only one also takes the bf16
// state from tensor memory (the output accumulators' columns are free there).
template <bool kStateOnly>
__global__ void __launch_bounds__(kFwdThreads, 1)
gdr_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_a,
               const __grid_constant__ CUtensorMap map_pg, const __grid_constant__ CUtensorMap map_h,
               const __grid_constant__ CUtensorMap map_o, const FwdParams p) {
  extern __shared__ unsigned char smem_dyn[];
  FwdSmem& s = *reinterpret_cast<FwdSmem*>(
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023)));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int entry = blockIdx.x / p.H, h = blockIdx.x - entry * p.H;
  const int seq = p.piece_map ? __ldg(p.piece_map + entry) : entry;
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
  const int warm_code = p.warmup ? __ldg(p.warmup + static_cast<size_t>(entry) * p.H + h) : (1 << 30);
  const int warm = warm_code & 0xFFFFFF;
  const bool use_h0 = (warm_code >> 30) & 1, use_piece_h0 = (warm_code >> 29) & 1, transition = (warm_code >> 28) & 1,
             skip = (warm_code >> 27) & 1;
  // iterations; iteration `it` handles chunk n = it - warm.  An EMPTY piece with a replay (warm > 0) is a state-only
  // run over the chunks in front of it: its final state is the state at that point of the sequence.
  const int total = ((nchunks > 0 || warm > 0) && !skip) ? warm + nchunks : 0;
  if (skip) return;  // nothing to do for this (entry, head): leave before any barrier or tensor memory is set up
  WaitCtx wc{&s.abort_flag, p.status_dev, 1, kWaitLimitCycles};

  if (tid == 0) {
    s.abort_flag = 0;
    for (int i = 0; i < 2; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 1); }
    for (int i = 0; i < kGateStages; ++i) { mbar_init(&s.gate_full[i], 64); mbar_init(&s.gate_empty[i], 12); }
    mbar_init(&s.uq_done, 1); mbar_init(&s.vd_done, 1); mbar_init(&s.s_done, 1); mbar_init(&s.o_done, 1);
    mbar_init(&s.qk_done, 1); mbar_init(&s.pq_ready, 4);
    mbar_init(&s.s_ready, 8); mbar_init(&s.s_scaled, 8); mbar_init(&s.w_ready, 8); mbar_init(&s.vp_ready, 8);
    mbar_init(&s.o_free, 4);
    mbar_init(&s.drain_bar, 1);
    fence_mbar_init();
    tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v); tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_pg); tma_prefetch_desc(&map_h); tma_prefetch_desc(&map_o);
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
      for (int it = 0; it < total; ++it) {
        const int st = it & 1;
        if (it >= 2) mbar_wait(wc, &s.empty[st], ((it >> 1) + 1) & 1, 1);
        // after an expiry the other roles run through without waiting; no further tiles are requested then (this
        // thread takes part in no barrier, and the byte counts of tiles that nobody waits for must not pile up)
        if (s.abort_flag) break;
        mbar_arrive_expect_tx(&s.full[st], kStageBytes);
        const int row = tok_begin + (it - warm) * kChunk;
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
    // ------------------------------------------------------------------ UMMA issuer: the whole warp runs the loop,
    // one elected lane issues (see elect_one)
    {
      constexpr uint32_t id64 = umma_idesc(128, 64, false, false, true);
      constexpr uint32_t id64_amn = umma_idesc(128, 64, true, false, true);
      constexpr uint32_t id128_bmn = umma_idesc(128, 128, false, true, true);
      constexpr uint32_t id_o = umma_idesc(64, 128, false, false, true);
      constexpr bool want_o = !kStateOnly;
      const uint64_t d_sbf = umma_desc_sw128(smem_u32(s.sbf), 16, 1024);
      const uint64_t d_vd = umma_desc_sw128(smem_u32(s.vd), 16, 1024);
      // stage-0 descriptors; stage 1 adds the stage stride to the address field (kept in registers)
      const uint64_t d_vmn0 = umma_desc_sw128(smem_u32(s.v[0]), 8192, 1024);
      const uint64_t d_kq0 = umma_desc_sw128(smem_u32(s.kq[0]), 16, 1024);
      const uint64_t d_kmn0 = umma_desc_sw128(smem_u32(s.kq[0]), 16384, 1024);
      const uint64_t d_a0 = umma_desc_sw128(smem_u32(s.a[0]), 16, 1024);
      const uint64_t d_pg0 = umma_desc_sw128(smem_u32(s.pg[0]), 16, 1024);
      // [K; Q] K^T of chunk `c` (stage c & 1) into the U columns: A = the whole 128-row k | q tile, B = its first 64
      // rows (k); rows 64-127 of the result are Q K^T.  Every barrier of this kernel completes exactly one phase per
      // iteration, replayed chunks included (their arrivals are trivial), so the phase of iteration `it` is it & 1.
      auto issue_qk = [&](int c) {
        const uint64_t d = desc_add(d_kq0, (c & 1) * 32768);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tm + kColUQ, desc_add(d, kq_off(kk)), desc_add(d, kq_off(kk)), id64, kk > 0);
        }
        __syncwarp();
      };
      for (int it = 0; it < total; ++it) {
        const int st = it & 1;
        const uint32_t ph = it & 1;
        const bool do_o = want_o && it >= warm;
        const uint64_t d_vmn = desc_add(d_vmn0, st * 16384), d_kq = desc_add(d_kq0, st * 32768),
                       d_kmn = desc_add(d_kmn0, st * 32768), d_a = desc_add(d_a0, st * 8192),
                       d_pg = desc_add(d_pg0, st * 8192);
        mbar_wait(wc, &s.full[st], (it >> 1) & 1, 2);
        tc_fence_after();
        if (want_o) {
          if (it == 0) {  // the first chunk has no earlier iteration to issue its Q K^T from
            if (do_o) issue_qk(0);
            if (elect_one()) umma_commit(&s.qk_done);
            __syncwarp();
          }
          // the output group has read this chunk's Q K^T out of the U columns (normally long ago: it was issued behind
          // the previous chunk's V_d products); waited for in replayed chunks too, which keeps that group within one
          // phase of this warp
          mbar_wait(wc, &s.pq_ready, ph, 22);
        }
        mbar_wait_spin(wc, &s.s_ready, ph, 3);
        tc_fence_after();
        if (elect_one()) {
          if (want_o) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)  // U^T = S^T K^T
              umma_ss(tm + kColUQ, desc_add(d_sbf, kq_off(kk)), desc_add(d_kq, kq_off(kk)), id64, kk > 0);
          } else {  // state-only runs: the bf16 state is an A operand in tensor memory (the output columns are free)
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_ts(tm + kColUQ, tm + kColOI + 8 * kk, desc_add(d_kq, kq_off(kk)), id64, kk > 0);
          }
          umma_commit(&s.uq_done);
        }
        __syncwarp();
        // the state-independent half of V_d goes behind U^T: it then runs beside the short W epilogue instead of beside the
        // conversion of the state, the longest stretch of the chain group
        if (!transition && elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)  // V_d^T = V^T A_g^T (A operand = the V tile as loaded, MN-major)
            umma_ss(tm + kColVD, desc_add(d_vmn, kk * 2048), desc_add(d_a, kk * 32), id64_amn, kk > 0);
        }
        __syncwarp();
        if (want_o) {  // OI = Q S: the accumulators of the previous chunk must have been drained
          if (it > 0) mbar_wait(wc, &s.o_free, (it - 1) & 1, 4);
          tc_fence_after();
          if (do_o && elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_ss(tm + kColOI, desc_add(d_kq, 8192 + kq_off(kk)), desc_add(d_sbf, kq_off(kk)), id_o, kk > 0);
          }
          __syncwarp();
        }
        mbar_wait_spin(wc, &s.w_ready, ph, 5);
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)  // V_d^T -= (gamma o U)^T A_g^T; A operand: bf16 pairs in the U columns
            umma_ts(tm + kColVD, tm + kColUQ + a_col(kk), desc_add(d_a, kk * 32), id64, (transition && kk == 0) ? 0 : 1);
          umma_commit(&s.vd_done);
        }
        __syncwarp();
        if (want_o && it + 1 < total) {
          // the U columns are dead from here until the next chunk's U: [K; Q] K^T of the next chunk goes there (its
          // tiles are in the other stage); it runs while the chain group forms V'
          if (it + 1 >= warm) {
            mbar_wait(wc, &s.full[st ^ 1], ((it + 1) >> 1) & 1, 24);
            tc_fence_after();
            issue_qk(it + 1);
          }
          if (elect_one()) umma_commit(&s.qk_done);
          __syncwarp();
        }
        mbar_wait_spin(wc, &s.vp_ready, ph, 7);
        mbar_wait_spin(wc, &s.s_scaled, ph, 9);
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)  // S^T += V'^T K; A operand: bf16 pairs in the V_d columns
            umma_ts(tm + kColS, tm + kColVD + a_col(kk), desc_add(d_kmn, kk * 2048), id128_bmn, 1);
          umma_commit(&s.s_done);
          if (do_o) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // OX = P_g V_d
              umma_ss(tm + kColOX, desc_add(d_pg, kk * 32), desc_add(d_vd, kk * 32), id_o, kk > 0);
          }
          umma_commit(&s.o_done);
          umma_commit(&s.empty[st]);
        }
        __syncwarp();
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ gate loader
    const int t = tid - 64;
    for (int it = 0; it < total; ++it) {
      const int n = it - warm, gs = it & (kGateStages - 1);
      if (it >= kGateStages) mbar_wait(wc, &s.gate_empty[gs], ((it >> 2) + 1) & 1, 10);
      const int len = min(kChunk, seq_len - n * kChunk);  // replayed chunks (n < 0) are always whole
      const long long row = static_cast<long long>(tok_begin) + static_cast<long long>(n) * kChunk;
      const float gl = __ldg(p.g_cum + (row + len - 1) * p.H + h);
      // (beta is folded into the A_g tile by the pre-kernel: this kernel never reads it)
      const float gi = (t < len) ? __ldg(p.g_cum + (row + t) * p.H + h) : gl;
      s.gate[gs][0][t] = gi;
      s.gate[gs][1][t] = fast_exp(gi);
      s.gate[gs][2][t] = (t < len) ? fast_exp(gl - gi) : 0.f;
      mbar_arrive(&s.gate_full[gs]);
    }
  } else if (warp < 12) {
    // ------------------------------------------------------------------ chain group (8 warps): per chunk
    //   state: TMEM -> bf16 operand (+ h), decay in TMEM;  W = V - gamma o U;  V_d and V' = rho o V_d
    // Warp w owns TMEM lanes 32*(w&3).. and, of every tile, the column half hf = (w-4)>>2.
    const int q4 = warp & 3, hf = (warp - 4) >> 2;
    const int v = q4 * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q4) * 32;
    {
      const int slot = p.h0_index ? __ldg(p.h0_index + seq) : seq;
      const float* src = (p.h0 && use_h0) ? p.h0 + (static_cast<size_t>(slot) * p.H + h) * kDim * kDim + v : nullptr;
      if (use_piece_h0) src = p.h0_piece + (static_cast<size_t>(seq) * p.H + h) * kDim * kDim + v;
#pragma unroll 1
      for (int pc = 0; pc < 2; ++pc) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kcol = 64 * hf + 32 * pc + i;
          r[i] = src ? __float_as_uint(__ldg(src + static_cast<size_t>(kcol) * kDim))
                     : ((transition && kcol == v) ? 0x3F800000u : 0u);
        }
        tmem_st32(tmem_addr(tm, lane_base, kColS + 64 * hf + 32 * pc), r);
      }
      tmem_wait_st();
    }
    for (int it = 0; it < total; ++it) {
      const int n = it - warm, gs = it & (kGateStages - 1);
      const uint32_t ph = it & 1;
      // ---- state -> bf16 operand, optional h, decay
      if (it > 0) {
        mbar_wait(wc, &s.s_done, (it - 1) & 1, 15);
        tc_fence_after();
      }
      mbar_wait(wc, &s.gate_full[gs], (it >> 2) & 1, 16);
      {
        const float gL = s.gate[gs][1][kChunk - 1];
        const bool store_h = (p.h_out != nullptr) && (n >= 0);
        constexpr bool state_only = kStateOnly;  // then the chain takes the bf16 state from tensor memory
        // both 32-column pieces are loaded before anything is stored, so only one TMEM round trip is exposed
        uint32_t r0[32], r1[32];
        tmem_ld32(tmem_addr(tm, lane_base, kColS + 64 * hf), r0);
        tmem_ld32(tmem_addr(tm, lane_base, kColS + 64 * hf + 32), r1);
        if (p.h_out != nullptr && !state_only) {  // the previous chunk's TMA store must have read the operand buffer;
          if (tid == 128) tma_store_wait_read<0>();  // waited for while the state is on its way from tensor memory
          asm volatile("bar.sync 2, 256;" ::: "memory");
        }
        tmem_wait_ld();
        uint32_t pk[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          pk[j] = pack_bf16(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
          pk[16 + j] = pack_bf16(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
        }
        if (state_only) {
          // chain part: bf16 pairs into the (unused) output columns, the A operand of U^T = S^T K^T
          tmem_st32(tmem_addr(tm, lane_base, kColOI + 32 * hf), pk);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s.s_ready);
          if (p.h_out != nullptr) {  // trailing part: the same values as the tile that the TMA store of h reads
            if (tid == 128) tma_store_wait_read<0>();
            asm volatile("bar.sync 2, 256;" ::: "memory");
          }
        }
        if (!state_only || p.h_out != nullptr) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<uint4*>(s.sbf + hf * 16384 + sw128(v, j * 16)) =
                make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            *reinterpret_cast<uint4*>(s.sbf + hf * 16384 + sw128(v, 64 + j * 16)) =
                make_uint4(pk[16 + 4 * j], pk[16 + 4 * j + 1], pk[16 + 4 * j + 2], pk[16 + 4 * j + 3]);
          }
          fence_async_smem();
        }
        if (!state_only) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&s.s_ready);
        }
        if (p.h_out != nullptr) {
          asm volatile("bar.sync 2, 256;" ::: "memory");  // all 8 warps have written (and fenced) their part
          if (store_h && tid == 128) {
            const int hr = static_cast<int>((static_cast<long long>(chunk_off + n) * p.H + h) * kDim);
            tma_store_3d(&map_h, s.sbf, 0, 0, hr);
            tma_store_3d(&map_h, s.sbf + 16384, 64, 0, hr);
            tma_store_commit();
          }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          r0[i] = __float_as_uint(__uint_as_float(r0[i]) * gL);
          r1[i] = __float_as_uint(__uint_as_float(r1[i]) * gL);
        }
        tmem_st32(tmem_addr(tm, lane_base, kColS + 64 * hf), r0);
        tmem_st32(tmem_addr(tm, lane_base, kColS + 64 * hf + 32), r1);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.s_scaled);
      }
      // ---- -(gamma_c U^T[v][c]) for c in [32 hf, 32 hf + 32): the state-dependent half of W = V - gamma o U
      mbar_wait(wc, &s.uq_done, ph, 13);
      tc_fence_after();
      {
        uint32_t u[32];
        tmem_ld32(tmem_addr(tm, lane_base, kColUQ + 32 * hf), u);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int c = 32 * hf + i;
          pk[i >> 1] = pack_bf16(-s.gate[gs][1][c] * __uint_as_float(u[i]), -s.gate[gs][1][c + 1] * __uint_as_float(u[i + 1]));
        }
        tmem_st16(tmem_addr(tm, lane_base, kColUQ + 32 * hf), pk);
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.w_ready);
      // ---- V_d^T and V'^T = rho o V_d^T
      mbar_wait(wc, &s.vd_done, ph, 14);
      tc_fence_after();
      {
        uint32_t d[32];
        tmem_ld32(tmem_addr(tm, lane_base, kColVD + 32 * hf), d);
        tmem_wait_ld();
        uint32_t pd[16], pp[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int c = 32 * hf + i;
          const float d0 = __uint_as_float(d[i]), d1 = __uint_as_float(d[i + 1]);
          pd[i >> 1] = pack_bf16(d0, d1);
          pp[i >> 1] = pack_bf16(s.gate[gs][2][c] * d0, s.gate[gs][2][c + 1] * d1);
        }
        tmem_st16(tmem_addr(tm, lane_base, kColVD + 32 * hf), pp);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(s.vd + sw128(v, hf * 64 + j * 16)) = make_uint4(pd[4 * j], pd[4 * j + 1], pd[4 * j + 2], pd[4 * j + 3]);
        tmem_wait_st();
      }
      tc_fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s.vp_ready); mbar_arrive(&s.gate_empty[gs]); }
    }
    if (p.h_out != nullptr && tid == 128) tma_store_wait_all<0>();
    // ---- final state
    if (total > 0) {
      mbar_wait(wc, &s.s_done, (total - 1) & 1, 17);
      tc_fence_after();
    }
    const int slot = p.ht_index ? __ldg(p.ht_index + entry) : entry;
    if (p.ht && slot >= 0) {
      float* dst = p.ht + (static_cast<size_t>(slot) * p.H + h) * kDim * kDim + v;
#pragma unroll 1
      for (int pc = 0; pc < 2; ++pc) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, lane_base, kColS + 64 * hf + 32 * pc), r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[static_cast<size_t>(64 * hf + 32 * pc + i) * kDim] = __uint_as_float(r[i]);
      }
    }
  } else {
    // ------------------------------------------------------------------ output group (4 warps)
    // o[c][:] = scale * gamma_c * OI[c][:] + OX[c][:]; thread (lane < 16) owns token row c = 16 * quarter + lane.
    // Before the finished chunk is drained, warps 14-15 - the two that can read TMEM lanes 64-127 - turn Q K^T of the
    // chunk AHEAD (parked in the U columns) into its P_g tile: P_g[r][j] = scale * exp(g_r - g_j) * (q_r . k_j), j <= r.
    const int q4 = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q4) * 32;
    const int c = 16 * q4 + (lane & 15);
    constexpr float kLog2e = 1.4426950408889634f;
    const float log2_scale = log2f(p.scale);
    auto ahead = [&](int ci) {
      const int n = ci - warm, gs = ci & (kGateStages - 1);
      mbar_wait(wc, &s.gate_full[gs], (ci >> 2) & 1, 19);
      if (!kStateOnly) mbar_wait(wc, &s.qk_done, ci & 1, 20);
      if (!kStateOnly && n >= 0 && q4 >= 2) {
        tc_fence_after();
        const int len = min(kChunk, seq_len - n * kChunk);
        const int r = 32 * (q4 - 2) + lane;   // token row; TMEM lane 64 + r
        const bool tile_store = p.pg_out != nullptr;
        if (tile_store) {  // the TMA stores of the earlier tiles have read their buffers
          if (tid == 448) tma_store_wait_read<0>();
          asm volatile("bar.sync 4, 64;" ::: "memory");
        }
        const float gr = kLog2e * s.gate[gs][0][r] + log2_scale;
        unsigned char* tile = s.pg[ci & 1];
        __nv_bfloat16* grow = tile_store ? p.pg_out + (static_cast<size_t>(tok_begin + n * kChunk + r) * p.H + h) * kChunk
                                         : nullptr;
        const bool whole = len == kChunk;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t qk[32];
          tmem_ld32(tmem_addr(tm, lane_base, kColUQ + 32 * half), qk);
          tmem_wait_ld();
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) {
            const int j0 = 32 * half + 8 * pc;
            uint4 x = make_uint4(0, 0, 0, 0);
            if (j0 <= r) {
              const float4 ga = *reinterpret_cast<const float4*>(&s.gate[gs][0][j0]);
              const float4 gb = *reinterpret_cast<const float4*>(&s.gate[gs][0][j0 + 4]);
              const float gj[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
              float y[8];
#pragma unroll
              for (int e = 0; e < 8; ++e)
                y[e] = (j0 + e <= r) ? exp2f(gr - kLog2e * gj[e]) * __uint_as_float(qk[8 * pc + e]) : 0.f;
              x = make_uint4(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]), pack_bf16(y[4], y[5]), pack_bf16(y[6], y[7]));
            }
            *reinterpret_cast<uint4*>(tile + sw128(r, (4 * half + pc) * 16)) = x;
            // a tail chunk's tile must not reach past the sequence end: its valid rows go out one by one
            if (tile_store && !whole && r < len) *(reinterpret_cast<uint4*>(grow) + 4 * half + pc) = x;
          }
        }
        fence_async_smem();
        if (tile_store) {
          asm volatile("bar.sync 4, 64;" ::: "memory");  // both warps have written (and fenced) their rows
          if (whole && tid == 448) {
            tma_store_3d(&map_pg, tile, 0, h, tok_begin + n * kChunk);
            tma_store_commit();
          }
        }
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.pq_ready);
    };
    if (total > 0) ahead(0);
    for (int it = 0; it < total; ++it) {
      const int n = it - warm, gs = it & (kGateStages - 1);
      const uint32_t ph = it & 1;
      if (it + 1 < total) ahead(it + 1);
      mbar_wait(wc, &s.gate_full[gs], (it >> 2) & 1, 18);
      mbar_wait(wc, &s.o_done, ph, 21);
      tc_fence_after();
      bool staged = false;
      if (!kStateOnly && n >= 0) {
        const int len = min(kChunk, seq_len - n * kChunk);
        // A whole chunk leaves through a shared-memory tile and two TMA stores (coalesced, and off the load/store
        // pipe that the chain group needs); a tail chunk is written row by row so that nothing past the sequence end
        // is touched.
        staged = len == kChunk;
        const bool wr = (lane < 16) && (c < len);
        const float f = p.scale * s.gate[gs][1][c];
        __nv_bfloat16* dst = p.o + (static_cast<size_t>(tok_begin + n * kChunk + (wr ? c : 0)) * p.H + h) * kDim;
        if (staged) {  // the previous chunk's TMA store has read the tile
          if (tid == 384) tma_store_wait_read<0>();
          asm volatile("bar.sync 3, 128;" ::: "memory");
        }
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          uint32_t oi[32], ox[32];
          tmem_ld32(tmem_addr(tm, lane_base, kColOI + 32 * pc), oi);
          tmem_ld32(tmem_addr(tm, lane_base, kColOX + 32 * pc), ox);
          tmem_wait_ld();
          if (wr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 x;
              x.x = pack_bf16(f * __uint_as_float(oi[8 * j]) + __uint_as_float(ox[8 * j]),
                              f * __uint_as_float(oi[8 * j + 1]) + __uint_as_float(ox[8 * j + 1]));
              x.y = pack_bf16(f * __uint_as_float(oi[8 * j + 2]) + __uint_as_float(ox[8 * j + 2]),
                              f * __uint_as_float(oi[8 * j + 3]) + __uint_as_float(ox[8 * j + 3]));
              x.z = pack_bf16(f * __uint_as_float(oi[8 * j + 4]) + __uint_as_float(ox[8 * j + 4]),
                              f * __uint_as_float(oi[8 * j + 5]) + __uint_as_float(ox[8 * j + 5]));
              x.w = pack_bf16(f * __uint_as_float(oi[8 * j + 6]) + __uint_as_float(ox[8 * j + 6]),
                              f * __uint_as_float(oi[8 * j + 7]) + __uint_as_float(ox[8 * j + 7]));
              if (staged) *reinterpret_cast<uint4*>(s.ostage + (pc >> 1) * 8192 + sw128(c, (pc & 1) * 64 + j * 16)) = x;
              else *reinterpret_cast<uint4*>(dst + 32 * pc + 8 * j) = x;
            }
          }
        }
      }
      // the accumulators have been read: the next chunk's output products may start
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s.o_free); mbar_arrive(&s.gate_empty[gs]); }
      if (staged) {
        fence_async_smem();
        asm volatile("bar.sync 3, 128;" ::: "memory");  // all four warps have written (and fenced) their rows
        if (tid == 384) {
          const int row0 = tok_begin + n * kChunk;
          tma_store_3d(&map_o, s.ostage, 0, h, row0);
          tma_store_3d(&map_o, s.ostage + 8192, 64, h, row0);
          tma_store_commit();
        }
      }
    }
    if (!kStateOnly && tid == 384) tma_store_wait_all<0>();
    if (!kStateOnly && tid == 448) tma_store_wait_all<0>();
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

extern "C" FQ_API int fq_gdr_fwd(const void* q, const void* k, const void* v, const void* Ag, void* Pg,
                                 const float* g_cumsum, const float* beta, const float* h0, float* ht,
                                 const int32_t* ht_index, void* o, void* h_out, int B, int T, int H, int Hg,
                                 const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq, int total_chunks,
                                 float scale, int32_t* status_dev, void* stream) {
  return fq_gdr_fwd_cp(q, k, v, Ag, Pg, g_cumsum, beta, h0, ht, ht_index, nullptr, nullptr, o, h_out, B, T, H, Hg,
                       cu_seqlens, chunk_offsets, n_seq, total_chunks, scale, status_dev, stream);
}

extern "C" FQ_API int fq_gdr_fwd_cp(const void* q, const void* k, const void* v, const void* Ag, void* Pg,
                                    const float* g_cumsum, const float* beta, const float* h0, float* ht,
                                    const int32_t* ht_index,
                                    const int32_t* h0_index, const int32_t* warmup, void* o, void* h_out, int B, int T,
                                    int H, int Hg, const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                                    int total_chunks, float scale, int32_t* status_dev, void* stream) {
  return fq_gdr_fwd_cp_ex(q, k, v, Ag, Pg, g_cumsum, beta, h0, ht, ht_index, h0_index, warmup, nullptr, n_seq, nullptr, o,
                          h_out, B, T, H, Hg, cu_seqlens, chunk_offsets, n_seq, total_chunks, scale, status_dev, stream);
}

extern "C" FQ_API int fq_gdr_fwd_cp_ex(const void* q, const void* k, const void* v, const void* Ag, void* Pg,
                                       const float* g_cumsum, const float* beta, const float* h0, float* ht,
                                       const int32_t* ht_index, const int32_t* h0_index, const int32_t* warmup,
                                       const int32_t* piece_map, int n_entries, const float* h0_piece, void* o,
                                       void* h_out, int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                                       const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale,
                                       int32_t* status_dev, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(n_entries > 0 && (piece_map != nullptr || n_entries == n_seq),
               "fq_gdr_fwd: a grid of entries other than the pieces needs piece_map");
  FQ_CHECK_ARG(piece_map == nullptr || (o == nullptr && h_out == nullptr),
               "fq_gdr_fwd: mapped entries are for state-only runs");
  FQ_CHECK_ARG(q && k && v && Ag && g_cumsum && beta, "fq_gdr_fwd: null input tensor");
  FQ_CHECK_ARG(B > 0 && T >= 0 && H > 0 && Hg > 0 && H % Hg == 0 && n_seq > 0 && total_chunks >= 0, "fq_gdr_fwd: bad sizes");
  FQ_CHECK_ARG((cu_seqlens == nullptr) == (chunk_offsets == nullptr),
               "fq_gdr_fwd: cu_seqlens and chunk_offsets must be given together");
  FQ_CHECK_ARG(cu_seqlens == nullptr || B == 1, "fq_gdr_fwd: packed batches need B == 1");
  FQ_CHECK_ARG(cu_seqlens != nullptr || n_seq == B, "fq_gdr_fwd: dense batches need n_seq == B");
  FQ_CHECK_ARG(warmup == nullptr || cu_seqlens != nullptr, "fq_gdr_fwd: warm-up tables need piece boundaries (cu_seqlens)");
  const uint64_t rows = static_cast<uint64_t>(B) * static_cast<uint64_t>(T);
  FQ_CHECK_ARG(rows > 0 && rows < (1ull << 31), "fq_gdr_fwd: token count out of range");
  CUtensorMap mq, mk, mv, ma, mpg, mh, mo;
  int rc;
  if ((rc = make_tmap_rows_heads_dim(&mq, q, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mk, k, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mv, v, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&ma, Ag, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  // the P_g tiles are an optional OUTPUT (kept for the backward); without it the map is never dereferenced
  if ((rc = make_tmap_rows_heads_dim(&mpg, Pg ? Pg : Ag, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  {
    const uint64_t hrows = static_cast<uint64_t>(total_chunks) * H * kDim;
    FQ_CHECK_ARG(hrows < (1ull << 31), "fq_gdr_fwd: too many chunks for the state tensor");
    // without h_out the map is never dereferenced; v stands in to keep the descriptor valid
    if (h_out) rc = make_tmap_rows_heads_dim(&mh, h_out, hrows, 1, kDim, kDim, 64);
    else rc = make_tmap_rows_heads_dim(&mh, v, rows, H, kDim, kChunk, 64);
    if (rc != FQ_OK) return rc;
  }
  // without o the map is never dereferenced; v stands in to keep the descriptor valid
  if ((rc = make_tmap_rows_heads_dim(&mo, o ? o : v, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  FwdParams p;
  p.g_cum = g_cumsum; p.beta = beta; p.h0 = h0; p.ht = ht; p.ht_index = ht_index; p.h0_index = h0_index;
  p.warmup = warmup; p.piece_map = piece_map; p.h0_piece = h0_piece;
  p.o = static_cast<__nv_bfloat16*>(o); p.h_out = static_cast<__nv_bfloat16*>(h_out);
  p.pg_out = o ? static_cast<__nv_bfloat16*>(Pg) : nullptr;
  p.H = H; p.Hg = Hg; p.scale = scale;
  p.sa = SeqArgs{T, cu_seqlens, chunk_offsets, n_seq, (T + kChunk - 1) / kChunk};
  p.status_dev = status_dev;
  const size_t smem = sizeof(FwdSmem) + 1024;
  {
    static std::atomic<unsigned long long> done0{0};
    const int rc_attr = set_smem_limit_once(reinterpret_cast<const void*>(gdr_fwd_kernel<false>), static_cast<int>(smem), &done0);
    if (rc_attr != FQ_OK) return rc_attr;
  }
  {
    static std::atomic<unsigned long long> done1{0};
    const int rc_attr = set_smem_limit_once(reinterpret_cast<const void*>(gdr_fwd_kernel<true>), static_cast<int>(smem), &done1);
    if (rc_attr != FQ_OK) return rc_attr;
  }
  const long long ctas = static_cast<long long>(n_entries) * H;
  FQ_CHECK_ARG(ctas < (1ll << 31), "fq_gdr_fwd: too many (sequence, head) pairs");
  if (o != nullptr && h_out != nullptr)  // a forward that keeps its states for a backward: the variant built for that
    return launch_gdr_fwd_train(mq, mk, mv, ma, mpg, mh, mo, p, static_cast<unsigned>(ctas), static_cast<cudaStream_t>(stream));
  auto kern = (o != nullptr) ? gdr_fwd_kernel<false> : gdr_fwd_kernel<true>;
  kern<<<static_cast<unsigned>(ctas), kFwdThreads, smem, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, ma, mpg, mh, mo, p);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

