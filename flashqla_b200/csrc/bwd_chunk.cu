// Backward, chunk-parallel part: given the state before each chunk (h, from the forward
// recurrence) and the state gradient after each chunk (dh, from bwd_dh.cu), every (chunk, V-head)
// unit is independent.  A persistent CTA walks units; per unit it runs six rounds of tcgen05 MMAs
// (M = 64: row = token of the chunk) with CUDA-core epilogues in between:
//
//   round 1  U = K S0 | D1 = K dS | D2 = P_g^T dO | accQ = dO S0^T
//            -> W = V - gamma o U, dV' = rho o D1 + D2, accQ *= scale*gamma, dg += rowsum(Q o accQ)
//   round 2  V' = A_g W | dW = A_g^T dV' | Z = S0^T dS (M = 128; only its trace = sum(dS o S0) is used, for dg_last)
//            -> dv = dW (output), dVg = -gamma o dW
//   round 3  K1 = V' dS^T | dPg = dO V'^T | dAg = dV' W^T | accK = dVg S0^T
//            -> dg += rowsum(K o accK); accK += rho o K1, dg -= rowsum(K o rho K1); dP = scale G o dPg;
//               dA = (G o dAg) beta_col; dg += rowsum of T = dPg o P_g + dAb o A_b; tiles T, T3 = dAb o A
//   round 4  accQ += dP K | accK += dP^T Q | X1 = A^T dA | column sums T^T 1, T3^T 1 (ones-vector MMAs)
//            -> dq, dg -= colsum(T), dbeta += colsum(T3)
//   round 5  X2 = X1 A^T | KK = K K^T
//            -> dL = -strict_lower(X2); dbeta += rowsum(dL o KK); T5 = beta_row dL
//   round 6  accK += T5 K + T5^T K  (dAs = T5 + T5^T, T5 = beta_row dL)  -> dk, dg, dbeta
//
// A_g and P_g come from kkt_solve.cu; S0 and dS arrive transposed ([v][k]) as the recurrences store them.
// dg is the gradient w.r.t. the chunk-local cumsum of the gate; the caller applies the reverse
// chunk cumsum.  dq / dk are written per V-head (bf16); the caller sums the heads of a QK group.
#include "flashqla.h"
#include "host.cuh"
#include "seq.cuh"

#include <mutex>

namespace fq {


constexpr int kBcThreads = 512;
constexpr int kStoreTid = 480;  // warp 15, lane 0: issues the TMA stores of dq, dk and dv (not one of the issuing warps)
constexpr uint32_t kBcLoadBytesA = 2 * 32768 + 2 * 16384;  // S0, dS, V, dO: requested a unit ahead
constexpr uint32_t kBcLoadBytesB = 2 * 16384 + 3 * 8192;  // K, Q, A, A_g, P_g: requested at the start of the unit

constexpr uint32_t kBcColU = 0;    // 128: U, then V', then K1, then X1 (0-63) / X2 (64-127)
constexpr uint32_t kBcColD1 = 128; // 128: D1 = K dS, then dW; later split into the two 64-column slots below
constexpr uint32_t kBcColQK = 128; // 64: dPg, then KK^T
constexpr uint32_t kBcColX = 192;  // 64: dAg, then the column sums
constexpr uint32_t kBcColK = 256;  // 128: D2 = P_g^T dO, then accK
constexpr uint32_t kBcColQ = 384;  // 128: accQ

struct BwdChunkSmem {
  // The tiles that a unit needs from its start (K, Q, A, A_g, P_g) and tiles that it only produces later (V', dVg,
  // dV', T) form pairs that swap roles from one unit to the next: the tiles of the CTA's next unit are loaded into
  // the partner buffers while the current unit finishes.  Pairs: kt/vp, qt/dvg, (at, ag)/dvp, pg/t12.
  unsigned char kt[16384];   // K  [64 c][128 k]  (two 64-row regions: k 0-63 | 64-127)
  unsigned char qt[16384];   // Q
  unsigned char wt[16384];   // V, rewritten as W
  unsigned char dot[16384];  // dO
  unsigned char dvp[16384];  // dV'  (computed)
  unsigned char dvg[16384];  // dVg  (computed)
  unsigned char vp[16384];   // V'
  unsigned char s0[32768];   // S0^T [128 v][128 k] (two 128-row regions: k 0-63 | 64-127), as stored by the recurrences
  unsigned char ds[32768];   // dS^T, same layout
  unsigned char at[8192];    // A   [64 i][64 j]
  unsigned char ag[8192];    // A_g -> dA -> dAs
  unsigned char pg[8192];    // P_g -> dP -> X1
  unsigned char t12[8192];   // T  = dPg o P_g + dAb o A_b   [64 i][64 j]
  unsigned char t3[8192];    // T3 = dAb o A                 [64 i][64 j]
  unsigned char ones[2048];  // 16 x 64 bf16 ones: B operand that turns an MMA into a column sum
  float g[kChunk], gam[kChunk], rho[kChunk], beta[kChunk];
  float dg_s[kChunk], db_s[kChunk];
  float dgl_s;
  uint64_t bar_tma_a, bar_tma_b, bar_mma;
  uint64_t drain_bar;  // only used by drain_after_abort
  uint32_t tmem_base;
  int abort_flag;
};

struct BwdChunkParams {
  const float* g_cum;
  const float* beta;
  __nv_bfloat16* dq;  // [rows, Hout, 128]
  __nv_bfloat16* dk;  // [rows, Hout, 128]
  float* dg;          // [rows, H]
  float* db;          // [rows, H]
  __nv_bfloat16* dv;  // [rows, H, 128]
  int H, Hg, total_chunks;
  int Hout;     // H: dq / dk per V-head;  Hg (grouped): the kernel sums the V-heads of a QK head itself - a CTA then
                // takes the heads of a group one after the other, stores the first head's tile and adds the others'
  float scale;
  SeqArgs sa;
  int* status_dev;
};

__device__ __forceinline__ uint32_t off64(int kk) { return (kk >> 2) * 8192 + (kk & 3) * 32; }
__device__ __forceinline__ uint32_t off128(int kk) { return (kk >> 2) * 16384 + (kk & 3) * 32; }

// Eight bf16 values of a tail chunk's row: stored, or (grouped output, later heads of a group) added to what the same
// thread stored for the earlier heads - the sum is formed in fp32 and rounded once, as the tile path does.  Kept out
// of line: only tail chunks come here, and the kernel's loop body is large as it is.
static __device__ __noinline__ void row_out(__nv_bfloat16* dst, uint4 x, bool accum) {
  uint4* ptr = reinterpret_cast<uint4*>(dst);
  if (accum) {
    const uint4 o = *ptr;
    x.x = pack_bf16(bf16_lo(o.x) + bf16_lo(x.x), bf16_hi(o.x) + bf16_hi(x.x));
    x.y = pack_bf16(bf16_lo(o.y) + bf16_lo(x.y), bf16_hi(o.y) + bf16_hi(x.y));
    x.z = pack_bf16(bf16_lo(o.z) + bf16_lo(x.z), bf16_hi(o.z) + bf16_hi(x.z));
    x.w = pack_bf16(bf16_lo(o.w) + bf16_lo(x.w), bf16_hi(o.w) + bf16_hi(x.w));
  }
  *ptr = x;
}

// sum over the 16 lanes of a half warp (lanes 0-15 and 16-31 reduce separately)
__device__ __forceinline__ float half_warp_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

__global__ void __launch_bounds__(kBcThreads, 1)
gdr_bwd_chunk_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                     const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_ag,
                     const __grid_constant__ CUtensorMap map_pg, const __grid_constant__ CUtensorMap map_h,
                     const __grid_constant__ CUtensorMap map_dh, const __grid_constant__ CUtensorMap map_dq,
                     const __grid_constant__ CUtensorMap map_dk, const __grid_constant__ CUtensorMap map_dv,
                     const BwdChunkParams p) {
  extern __shared__ unsigned char smem_dyn[];
  BwdChunkSmem& s = *reinterpret_cast<BwdChunkSmem*>(
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023)));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // warp w: TMEM lane quarter q4 = w & 3 (token rows 16 q4 .. +15 in lanes 0-15), column quarter cq = w >> 2:
  // 32 columns of a 128-column accumulator (half hf, piece pc), 16 columns of a 64-column one
  const int q4 = warp & 3, cq = warp >> 2, hf = cq >> 1, pc = cq & 1;
  const bool active = lane < 16;
  const int row = active ? (16 * q4 + lane) : 0;
  const uint32_t lane_base = static_cast<uint32_t>(q4) * 32;
  WaitCtx wc{&s.abort_flag, p.status_dev, 3, kWaitLimitCycles};
  const int heads_per_group = p.H / p.Hg;

  if (tid == 0) {
    s.abort_flag = 0;
    mbar_init(&s.bar_tma_a, 1);
    mbar_init(&s.bar_tma_b, 1);
    mbar_init(&s.bar_mma, 4);  // four issuing threads per round, one commit each
    mbar_init(&s.drain_bar, 4);
    fence_mbar_init();
    tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v); tma_prefetch_desc(&map_do);
    tma_prefetch_desc(&map_a); tma_prefetch_desc(&map_h);
    tma_prefetch_desc(&map_dh); tma_prefetch_desc(&map_ag); tma_prefetch_desc(&map_pg);
  }
  for (int i = tid; i < 512; i += kBcThreads) reinterpret_cast<uint32_t*>(s.ones)[i] = 0x3F803F80u;
  fence_async_smem();
  if (warp == 0) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;
  const uint32_t swt = smem_u32(s.wt), sdot = smem_u32(s.dot), ss0 = smem_u32(s.s0), sds = smem_u32(s.ds),
                 st3 = smem_u32(s.t3), sones = smem_u32(s.ones);
  // buffers that swap roles between units (see BwdChunkSmem)
  unsigned char *b_kt = s.kt, *b_vp = s.vp, *b_qt = s.qt, *b_dvg = s.dvg, *b_at = s.at, *b_dvp = s.dvp, *b_pg = s.pg,
                *b_t12 = s.t12;
  constexpr uint32_t id64_128_kk = umma_idesc(64, 128, false, false, true);
  constexpr uint32_t id64_128_kmn = umma_idesc(64, 128, false, true, true);
  constexpr uint32_t id64_128_mnmn = umma_idesc(64, 128, true, true, true);
  constexpr uint32_t id64_64_kk = umma_idesc(64, 64, false, false, true);
  constexpr uint32_t id64_64_mnmn = umma_idesc(64, 64, true, true, true);
  constexpr uint32_t id64_16_mnk = umma_idesc(64, 16, true, false, true);
  constexpr uint32_t id128_128_kk = umma_idesc(128, 128, false, false, true);

  uint32_t tma_phase = 0, mma_phase = 0;
  // S0, dS, V and dO are dead once the third round of products has completed, so the tiles of the CTA's next unit
  // are requested there and land while the rest of the unit runs
  auto load_a = [&](int chunk, int h) {
    const ChunkPos cp = chunk_lookup(p.sa, chunk);
    mbar_arrive_expect_tx(&s.bar_tma_a, kBcLoadBytesA);
    const int r0 = cp.tok0;
    tma_load_3d(s.wt, &map_v, &s.bar_tma_a, 0, h, r0);
    tma_load_3d(s.wt + 8192, &map_v, &s.bar_tma_a, 64, h, r0);
    tma_load_3d(s.dot, &map_do, &s.bar_tma_a, 0, h, r0);
    tma_load_3d(s.dot + 8192, &map_do, &s.bar_tma_a, 64, h, r0);
    const int hr = static_cast<int>((static_cast<long long>(chunk) * p.H + h) * kDim);
    tma_load_3d(s.s0, &map_h, &s.bar_tma_a, 0, 0, hr);
    tma_load_3d(s.s0 + 16384, &map_h, &s.bar_tma_a, 64, 0, hr);
    tma_load_3d(s.ds, &map_dh, &s.bar_tma_a, 0, 0, hr);
    tma_load_3d(s.ds + 16384, &map_dh, &s.bar_tma_a, 64, 0, hr);
  };
  // part 0: K, Q, A, A_g (and the byte count of the whole group); part 1: P_g
  auto load_b = [&](int chunk, int h, int part, unsigned char* dk, unsigned char* dq, unsigned char* da,
                    unsigned char* dpg) {
    const int hg = h / heads_per_group;
    const ChunkPos cp = chunk_lookup(p.sa, chunk);
    const int r0 = cp.tok0;
    if (part != 1) {
      mbar_arrive_expect_tx(&s.bar_tma_b, kBcLoadBytesB);
      tma_load_3d(dk, &map_k, &s.bar_tma_b, 0, hg, r0);
      tma_load_3d(dk + 8192, &map_k, &s.bar_tma_b, 64, hg, r0);
      tma_load_3d(dq, &map_q, &s.bar_tma_b, 0, hg, r0);
      tma_load_3d(dq + 8192, &map_q, &s.bar_tma_b, 64, hg, r0);
      tma_load_3d(da, &map_a, &s.bar_tma_b, 0, h, r0);
      tma_load_3d(da + 8192, &map_ag, &s.bar_tma_b, 0, h, r0);
    }
    if (part != 0) tma_load_3d(dpg, &map_pg, &s.bar_tma_b, 0, h, r0);
  };
  // Units (chunk, head) are walked with a stride of one grid; the index pair is stepped without divisions.  Grouped
  // output: the stride runs over (chunk, QK head) pairs and the V-heads of the pair follow one another (index j).
  const bool grouped = p.Hout != p.H;
  const int Hw = grouped ? p.Hg : p.H, Gw = grouped ? heads_per_group : 1;
  int oc = static_cast<int>(blockIdx.x) / Hw, oh = static_cast<int>(blockIdx.x) - oc * Hw, j = 0;
  const int step_c = static_cast<int>(gridDim.x) / Hw, step_h = static_cast<int>(gridDim.x) - step_c * Hw;
  int chunk = oc, h = oh * Gw;
  if (tid == 0 && chunk < p.total_chunks) load_a(chunk, h);

  // raw gate values of a unit: threads 0-63 fetch them one unit ahead, so that the loads are not waited for
  float gl_n = 0.f, gi_n = 0.f, bi_n = 0.f;
  auto fetch_gates = [&](int chunk, int h) {
    const ChunkPos cp = chunk_lookup(p.sa, chunk);
    const size_t base = static_cast<size_t>(cp.tok0) * p.H + h;
    gl_n = __ldg(p.g_cum + base + static_cast<size_t>(cp.len - 1) * p.H);
    gi_n = gl_n;
    bi_n = 0.f;
    if (tid < cp.len) {
      gi_n = __ldg(p.g_cum + base + static_cast<size_t>(tid) * p.H);
      bi_n = __ldg(p.beta + base + static_cast<size_t>(tid) * p.H);
    }
  };
  if (tid < kChunk && chunk < p.total_chunks) fetch_gates(chunk, h);
#pragma unroll 1
  for (int iter = 0; chunk < p.total_chunks; ++iter) {
    int noc = oc, noh = oh, nj = j + 1;  // this CTA's next unit
    if (nj >= Gw) {
      nj = 0; noc = oc + step_c; noh = oh + step_h;
      if (noh >= Hw) { noh -= Hw; ++noc; }
    }
    const int nchunk = noc, nh = noh * Gw + nj;
    const bool has_next = nchunk < p.total_chunks;
    const bool accum = grouped && j > 0;   // dq / dk of this unit are added to the group's
    const int ho = grouped ? h / heads_per_group : h;
    const int hg = h / heads_per_group;
    const ChunkPos cp = chunk_lookup(p.sa, chunk);
    const int len = cp.len;
    const bool whole = len == kChunk;  // then dq and dk leave by TMA; a tail chunk is written row by row
    unsigned char* b_ag = b_at + 8192;
    const uint32_t skt = smem_u32(b_kt), sqt = smem_u32(b_qt), sdvp = smem_u32(b_dvp), sdvg = smem_u32(b_dvg),
                   svp = smem_u32(b_vp), sat = smem_u32(b_at), sag = smem_u32(b_ag), spg = smem_u32(b_pg),
                   st12 = smem_u32(b_t12);
    // dq and dk of a whole chunk leave through the (dead) Q and K tiles and TMA stores issued by thread kStoreTid; those
    // tiles are written again in this unit's second round, after the syncs below
    if (tid == kStoreTid) tma_store_wait_read<0>();
    __syncthreads();  // the previous unit's shared-memory reads are complete
    // after an expiry no further unit is started (every thread reads the flag here, after the barrier and before any
    // wait of this unit, so all of them see the same value)
    if (s.abort_flag) break;

    if (tid == 0 && iter == 0) load_b(chunk, h, 2, b_kt, b_qt, b_at, b_pg);  // later units: requested a unit ahead
    if (tid < kChunk) {
      const float gl = gl_n, gi = gi_n, bi = bi_n;
      s.g[tid] = gi;
      s.gam[tid] = fast_exp(gi);
      s.rho[tid] = (tid < len) ? fast_exp(gl - gi) : 0.f;
      s.beta[tid] = bi;
      s.dg_s[tid] = 0.f;
      s.db_s[tid] = 0.f;
      if (tid == 0) s.dgl_s = 0.f;
    }
    __syncthreads();
    mbar_wait(wc, &s.bar_tma_a, tma_phase, 1);
    mbar_wait(wc, &s.bar_tma_b, tma_phase, 8);
    tma_phase ^= 1;

    // ---- pre-pass on shared memory: zero the rows past the sequence end
    if (len < kChunk) {
      unsigned char* tiles[4] = {b_kt, b_qt, s.wt, s.dot};
      const int nrows = kChunk - len;
      for (int idx = tid; idx < nrows * 16; idx += kBcThreads) {
        const int r = len + (idx >> 4), pc = idx & 15;
        const uint32_t off = (pc >> 3) * 8192 + r * 128 + (pc & 7) * 16;
#pragma unroll
        for (int t6 = 0; t6 < 4; ++t6) *reinterpret_cast<uint4*>(tiles[t6] + off) = make_uint4(0, 0, 0, 0);
        if (pc < 8) {
          *reinterpret_cast<uint4*>(b_at + r * 128 + pc * 16) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(b_ag + r * 128 + pc * 16) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(b_pg + r * 128 + pc * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      __syncthreads();
    }
    fence_async_smem();
    __syncthreads();

    const float gam_r = s.gam[row], rho_r = s.rho[row];

    // ================================================================== round 1
    if (warp < 4 && elect_one()) {  // the products of a round are issued by one elected lane of each of four warps
      tc_fence_after();
      if (warp == 0) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // U = K S0
          umma_ss(tm + kBcColU, desc_add(umma_desc_sw128(skt, 16, 1024), off64(kk)), desc_add(umma_desc_sw128(ss0, 16, 1024), off128(kk)),
                  id64_128_kk, kk > 0);
      } else if (warp == 1) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // D1 = K dS
          umma_ss(tm + kBcColD1, desc_add(umma_desc_sw128(skt, 16, 1024), off64(kk)), desc_add(umma_desc_sw128(sds, 16, 1024), off128(kk)),
                  id64_128_kk, kk > 0);
      } else if (warp == 2) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // D2 = P_g^T dO
          umma_ss(tm + kBcColK, desc_add(umma_desc_sw128(spg, 8192, 1024), kk * 2048), desc_add(umma_desc_sw128(sdot, 8192, 1024), kk * 2048),
                  id64_128_mnmn, kk > 0);
      } else if (warp == 3) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // accQ = dO S0^T
          umma_ss(tm + kBcColQ, desc_add(umma_desc_sw128(sdot, 16, 1024), off64(kk)), desc_add(umma_desc_sw128(ss0, 16384, 1024), kk * 2048),
                  id64_128_kmn, kk > 0);
      }
      umma_commit(&s.bar_mma);
    }
    __syncwarp();
    // while the first round runs: the next unit's gate values
    if (tid < kChunk && has_next) fetch_gates(nchunk, nh);
    mbar_wait(wc, &s.bar_mma, mma_phase, 2);
    mma_phase ^= 1;
    tc_fence_after();
    {
      // W = V - gamma o U (in place over V);  dV' = rho o D1 + D2
      {
        uint32_t u[32];
        tmem_ld32(tmem_addr(tm, lane_base, kBcColU + 64 * hf + 32 * pc), u);
        tmem_wait_ld();
        if (active) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4* ptr = reinterpret_cast<uint4*>(s.wt + hf * 8192 + sw128(row, (4 * pc + ch) * 16));
            uint4 x = *ptr;
            uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              xw[e] = pack_bf16(bf16_lo(xw[e]) - gam_r * __uint_as_float(u[8 * ch + 2 * e]),
                                bf16_hi(xw[e]) - gam_r * __uint_as_float(u[8 * ch + 2 * e + 1]));
            *ptr = x;
          }
        }
        uint32_t d2[32];
        tmem_ld32(tmem_addr(tm, lane_base, kBcColD1 + 64 * hf + 32 * pc), u);
        tmem_ld32(tmem_addr(tm, lane_base, kBcColK + 64 * hf + 32 * pc), d2);
        tmem_wait_ld();
        if (active) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 x;
            uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              xw[e] = pack_bf16(rho_r * __uint_as_float(u[8 * ch + 2 * e]) + __uint_as_float(d2[8 * ch + 2 * e]),
                                rho_r * __uint_as_float(u[8 * ch + 2 * e + 1]) + __uint_as_float(d2[8 * ch + 2 * e + 1]));
            *reinterpret_cast<uint4*>(b_dvp + hf * 8192 + sw128(row, (4 * pc + ch) * 16)) = x;
          }
        }
      }
      // accQ *= scale * gamma (written back); dg += rowsum(Q o accQ)
      float part = 0.f;
      {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, lane_base, kBcColQ + 64 * hf + 32 * pc), r);
        tmem_wait_ld();
        const float f = p.scale * gam_r;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const uint4 qv = *reinterpret_cast<const uint4*>(b_qt + hf * 8192 + sw128(row, (4 * pc + ch) * 16));
          const uint32_t* qw = reinterpret_cast<const uint32_t*>(&qv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float x0 = f * __uint_as_float(r[8 * ch + 2 * e]), x1 = f * __uint_as_float(r[8 * ch + 2 * e + 1]);
            part += bf16_lo(qw[e]) * x0 + bf16_hi(qw[e]) * x1;
            r[8 * ch + 2 * e] = __float_as_uint(x0);
            r[8 * ch + 2 * e + 1] = __float_as_uint(x1);
          }
        }
        tmem_st32(tmem_addr(tm, lane_base, kBcColQ + 64 * hf + 32 * pc), r);
      }
      if (active) atomicAdd(&s.dg_s[row], part);
      tmem_wait_st();
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();

    // ================================================================== round 2: V' = A_g W, dW = A_g^T dV'
    if (warp < 4 && elect_one()) {  // the products of a round are issued by one elected lane of each of four warps
      tc_fence_after();
      if (warp == 0) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kBcColU, desc_add(umma_desc_sw128(sag, 16, 1024), kk * 32), desc_add(umma_desc_sw128(swt, 8192, 1024), kk * 2048),
                  id64_128_kmn, kk > 0);
      } else if (warp == 1) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kBcColD1, desc_add(umma_desc_sw128(sag, 8192, 1024), kk * 2048), desc_add(umma_desc_sw128(sdvp, 8192, 1024), kk * 2048),
                  id64_128_mnmn, kk > 0);
      } else if (warp == 2) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // Z = S0^T-tile (dS^T-tile)^T [128 v x 128 v']: its trace is sum(dS o S0)
          umma_ss(tm + kBcColK, desc_add(umma_desc_sw128(ss0, 16, 1024), off128(kk)), desc_add(umma_desc_sw128(sds, 16, 1024), off128(kk)),
                  id128_128_kk, kk > 0);
      }
      umma_commit(&s.bar_mma);
    }
    __syncwarp();
    mbar_wait(wc, &s.bar_mma, mma_phase, 3);
    mma_phase ^= 1;
    tc_fence_after();
    {
      if (cq == 0) {
        // gamma_last * sum(dS o S0) = gamma_last * trace(Z): lane v of this warp's quarter picks column v
        uint32_t z[32];
        tmem_ld32(tmem_addr(tm, lane_base, kBcColK + 32 * q4), z);
        tmem_wait_ld();
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) d = (lane == i) ? __uint_as_float(z[i]) : d;
        d += __shfl_xor_sync(0xffffffffu, d, 16);
        d = half_warp_sum(d);
        if (lane == 0) atomicAdd(&s.dgl_s, d * s.gam[kChunk - 1]);
      }
      __nv_bfloat16* dvdst = p.dv + (static_cast<size_t>(cp.tok0 + row) * p.H + h) * kDim + 64 * hf;
      {
        uint32_t r[32], w2[32];
        tmem_ld32(tmem_addr(tm, lane_base, kBcColU + 64 * hf + 32 * pc), r);
        tmem_ld32(tmem_addr(tm, lane_base, kBcColD1 + 64 * hf + 32 * pc), w2);
        tmem_wait_ld();
        if (active) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 x, y, z;
            x.x = pack_bf16(__uint_as_float(r[8 * ch]), __uint_as_float(r[8 * ch + 1]));
            x.y = pack_bf16(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
            x.z = pack_bf16(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
            x.w = pack_bf16(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
            *reinterpret_cast<uint4*>(b_vp + hf * 8192 + sw128(row, (4 * pc + ch) * 16)) = x;
            uint32_t* yw = reinterpret_cast<uint32_t*>(&y);
            uint32_t* zw = reinterpret_cast<uint32_t*>(&z);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float d0 = __uint_as_float(w2[8 * ch + 2 * e]), d1 = __uint_as_float(w2[8 * ch + 2 * e + 1]);
              yw[e] = pack_bf16(d0, d1);                      // dv
              zw[e] = pack_bf16(-gam_r * d0, -gam_r * d1);    // dVg
            }
            *reinterpret_cast<uint4*>(b_dvg + hf * 8192 + sw128(row, (4 * pc + ch) * 16)) = z;
            // whole chunk: the two 64-column halves of dv go into the T and T3 tiles (free until the third round's
            // epilogue) and leave by TMA below
            if (whole) *reinterpret_cast<uint4*>((hf ? s.t3 : b_t12) + sw128(row, (4 * pc + ch) * 16)) = y;
            else if (row < len) *reinterpret_cast<uint4*>(dvdst + 32 * pc + 8 * ch) = y;
          }
        }
      }
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();
    if (whole && tid == kStoreTid) {
      tma_store_3d(&map_dv, b_t12, 0, h, cp.tok0);
      tma_store_3d(&map_dv, s.t3, 64, h, cp.tok0);
      tma_store_commit();
    }

    // ================================================================== round 3
    if (warp < 4 && elect_one()) {  // the products of a round are issued by one elected lane of each of four warps
      tc_fence_after();
      if (warp == 0) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tm + kBcColU, desc_add(umma_desc_sw128(svp, 16, 1024), off64(kk)), desc_add(umma_desc_sw128(sds, 16384, 1024), kk * 2048),
                  id64_128_kmn, kk > 0);
      } else if (warp == 1) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tm + kBcColQK, desc_add(umma_desc_sw128(sdot, 16, 1024), off64(kk)), desc_add(umma_desc_sw128(svp, 16, 1024), off64(kk)),
                  id64_64_kk, kk > 0);
      } else if (warp == 2) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tm + kBcColX, desc_add(umma_desc_sw128(sdvp, 16, 1024), off64(kk)), desc_add(umma_desc_sw128(swt, 16, 1024), off64(kk)),
                  id64_64_kk, kk > 0);
      } else if (warp == 3) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // accK = dVg S0^T
          umma_ss(tm + kBcColK, desc_add(umma_desc_sw128(sdvg, 16, 1024), off64(kk)), desc_add(umma_desc_sw128(ss0, 16384, 1024), kk * 2048),
                  id64_128_kmn, kk > 0);
      }
      umma_commit(&s.bar_mma);
    }
    __syncwarp();
    mbar_wait(wc, &s.bar_mma, mma_phase, 4);
    mma_phase ^= 1;
    tc_fence_after();
    if (whole) {  // the TMA store of dv has read the T / T3 tiles, which this round's epilogue writes
      if (tid == kStoreTid) tma_store_wait_read<0>();
      __syncthreads();
    }
    // The tiles that round three read last are dead from here on; two threads request this CTA's next unit there:
    // S0, dS, V, dO in place, and K, Q, A, A_g into V', dVg and dV'.  They land while rounds three to six finish.
    if (has_next && (warp == 2 || warp == 3)) {
      if (elect_one()) {
        if (warp == 2) load_a(nchunk, nh);
        else load_b(nchunk, nh, 0, b_vp, b_dvg, b_dvp, b_t12);
      }
      __syncwarp();
    }
    {
      // dg += rowsum(K o accK); then accK += rho o K1 ; kk = rowsum(K o rho K1)
      float kkp = 0.f, kap = 0.f;
      {
        uint32_t r[32], a2[32];
        tmem_ld32(tmem_addr(tm, lane_base, kBcColU + 64 * hf + 32 * pc), r);
        tmem_ld32(tmem_addr(tm, lane_base, kBcColK + 64 * hf + 32 * pc), a2);
        tmem_wait_ld();
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const uint4 kv = *reinterpret_cast<const uint4*>(b_kt + hf * 8192 + sw128(row, (4 * pc + ch) * 16));
          const uint32_t* kw = reinterpret_cast<const uint32_t*>(&kv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float x0 = rho_r * __uint_as_float(r[8 * ch + 2 * e]), x1 = rho_r * __uint_as_float(r[8 * ch + 2 * e + 1]);
            kap += bf16_lo(kw[e]) * __uint_as_float(a2[8 * ch + 2 * e]) + bf16_hi(kw[e]) * __uint_as_float(a2[8 * ch + 2 * e + 1]);
            kkp += bf16_lo(kw[e]) * x0 + bf16_hi(kw[e]) * x1;
            a2[8 * ch + 2 * e] = __float_as_uint(__uint_as_float(a2[8 * ch + 2 * e]) + x0);
            a2[8 * ch + 2 * e + 1] = __float_as_uint(__uint_as_float(a2[8 * ch + 2 * e + 1]) + x1);
          }
        }
        tmem_st32(tmem_addr(tm, lane_base, kBcColK + 64 * hf + 32 * pc), a2);
      }
      if (!active) kkp = 0.f;
      if (active) atomicAdd(&s.dg_s[row], kap - kkp);
      const float kks = half_warp_sum(kkp);
      if (lane == 0) atomicAdd(&s.dgl_s, kks);
      // dPg and dAg -> dP, dA, T, T3 tiles and the row sums of T: this warp's 16 columns.  Only lanes 0-15 hold
      // accumulator rows (M = 64), so each of them hands half of its columns to lane + 16: all 32 lanes work on
      // 8 columns (one 16-byte piece of the tile row).
      uint32_t r1[16], r2[16];
      tmem_ld16(tmem_addr(tm, lane_base, kBcColQK + 16 * cq), r1);
      tmem_ld16(tmem_addr(tm, lane_base, kBcColX + 16 * cq), r2);
      tmem_wait_ld();
      const int up = lane >> 4;                 // 0: columns 0-7 of the piece, 1: columns 8-15
      const int row2 = 16 * q4 + (lane & 15);   // row served by this lane
      const float g_r2 = s.g[row2];
      float a1[8], a2[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t h1 = __shfl_sync(0xffffffffu, r1[8 + i], lane & 15);
        const uint32_t h2 = __shfl_sync(0xffffffffu, r2[8 + i], lane & 15);
        a1[i] = __uint_as_float(up ? h1 : r1[i]);
        a2[i] = __uint_as_float(up ? h2 : r2[i]);
      }
      float rows = 0.f;
      {
        const uint32_t so = sw128(row2, (2 * cq + up) * 16);
        const uint4 pgv = *reinterpret_cast<const uint4*>(b_pg + so);
        const uint4 av = *reinterpret_cast<const uint4*>(b_at + so);
        const uint32_t* pw = reinterpret_cast<const uint32_t*>(&pgv);
        const uint32_t* aw = reinterpret_cast<const uint32_t*>(&av);
        uint4 dpv, dav, t12v, t3v;
        uint32_t* dpw = reinterpret_cast<uint32_t*>(&dpv);
        uint32_t* daw = reinterpret_cast<uint32_t*>(&dav);
        uint32_t* t12w = reinterpret_cast<uint32_t*>(&t12v);
        uint32_t* t3w = reinterpret_cast<uint32_t*>(&t3v);
        const int jb = 16 * cq + 8 * up;
        const float4 gj0 = *reinterpret_cast<const float4*>(&s.g[jb]);
        const float4 gj1 = *reinterpret_cast<const float4*>(&s.g[jb + 4]);
        const float4 bj0 = *reinterpret_cast<const float4*>(&s.beta[jb]);
        const float4 bj1 = *reinterpret_cast<const float4*>(&s.beta[jb + 4]);
        const float gj[8] = {gj0.x, gj0.y, gj0.z, gj0.w, gj1.x, gj1.y, gj1.z, gj1.w};
        const float bjv[8] = {bj0.x, bj0.y, bj0.z, bj0.w, bj1.x, bj1.y, bj1.z, bj1.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float dpo[2], dao[2], t12o[2], t3o[2];
#pragma unroll
          for (int z = 0; z < 2; ++z) {
            const int j = jb + 2 * e + z;
            const bool keep = j <= row2;
            const float G = keep ? fast_exp(g_r2 - gj[2 * e + z]) : 0.f;
            const float pgx = z ? bf16_hi(pw[e]) : bf16_lo(pw[e]);
            const float ax = z ? bf16_hi(aw[e]) : bf16_lo(aw[e]);
            const float dpg = a1[2 * e + z];
            const float dab = G * a2[2 * e + z];
            const float bj = bjv[2 * e + z];
            t12o[z] = keep ? (dpg * pgx + dab * ax * bj) : 0.f;
            t3o[z] = dab * ax;
            dpo[z] = p.scale * G * dpg;
            dao[z] = dab * bj;
          }
          dpw[e] = pack_bf16(dpo[0], dpo[1]);
          daw[e] = pack_bf16(dao[0], dao[1]);
          t12w[e] = pack_bf16(t12o[0], t12o[1]);
          // the row sums use the rounded values that the column-sum MMA sees, so the diagonal terms cancel exactly
          rows += bf16_lo(t12w[e]) + bf16_hi(t12w[e]);
          t3w[e] = pack_bf16(t3o[0], t3o[1]);
        }
        *reinterpret_cast<uint4*>(b_pg + so) = dpv;
        *reinterpret_cast<uint4*>(b_ag + so) = dav;
        *reinterpret_cast<uint4*>(b_t12 + so) = t12v;
        *reinterpret_cast<uint4*>(s.t3 + so) = t3v;
      }
      rows += __shfl_xor_sync(0xffffffffu, rows, 16);
      if (active) atomicAdd(&s.dg_s[row], rows);
      tmem_wait_st();
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();

    // ================================================================== round 4
    if (warp < 4 && elect_one()) {  // the products of a round are issued by one elected lane of each of four warps
      tc_fence_after();
      if (warp == 0) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kBcColQ, desc_add(umma_desc_sw128(spg, 16, 1024), kk * 32), desc_add(umma_desc_sw128(skt, 8192, 1024), kk * 2048),
                  id64_128_kmn, 1);
      } else if (warp == 1) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kBcColK, desc_add(umma_desc_sw128(spg, 8192, 1024), kk * 2048), desc_add(umma_desc_sw128(sqt, 8192, 1024), kk * 2048),
                  id64_128_mnmn, 1);
      } else if (warp == 2) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kBcColU, desc_add(umma_desc_sw128(sat, 8192, 1024), kk * 2048), desc_add(umma_desc_sw128(sag, 8192, 1024), kk * 2048),
                  id64_64_mnmn, kk > 0);
      } else if (warp == 3) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // column sums: D[j][:] = sum_i T[i][j]
          umma_ss(tm + kBcColX, desc_add(umma_desc_sw128(st12, 8192, 1024), kk * 2048), desc_add(umma_desc_sw128(sones, 16, 1024), kk * 32),
                  id64_16_mnk, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kBcColX + 16, desc_add(umma_desc_sw128(st3, 8192, 1024), kk * 2048), desc_add(umma_desc_sw128(sones, 16, 1024), kk * 32),
                  id64_16_mnk, kk > 0);
      }
      umma_commit(&s.bar_mma);
    }
    __syncwarp();
    mbar_wait(wc, &s.bar_mma, mma_phase, 5);
    mma_phase ^= 1;
    tc_fence_after();
    {
      uint32_t r[32];
      {
        uint32_t x1[16];
        tmem_ld16(tmem_addr(tm, lane_base, kBcColU + 16 * cq), x1);
        tmem_wait_ld();
        if (active) {
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            uint4 x;
            x.x = pack_bf16(__uint_as_float(x1[8 * ch]), __uint_as_float(x1[8 * ch + 1]));
            x.y = pack_bf16(__uint_as_float(x1[8 * ch + 2]), __uint_as_float(x1[8 * ch + 3]));
            x.z = pack_bf16(__uint_as_float(x1[8 * ch + 4]), __uint_as_float(x1[8 * ch + 5]));
            x.w = pack_bf16(__uint_as_float(x1[8 * ch + 6]), __uint_as_float(x1[8 * ch + 7]));
            *reinterpret_cast<uint4*>(b_pg + sw128(row, (2 * cq + ch) * 16)) = x;
          }
        }
      }
      // column sums of T and T3 (every column of the small accumulators holds the same sum)
      if (cq == 0) {
        uint32_t c12[16], c3[16];
        tmem_ld16(tmem_addr(tm, lane_base, kBcColX), c12);
        tmem_ld16(tmem_addr(tm, lane_base, kBcColX + 16), c3);
        tmem_wait_ld();
        if (active) {
          atomicAdd(&s.dg_s[row], -__uint_as_float(c12[0]));
          atomicAdd(&s.db_s[row], __uint_as_float(c3[0]));
        }
      }
      // dq
      __nv_bfloat16* dst = p.dq + (static_cast<size_t>(cp.tok0 + row) * p.Hout + ho) * kDim + 64 * hf;
      {
        tmem_ld32(tmem_addr(tm, lane_base, kBcColQ + 64 * hf + 32 * pc), r);
        tmem_wait_ld();
        if (active && (row < len || whole)) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 x;
            x.x = pack_bf16(__uint_as_float(r[8 * ch]), __uint_as_float(r[8 * ch + 1]));
            x.y = pack_bf16(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
            x.z = pack_bf16(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
            x.w = pack_bf16(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
            // whole chunk: into the Q tile (dead since this round's products completed), stored by TMA below
            if (whole) *reinterpret_cast<uint4*>(b_qt + hf * 8192 + sw128(row, (4 * pc + ch) * 16)) = x;
            else row_out(dst + 32 * pc + 8 * ch, x, accum);
          }
        }
      }
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();
    if (whole && tid == kStoreTid) {
      if (accum) {  // the group's earlier tiles (stored or added by this thread) are complete in global memory
        tma_store_wait_all<0>();
        tma_reduce_add_3d(&map_dq, b_qt, 0, ho, cp.tok0);
        tma_reduce_add_3d(&map_dq, b_qt + 8192, 64, ho, cp.tok0);
      } else {
        tma_store_3d(&map_dq, b_qt, 0, ho, cp.tok0);
        tma_store_3d(&map_dq, b_qt + 8192, 64, ho, cp.tok0);
      }
      tma_store_commit();
    }

    // ================================================================== round 5
    if (warp < 4 && elect_one()) {  // the products of a round are issued by one elected lane of each of four warps
      tc_fence_after();
      if (warp == 0) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm + kBcColU + 64, desc_add(umma_desc_sw128(spg, 16, 1024), kk * 32), desc_add(umma_desc_sw128(sat, 16, 1024), kk * 32),
                  id64_64_kk, kk > 0);
      } else if (warp == 1) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tm + kBcColQK, desc_add(umma_desc_sw128(skt, 16, 1024), off64(kk)), desc_add(umma_desc_sw128(skt, 16, 1024), off64(kk)),
                  id64_64_kk, kk > 0);
      }
      umma_commit(&s.bar_mma);
      // T was last read in round four: the next unit's P_g goes there
      if (warp == 3 && has_next) load_b(nchunk, nh, 1, b_vp, b_dvg, b_dvp, b_t12);
    }
    __syncwarp();
    mbar_wait(wc, &s.bar_mma, mma_phase, 6);
    mma_phase ^= 1;
    tc_fence_after();
    {
      uint32_t x2[16], kk2[16];
      tmem_ld16(tmem_addr(tm, lane_base, kBcColU + 64 + 16 * cq), x2);
      tmem_ld16(tmem_addr(tm, lane_base, kBcColQK + 16 * cq), kk2);
      tmem_wait_ld();
      // as in round 3, lane + 16 takes over columns 8-15 of the row held by lane
      const int up = lane >> 4;
      const int row2 = 16 * q4 + (lane & 15);
      const float beta_r2 = s.beta[row2];
      float dbr = 0.f;
      // Only the lower triangle T5 = beta_row o dL is stored (8 columns per lane, row-contiguous); round 6 applies
      // it and its transpose, which together are dAs = T5 + T5^T.
      uint32_t tw[4];
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        float o2[2];
#pragma unroll
        for (int z = 0; z < 2; ++z) {
          const uint32_t hx = __shfl_sync(0xffffffffu, x2[8 + i + z], lane & 15);
          const uint32_t hk = __shfl_sync(0xffffffffu, kk2[8 + i + z], lane & 15);
          const float xv = __uint_as_float(up ? hx : x2[i + z]);
          const float kv = __uint_as_float(up ? hk : kk2[i + z]);
          const int j = 16 * cq + 8 * up + i + z;
          const float dL = (j < row2) ? -xv : 0.f;
          dbr += dL * kv;
          o2[z] = beta_r2 * dL;
        }
        tw[i >> 1] = pack_bf16(o2[0], o2[1]);
      }
      *reinterpret_cast<uint4*>(b_ag + sw128(row2, (2 * cq + up) * 16)) = make_uint4(tw[0], tw[1], tw[2], tw[3]);
      dbr += __shfl_xor_sync(0xffffffffu, dbr, 16);
      if (active) atomicAdd(&s.db_s[row], dbr);
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();

    // ================================================================== round 6
    if (warp < 4 && elect_one()) {  // the products of a round are issued by one elected lane of each of four warps
      tc_fence_after();
      if (warp == 0) {
        // both groups add to the same accumulator: one thread issues them, so that the order of the fp32 additions
        // (and with it every bit of dk) is the same from run to run
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // accK += T5 K
          umma_ss(tm + kBcColK, desc_add(umma_desc_sw128(sag, 16, 1024), kk * 32), desc_add(umma_desc_sw128(skt, 8192, 1024), kk * 2048),
                  id64_128_kmn, 1);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // accK += T5^T K
          umma_ss(tm + kBcColK, desc_add(umma_desc_sw128(sag, 8192, 1024), kk * 2048), desc_add(umma_desc_sw128(skt, 8192, 1024), kk * 2048),
                  id64_128_mnmn, 1);
      }
      umma_commit(&s.bar_mma);
    }
    __syncwarp();
    mbar_wait(wc, &s.bar_mma, mma_phase, 7);
    mma_phase ^= 1;
    tc_fence_after();
    {
      __nv_bfloat16* dst = p.dk + (static_cast<size_t>(cp.tok0 + row) * p.Hout + ho) * kDim + 64 * hf;
      {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tm, lane_base, kBcColK + 64 * hf + 32 * pc), r);
        tmem_wait_ld();
        if (active && (row < len || whole)) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 x;
            x.x = pack_bf16(__uint_as_float(r[8 * ch]), __uint_as_float(r[8 * ch + 1]));
            x.y = pack_bf16(__uint_as_float(r[8 * ch + 2]), __uint_as_float(r[8 * ch + 3]));
            x.z = pack_bf16(__uint_as_float(r[8 * ch + 4]), __uint_as_float(r[8 * ch + 5]));
            x.w = pack_bf16(__uint_as_float(r[8 * ch + 6]), __uint_as_float(r[8 * ch + 7]));
            // whole chunk: into the K tile (dead since this round's products completed), stored by TMA below
            if (whole) *reinterpret_cast<uint4*>(b_kt + hf * 8192 + sw128(row, (4 * pc + ch) * 16)) = x;
            else row_out(dst + 32 * pc + 8 * ch, x, accum);
          }
        }
      }
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();
    if (whole && tid == kStoreTid) {
      if (accum) {  // (the wait before this unit's dq tile covered the group's earlier dk tiles as well)
        tma_reduce_add_3d(&map_dk, b_kt, 0, ho, cp.tok0);
        tma_reduce_add_3d(&map_dk, b_kt + 8192, 64, ho, cp.tok0);
      } else {
        tma_store_3d(&map_dk, b_kt, 0, ho, cp.tok0);
        tma_store_3d(&map_dk, b_kt + 8192, 64, ho, cp.tok0);
      }
      tma_store_commit();
    }
    if (tid < kChunk) {
      // the padded rows of a tail chunk share the gate of the last valid token
      float dgv = s.dg_s[tid];
      if (tid == len - 1) {
        for (int t2 = len; t2 < kChunk; ++t2) dgv += s.dg_s[t2];
        dgv += s.dgl_s;
      }
      if (tid < len) {
        const size_t o = static_cast<size_t>(cp.tok0 + tid) * p.H + h;
        p.dg[o] = dgv;
        p.db[o] = s.db_s[tid];
      }
    }
    {  // the paired buffers swap roles
      unsigned char* t;
      t = b_kt; b_kt = b_vp; b_vp = t;
      t = b_qt; b_qt = b_dvg; b_dvg = t;
      t = b_at; b_at = b_dvp; b_dvp = t;
      t = b_pg; b_pg = b_t12; b_t12 = t;
    }
    oc = noc; oh = noh; j = nj;
    chunk = nchunk;
    h = nh;
  }

  if (tid == kStoreTid) tma_store_wait_all<0>();
  tc_fence_before();
  __syncthreads();
  if (s.abort_flag) {  // a wait expired somewhere in the CTA (the same value for every thread: all loops are done)
    drain_after_abort(warp < 4 && elect_one(), &s.drain_bar);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tm, 512);
}

// Sum of the G V-heads of every QK head: in [rows, H, 128] bf16 -> out [rows, Hg, 128] bf16 (fp32 accumulate).
// One launch serves up to two tensors (dq and dk of the backward): blockIdx.y picks the pair.
__global__ void __launch_bounds__(256) group_reduce_kernel(const __nv_bfloat16* __restrict__ in0,
                                                          __nv_bfloat16* __restrict__ out0,
                                                          const __nv_bfloat16* __restrict__ in1,
                                                          __nv_bfloat16* __restrict__ out1, long long rows, int H, int Hg) {
  const __nv_bfloat16* __restrict__ in = blockIdx.y ? in1 : in0;
  __nv_bfloat16* __restrict__ out = blockIdx.y ? out1 : out0;
  const int G = H / Hg;
  const long long total = rows * Hg * (kDim / 8);
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int piece = static_cast<int>(idx % (kDim / 8));
    const long long rh = idx / (kDim / 8);
    const int hg = static_cast<int>(rh % Hg);
    const long long r = rh / Hg;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int i = 0; i < G; ++i) {
      const uint4 x = __ldg(reinterpret_cast<const uint4*>(in + ((r * H + hg * G + i) * kDim)) + piece);
      const uint32_t* xw = reinterpret_cast<const uint32_t*>(&x);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += bf16_lo(xw[e]);
        acc[2 * e + 1] += bf16_hi(xw[e]);
      }
    }
    uint4 y;
    y.x = pack_bf16(acc[0], acc[1]);
    y.y = pack_bf16(acc[2], acc[3]);
    y.z = pack_bf16(acc[4], acc[5]);
    y.w = pack_bf16(acc[6], acc[7]);
    *(reinterpret_cast<uint4*>(out + (r * Hg + hg) * kDim) + piece) = y;
  }
}

// Launch of group_reduce_kernel for one tensor (in1 == nullptr) or two; 16 CTAs of 256 threads per SM at most.
static int launch_group_reduce(const void* in0, void* out0, const void* in1, void* out1, long long rows, int H, int Hg,
                               cudaStream_t st) {
  const long long total = rows * Hg * (kDim / 8);
  const long long blocks = (total + 255) / 256;
  const long long cap = 16LL * sm_count();
  dim3 grid(static_cast<unsigned>(blocks < cap ? blocks : cap), in1 ? 2 : 1);
  group_reduce_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in0), static_cast<__nv_bfloat16*>(out0),
                                            static_cast<const __nv_bfloat16*>(in1), static_cast<__nv_bfloat16*>(out1), rows,
                                            H, Hg);
  return cudaGetLastError() == cudaSuccess ? FQ_OK : FQ_ERR_CUDA;
}

}  // namespace fq

static int bwd_chunk_launch(const void* q, const void* k, const void* v, const void* A, const void* Ag, const void* Pg,
                            const void* dout, const void* h, const void* dh, const float* g_cumsum, const float* beta,
                            void* dq, void* dk, void* dv, float* dg, float* db, int B, int T, int H, int Hg,
                            const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq, int total_chunks,
                            float scale, int32_t* status_dev, void* stream, bool grouped) {
  using namespace fq;
  const int Hout = grouped ? Hg : H;
  FQ_CHECK_ARG(q && k && v && A && Ag && Pg && dout && dv && h && dh && g_cumsum && beta && dq && dk && dg && db,
               "fq_gdr_bwd_chunk: null tensor");
  FQ_CHECK_ARG(B > 0 && T >= 0 && H > 0 && Hg > 0 && H % Hg == 0 && n_seq > 0 && total_chunks >= 0,
               "fq_gdr_bwd_chunk: bad sizes");
  FQ_CHECK_ARG((cu_seqlens == nullptr) == (chunk_offsets == nullptr),
               "fq_gdr_bwd_chunk: cu_seqlens and chunk_offsets must be given together");
  FQ_CHECK_ARG(cu_seqlens == nullptr || B == 1, "fq_gdr_bwd_chunk: packed batches need B == 1");
  FQ_CHECK_ARG(cu_seqlens != nullptr || n_seq == B, "fq_gdr_bwd_chunk: dense batches need n_seq == B");
  if (total_chunks == 0) return FQ_OK;
  const uint64_t rows = static_cast<uint64_t>(B) * static_cast<uint64_t>(T);
  const uint64_t hrows = static_cast<uint64_t>(total_chunks) * H * kDim;
  FQ_CHECK_ARG(rows > 0 && rows < (1ull << 31) && hrows < (1ull << 31), "fq_gdr_bwd_chunk: sizes out of range");
  CUtensorMap mq, mk, mv, mdo, ma, mag, mpg, mh, mdh, mdq, mdk, mdv;
  int rc;
  if ((rc = make_tmap_rows_heads_dim(&mq, q, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mk, k, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mv, v, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdo, dout, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&ma, A, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mag, Ag, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mpg, Pg, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mh, h, hrows, 1, kDim, kDim, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdh, dh, hrows, 1, kDim, kDim, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdq, dq, rows, Hout, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdk, dk, rows, Hout, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdv, dv, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  BwdChunkParams p;
  p.g_cum = g_cumsum; p.beta = beta;
  p.dq = static_cast<__nv_bfloat16*>(dq); p.dk = static_cast<__nv_bfloat16*>(dk); p.dg = dg; p.db = db;
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.H = H; p.Hg = Hg; p.Hout = Hout; p.total_chunks = total_chunks; p.scale = scale;
  p.sa = SeqArgs{T, cu_seqlens, chunk_offsets, n_seq, (T + kChunk - 1) / kChunk};
  p.status_dev = status_dev;
  const size_t smem = sizeof(BwdChunkSmem) + 1024;
  {
    static std::atomic<unsigned long long> done0{0};
    const int rc_attr = set_smem_limit_once(reinterpret_cast<const void*>(gdr_bwd_chunk_kernel), static_cast<int>(smem), &done0);
    if (rc_attr != FQ_OK) return rc_attr;
  }
  const long long units = static_cast<long long>(total_chunks) * Hout;  // strides of the unit walk (see the kernel)
  const int grid = static_cast<int>(units < sm_count() ? units : sm_count());
  gdr_bwd_chunk_kernel<<<grid, kBcThreads, smem, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, mdo, ma, mag, mpg, mh,
                                                                                      mdh, mdq, mdk, mdv, p);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_gdr_bwd_chunk(const void* q, const void* k, const void* v, const void* A, const void* Ag,
                                       const void* Pg, const void* dout, const void* h, const void* dh,
                                       const float* g_cumsum, const float* beta, void* dq, void* dk, void* dv, float* dg,
                                       float* db,
                                       int B, int T, int H, int Hg, const int32_t* cu_seqlens,
                                       const int32_t* chunk_offsets, int n_seq, int total_chunks, float scale,
                                       int32_t* status_dev, void* stream) {
  return bwd_chunk_launch(q, k, v, A, Ag, Pg, dout, h, dh, g_cumsum, beta, dq, dk, dv, dg, db, B, T, H, Hg, cu_seqlens,
                          chunk_offsets, n_seq, total_chunks, scale, status_dev, stream, false);
}

extern "C" FQ_API int fq_gdr_bwd_chunk_grouped(const void* q, const void* k, const void* v, const void* A, const void* Ag,
                                               const void* Pg, const void* dout, const void* h, const void* dh,
                                               const float* g_cumsum, const float* beta, void* dq, void* dk, void* dv,
                                               float* dg, float* db, int B, int T, int H, int Hg,
                                               const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                                               int total_chunks, float scale, int32_t* status_dev, void* stream) {
  return bwd_chunk_launch(q, k, v, A, Ag, Pg, dout, h, dh, g_cumsum, beta, dq, dk, dv, dg, db, B, T, H, Hg, cu_seqlens,
                          chunk_offsets, n_seq, total_chunks, scale, status_dev, stream, true);
}

extern "C" FQ_API int fq_group_reduce(const void* in, void* out, long long rows, int H, int Hg, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(in && out && rows >= 0 && H > 0 && Hg > 0 && H % Hg == 0, "fq_group_reduce: bad arguments");
  if (rows == 0) return FQ_OK;
  if (launch_group_reduce(in, out, nullptr, nullptr, rows, H, Hg, static_cast<cudaStream_t>(stream)) != FQ_OK) {
    set_error("fq_group_reduce: launch failed");
    return FQ_ERR_CUDA;
  }
  return FQ_OK;
}

extern "C" FQ_API int fq_group_reduce_pair(const void* in_a, void* out_a, const void* in_b, void* out_b, long long rows,
                                           int H, int Hg, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(in_a && out_a && in_b && out_b && rows >= 0 && H > 0 && Hg > 0 && H % Hg == 0,
               "fq_group_reduce_pair: bad arguments");
  if (rows == 0) return FQ_OK;
  if (launch_group_reduce(in_a, out_a, in_b, out_b, rows, H, Hg, static_cast<cudaStream_t>(stream)) != FQ_OK) {
    set_error("fq_group_reduce_pair: launch failed");
    return FQ_ERR_CUDA;
  }
  return FQ_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the chunk-parallel backward for grouped heads (Hg < H).
//
// The regular path needs two [rows, H, 128] bf16 buffers for the per-V-head dq / dk that
// fq_group_reduce then sums; the caller allocates them.  Some callers cannot allocate device
// memory at the point where they run the backward: code that executes inside a region where the
// framework's allocator is frozen (a memory-planned inference/training step whose buffers were all
// assigned ahead of time), or a host without a caching allocator that would have to pay a
// cudaMalloc (which synchronises the device) on every call.  For them the two buffers live in a
// fixed array that is part of the library image.
namespace fq {
constexpr size_t kNoAllocScratchBytes = 32ull << 20;  // 2 buffers of rows*H*128 bf16  ->  rows*H <= 65536
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
}  // namespace fq

extern "C" FQ_API int fq_gdr_bwd_chunk_gva_noalloc(const void* q, const void* k, const void* v, const void* A,
                                                   const void* Ag, const void* Pg, const void* dout, const void* h,
                                                   const void* dh, const float* g_cumsum, const float* beta, void* dq,
                                                   void* dk, void* dv, float* dg, float* db, int B, int T, int H, int Hg,
                                                   const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n_seq,
                                                   int total_chunks, float scale, int32_t* status_dev, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(q && k && v && A && Ag && Pg && dout && dv && h && dh && g_cumsum && beta && dq && dk && dg && db,
               "fq_gdr_bwd_chunk_gva_noalloc: null tensor");
  FQ_CHECK_ARG(B > 0 && T >= 0 && H > 0 && Hg > 0 && H % Hg == 0 && n_seq > 0 && total_chunks >= 0,
               "fq_gdr_bwd_chunk_gva_noalloc: bad sizes");
  FQ_CHECK_ARG((cu_seqlens == nullptr) == (chunk_offsets == nullptr),
               "fq_gdr_bwd_chunk_gva_noalloc: cu_seqlens and chunk_offsets must be given together");
  FQ_CHECK_ARG(cu_seqlens == nullptr || B == 1, "fq_gdr_bwd_chunk_gva_noalloc: packed batches need B == 1");
  FQ_CHECK_ARG(cu_seqlens != nullptr || n_seq == B, "fq_gdr_bwd_chunk_gva_noalloc: dense batches need n_seq == B");
  const uint64_t rows = static_cast<uint64_t>(B) * static_cast<uint64_t>(T);
  const uint64_t per_buffer = rows * static_cast<uint64_t>(H) * kDim * 2;
  if (2 * per_buffer > kNoAllocScratchBytes) {
    set_error("fq_gdr_bwd_chunk_gva_noalloc: B*T*H = %llu exceeds the built-in scratch (limit B*T*H <= %llu); "
              "use fq_gdr_bwd_chunk + fq_group_reduce with caller-provided buffers",
              (unsigned long long)(rows * H), (unsigned long long)(kNoAllocScratchBytes / (4 * kDim)));
    return FQ_ERR_WORKSPACE;
  }
  if (total_chunks == 0) return FQ_OK;
  const uint64_t hrows = static_cast<uint64_t>(total_chunks) * H * kDim;
  FQ_CHECK_ARG(rows > 0 && rows < (1ull << 31) && hrows < (1ull << 31), "fq_gdr_bwd_chunk_gva_noalloc: sizes out of range");

  // One-time set-up per device, with that device current: resolve the device address of the scratch
  // array (its name is only a host-side handle) and raise the kernel's shared-memory limit.  The
  // cache is filled under a mutex, so first calls from several host threads are safe.
  static unsigned char* scratch_dev[64] = {nullptr};
  static std::mutex setup_mutex;
  int dev = 0;
  FQ_CHECK_CUDA(cudaGetDevice(&dev));
  FQ_CHECK_ARG(dev >= 0 && dev < 64, "fq_gdr_bwd_chunk_gva_noalloc: device index out of range");
  const size_t smem = sizeof(BwdChunkSmem) + 1024;
  {
    std::lock_guard<std::mutex> lock(setup_mutex);
    if (scratch_dev[dev] == nullptr) {
      void* ptr = nullptr;
      FQ_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
      FQ_CHECK_CUDA(cudaFuncSetAttribute(gdr_bwd_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      scratch_dev[dev] = static_cast<unsigned char*>(ptr);
    }
  }
  __nv_bfloat16* dq_h = reinterpret_cast<__nv_bfloat16*>(scratch_dev[dev]);
  __nv_bfloat16* dk_h = reinterpret_cast<__nv_bfloat16*>(scratch_dev[dev] + per_buffer);

  CUtensorMap mq, mk, mv, mdo, ma, mag, mpg, mh, mdh, mdq, mdk, mdv;
  int rc;
  if ((rc = make_tmap_rows_heads_dim(&mq, q, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mk, k, rows, Hg, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mv, v, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdo, dout, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&ma, A, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mag, Ag, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mpg, Pg, rows, H, kChunk, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mh, h, hrows, 1, kDim, kDim, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdh, dh, hrows, 1, kDim, kDim, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdq, dq_h, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdk, dk_h, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mdv, dv, rows, H, kDim, kChunk, 64)) != FQ_OK) return rc;
  BwdChunkParams p;
  p.g_cum = g_cumsum; p.beta = beta;
  p.dq = dq_h; p.dk = dk_h; p.dg = dg; p.db = db;
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.H = H; p.Hg = Hg; p.Hout = H; p.total_chunks = total_chunks; p.scale = scale;
  p.sa = SeqArgs{T, cu_seqlens, chunk_offsets, n_seq, (T + kChunk - 1) / kChunk};
  p.status_dev = status_dev;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long units = static_cast<long long>(total_chunks) * H;
  const int grid = static_cast<int>(units < sm_count() ? units : sm_count());
  gdr_bwd_chunk_kernel<<<grid, kBcThreads, smem, st>>>(mq, mk, mv, mdo, ma, mag, mpg, mh, mdh, mdq, mdk, mdv, p);
  FQ_CHECK_CUDA(cudaGetLastError());
  // Every token row of both scratch buffers was just written (each row belongs to exactly one
  // chunk), so nothing has to be cleared before the sum reads them.
  if (launch_group_reduce(dq_h, dq, dk_h, dk, static_cast<long long>(rows), H, Hg, st) != FQ_OK) {
    set_error("fq_gdr_bwd_chunk_gva_noalloc: head-sum launch failed");
    return FQ_ERR_CUDA;
  }
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

