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

// One warp per (piece, head): lane l looks at the (32 i + l)-th chunk away from the piece, the running log-decay is an
// inclusive warp scan, and the first chunk at which it drops below the threshold ends the replay.  `w_cap` bounds
// the walk (0 = no bound): a replay that would be longer is reported as w_cap + 1 chunks without looking further,
// which is all that the transition-matrix fallback needs to know.
// The walk of one warp: returns (in every lane) the code of the replay - w chunks, or avail | bit 30 when the end of
// the sequence is reached first, or limit = w_cap + 1 when the walk gave up at the cap.
__device__ __forceinline__ int scan_replay(const float* __restrict__ g_cum, long long edge, int avail, int last_len,
                                           bool reverse, int H, int h, float threshold, int w_cap, int lane) {
  // forward: chunks before the piece, walking backwards from its first token `edge`; reverse (state gradient): chunks
  // after the piece, walking forwards from the first token after it (`edge`), `last_len` = tokens in the sequence's
  // last chunk
  const int limit = (w_cap > 0 && w_cap + 1 < avail) ? w_cap + 1 : avail;
  float carry = 0.f;
  int w = -1;
  for (int base = 0; base < limit && w < 0; base += 32) {
    const int c = base + lane;
    float x = 0.f;
    if (c < limit) {
      long long tok;
      if (!reverse) tok = edge - static_cast<long long>(c) * kChunk - 1;
      else tok = edge + static_cast<long long>(c) * kChunk + ((c == avail - 1) ? last_len : kChunk) - 1;
      x = __ldg(g_cum + tok * H + h);
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    x += carry;
    const unsigned hit = __ballot_sync(0xffffffffu, c < limit && x < threshold);
    if (hit) w = base + __ffs(hit);  // chunks replayed = index of the first hit + 1
    carry = __shfl_sync(0xffffffffu, x, 31);
  }
  if (w > 0) return w;                           // decayed after w chunks
  if (limit == avail) return avail | (1 << 30);  // reached the end of the sequence: exact
  return limit;                                  // gave up at the cap
}

__global__ void __launch_bounds__(128) cp_warmup_kernel(const float* __restrict__ g_cum,
                                                       const int* __restrict__ piece_start,
                                                       const int* __restrict__ piece_first_chunk,
                                                       int* __restrict__ warmup, int n_pieces, int H, float threshold,
                                                       int reverse, const int* __restrict__ piece_chunks_after,
                                                       int w_cap, const int* __restrict__ piece_seq,
                                                       int* __restrict__ flags) {
  const int idx = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (idx >= n_pieces * H) return;
  const int piece = idx / H, h = idx - piece * H;
  const int avail = reverse ? __ldg(piece_chunks_after + piece) : __ldg(piece_first_chunk + piece);
  const int last_len = reverse ? __ldg(piece_first_chunk + piece) : kChunk;
  const int code = scan_replay(g_cum, __ldg(piece_start + piece), avail, last_len, reverse != 0, H, h, threshold, w_cap, lane);
  if (lane == 0) {
    warmup[idx] = code;
    // a replay of more than w_cap chunks: the (sequence, head) pair takes the transition-matrix route (see below)
    if (flags != nullptr && (code & 0xFFFFFF) > w_cap) atomicOr(flags + __ldg(piece_seq + piece) * H + h, 1);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Transition-matrix fallback.  A replay of more than `w_cap` chunks costs more than it saves (a head whose gate
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

// Codes of the reverse direction (state gradient) for the pairs flagged by the forward plan: every piece but the last
// of its sequence starts from the corrected gradient e_r (bit 29); the gradient pass runs every piece but the first from
// zero (the last one from dht, bit 30) with no replay, its left-edge gradient is C_r.
__global__ void __launch_bounds__(128) cp_resolve_reverse_kernel(const int* __restrict__ warmup_in,
                                                                const int* __restrict__ piece_seq,
                                                                const int* __restrict__ chunks_before,
                                                                const int* __restrict__ chunks_after,
                                                                const int* __restrict__ flags,
                                                                int* __restrict__ warmup_out, int* __restrict__ pass1,
                                                                int n_pieces, int H) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_pieces * H) return;
  const int piece = idx / H, h = idx - piece * H;
  const bool flagged = __ldg(flags + __ldg(piece_seq + piece) * H + h) != 0;
  const bool first = __ldg(chunks_before + piece) == 0, last = __ldg(chunks_after + piece) == 0;
  warmup_out[idx] = (flagged && !last) ? (1 << 29) : __ldg(warmup_in + idx);
  pass1[idx] = (flagged && !first) ? (last ? (1 << 30) : 0) : (1 << 27);
}

// Gate scans (both directions if codes_rev is given), flag and codes of one (sequence, head) in ONE launch: a CTA per
// pair, a warp per piece for the scans, then - the flag being known inside the CTA - a thread per piece for the codes.
// Same results as fq_cp_warmup (+ reverse) followed by fq_cp_transition_plan(_reverse).
__global__ void __launch_bounds__(256) cp_plan_kernel(const float* __restrict__ g_cum, const int* __restrict__ piece_start,
                                                     const int* __restrict__ piece_end,
                                                     const int* __restrict__ chunks_before,
                                                     const int* __restrict__ chunks_after,
                                                     const int* __restrict__ last_chunk_len,
                                                     const int* __restrict__ seq_piece_offsets, int* __restrict__ flags,
                                                     int* __restrict__ codes, int* __restrict__ pass1,
                                                     int* __restrict__ codes_rev, int* __restrict__ pass1_rev,
                                                     int n_pieces, int H, float threshold, int w_cap) {
  __shared__ int any_far;
  const int seq = blockIdx.x / H, h = blockIdx.x - seq * H;
  const int p0 = __ldg(seq_piece_offsets + seq), p1 = __ldg(seq_piece_offsets + seq + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) any_far = 0;
  __syncthreads();
  for (int piece = p0 + warp; piece < p1; piece += 8) {
    const int cf = scan_replay(g_cum, __ldg(piece_start + piece), __ldg(chunks_before + piece), kChunk, false, H, h,
                               threshold, w_cap, lane);
    int cr = 0;
    if (codes_rev != nullptr)
      cr = scan_replay(g_cum, __ldg(piece_end + piece), __ldg(chunks_after + piece), __ldg(last_chunk_len + piece), true, H,
                       h, threshold, w_cap, lane);
    if (lane == 0) {
      codes[piece * H + h] = cf;
      if (codes_rev != nullptr) codes_rev[piece * H + h] = cr;
      if ((cf & 0xFFFFFF) > w_cap || (cr & 0xFFFFFF) > w_cap) atomicOr(&any_far, 1);
    }
  }
  __syncthreads();  // also makes this CTA's own global writes above visible to its threads below
  const bool flagged = any_far != 0;
  if (threadIdx.x == 0) flags[seq * H + h] = flagged ? 1 : 0;
  constexpr int kSkip = 1 << 27;
  for (int piece = p0 + threadIdx.x; piece < p1; piece += 256) {
    const int idx = piece * H + h;
    const bool first = __ldg(chunks_before + piece) == 0, last = __ldg(chunks_after + piece) == 0;
    if (flagged && !first) codes[idx] = 1 << 29;
    pass1[idx] = (flagged && !last) ? (first ? (1 << 30) : 0) : kSkip;               // B_r
    pass1[n_pieces * H + idx] = (flagged && !last && !first) ? (1 << 28) : kSkip;    // T_r
    if (codes_rev != nullptr) {
      if (flagged && !last) codes_rev[idx] = 1 << 29;
      pass1_rev[idx] = (flagged && !first) ? (last ? (1 << 30) : 0) : kSkip;
    }
  }
}

__device__ __forceinline__ void mma_tf32_1688(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// x = hi + lo with both parts representable in TF32 (the split that makes three TF32 products as good as fp32)
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
  const float r = x - __uint_as_float(hi);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(r));
}

// h0_{r+1} = T_r h0_r + B_r for the pieces of one flagged (sequence, head); a CTA (8 warps) owns kChainCols of the 128
// state columns, warp w the rows 16 w .. 16 w + 15.  The 128 x 128 x kChainCols product of a step runs on the warp-level
// tensor path with split TF32 operands (hi*hi + lo*hi + hi*lo: fp32-grade); the step's T_r fragments come straight
// from global memory (they were written by the state pass just before and sit in L2), the state slice goes through
// shared memory.  bt: [2 * n_pieces, H, 128, 128] fp32 (B_r in slot r, T_r in slot n_pieces + r);
// h0_piece: [n_pieces, H, 128, 128].
constexpr int kChainCols = 16;
constexpr int kChainLd = kChainCols + 8;  // row stride of the state slice: conflict-free B fragments

// kReverse: the chain of the state gradient, e_{r-1} = T_r^T e_r + C_r from the last piece down (add = C, out = e).
template <bool kReverse>
__global__ void __launch_bounds__(256) cp_chain_kernel(const float* __restrict__ add, const float* __restrict__ tmat,
                                                      float* __restrict__ out, const int* __restrict__ flags,
                                                      const int* __restrict__ seq_piece_offsets, int H, int compose,
                                                      const float* __restrict__ init) {
  __shared__ float sx[kDim * kChainLd];
  const int seq = blockIdx.x / H, h = blockIdx.x - seq * H, c0 = blockIdx.y * kChainCols;
  if (__ldg(flags + seq * H + h) == 0) return;
  const int p0 = __ldg(seq_piece_offsets + seq), p1 = __ldg(seq_piece_offsets + seq + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int m0 = warp * 16;
  const size_t mat = static_cast<size_t>(kDim) * kDim;
  const int steps = p1 - p0 - 1;
  if (init != nullptr) {
    // the chain starts from a given state (gradient) of this head instead of from B (C) of its first piece: every
    // step, the first included, applies its transition matrix
    const float* src = init + static_cast<size_t>(h) * mat;
    for (int i = threadIdx.x; i < kDim * kChainCols; i += 256) {
      const int row = i / kChainCols, col = i - row * kChainCols;
      sx[row * kChainLd + col] = __ldg(src + static_cast<size_t>(row) * kDim + c0 + col);
    }
    __syncthreads();
  }
  for (int st = 0; st < steps; ++st) {
    const int r = kReverse ? p1 - 1 - st : p0 + st;  // piece whose (T, add) pair this step applies
    // accumulators start from B_r (C_r): rows m0+g and m0+g+8, column pairs c0 + 8 n + 2 t.  compose: the chain of
    // the transition matrices alone, X_1 = T_first, X_{r+1} = T_r X_r (the first step starts from T, later ones from 0)
    const float* B = (compose ? tmat : add) + (static_cast<size_t>(r) * H + h) * mat;
    const bool have_b = !compose || st == 0;
    float acc[kChainCols / 8][4];
#pragma unroll
    for (int n = 0; n < kChainCols / 8; ++n) {
      float2 lo = make_float2(0.f, 0.f), hi = lo;
      if (have_b) {
        lo = __ldg(reinterpret_cast<const float2*>(B + static_cast<size_t>(m0 + g) * kDim + c0 + 8 * n + 2 * t));
        hi = __ldg(reinterpret_cast<const float2*>(B + static_cast<size_t>(m0 + g + 8) * kDim + c0 + 8 * n + 2 * t));
      }
      acc[n][0] = lo.x; acc[n][1] = lo.y; acc[n][2] = hi.x; acc[n][3] = hi.y;
    }
    float acc1[kChainCols / 8][4], acc2[kChainCols / 8][4];
#pragma unroll
    for (int n = 0; n < kChainCols / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc1[n][e] = acc2[n][e] = 0.f;
    if (st > 0 || init != nullptr) {
      const float* Tm = tmat + (static_cast<size_t>(r) * H + h) * mat;
      float ta[16][4];  // the A fragments of all sixteen k-steps: one round trip to L2 per step of the chain
#pragma unroll
      for (int ks = 0; ks < 16; ++ks) {
        const int k0 = 8 * ks;
        if (!kReverse) {
          ta[ks][0] = __ldg(Tm + static_cast<size_t>(m0 + g) * kDim + k0 + t);
          ta[ks][1] = __ldg(Tm + static_cast<size_t>(m0 + g + 8) * kDim + k0 + t);
          ta[ks][2] = __ldg(Tm + static_cast<size_t>(m0 + g) * kDim + k0 + t + 4);
          ta[ks][3] = __ldg(Tm + static_cast<size_t>(m0 + g + 8) * kDim + k0 + t + 4);
        } else {  // A = T^T
          ta[ks][0] = __ldg(Tm + static_cast<size_t>(k0 + t) * kDim + m0 + g);
          ta[ks][1] = __ldg(Tm + static_cast<size_t>(k0 + t) * kDim + m0 + g + 8);
          ta[ks][2] = __ldg(Tm + static_cast<size_t>(k0 + t + 4) * kDim + m0 + g);
          ta[ks][3] = __ldg(Tm + static_cast<size_t>(k0 + t + 4) * kDim + m0 + g + 8);
        }
      }
#pragma unroll
      for (int ks = 0; ks < 16; ++ks) {
        const int k0 = 8 * ks;
        uint32_t ah[4], al[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) split_tf32(ta[ks][e], ah[e], al[e]);
#pragma unroll
        for (int n = 0; n < kChainCols / 8; ++n) {
          uint32_t bh[2], bl[2];
          split_tf32(sx[(k0 + t) * kChainLd + 8 * n + g], bh[0], bl[0]);
          split_tf32(sx[(k0 + t + 4) * kChainLd + 8 * n + g], bh[1], bl[1]);
          mma_tf32_1688(acc1[n], al, bh);  // three independent accumulation chains per tile
          mma_tf32_1688(acc2[n], ah, bl);
          mma_tf32_1688(acc[n], ah, bh);
        }
      }
    }
#pragma unroll
    for (int n = 0; n < kChainCols / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[n][e] += acc1[n][e] + acc2[n][e];
    __syncthreads();  // every warp has read the old state slice
    float* dst = out + (static_cast<size_t>(kReverse ? r - 1 : r + 1) * H + h) * mat;
#pragma unroll
    for (int n = 0; n < kChainCols / 8; ++n) {
      const int col = 8 * n + 2 * t;
      *reinterpret_cast<float2*>(&sx[(m0 + g) * kChainLd + col]) = make_float2(acc[n][0], acc[n][1]);
      *reinterpret_cast<float2*>(&sx[(m0 + g + 8) * kChainLd + col]) = make_float2(acc[n][2], acc[n][3]);
      *reinterpret_cast<float2*>(dst + static_cast<size_t>(m0 + g) * kDim + c0 + col) = make_float2(acc[n][0], acc[n][1]);
      *reinterpret_cast<float2*>(dst + static_cast<size_t>(m0 + g + 8) * kDim + c0 + col) = make_float2(acc[n][2], acc[n][3]);
    }
    __syncthreads();
  }
}

}  // namespace fq

extern "C" FQ_API int fq_cp_warmup(const float* g_cumsum, const int32_t* piece_edge, const int32_t* piece_aux,
                                   const int32_t* piece_chunks_after, int32_t* warmup, int n_pieces, int H,
                                   float threshold, int reverse, int w_cap, const int32_t* piece_seq, int32_t* flags,
                                   void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(g_cumsum && piece_edge && piece_aux && warmup, "fq_cp_warmup: null tensor");
  FQ_CHECK_ARG(!reverse || piece_chunks_after, "fq_cp_warmup: the reverse scan needs piece_chunks_after");
  FQ_CHECK_ARG(n_pieces > 0 && H > 0 && threshold < 0.f, "fq_cp_warmup: bad arguments");
  FQ_CHECK_ARG(w_cap >= 0, "fq_cp_warmup: bad cap");
  FQ_CHECK_ARG(flags == nullptr || (piece_seq != nullptr && w_cap > 0), "fq_cp_warmup: flags need piece_seq and a cap");
  const long long total = static_cast<long long>(n_pieces) * H;  // one warp each, four warps per CTA
  cp_warmup_kernel<<<static_cast<unsigned>((total + 3) / 4), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      g_cumsum, piece_edge, piece_aux, warmup, n_pieces, H, threshold, reverse, piece_chunks_after, w_cap, piece_seq, flags);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_cp_transition_plan(const int32_t* warmup_in, const int32_t* piece_seq,
                                            const int32_t* chunks_before, const int32_t* chunks_after,
                                            const int32_t* flags, int32_t* warmup_out, int32_t* pass1_codes,
                                            int n_pieces, int H, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(warmup_in && piece_seq && chunks_before && chunks_after && flags && warmup_out && pass1_codes,
               "fq_cp_transition_plan: null tensor");
  FQ_CHECK_ARG(n_pieces > 0 && H > 0, "fq_cp_transition_plan: bad arguments");
  const int total = n_pieces * H;
  cp_resolve_kernel<<<(total + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      warmup_in, piece_seq, chunks_before, chunks_after, flags, warmup_out, pass1_codes, n_pieces, H);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_cp_chain(const float* bt, float* h0_piece, const int32_t* flags,
                                  const int32_t* seq_piece_offsets, int n_pieces, int n_seq, int H, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(bt && h0_piece && flags && seq_piece_offsets, "fq_cp_chain: null tensor");
  FQ_CHECK_ARG(n_pieces > 0 && n_seq > 0 && H > 0, "fq_cp_chain: bad arguments");
  dim3 grid(static_cast<unsigned>(n_seq) * H, kDim / kChainCols);
  const float* tmat = bt + static_cast<size_t>(n_pieces) * H * kDim * kDim;
  cp_chain_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(bt, tmat, h0_piece, flags, seq_piece_offsets, H, 0, nullptr);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_cp_transition_plan_reverse(const int32_t* warmup_in, const int32_t* piece_seq,
                                                    const int32_t* chunks_before, const int32_t* chunks_after,
                                                    const int32_t* flags, int32_t* warmup_out, int32_t* pass1_codes,
                                                    int n_pieces, int H, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(warmup_in && piece_seq && chunks_before && chunks_after && flags && warmup_out && pass1_codes,
               "fq_cp_transition_plan_reverse: null tensor");
  FQ_CHECK_ARG(n_pieces > 0 && H > 0, "fq_cp_transition_plan_reverse: bad arguments");
  const int total = n_pieces * H;
  cp_resolve_reverse_kernel<<<(total + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      warmup_in, piece_seq, chunks_before, chunks_after, flags, warmup_out, pass1_codes, n_pieces, H);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_cp_chain_reverse(const float* c, const float* tmat, float* dht_piece, const int32_t* flags,
                                          const int32_t* seq_piece_offsets, int n_pieces, int n_seq, int H,
                                          void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(c && tmat && dht_piece && flags && seq_piece_offsets, "fq_cp_chain_reverse: null tensor");
  FQ_CHECK_ARG(n_pieces > 0 && n_seq > 0 && H > 0, "fq_cp_chain_reverse: bad arguments");
  dim3 grid(static_cast<unsigned>(n_seq) * H, kDim / kChainCols);
  cp_chain_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(c, tmat, dht_piece, flags, seq_piece_offsets, H, 0, nullptr);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_cp_plan(const float* g_cumsum, const int32_t* piece_start, const int32_t* piece_end,
                                 const int32_t* chunks_before, const int32_t* chunks_after,
                                 const int32_t* last_chunk_len, const int32_t* seq_piece_offsets, int32_t* flags,
                                 int32_t* codes, int32_t* pass1_codes, int32_t* codes_rev, int32_t* pass1_rev,
                                 int n_pieces, int n_seq, int H, float threshold, int w_cap, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(g_cumsum && piece_start && piece_end && chunks_before && chunks_after && last_chunk_len &&
                   seq_piece_offsets && flags && codes && pass1_codes,
               "fq_cp_plan: null tensor");
  FQ_CHECK_ARG((codes_rev == nullptr) == (pass1_rev == nullptr), "fq_cp_plan: the reverse tables come together");
  FQ_CHECK_ARG(n_pieces > 0 && n_seq > 0 && H > 0 && threshold < 0.f && w_cap > 0, "fq_cp_plan: bad arguments");
  cp_plan_kernel<<<static_cast<unsigned>(n_seq) * H, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      g_cumsum, piece_start, piece_end, chunks_before, chunks_after, last_chunk_len, seq_piece_offsets, flags, codes,
      pass1_codes, codes_rev, pass1_rev, n_pieces, H, threshold, w_cap);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_cp_chain_ex(const float* add, const float* tmat, float* out, const int32_t* flags,
                                     const int32_t* seq_piece_offsets, const float* init, int n_seq, int H, int reverse,
                                     int compose, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(tmat && out && flags && seq_piece_offsets, "fq_cp_chain_ex: null tensor");
  FQ_CHECK_ARG(add != nullptr || compose, "fq_cp_chain_ex: the additive terms are missing");
  FQ_CHECK_ARG(!(compose && (reverse || init)), "fq_cp_chain_ex: compose goes with neither reverse nor init");
  FQ_CHECK_ARG(n_seq > 0 && H > 0, "fq_cp_chain_ex: bad arguments");
  dim3 grid(static_cast<unsigned>(n_seq) * H, kDim / kChainCols);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (reverse) cp_chain_kernel<true><<<grid, 256, 0, st>>>(add, tmat, out, flags, seq_piece_offsets, H, 0, init);
  else cp_chain_kernel<false><<<grid, 256, 0, st>>>(add, tmat, out, flags, seq_piece_offsets, H, compose, init);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}
