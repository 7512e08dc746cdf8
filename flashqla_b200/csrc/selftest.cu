// Self-test of the tensor-core plumbing used by the recurrence kernels: TMA tiles with 128-byte
// swizzle -> UMMA (tcgen05.mma) with shared-memory or tensor-memory operands -> TMEM -> registers.
// One CTA, one 128x128 problem; `mode` picks the operand forms:
//   0  D = A * B^T            A, B K-major tiles from TMA                (M=128, N=128, K=128)
//   1  D = A[:, :64] * B[:64] A K-major, B MN-major (rows of B = contraction index)  (K=64)
//   2  as 0, but A is written to shared memory by CUDA cores with the manual swizzle
//   3  D[:64] = A[:64] * B^T  M = 64 (rows live in lanes 0-15 of each 32-lane quarter)
//   4  as 0, but A is staged in tensor memory (bf16 pairs packed in 32-bit columns)
//   5  D = A[:64]^T * B[:, :64]^T   A MN-major (rows of A = contraction index)       (K=64)
//   6  D = A * B^T with N = 64 twice: columns 0-63 from B rows 0-63, 64-127 from rows 64-127
#include "flashqla.h"
#include "host.cuh"

namespace fq {

struct SelfTestSmem {
  unsigned char a[32768];  // two 128-row x 128-byte regions
  unsigned char b[32768];
  uint64_t bar_tma;
  uint64_t bar_mma;
  uint64_t drain_bar;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(128) selftest_kernel(const __grid_constant__ CUtensorMap map_a128,
                                                      const __grid_constant__ CUtensorMap map_a64,
                                                      const __grid_constant__ CUtensorMap map_b128,
                                                      const __grid_constant__ CUtensorMap map_b64,
                                                      const __nv_bfloat16* __restrict__ a_glob, float* __restrict__ d,
                                                      int mode, int* status_dev) {
  extern __shared__ unsigned char smem_dyn[];
  SelfTestSmem& s = *reinterpret_cast<SelfTestSmem*>(
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023)));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wc{&s.abort_flag, status_dev, 15, kWaitLimitCycles};
  constexpr uint32_t kCols = 256;

  if (tid == 0) {
    s.abort_flag = 0;
    mbar_init(&s.bar_tma, 1);
    mbar_init(&s.bar_mma, 1);
    mbar_init(&s.drain_bar, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&s.tmem_base, kCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;

  // ---- stage operands
  if (tid == 0) {
    const uint32_t a_bytes = (mode == 0 || mode == 3 || mode == 6) ? 32768u : (mode == 1 || mode == 5) ? 16384u : 0u;
    const uint32_t b_bytes = (mode == 1 || mode == 5) ? 16384u : 32768u;
    mbar_arrive_expect_tx(&s.bar_tma, a_bytes + b_bytes);
    if (mode == 0 || mode == 3 || mode == 6) {
      tma_load_3d(s.a, &map_a128, &s.bar_tma, 0, 0, 0);
      tma_load_3d(s.a + 16384, &map_a128, &s.bar_tma, 64, 0, 0);
    } else if (mode == 1) {
      tma_load_3d(s.a, &map_a128, &s.bar_tma, 0, 0, 0);
    } else if (mode == 5) {
      tma_load_3d(s.a, &map_a64, &s.bar_tma, 0, 0, 0);
      tma_load_3d(s.a + 16384, &map_a64, &s.bar_tma, 64, 0, 0);
    }
    if (mode == 0 || mode == 2 || mode == 3 || mode == 4 || mode == 6) {
      tma_load_3d(s.b, &map_b128, &s.bar_tma, 0, 0, 0);
      tma_load_3d(s.b + 16384, &map_b128, &s.bar_tma, 64, 0, 0);
    } else if (mode == 1) {
      tma_load_3d(s.b, &map_b64, &s.bar_tma, 0, 0, 0);
      tma_load_3d(s.b + 16384, &map_b64, &s.bar_tma, 64, 0, 0);
    } else if (mode == 5) {
      tma_load_3d(s.b, &map_b128, &s.bar_tma, 0, 0, 0);
    }
  }
  if (mode == 2) {  // A through CUDA cores: thread = row, 16-byte pieces at swizzled offsets
    const uint4* src = reinterpret_cast<const uint4*>(a_glob + static_cast<size_t>(tid) * 128);
#pragma unroll
    for (int pc = 0; pc < 16; ++pc) {
      const uint4 v = __ldg(src + pc);
      *reinterpret_cast<uint4*>(s.a + (pc >> 3) * 16384 + sw128(tid, (pc & 7) * 16)) = v;
    }
    fence_async_smem();
  }
  if (mode == 4) {  // A into tensor memory columns [128, 192): lane = row, column c holds k = 2c, 2c+1
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a_glob + static_cast<size_t>(tid) * 128);
#pragma unroll
    for (int cb = 0; cb < 2; ++cb) {
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = __ldg(src + cb * 32 + i);
      tmem_st32(tmem_addr(tm, warp * 32, 128 + cb * 32), r);
    }
    tmem_wait_st();
    tc_fence_before();
  }
  __syncthreads();

  // ---- issue the MMAs
  if (tid == 0) {
    tc_fence_after();
    mbar_wait(wc, &s.bar_tma, 0, 1);
    {
      tc_fence_after();
      const uint32_t sa = smem_u32(s.a), sb = smem_u32(s.b);
      if (mode == 0 || mode == 2) {
        const uint32_t idesc = umma_idesc(128, 128, false, false, true);
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_ss(tm, umma_desc_sw128(sa + off, 16, 1024), umma_desc_sw128(sb + off, 16, 1024), idesc, kk > 0);
        }
      } else if (mode == 6) {
        const uint32_t idesc = umma_idesc(128, 64, false, false, true);
        for (int half = 0; half < 2; ++half)
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
            umma_ss(tm + half * 64, umma_desc_sw128(sa + off, 16, 1024),
                    umma_desc_sw128(sb + off + half * 8192, 16, 1024), idesc, kk > 0);
          }
      } else if (mode == 3) {
        const uint32_t idesc = umma_idesc(64, 128, false, false, true);
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_ss(tm, umma_desc_sw128(sa + off, 16, 1024), umma_desc_sw128(sb + off, 16, 1024), idesc, kk > 0);
        }
      } else if (mode == 4) {
        const uint32_t idesc = umma_idesc(128, 128, false, false, true);
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_ts(tm, tm + 128 + kk * 8, umma_desc_sw128(sb + off, 16, 1024), idesc, kk > 0);
        }
      } else if (mode == 1) {
        const uint32_t idesc = umma_idesc(128, 128, false, true, true);
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm, umma_desc_sw128(sa + kk * 32, 16, 1024), umma_desc_sw128(sb + kk * 2048, 16384, 1024), idesc,
                  kk > 0);
      } else if (mode == 5) {
        const uint32_t idesc = umma_idesc(128, 128, true, false, true);
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tm, umma_desc_sw128(sa + kk * 2048, 16384, 1024), umma_desc_sw128(sb + kk * 32, 16, 1024), idesc,
                  kk > 0);
      }
      umma_commit(&s.bar_mma);
    }
  }
  __syncwarp();

  // ---- epilogue: TMEM -> registers -> global
  mbar_wait(wc, &s.bar_mma, 0, 2);
  tc_fence_after();
  {
#pragma unroll 1
    for (int cb = 0; cb < 4; ++cb) {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tm, warp * 32, cb * 32), r);
      tmem_wait_ld();
      if (mode == 3) {
        if (lane < 16) {
          float* dst = d + static_cast<size_t>(warp * 16 + lane) * 128 + cb * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) dst[i] = __uint_as_float(r[i]);
        }
      } else {
        float* dst = d + static_cast<size_t>(warp * 32 + lane) * 128 + cb * 32;
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[i] = __uint_as_float(r[i]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (s.abort_flag) {
    drain_after_abort(tid == 0, &s.drain_bar);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tm, kCols);
}

// A wait that nobody satisfies, with a caller-chosen (short) limit: the safe way to see the expiry path of the
// kernels' bounded waits at work.  Warp 2 waits on an mbarrier without arrivals; the other warps wait on a second
// barrier that warp 2 would arrive on afterwards.  Expected: warp 2's wait gives up after `limit` cycles, writes
// (14 << 12) + 5 to the status word and raises the abort flag; the other warps' waits stop at once; the CTA runs to
// its end, releases its tensor memory and writes 1 to `done`.  Nothing traps, faults or spins without a bound.
struct ExpirySmem {
  uint64_t never, after, drain_bar;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(128) wait_expiry_kernel(int* status_dev, int* done, long long limit) {
  __shared__ ExpirySmem s;
  const int tid = threadIdx.x, warp = tid >> 5;
  WaitCtx wc{&s.abort_flag, status_dev, 14, limit};
  if (tid == 0) {
    s.abort_flag = 0;
    mbar_init(&s.never, 1);
    mbar_init(&s.after, 1);
    mbar_init(&s.drain_bar, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&s.tmem_base, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = s.tmem_base;
  if (warp == 2) {
    mbar_wait(wc, &s.never, 0, 5);
  } else {
    // would be released by warp 2 in a run without the expiry; here the raised flag ends the wait
    WaitCtx wc_long{&s.abort_flag, status_dev, 14, kWaitLimitCycles};
    mbar_wait(wc_long, &s.after, 0, 6);
  }
  tc_fence_before();
  __syncthreads();
  if (s.abort_flag) {
    drain_after_abort(tid == 0, &s.drain_bar);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(tm, 64);
  if (tid == 0) *done = 1;
}

}  // namespace fq

extern "C" FQ_API int fq_selftest_umma(const void* a, const void* b, float* d, int mode, int32_t* status_dev,
                                       void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(a && b && d, "fq_selftest_umma: null tensor");
  FQ_CHECK_ARG(mode >= 0 && mode <= 6, "fq_selftest_umma: mode must be 0..6");
  CUtensorMap ma128, ma64, mb128, mb64;
  int rc;
  if ((rc = make_tmap_rows_heads_dim(&ma128, a, 128, 1, 128, 128, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&ma64, a, 128, 1, 128, 64, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mb128, b, 128, 1, 128, 128, 64)) != FQ_OK) return rc;
  if ((rc = make_tmap_rows_heads_dim(&mb64, b, 128, 1, 128, 64, 64)) != FQ_OK) return rc;
  const size_t smem = sizeof(SelfTestSmem) + 1024;
  {
    static std::atomic<unsigned long long> done{0};
    const int rc_attr = set_smem_limit_once(reinterpret_cast<const void*>(selftest_kernel), static_cast<int>(smem), &done);
    if (rc_attr != FQ_OK) return rc_attr;
  }
  selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(ma128, ma64, mb128, mb64,
                                                                         static_cast<const __nv_bfloat16*>(a), d, mode,
                                                                         status_dev);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_selftest_wait_expiry(int32_t* status_dev, int32_t* done_dev, long long limit_cycles,
                                              void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(status_dev && done_dev, "fq_selftest_wait_expiry: null pointer");
  FQ_CHECK_ARG(limit_cycles > 0 && limit_cycles <= 100000000LL,
               "fq_selftest_wait_expiry: the limit must be between 1 and 1e8 cycles (this test is meant to end at once)");
  wait_expiry_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(status_dev, done_dev, limit_cycles);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}
