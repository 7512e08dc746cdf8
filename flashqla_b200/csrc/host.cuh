// Host-side helpers shared by the C-ABI entry points: error reporting, TMA descriptor
// construction through the driver entry point (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "common.cuh"

namespace fq {

// Thread-local message returned by fq_last_error().
char* last_error_buf();
void set_error(const char* fmt, ...);

#define FQ_CHECK_ARG(cond, ...)      \
  do {                               \
    if (!(cond)) {                   \
      ::fq::set_error(__VA_ARGS__);  \
      return FQ_ERR_INVALID;   \
    }                                \
  } while (0)

#define FQ_CHECK_CUDA(expr)                                                                  \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess) {                                                                 \
      ::fq::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return FQ_ERR_CUDA;                                                             \
    }                                                                                        \
  } while (0)

// Tensor map over a [rows][heads][dim] bf16/fp16 tensor (dim contiguous, heads next, rows
// slowest) with a box of `box_dim` x 1 x `box_rows` elements and 128-byte swizzle.
// Returns FQ_OK or an error code.
int make_tmap_rows_heads_dim(CUtensorMap* out, const void* base, uint64_t rows, uint64_t heads, uint64_t dim,
                             uint32_t box_rows, uint32_t box_dim);

// Raises the dynamic shared-memory limit of kernel `func` to `bytes` on the current device, once per device
// (`done_mask`: one bit per device index, owned by the caller as a function-local static).  Safe to call from
// several host threads at once.  Returns FQ_OK or an error code.
int set_smem_limit_once(const void* func, int bytes, std::atomic<unsigned long long>* done_mask);

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace fq
