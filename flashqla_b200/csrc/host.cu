// Host utilities: error string, driver entry point for tensor-map encoding, version.
#include "host.cuh"

#include <stdarg.h>
#include <atomic>
#include <string.h>

#include "flashqla.h"

namespace fq {

char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int make_tmap_rows_heads_dim(CUtensorMap* out, const void* base, uint64_t rows, uint64_t heads, uint64_t dim,
                             uint32_t box_rows, uint32_t box_dim) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return FQ_ERR_CUDA;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_error("tensor base address must be 16-byte aligned for TMA");
    return FQ_ERR_INVALID;
  }
  // The encoder is a driver call and needs a current context.  A host thread that has only selected a device
  // (e.g. an autograd worker thread whose first CUDA work is this call) has none yet: re-selecting the current
  // device through the runtime initialises the device's primary context and binds it to the thread.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) {
      set_error("no usable CUDA context on this thread: %s", cudaGetErrorString(cudaGetLastError()));
      return FQ_ERR_CUDA;
    }
    ctx_bound = true;
  }
  cuuint64_t gdim[3] = {dim, heads, rows};
  cuuint64_t gstride[2] = {dim * 2, heads * dim * 2};  // bytes, for dims 1 and 2
  cuuint32_t box[3] = {box_dim, 1, box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu heads=%llu dim=%llu)", (int)r,
              (unsigned long long)rows, (unsigned long long)heads, (unsigned long long)dim);
    return FQ_ERR_CUDA;
  }
  return FQ_OK;
}

int set_smem_limit_once(const void* func, int bytes, std::atomic<unsigned long long>* done_mask) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_error("cudaGetDevice failed: %s", cudaGetErrorString(e));
    return FQ_ERR_CUDA;
  }
  const unsigned long long bit = (dev >= 0 && dev < 64) ? (1ull << dev) : 0ull;
  if (bit && (done_mask->load(std::memory_order_acquire) & bit)) return FQ_OK;
  // idempotent: two host threads that get here together both set the same value
  e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(MaxDynamicSharedMemorySize=%d) failed: %s", bytes, cudaGetErrorString(e));
    return FQ_ERR_CUDA;
  }
  if (bit) done_mask->fetch_or(bit, std::memory_order_release);
  return FQ_OK;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace fq

extern "C" {
FQ_API int fq_version(void) { return 100; }
FQ_API const char* fq_last_error(void) { return fq::last_error_buf(); }
}
