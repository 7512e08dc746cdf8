// Row-wise L2 normalisation of q / k over the head dimension (128): y = x * rsqrt(sum(x^2) + eps), and its
// backward dx = r * dy - x * r^3 * (x . dy) with r = rsqrt(sum(x^2) + eps) recomputed from x.
// One warp per row (32 lanes x 4 bf16 = 8 bytes per lane); fp32 arithmetic in registers, one pass over HBM
// (2 bytes read + 2 bytes written per element forward, 4 + 2 backward).
#include "flashqla.h"
#include "host.cuh"

namespace fq {

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__global__ void __launch_bounds__(256) l2norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                         long long rows, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(x + r * kDim) + lane);
    const float a0 = bf16_lo(v.x), a1 = bf16_hi(v.x), a2 = bf16_lo(v.y), a3 = bf16_hi(v.y);
    const float rinv = rsqrtf(warp_sum(a0 * a0 + a1 * a1 + a2 * a2 + a3 * a3) + eps);
    uint2 o;
    o.x = pack_bf16(a0 * rinv, a1 * rinv);
    o.y = pack_bf16(a2 * rinv, a3 * rinv);
    *(reinterpret_cast<uint2*>(y + r * kDim) + lane) = o;
  }
}

__global__ void __launch_bounds__(256) l2norm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                                         __nv_bfloat16* __restrict__ dx, long long rows, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(x + r * kDim) + lane);
    const uint2 d = __ldg(reinterpret_cast<const uint2*>(dy + r * kDim) + lane);
    const float a[4] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y)};
    const float g[4] = {bf16_lo(d.x), bf16_hi(d.x), bf16_lo(d.y), bf16_hi(d.y)};
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { ss += a[i] * a[i]; dot += a[i] * g[i]; }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float rinv = rsqrtf(ss + eps);
    const float c = dot * rinv * rinv * rinv;
    uint2 o;
    o.x = pack_bf16(rinv * g[0] - c * a[0], rinv * g[1] - c * a[1]);
    o.y = pack_bf16(rinv * g[2] - c * a[2], rinv * g[3] - c * a[3]);
    *(reinterpret_cast<uint2*>(dx + r * kDim) + lane) = o;
  }
}

static int l2norm_grid(long long rows) {
  const long long blocks = (rows + 7) / 8;  // 8 warps (rows) per block
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return static_cast<int>(blocks < cap ? blocks : cap);
}

}  // namespace fq

extern "C" FQ_API int fq_l2norm_fwd(const void* x, void* y, long long rows, float eps, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(x && y && rows >= 0, "fq_l2norm_fwd: bad arguments");
  if (rows == 0) return FQ_OK;
  l2norm_fwd_kernel<<<l2norm_grid(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), rows, eps);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}

extern "C" FQ_API int fq_l2norm_bwd(const void* x, const void* dy, void* dx, long long rows, float eps, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(x && dy && dx && rows >= 0, "fq_l2norm_bwd: bad arguments");
  if (rows == 0) return FQ_OK;
  l2norm_bwd_kernel<<<l2norm_grid(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), rows, eps);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}
