// Token-by-token recurrence of the gated delta rule: the decode side of the chunked prefill (it consumes the final
// state that the forward writes and produces the state the next call starts from).  Per (sequence, V-head), for
// each of the T new tokens:
//
//   S <- e^{g} S;   v' = beta (v - S^T k);   S <- S + k v'^T;   o = scale * S^T q
//
// The state [K = 128][V = 128] (fp32, 64 KiB) is the only large operand: one pass reads it, keeps it in
// registers over the T tokens and writes it back, i.e. the kernel is bound by 128 KiB of HBM traffic per head.
// A CTA of 128 threads owns 32 columns v of one head (4 CTAs per head keep enough loads in flight when there are
// few heads): thread (kq, lane) holds S[32 kq .. 32 kq + 31][v], so every global access of a warp is one 128-byte
// row segment; the two dot products reduce over the four kq groups through shared memory.
#include "flashqla.h"
#include "host.cuh"

namespace fq {

constexpr int kDecThreads = 128;
constexpr int kDecCols = 32;  // V columns per CTA

__global__ void __launch_bounds__(kDecThreads) gdr_recurrent_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const float* __restrict__ g, const float* __restrict__ beta, const float* __restrict__ state_in,
    float* __restrict__ state_out, __nv_bfloat16* __restrict__ o, int T, int H, int Hg, float scale) {
  __shared__ float ks[kDim], qs[kDim];
  __shared__ float red[4][kDecCols];
  const int tid = threadIdx.x, lane = tid & 31, kq = tid >> 5;
  const int vs = blockIdx.x & 3;
  const int head = blockIdx.x >> 2;  // n * H + h
  const int n = head / H, h = head - n * H;
  const int hg = h / (H / Hg);
  const int vcol = vs * kDecCols + lane;

  float s[32];
  const size_t sbase = (static_cast<size_t>(head) * kDim + 32 * kq) * kDim + vcol;
  if (state_in != nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i) s[i] = __ldg(state_in + sbase + static_cast<size_t>(i) * kDim);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) s[i] = 0.f;
  }

  for (int t = 0; t < T; ++t) {
    const size_t tok = static_cast<size_t>(n) * T + t;
    __syncthreads();  // the previous token's reads of ks / qs / red are complete
    ks[tid] = __bfloat162float(k[(tok * Hg + hg) * kDim + tid]);
    qs[tid] = __bfloat162float(q[(tok * Hg + hg) * kDim + tid]);
    const float gam = __expf(__ldg(g + tok * H + h));
    const float bt = __ldg(beta + tok * H + h);
    const float vv = __bfloat162float(v[(tok * H + h) * kDim + vcol]);
    __syncthreads();
    float pred = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      s[i] *= gam;
      pred += s[i] * ks[32 * kq + i];
    }
    red[kq][lane] = pred;
    __syncthreads();
    const float vnew = bt * (vv - (red[0][lane] + red[1][lane] + red[2][lane] + red[3][lane]));
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      s[i] += ks[32 * kq + i] * vnew;
      acc += s[i] * qs[32 * kq + i];
    }
    __syncthreads();  // every thread has read red before it is reused
    red[kq][lane] = acc;
    __syncthreads();
    if (kq == 0)
      o[(tok * H + h) * kDim + vcol] =
          __float2bfloat16(scale * (red[0][lane] + red[1][lane] + red[2][lane] + red[3][lane]));
  }
  if (state_out != nullptr) {
#pragma unroll
    for (int i = 0; i < 32; ++i) state_out[sbase + static_cast<size_t>(i) * kDim] = s[i];
  }
}

}  // namespace fq

extern "C" FQ_API int fq_gdr_recurrent(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                       const float* state_in, float* state_out, void* o, int N, int T, int H, int Hg,
                                       float scale, void* stream) {
  using namespace fq;
  FQ_CHECK_ARG(q && k && v && g && beta && o, "fq_gdr_recurrent: null tensor");
  FQ_CHECK_ARG(N > 0 && T > 0 && H > 0 && Hg > 0 && H % Hg == 0, "fq_gdr_recurrent: bad sizes");
  const long long ctas = 4LL * N * H;
  FQ_CHECK_ARG(ctas < (1LL << 31), "fq_gdr_recurrent: too many (sequence, head) pairs");
  gdr_recurrent_kernel<<<static_cast<unsigned>(ctas), kDecThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      g, beta, state_in, state_out, static_cast<__nv_bfloat16*>(o), T, H, Hg, scale);
  FQ_CHECK_CUDA(cudaGetLastError());
  return FQ_OK;
}
