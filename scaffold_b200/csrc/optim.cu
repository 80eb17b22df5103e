// Global-norm gradient clipping fused with the Adam update over flat fp32
// parameter / gradient / moment buffers.
//
//   sb_grad_sumsq   two-stage deterministic sum of squares -> norm (device scalar)
//   sb_adam_step    g' = g * min(1, max_norm / (norm + 1e-6)) * inv_scale, then the
//                   Adam update of torch.optim.Adam (no weight decay, no amsgrad);
//                   the clip coefficient is read on the device, so the step needs
//                   no host synchronisation.
//
// Role of the reference: clip_grad_norm_(1.0) + fused Adam in
// ScaFFold/utils/trainer.py:678-694.
#include "common.cuh"
#include "host_api.h"

namespace sb {

constexpr int OPT_THREADS = 256;

__global__ void __launch_bounds__(OPT_THREADS) sumsq_partial_kernel(const float* __restrict__ g, long long n,
                                                                    float* __restrict__ partials) {
  __shared__ float red[OPT_THREADS / 32];
  float acc = 0.f;
  const long long n4 = n / 4;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < n4; i += (long long)gridDim.x * OPT_THREADS) {
    const float4 v = __ldg(g4 + i);
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - n4 * 4)) {
    const float v = g[n4 * 4 + threadIdx.x];
    acc += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = 0.f;
#pragma unroll
    for (int w = 0; w < OPT_THREADS / 32; ++w) r += red[w];
    partials[blockIdx.x] = r;
  }
}

__global__ void sumsq_finalize_kernel(const float* __restrict__ partials, int nblocks, float* __restrict__ out) {
  // single thread, index order: deterministic
  double acc = 0.0;
  for (int i = 0; i < nblocks; ++i) acc += (double)partials[i];
  out[0] = (float)sqrt(acc);
}

__global__ void __launch_bounds__(OPT_THREADS) adam_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                           float* __restrict__ m, float* __restrict__ v, long long n,
                                                           float lr, float b1, float b2, float eps, float bc1,
                                                           float bc2_sqrt, float max_norm,
                                                           const float* __restrict__ norm, float grad_scale) {
  float coef = grad_scale;
  if (max_norm > 0.f && norm != nullptr) {
    const float c = max_norm / (norm[0] * grad_scale + 1e-6f);
    coef *= c < 1.f ? c : 1.f;
  }
  const float step_size = lr / bc1;
  for (long long i = (long long)blockIdx.x * OPT_THREADS + threadIdx.x; i < n; i += (long long)gridDim.x * OPT_THREADS) {
    const float gi = g[i] * coef;
    const float mi = m[i] + (gi - m[i]) * (1.f - b1);       // lerp, as torch does
    const float vi = v[i] * b2 + gi * gi * (1.f - b2);
    m[i] = mi;
    v[i] = vi;
    const float denom = sqrtf(vi) / bc2_sqrt + eps;
    p[i] -= step_size * mi / denom;
  }
}

}  // namespace sb

using namespace sb;

extern "C" int sb_opt_blocks(long long n) {
  long long b = (n / 4 + OPT_THREADS - 1) / OPT_THREADS;
  const long long cap = 148LL * 8;
  return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}

extern "C" int sb_grad_norm(const float* g, long long n, float* partials, float* norm_out, cudaStream_t stream) {
  if ((reinterpret_cast<uintptr_t>(g) & 15) != 0) return SB_ERR_ALIGN;
  const int blocks = sb_opt_blocks(n);
  sumsq_partial_kernel<<<blocks, OPT_THREADS, 0, stream>>>(g, n, partials);
  sb_count_launch(1);
  sumsq_finalize_kernel<<<1, 1, 0, stream>>>(partials, blocks, norm_out);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_adam_step(float* p, const float* g, float* m, float* v, long long n, float lr, float b1, float b2,
                            float eps, int step, float max_norm, const float* norm, float grad_scale,
                            cudaStream_t stream) {
  const float bc1 = 1.f - powf(b1, (float)step);
  const float bc2_sqrt = sqrtf(1.f - powf(b2, (float)step));
  const int blocks = sb_opt_blocks(n) * 2;
  adam_kernel<<<blocks, OPT_THREADS, 0, stream>>>(p, g, m, v, n, lr, b1, b2, eps, bc1, bc2_sqrt, max_norm, norm,
                                                  grad_scale);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
