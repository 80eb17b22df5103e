// Fused segmentation loss: softmax cross-entropy (class-weighted) + soft Dice
// sums in ONE pass over the logits, and the gradient w.r.t. the logits in one
// more pass; plus the hard-Dice (argmax) counts of the validation metric.
//
// Logits are voxel-major bf16 [N, S, CP] (CP = classes padded to a multiple of
// 8, at most 32), labels int16/int32/int64 [N, S]. No fp32 probability tensor,
// no one-hot tensor and no log-softmax tensor is ever written: every thread
// keeps one voxel's classes in registers.
//
// Pass 1 (loss_sums_kernel): per sample n and class c
//     P[n][c] = sum_v p_c(v)        Q[n][c] = sum_v [y(v) = c]
//     I[n][c] = sum_v p_c(v) [y(v) = c]
//   and CE numerator sum_v w[y] * (-log p_y), denominator sum_v w[y].
//   Block partials go to a workspace; loss_finalize_kernel adds them in index
//   order (deterministic) into sums[N][C][3] and ce[2].
// Pass 2 (loss_grad_kernel): with per-(n,c) coefficients alpha, beta of
//   dL/dp_c(v) = alpha[n][c] * [y(v)=c] + beta[n][c] and k_ce = g / denominator:
//     dlogit_j = k_ce * w[y] * (p_j - [y=j]) + p_j * (a_j - sum_c a_c p_c)
//
// A label outside [0, C) (a dataset with more categories than the model, an ignore
// value) is never used as an index: the voxel gets weight 0 in the cross entropy and
// belongs to no class in the Dice sums, and the kernels record ST_BAD_ARG (site 61 /
// 62, detail = label value) in the status word so that the host can raise.
//
// Role of the reference: ScaFFold/utils/trainer.py:635-664,
// ScaFFold/utils/losses.py:117-205, ScaFFold/utils/dice_score.py:101-136,
// ScaFFold/utils/evaluate.py:178-193.
#include "common.cuh"
#include "host_api.h"

namespace sb {

constexpr int LOSS_THREADS = 256;
constexpr int LOSS_MAXC = 32;

__device__ __forceinline__ long long load_label(const void* labels, int kind, long long i) {
  if (kind == 2) return reinterpret_cast<const short*>(labels)[i];
  if (kind == 4) return reinterpret_cast<const int*>(labels)[i];
  return reinterpret_cast<const long long*>(labels)[i];
}

template <int CP>
__device__ __forceinline__ void load_logits(const __nv_bfloat16* p, float (&f)[CP]) {
#pragma unroll
  for (int i = 0; i < CP / 8; ++i) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p) + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(h[j]);
      f[i * 8 + 2 * j] = t.x;
      f[i * 8 + 2 * j + 1] = t.y;
    }
  }
}

// softmax over the first C of CP entries; returns log-sum-exp
template <int CP>
__device__ __forceinline__ float softmax_regs(float (&f)[CP], int C) {
  float m = -INFINITY;
#pragma unroll
  for (int c = 0; c < CP; ++c)
    if (c < C) m = fmaxf(m, f[c]);
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < CP; ++c) {
    f[c] = c < C ? __expf(f[c] - m) : 0.f;
    s += f[c];
  }
  const float inv = 1.f / s;
#pragma unroll
  for (int c = 0; c < CP; ++c) f[c] *= inv;
  return m + __logf(s);
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = 0.f;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 0; w < LOSS_THREADS / 32; ++w) r += red[w];
  }
  return r;  // valid on thread 0
}

// workspace layout per (n, block): [3*C + 2] floats: P[c], Q[c], I[c], ce_num, ce_den
template <int CP>
__global__ void __launch_bounds__(LOSS_THREADS) loss_sums_kernel(const __nv_bfloat16* __restrict__ logits,
                                                                 const void* __restrict__ labels, int label_kind,
                                                                 const float* __restrict__ cw, float* __restrict__ ws,
                                                                 int C, long long S, int argmax_mode,
                                                                 uint32_t* __restrict__ status) {
  __shared__ float red[LOSS_THREADS / 32];
  const int n = blockIdx.y;
  float P[CP], Q[CP], I[CP];
#pragma unroll
  for (int c = 0; c < CP; ++c) { P[c] = 0.f; Q[c] = 0.f; I[c] = 0.f; }
  float ce_num = 0.f, ce_den = 0.f;
  // two voxels per iteration: both voxels' logits and labels are requested before either is used
  const long long stride = (long long)gridDim.x * LOSS_THREADS;
  auto voxel = [&](float (&f)[CP], const long long y_raw) {
    const bool y_ok = y_raw >= 0 && y_raw < C;
    const int y = y_ok ? (int)y_raw : -1;
    if (!y_ok) report(status, ST_BAD_ARG, 61, (uint32_t)y_raw, (uint32_t)n);
    float ly = 0.f;
#pragma unroll
    for (int c = 0; c < CP; ++c)
      if (c == y) ly = f[c];
    const float lse = softmax_regs<CP>(f, C);  // f now holds probabilities
    if (argmax_mode) {
      // hard prediction: one-hot of the first maximum
      int best = 0;
      float bv = f[0];
#pragma unroll
      for (int c = 1; c < CP; ++c)
        if (c < C && f[c] > bv) { bv = f[c]; best = c; }
#pragma unroll
      for (int c = 0; c < CP; ++c) f[c] = c == best ? 1.f : 0.f;
    }
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      P[c] += f[c];
      if (c == y) { Q[c] += 1.f; I[c] += f[c]; }
    }
    const float wy = y_ok ? (cw ? cw[y] : 1.f) : 0.f;
    ce_num += wy * (lse - ly);
    ce_den += wy;
  };
  long long v = (long long)blockIdx.x * LOSS_THREADS + threadIdx.x;
  for (; v + stride < S; v += 2 * stride) {
    float f0[CP], f1[CP];
    load_logits<CP>(logits + ((long long)n * S + v) * CP, f0);
    load_logits<CP>(logits + ((long long)n * S + v + stride) * CP, f1);
    const long long y0 = load_label(labels, label_kind, (long long)n * S + v);
    const long long y1 = load_label(labels, label_kind, (long long)n * S + v + stride);
    voxel(f0, y0);
    voxel(f1, y1);
  }
  for (; v < S; v += stride) {
    float f0[CP];
    load_logits<CP>(logits + ((long long)n * S + v) * CP, f0);
    voxel(f0, load_label(labels, label_kind, (long long)n * S + v));
  }
  float* dst = ws + ((long long)n * gridDim.x + blockIdx.x) * (3 * C + 2);
#pragma unroll
  for (int c = 0; c < CP; ++c) {
    if (c < C) {
      float r = block_sum(P[c], red);
      if (threadIdx.x == 0) dst[c] = r;
      r = block_sum(Q[c], red);
      if (threadIdx.x == 0) dst[C + c] = r;
      r = block_sum(I[c], red);
      if (threadIdx.x == 0) dst[2 * C + c] = r;
    }
  }
  float r = block_sum(ce_num, red);
  if (threadIdx.x == 0) dst[3 * C] = r;
  r = block_sum(ce_den, red);
  if (threadIdx.x == 0) dst[3 * C + 1] = r;
}

// out[n][k] = sum_b ws[n][b][k], k < 3C+2 (double accumulation, index order)
__global__ void loss_finalize_kernel(const float* __restrict__ ws, float* __restrict__ out, int nblocks, int K) {
  const int n = blockIdx.x;
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    double acc = 0.0;
    for (int b = 0; b < nblocks; ++b) acc += (double)ws[((long long)n * nblocks + b) * K + k];
    out[(long long)n * K + k] = (float)acc;
  }
}

template <int CP>
__global__ void __launch_bounds__(LOSS_THREADS) loss_grad_kernel(const __nv_bfloat16* __restrict__ logits,
                                                                 const void* __restrict__ labels, int label_kind,
                                                                 const float* __restrict__ cw,
                                                                 const float* __restrict__ coef,  // [N][2][C]
                                                                 const float* __restrict__ kce,   // [1]
                                                                 __nv_bfloat16* __restrict__ dlogits, int C,
                                                                 long long S, uint32_t* __restrict__ status) {
  const int n = blockIdx.y;
  float alpha[CP], beta[CP];
#pragma unroll
  for (int c = 0; c < CP; ++c) {
    alpha[c] = c < C ? coef[((long long)n * 2 + 0) * C + c] : 0.f;
    beta[c] = c < C ? coef[((long long)n * 2 + 1) * C + c] : 0.f;
  }
  const float k_ce = kce[0];
  auto voxel = [&](float (&f)[CP], const long long y_raw, const long long off) {
    const bool y_ok = y_raw >= 0 && y_raw < C;
    const int y = y_ok ? (int)y_raw : -1;
    if (!y_ok) report(status, ST_BAD_ARG, 62, (uint32_t)y_raw, (uint32_t)n);
    softmax_regs<CP>(f, C);
    const float wy = y_ok ? (cw ? cw[y] : 1.f) * k_ce : 0.f;
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      const float a = beta[c] + (c == y ? alpha[c] : 0.f);
      dot += a * f[c];
    }
    float g[CP];
#pragma unroll
    for (int c = 0; c < CP; ++c) {
      const float a = beta[c] + (c == y ? alpha[c] : 0.f);
      g[c] = c < C ? wy * (f[c] - (c == y ? 1.f : 0.f)) + f[c] * (a - dot) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < CP / 8; ++i) {
      uint4 o;
      o.x = pack_bf16x2(g[i * 8 + 0], g[i * 8 + 1]);
      o.y = pack_bf16x2(g[i * 8 + 2], g[i * 8 + 3]);
      o.z = pack_bf16x2(g[i * 8 + 4], g[i * 8 + 5]);
      o.w = pack_bf16x2(g[i * 8 + 6], g[i * 8 + 7]);
      reinterpret_cast<uint4*>(dlogits + off)[i] = o;
    }
  };
  // two voxels per iteration: both voxels' logits and labels are requested before either is used
  const long long stride = (long long)gridDim.x * LOSS_THREADS;
  long long v = (long long)blockIdx.x * LOSS_THREADS + threadIdx.x;
  for (; v + stride < S; v += 2 * stride) {
    float f0[CP], f1[CP];
    const long long off0 = ((long long)n * S + v) * CP, off1 = ((long long)n * S + v + stride) * CP;
    load_logits<CP>(logits + off0, f0);
    load_logits<CP>(logits + off1, f1);
    const long long y0 = load_label(labels, label_kind, (long long)n * S + v);
    const long long y1 = load_label(labels, label_kind, (long long)n * S + v + stride);
    voxel(f0, y0, off0);
    voxel(f1, y1, off1);
  }
  for (; v < S; v += stride) {
    float f0[CP];
    const long long off0 = ((long long)n * S + v) * CP;
    load_logits<CP>(logits + off0, f0);
    voxel(f0, load_label(labels, label_kind, (long long)n * S + v), off0);
  }
}

}  // namespace sb

using namespace sb;

extern "C" int sb_loss_blocks(long long S) {
  long long b = (S + LOSS_THREADS - 1) / LOSS_THREADS;
  const long long cap = 148LL * 4;
  return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}

// sums: [N][3C+2] floats; ws: [N][blocks][3C+2]
// largest class count of the fused kernels (callers route wider heads to the framework formula)
extern "C" int sb_loss_max_classes(void) { return LOSS_MAXC; }

extern "C" int sb_loss_sums(const void* logits, const void* labels, int label_kind, const float* cw, float* ws,
                            float* sums, int N, long long S, int C, int CP, int argmax_mode, uint32_t* status,
                            cudaStream_t stream) {
  if (C > CP || CP % 8 != 0 || CP > LOSS_MAXC) return SB_ERR_SHAPE;
  if (label_kind != 2 && label_kind != 4 && label_kind != 8) return SB_ERR_SHAPE;
  const int blocks = sb_loss_blocks(S);
  dim3 grid(blocks, N);
  const __nv_bfloat16* lg = (const __nv_bfloat16*)logits;
  switch (CP) {
    case 8: loss_sums_kernel<8><<<grid, LOSS_THREADS, 0, stream>>>(lg, labels, label_kind, cw, ws, C, S, argmax_mode, status); sb_count_launch(1); break;
    case 16: loss_sums_kernel<16><<<grid, LOSS_THREADS, 0, stream>>>(lg, labels, label_kind, cw, ws, C, S, argmax_mode, status); sb_count_launch(1); break;
    case 24: loss_sums_kernel<24><<<grid, LOSS_THREADS, 0, stream>>>(lg, labels, label_kind, cw, ws, C, S, argmax_mode, status); sb_count_launch(1); break;
    case 32: loss_sums_kernel<32><<<grid, LOSS_THREADS, 0, stream>>>(lg, labels, label_kind, cw, ws, C, S, argmax_mode, status); sb_count_launch(1); break;
    default: return SB_ERR_SHAPE;
  }
  loss_finalize_kernel<<<N, 128, 0, stream>>>(ws, sums, blocks, 3 * C + 2);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_loss_grad(const void* logits, const void* labels, int label_kind, const float* cw,
                            const float* coef, const float* kce, void* dlogits, int N, long long S, int C, int CP,
                            uint32_t* status, cudaStream_t stream) {
  if (C > CP || CP % 8 != 0 || CP > LOSS_MAXC) return SB_ERR_SHAPE;
  const int blocks = sb_loss_blocks(S) * 2;
  dim3 grid(blocks, N);
  const __nv_bfloat16* lg = (const __nv_bfloat16*)logits;
  __nv_bfloat16* dl = (__nv_bfloat16*)dlogits;
  switch (CP) {
    case 8: loss_grad_kernel<8><<<grid, LOSS_THREADS, 0, stream>>>(lg, labels, label_kind, cw, coef, kce, dl, C, S, status); sb_count_launch(1); break;
    case 16: loss_grad_kernel<16><<<grid, LOSS_THREADS, 0, stream>>>(lg, labels, label_kind, cw, coef, kce, dl, C, S, status); sb_count_launch(1); break;
    case 24: loss_grad_kernel<24><<<grid, LOSS_THREADS, 0, stream>>>(lg, labels, label_kind, cw, coef, kce, dl, C, S, status); sb_count_launch(1); break;
    case 32: loss_grad_kernel<32><<<grid, LOSS_THREADS, 0, stream>>>(lg, labels, label_kind, cw, coef, kce, dl, C, S, status); sb_count_launch(1); break;
    default: return SB_ERR_SHAPE;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
