// 2x2x2 max-pool for channels-last bf16 activations, forward and backward.
//
// One thread owns 8 channels (a 16-byte vector) of one OUTPUT voxel: forward
// reads its 8 input voxels and stores the maximum; backward recomputes which
// input produced the maximum (first match in (kd,kh,kw) order, the rule ATen
// uses) and writes the full 2x2x2 input-gradient block, so no index tensor is
// kept and dx needs no zero fill. Odd trailing planes (floor mode) get zeros.
//
// Role of the reference: nn.MaxPool3d(2) in ScaFFold/unet/unet_parts.py:159-171.
#include "common.cuh"
#include "host_api.h"

namespace sb {

__device__ __forceinline__ void unpack8p(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__global__ void __launch_bounds__(256) maxpool2_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                           __nv_bfloat16* __restrict__ y, int N, int D, int H,
                                                           int W, int C) {
  const int OD = D / 2, OH = H / 2, OW = W / 2, C8 = C / 8;
  const long long total = (long long)N * OD * OH * OW * C8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int c8 = (int)(t % C8); t /= C8;
    const int ow = (int)(t % OW); t /= OW;
    const int oh = (int)(t % OH); t /= OH;
    const int od = (int)(t % OD); t /= OD;
    const int n = (int)t;
    float m[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) m[j] = -INFINITY;
    bool nan[8] = {false, false, false, false, false, false, false, false};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int kd = k >> 2, kh = (k >> 1) & 1, kw = k & 1;
      const long long v = (((long long)n * D + (2 * od + kd)) * H + (2 * oh + kh)) * W + (2 * ow + kw);
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + v * C + c8 * 8));
      float f[8];
      unpack8p(raw, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (f[j] != f[j]) nan[j] = true;
        m[j] = fmaxf(m[j], f[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (nan[j]) m[j] = __int_as_float(0x7fc00000);
    uint4 o;
    o.x = pack_bf16x2(m[0], m[1]);
    o.y = pack_bf16x2(m[2], m[3]);
    o.z = pack_bf16x2(m[4], m[5]);
    o.w = pack_bf16x2(m[6], m[7]);
    *reinterpret_cast<uint4*>(y + i * 8) = o;
  }
}

__global__ void __launch_bounds__(256) maxpool2_bwd_kernel(const __nv_bfloat16* __restrict__ gy,
                                                           const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ y,
                                                           __nv_bfloat16* __restrict__ gx, int N, int D, int H,
                                                           int W, int C) {
  const int OD = D / 2, OH = H / 2, OW = W / 2, C8 = C / 8;
  const long long total = (long long)N * OD * OH * OW * C8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int c8 = (int)(t % C8); t /= C8;
    const int ow = (int)(t % OW); t /= OW;
    const int oh = (int)(t % OH); t /= OH;
    const int od = (int)(t % OD); t /= OD;
    const int n = (int)t;
    const uint4 ry = __ldg(reinterpret_cast<const uint4*>(y + i * 8));
    const uint4 rg = __ldg(reinterpret_cast<const uint4*>(gy + i * 8));
    const unsigned short* ys = reinterpret_cast<const unsigned short*>(&ry);
    const unsigned short* gs = reinterpret_cast<const unsigned short*>(&rg);
    unsigned taken = 0;  // bit j: channel j already routed
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int kd = k >> 2, kh = (k >> 1) & 1, kw = k & 1;
      const long long v = (((long long)n * D + (2 * od + kd)) * H + (2 * oh + kh)) * W + (2 * ow + kw);
      const uint4 rx = __ldg(reinterpret_cast<const uint4*>(x + v * C + c8 * 8));
      const unsigned short* xs = reinterpret_cast<const unsigned short*>(&rx);
      uint4 o;
      unsigned short* os = reinterpret_cast<unsigned short*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // bitwise equality with the stored maximum; a NaN maximum matches the first NaN input
        const bool isnan_y = (ys[j] & 0x7fff) > 0x7f80;
        const bool isnan_x = (xs[j] & 0x7fff) > 0x7f80;
        const bool same = isnan_y ? isnan_x : (xs[j] == ys[j] || ((xs[j] | ys[j]) & 0x7fff) == 0);
        const bool hit = same && !((taken >> j) & 1u);
        if (hit) taken |= 1u << j;
        os[j] = hit ? gs[j] : (unsigned short)0;
      }
      *reinterpret_cast<uint4*>(gx + v * C + c8 * 8) = o;
    }
  }
}

// Forward that also records, per output element, WHICH of its eight inputs is the maximum (one byte per channel,
// eight channels = one 64-bit word per thread; first match in (kd,kh,kw) order, a NaN wins over numbers and the first
// NaN over later ones: the rule of the kernels above). The backward pass below then needs neither x nor y: it reads
// gy and the index words (3/16 of a volume) and writes gx, instead of reading a whole volume of x again.
__global__ void __launch_bounds__(256) maxpool2_fwd_idx_kernel(const __nv_bfloat16* __restrict__ x,
                                                               __nv_bfloat16* __restrict__ y,
                                                               unsigned long long* __restrict__ idx, int N, int D,
                                                               int H, int W, int C) {
  const int OD = D / 2, OH = H / 2, OW = W / 2, C8 = C / 8;
  const long long total = (long long)N * OD * OH * OW * C8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int c8 = (int)(t % C8); t /= C8;
    const int ow = (int)(t % OW); t /= OW;
    const int oh = (int)(t % OH); t /= OH;
    const int od = (int)(t % OD); t /= OD;
    const int n = (int)t;
    float m[8];
    unsigned int bi[8];  // index k of channel j's maximum
    uint4 raw[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int kd = k >> 2, kh = (k >> 1) & 1, kw = k & 1;
      const long long v = (((long long)n * D + (2 * od + kd)) * H + (2 * oh + kh)) * W + (2 * ow + kw);
      raw[k] = __ldg(reinterpret_cast<const uint4*>(x + v * C + c8 * 8));
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float f[8];
      unpack8p(raw[k], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (k == 0) {
          m[j] = f[j];
          bi[j] = 0u;
        } else if (m[j] == m[j] && (f[j] != f[j] || f[j] > m[j])) {  // keep a NaN; else take a NaN or a larger value
          m[j] = f[j];
          bi[j] = (unsigned int)k;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (m[j] != m[j]) m[j] = __int_as_float(0x7fc00000);
    uint4 o;
    o.x = pack_bf16x2(m[0], m[1]);
    o.y = pack_bf16x2(m[2], m[3]);
    o.z = pack_bf16x2(m[4], m[5]);
    o.w = pack_bf16x2(m[6], m[7]);
    *reinterpret_cast<uint4*>(y + i * 8) = o;
    // byte j of the index word: channel j's winner
    const unsigned int lo = bi[0] | (bi[1] << 8) | (bi[2] << 16) | (bi[3] << 24);
    const unsigned int hi = bi[4] | (bi[5] << 8) | (bi[6] << 16) | (bi[7] << 24);
    idx[i] = (unsigned long long)lo | ((unsigned long long)hi << 32);
  }
}

__global__ void __launch_bounds__(256) maxpool2_bwd_idx_kernel(const __nv_bfloat16* __restrict__ gy,
                                                               const unsigned long long* __restrict__ idx,
                                                               __nv_bfloat16* __restrict__ gx, int N, int D, int H,
                                                               int W, int C) {
  const int OD = D / 2, OH = H / 2, OW = W / 2, C8 = C / 8;
  const long long total = (long long)N * OD * OH * OW * C8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i;
    const int c8 = (int)(t % C8); t /= C8;
    const int ow = (int)(t % OW); t /= OW;
    const int oh = (int)(t % OH); t /= OH;
    const int od = (int)(t % OD); t /= OD;
    const int n = (int)t;
    const uint4 rg = __ldg(reinterpret_cast<const uint4*>(gy + i * 8));
    const unsigned long long which = __ldg(idx + i);
    const unsigned short* gs = reinterpret_cast<const unsigned short*>(&rg);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int kd = k >> 2, kh = (k >> 1) & 1, kw = k & 1;
      const long long v = (((long long)n * D + (2 * od + kd)) * H + (2 * oh + kh)) * W + (2 * ow + kw);
      uint4 o;
      unsigned short* os = reinterpret_cast<unsigned short*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) os[j] = ((which >> (8 * j)) & 0xffull) == (unsigned long long)k ? gs[j] : (unsigned short)0;
      *reinterpret_cast<uint4*>(gx + v * C + c8 * 8) = o;
    }
  }
}

// zero the planes a floor-mode pool never reads (odd extents)
__global__ void maxpool2_bwd_tail_kernel(__nv_bfloat16* gx, int N, int D, int H, int W, int C) {
  const long long total = (long long)N * D * H * W;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total;
       v += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(v % W), h = (int)((v / W) % H), d = (int)((v / ((long long)W * H)) % D);
    if (w >= (W / 2) * 2 || h >= (H / 2) * 2 || d >= (D / 2) * 2)
      for (int c = 0; c < C; ++c) gx[v * C + c] = __float2bfloat16(0.f);
  }
}

}  // namespace sb

using namespace sb;

static int pool_grid(long long total) {
  long long b = (total + 255) / 256;
  const long long cap = 148LL * 16;
  return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}

extern "C" int sb_maxpool2_fwd(const void* x, void* y, int N, int D, int H, int W, int C, cudaStream_t stream) {
  if (C % 8 != 0 || D < 2 || H < 2 || W < 2) return SB_ERR_SHAPE;
  const long long total = (long long)N * (D / 2) * (H / 2) * (W / 2) * (C / 8);
  maxpool2_fwd_kernel<<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, N, D, H, W, C);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_maxpool2_bwd(const void* gy, const void* x, const void* y, void* gx, int N, int D, int H, int W,
                               int C, cudaStream_t stream) {
  if (C % 8 != 0 || D < 2 || H < 2 || W < 2) return SB_ERR_SHAPE;
  const long long total = (long long)N * (D / 2) * (H / 2) * (W / 2) * (C / 8);
  maxpool2_bwd_kernel<<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)gy, (const __nv_bfloat16*)x,
                                                            (const __nv_bfloat16*)y, (__nv_bfloat16*)gx, N, D, H, W, C);
  sb_count_launch(1);
  if ((D | H | W) & 1) {
    maxpool2_bwd_tail_kernel<<<pool_grid((long long)N * D * H * W), 256, 0, stream>>>((__nv_bfloat16*)gx, N, D, H, W, C);
    sb_count_launch(1);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// Forward that also writes the index words (N * D/2 * H/2 * W/2 * C/8 of them) for sb_maxpool2_bwd_idx.
extern "C" int sb_maxpool2_fwd_idx(const void* x, void* y, void* idx, int N, int D, int H, int W, int C,
                                   cudaStream_t stream) {
  if (C % 8 != 0 || D < 2 || H < 2 || W < 2 || idx == nullptr) return SB_ERR_SHAPE;
  const long long total = (long long)N * (D / 2) * (H / 2) * (W / 2) * (C / 8);
  maxpool2_fwd_idx_kernel<<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y,
                                                                (unsigned long long*)idx, N, D, H, W, C);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// Backward from the index words: reads gy and idx only.
extern "C" int sb_maxpool2_bwd_idx(const void* gy, const void* idx, void* gx, int N, int D, int H, int W, int C,
                                   cudaStream_t stream) {
  if (C % 8 != 0 || D < 2 || H < 2 || W < 2 || idx == nullptr) return SB_ERR_SHAPE;
  const long long total = (long long)N * (D / 2) * (H / 2) * (W / 2) * (C / 8);
  maxpool2_bwd_idx_kernel<<<pool_grid(total), 256, 0, stream>>>((const __nv_bfloat16*)gy,
                                                                (const unsigned long long*)idx, (__nv_bfloat16*)gx, N,
                                                                D, H, W, C);
  sb_count_launch(1);
  if ((D | H | W) & 1) {
    maxpool2_bwd_tail_kernel<<<pool_grid((long long)N * D * H * W), 256, 0, stream>>>((__nv_bfloat16*)gx, N, D, H, W, C);
    sb_count_launch(1);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
