// Column sums of a voxel-major bf16 matrix [M, C] in fp32: the bias gradient of a convolution
// (sum of the output gradient over voxels). Two deterministic stages: per-block partial sums in a
// fixed order, then one block adds the partials in block order.
//
// Role of the reference: the bias gradient autograd computes for nn.Conv3d / nn.ConvTranspose3d
// (ScaFFold/unet/unet_parts.py:118-155 uses biased transposed convolutions).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "host_api.h"

namespace sb {

constexpr int CS_THREADS = 256;

__global__ void __launch_bounds__(CS_THREADS) colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, long long M,
                                                                    int C, float* __restrict__ part) {
  __shared__ float sm[CS_THREADS * 8];
  const int tpv = C / 8;                // threads per row
  const int rpb = CS_THREADS / tpv;     // rows per block iteration
  const int oct = threadIdx.x % tpv, rl = threadIdx.x / tpv;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (rl < rpb) {
    const long long stride = (long long)gridDim.x * rpb;
    auto add = [&](const uint4 raw) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    };
    long long r = (long long)blockIdx.x * rpb + rl;
    for (; r + stride < M; r += 2 * stride) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(x + r * C + oct * 8));
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(x + (r + stride) * C + oct * 8));
      add(a);
      add(b);
    }
    for (; r < M; r += stride) add(__ldg(reinterpret_cast<const uint4*>(x + r * C + oct * 8)));
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) sm[threadIdx.x * 8 + i] = acc[i];
  __syncthreads();
  for (int ch = threadIdx.x; ch < C; ch += CS_THREADS) {
    const int o = ch / 8, j = ch % 8;
    float s = 0.f;
    for (int v = 0; v < rpb; ++v) s += sm[(v * tpv + o) * 8 + j];
    part[(long long)blockIdx.x * C + ch] = s;
  }
}

// one warp per channel: lanes take the partials b = lane, lane + 32, ... in order, then a fixed shuffle tree
__global__ void __launch_bounds__(CS_THREADS) colsum_final_kernel(const float* __restrict__ part, int nblocks, int C,
                                                                  float* __restrict__ out, int n_out) {
  const int ch = blockIdx.x * (CS_THREADS / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (ch >= n_out) return;
  float s = 0.f;
  for (int b = lane; b < nblocks; b += 32) s += part[(long long)b * C + ch];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[ch] = s;
}

}  // namespace sb

// x bf16 [M, C] (C a multiple of 8, at most 2048), out fp32 [n_out] (n_out <= C), work fp32 [sb_colsum_blocks() * C]
extern "C" int sb_colsum_blocks(void) { return 592; }
extern "C" int sb_colsum(const void* x, long long M, int C, float* out, int n_out, float* work, cudaStream_t stream) {
  if (C % 8 != 0 || C / 8 > sb::CS_THREADS || n_out > C || M <= 0) return SB_ERR_SHAPE;
  const int rpb = sb::CS_THREADS / (C / 8);
  long long want = (M + rpb - 1) / rpb;
  const int nblocks = (int)(want < 592 ? want : 592);
  sb::colsum_partial_kernel<<<nblocks, sb::CS_THREADS, 0, stream>>>((const __nv_bfloat16*)x, M, C, work);
  const int cpb = sb::CS_THREADS / 32;
  sb::colsum_final_kernel<<<(n_out + cpb - 1) / cpb, sb::CS_THREADS, 0, stream>>>(work, nblocks, C, out, n_out);
  sb_count_launch(2);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
