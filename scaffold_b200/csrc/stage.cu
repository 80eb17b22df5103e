// Input staging: a channel-major volume [N, C, S] (fp32 as the data loader delivers it, or bf16) with few
// channels becomes the voxel-major bf16 operand [N, S, 16 or 32] of the stem convolution in one pass: layout
// change, down-cast and zero padding of the channels, one 32-byte store per voxel.
//
// Role of the reference: the `.to(device, dtype, memory_format=channels_last_3d)` of a batch
// (ScaFFold/utils/trainer.py:575-583).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "host_api.h"

namespace sb {

template <typename T>
__global__ void __launch_bounds__(256) stage_input_kernel(const T* __restrict__ x, int C, long long S,
                                                          __nv_bfloat16* __restrict__ y, long long total, int cpad) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long n = i / S, v = i - n * S;
    const T* src = x + n * C * S + v;
    __align__(16) __nv_bfloat16 out[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) out[c] = c < C ? __float2bfloat16((float)src[(long long)c * S]) : __float2bfloat16(0.f);
    uint4* dst = reinterpret_cast<uint4*>(y + i * cpad);
    dst[0] = reinterpret_cast<const uint4*>(out)[0];
    dst[1] = reinterpret_cast<const uint4*>(out)[1];
    if (cpad == 32) {  // channels 16..31 are padding
      dst[2] = make_uint4(0u, 0u, 0u, 0u);
      dst[3] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

}  // namespace sb

// x: [N, C, S] contiguous, C <= 16, is_bf16 selects the element type; y: bf16 [N, S, cpad], cpad 16 or 32
extern "C" int sb_stage_input(const void* x, int is_bf16, int N, int C, long long S, void* y, int cpad,
                              cudaStream_t stream) {
  if (C < 1 || C > 16 || N < 1 || S < 1 || (cpad != 16 && cpad != 32)) return SB_ERR_SHAPE;
  const long long total = (long long)N * S;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (is_bf16)
    sb::stage_input_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, C, S, (__nv_bfloat16*)y, total, cpad);
  else
    sb::stage_input_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)x, C, S, (__nv_bfloat16*)y, total, cpad);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
