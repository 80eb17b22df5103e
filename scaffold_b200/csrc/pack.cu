// Weight packing for the 3x3x3 convolution kernels: one pass over the fp32 master weights
// [Cout][Cin][27] writes every bf16 operand layout the step needs.
//
//   fwd    [27][cout_pad][cin_pad]   taps in (kd,kh,kw) order          (forward, generic / plane kernels)
//   dgrad  [27][cin_pad][cout_pad]   transposed, taps flipped           (backward-data as a forward conv)
//   *_kd   the same two with taps reordered to (kh, kw, 2-kd)           (kd-fused plane kernel)
//
// Input channels may belong to two concatenated sources whose first part is zero-padded
// (real0 channels stored in pad0 slots); padding positions are never written, so the buffers are
// zeroed once by the caller and reused every step.
//
// Role of the reference: the weight re-layout that triton_conv3d's adapters do with torch ops before
// each launch (triton_conv3d/gather_gemm.py:344-420); here it is one kernel per layer (first use) or one
// kernel for the whole model (sb_pack_conv3_batch, launched by the optimizer right after the update).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "host_api.h"

namespace sb {

constexpr int PK_T = 32;  // tile of output and input channels

__device__ __forceinline__ int kd_pos(int p) {  // (kd,kh,kw) index -> (kh,kw,2-kd) index
  const int kd = p / 9, r = p - kd * 9;
  return r * 3 + (2 - kd);
}

// tap (kd,kh,kw) with two axes exchanged: 1 kd <-> kh, 2 kd <-> kw (an involution)
__device__ __forceinline__ int swap_tap(int tap, int mode) {
  if (mode == 0) return tap;
  const int kd = tap / 9, kh = (tap / 3) % 3, kw = tap % 3;
  return mode == 1 ? (kh * 9 + kd * 3 + kw) : (kw * 9 + kh * 3 + kd);
}

// Tile in shared memory as [tap][co][ci], rows padded to 34 elements so that the transposed read of the
// backward-data layouts spreads over the banks. Global reads are contiguous runs of 32 x 27 floats; global
// writes are 16-byte pieces of 64-byte rows.
constexpr int PK_LD = PK_T + 2;
constexpr int PK_PLANE = PK_T * PK_LD + 2;  // one tap's plane; the odd word count spreads taps over banks

// One 32 x 32 (output x input channel) tile of one layer; `tile` is the CTA's dynamic shared memory.
__device__ __forceinline__ void pack_tile(const SbPackArgs& a, const int bx, const int by, __nv_bfloat16* tile) {
  __nv_bfloat16* const o_fwd = (__nv_bfloat16*)a.fwd;
  __nv_bfloat16* const o_fwd_kd = (__nv_bfloat16*)a.fwd_kd;
  __nv_bfloat16* const o_dgrad = (__nv_bfloat16*)a.dgrad;
  __nv_bfloat16* const o_dgrad_kd = (__nv_bfloat16*)a.dgrad_kd;
  const int co0 = bx * PK_T, ci0 = by * PK_T;
  const int nco = min(PK_T, a.cout - co0), nci = min(PK_T, a.cin - ci0);
  const int run = nci * 27;
  if (nci == PK_T && (a.cin % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.w) & 15) == 0)) {
    // full tile: each row is 864 contiguous floats starting on a 16-byte boundary; 16-byte loads, two in flight
    constexpr int V = PK_T * 27 / 4;  // float4 per row
    for (int i = threadIdx.x; i < PK_T * V; i += 2 * blockDim.x) {
      float4 v[2];
      int rr[2], jj[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int iu = i + u * blockDim.x;
        rr[u] = iu / V;
        jj[u] = (iu - rr[u] * V) * 4;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (iu < PK_T * V && rr[u] < nco)
          v[u] = __ldg(reinterpret_cast<const float4*>(a.w + ((long long)(co0 + rr[u]) * a.cin + ci0) * 27 + jj[u]));
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (i + u * blockDim.x >= PK_T * V) continue;
        const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = jj[u] + q;
          const int ci = j / 27, tap = swap_tap(j - ci * 27, a.tap_swap);
          tile[tap * PK_PLANE + rr[u] * PK_LD + ci] = __float2bfloat16(e[q]);
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < PK_T * PK_T * 27; i += blockDim.x) {
      const int r = i / (PK_T * 27), j = i - r * (PK_T * 27);
      const int ci = j / 27, tap = swap_tap(j - ci * 27, a.tap_swap);
      float v = 0.f;
      if (r < nco && j < run) v = a.w[((long long)(co0 + r) * a.cin + ci0) * 27 + j];
      tile[tap * PK_PLANE + r * PK_LD + ci] = __float2bfloat16(v);
    }
  }
  __syncthreads();
  // Where the tile's 32 input channels land: contiguous unless the tile straddles the end of a padded source.
  const int cp0 = ci0 < a.real0 ? ci0 : ci0 - a.real0 + a.pad0;
  const bool contiguous = (ci0 >= a.real0 || ci0 + nci <= a.real0);
  const bool vec_f = contiguous && nci == PK_T && (cp0 % 8 == 0) && (a.cin_pad % 8 == 0);
  const bool vec_d = nco == PK_T && (a.cout_pad % 8 == 0);
  if (o_fwd || o_fwd_kd) {
    const long long tapsz = (long long)a.cout_pad * a.cin_pad;
    if (vec_f) {
      for (int i = threadIdx.x; i < 27 * nco * 4; i += blockDim.x) {
        const int q = i & 3, co = (i >> 2) % nco, tap = (i >> 2) / nco;
        const __nv_bfloat16* src = &tile[tap * PK_PLANE + co * PK_LD + q * 8];
        uint4 v;
        v.x = *reinterpret_cast<const uint32_t*>(src);
        v.y = *reinterpret_cast<const uint32_t*>(src + 2);
        v.z = *reinterpret_cast<const uint32_t*>(src + 4);
        v.w = *reinterpret_cast<const uint32_t*>(src + 6);
        const long long off = ((long long)(co0 + co)) * a.cin_pad + cp0 + q * 8;
        if (o_fwd) *reinterpret_cast<uint4*>(o_fwd + tap * tapsz + off) = v;
        if (o_fwd_kd) *reinterpret_cast<uint4*>(o_fwd_kd + kd_pos(tap) * tapsz + off) = v;
      }
    } else {
      for (int i = threadIdx.x; i < 27 * nco * PK_T; i += blockDim.x) {
        const int ci = i % PK_T, co = (i / PK_T) % nco, tap = i / (PK_T * nco);
        if (ci >= nci) continue;
        const int c = ci0 + ci;
        const int cp = c < a.real0 ? c : c - a.real0 + a.pad0;
        const __nv_bfloat16 v = tile[tap * PK_PLANE + co * PK_LD + ci];
        const long long off = ((long long)(co0 + co)) * a.cin_pad + cp;
        if (o_fwd) o_fwd[tap * tapsz + off] = v;
        if (o_fwd_kd) o_fwd_kd[kd_pos(tap) * tapsz + off] = v;
      }
    }
  }
  if (o_dgrad || o_dgrad_kd) {
    const long long tapsz = (long long)a.cin_pad * a.cout_pad;
    if (vec_d) {
      for (int i = threadIdx.x; i < 27 * nci * 4; i += blockDim.x) {
        const int q = i & 3, ci = (i >> 2) % nci, tap = (i >> 2) / nci;
        const int c = ci0 + ci;
        const int cp = c < a.real0 ? c : c - a.real0 + a.pad0;
        __nv_bfloat16 e[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) e[k] = tile[tap * PK_PLANE + (q * 8 + k) * PK_LD + ci];
        uint4 v;
        v.x = (uint32_t)__bfloat16_as_ushort(e[0]) | ((uint32_t)__bfloat16_as_ushort(e[1]) << 16);
        v.y = (uint32_t)__bfloat16_as_ushort(e[2]) | ((uint32_t)__bfloat16_as_ushort(e[3]) << 16);
        v.z = (uint32_t)__bfloat16_as_ushort(e[4]) | ((uint32_t)__bfloat16_as_ushort(e[5]) << 16);
        v.w = (uint32_t)__bfloat16_as_ushort(e[6]) | ((uint32_t)__bfloat16_as_ushort(e[7]) << 16);
        const long long off = (long long)cp * a.cout_pad + co0 + q * 8;
        const int p = 26 - tap;
        if (o_dgrad) *reinterpret_cast<uint4*>(o_dgrad + p * tapsz + off) = v;
        if (o_dgrad_kd) *reinterpret_cast<uint4*>(o_dgrad_kd + kd_pos(p) * tapsz + off) = v;
      }
    } else {
      for (int i = threadIdx.x; i < 27 * nci * PK_T; i += blockDim.x) {
        const int co = i % PK_T, ci = (i / PK_T) % nci, tap = i / (PK_T * nci);
        if (co >= nco) continue;
        const int c = ci0 + ci;
        const int cp = c < a.real0 ? c : c - a.real0 + a.pad0;
        const __nv_bfloat16 v = tile[tap * PK_PLANE + co * PK_LD + ci];
        const long long off = (long long)cp * a.cout_pad + (co0 + co);
        const int p = 26 - tap;
        if (o_dgrad) o_dgrad[p * tapsz + off] = v;
        if (o_dgrad_kd) o_dgrad_kd[kd_pos(p) * tapsz + off] = v;
      }
    }
  }
}

__global__ void __launch_bounds__(256) pack_conv3_kernel(SbPackArgs a) {
  extern __shared__ __nv_bfloat16 tile[];  // [27] planes of [PK_T][PK_LD]
  pack_tile(a, blockIdx.x, blockIdx.y, tile);
}

// All layers of a model in one launch: block b belongs to the job with tile0 <= b < tile0 + tiles.
__global__ void __launch_bounds__(256) pack_conv3_batch_kernel(const SbPackJob* __restrict__ jobs, int njobs) {
  extern __shared__ __nv_bfloat16 tile[];
  __shared__ int job_s;
  if (threadIdx.x == 0) {
    int j = 0;
    while (j + 1 < njobs && (int)blockIdx.x >= jobs[j + 1].tile0) ++j;
    job_s = j;
  }
  __syncthreads();
  const SbPackJob& jb = jobs[job_s];
  const int t = blockIdx.x - jb.tile0;
  pack_tile(jb.a, t % jb.tiles_x, t / jb.tiles_x, tile);
}

}  // namespace sb

static int pack_configure(int smem) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sb::pack_conv3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaFuncSetAttribute(sb::pack_conv3_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return SB_ERR_DRIVER;
    configured = true;
  }
  return 0;
}

static bool pack_args_ok(const SbPackArgs* a) {
  return !(a->cout <= 0 || a->cin <= 0 || a->real0 > a->pad0 || a->cin - a->real0 + a->pad0 > a->cin_pad ||
           a->cout > a->cout_pad || a->tap_swap < 0 || a->tap_swap > 2);
}

// Fills tile0 / tiles_x of `njobs` host-side jobs (validating each) and returns the total tile count, or -1.
extern "C" long long sb_pack_conv3_plan(SbPackJob* jobs, int njobs) {
  long long total = 0;
  for (int j = 0; j < njobs; ++j) {
    if (!pack_args_ok(&jobs[j].a)) return -1;
    jobs[j].tile0 = (int)total;
    jobs[j].tiles_x = (jobs[j].a.cout + sb::PK_T - 1) / sb::PK_T;
    total += (long long)jobs[j].tiles_x * ((jobs[j].a.cin + sb::PK_T - 1) / sb::PK_T);
    if (total > 0x7fffffffLL) return -1;
  }
  return total;
}

// dev_jobs: the planned job table copied to device memory by the caller (it stays valid while buffers persist).
extern "C" int sb_pack_conv3_batch(const SbPackJob* dev_jobs, int njobs, long long total_tiles, cudaStream_t stream) {
  const int smem = 27 * sb::PK_PLANE * (int)sizeof(__nv_bfloat16);
  int rc = pack_configure(smem);
  if (rc) return rc;
  if (njobs < 1 || total_tiles < 1 || dev_jobs == nullptr) return SB_ERR_SHAPE;
  sb::pack_conv3_batch_kernel<<<(unsigned)total_tiles, 256, smem, stream>>>(dev_jobs, njobs);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_pack_conv3(const SbPackArgs* a, cudaStream_t stream) {
  const int smem = 27 * sb::PK_PLANE * (int)sizeof(__nv_bfloat16);
  int rc = pack_configure(smem);
  if (rc) return rc;
  if (!pack_args_ok(a)) return SB_ERR_SHAPE;
  dim3 grid((a->cout + sb::PK_T - 1) / sb::PK_T, (a->cin + sb::PK_T - 1) / sb::PK_T);
  sb::pack_conv3_kernel<<<grid, 256, smem, stream>>>(*a);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
