// Halo traffic of a depth-sharded volume over peer memory (NVLink P2P stores).
//
//   halo_push_kernel    copies boundary planes of this rank's activation (or of a
//                       gradient slab) straight into the NEIGHBOUR's landing buffer
//                       with 16-byte stores, then publishes an epoch in the
//                       neighbour's flag word (st.release.sys). No packing pass, no
//                       NCCL call; the consumer convolution waits on the flag only
//                       in the tiles that touch the halo.
//   halo_accum_kernel   backward: waits (bounded) for the neighbour's gradient slab
//                       and adds it into this rank's boundary plane.
//
// A depth plane of an NDHWC tensor is one contiguous run per sample, so a slab is
// N runs of H*W*C elements.
//
// Role of the reference: _exchange_forward / _exchange_backward,
// ScaFFold/unet/conv3d.py:748-841 (NCCL batch_isend_irecv + cat / add_).
#include "common.cuh"
#include "host_api.h"

namespace sb {

constexpr int HALO_MAX_COPIES = 8;
constexpr int HALO_THREADS = 256;

struct HaloCopy {
  const uint4* src;       // first plane to send (sample 0)
  uint4* dst;             // landing region in the neighbour's memory (sample 0)
  long long src_stride;   // uint4 per sample in the source tensor
  long long dst_stride;   // uint4 per sample in the landing region
  long long plane;        // uint4 per plane
  uint32_t* flag;         // neighbour's flag word to publish into (may repeat across copies)
};

struct HaloPushParams {
  HaloCopy c[HALO_MAX_COPIES];
  int ncopies, N;
  uint32_t epoch;
  uint32_t* counter;      // local scratch word: CTAs finished
};

__device__ __forceinline__ void halo_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t halo_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(HALO_THREADS) halo_push_kernel(const HaloPushParams p) {
  for (int k = 0; k < p.ncopies; ++k) {
    const HaloCopy& c = p.c[k];
    const long long total = c.plane * p.N;
    for (long long i = (long long)blockIdx.x * HALO_THREADS + threadIdx.x; i < total;
         i += (long long)gridDim.x * HALO_THREADS) {
      const long long n = i / c.plane, e = i - n * c.plane;
      c.dst[n * c.dst_stride + e] = __ldg(c.src + n * c.src_stride + e);
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ uint32_t last_s;
  if (threadIdx.x == 0) last_s = (atomicAdd(p.counter, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (last_s && threadIdx.x == 0) {
    *p.counter = 0u;
    for (int k = 0; k < p.ncopies; ++k) {
      bool seen = false;
      for (int j = 0; j < k; ++j) seen |= p.c[j].flag == p.c[k].flag;
      if (!seen) halo_st_release(p.c[k].flag, p.epoch);
    }
  }
}

struct HaloAccumParams {
  __nv_bfloat16* dst;          // boundary plane of this rank's gradient (sample 0)
  const __nv_bfloat16* slab;   // landed slab (sample 0), `slab_ld` channels per voxel
  long long dst_stride, slab_stride;  // elements per sample
  long long voxels;            // voxels per plane
  int C, slab_ld, c_off, N;
  const uint32_t* flag;
  uint32_t epoch;
  long long wait_ticks;
  uint32_t* status;
};

__global__ void __launch_bounds__(HALO_THREADS) halo_accum_kernel(const HaloAccumParams p) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    int ok = 1;
    const long long t0 = clock64();
    while ((int)(halo_ld_acquire(p.flag) - p.epoch) < 0) {
      if (clock64() - t0 > p.wait_ticks) {
        report(p.status, ST_FLAG_TIMEOUT, 51, blockIdx.x, p.epoch);
        ok = 0;
        break;
      }
      __nanosleep(64);
    }
    ok_s = ok;
  }
  __syncthreads();
  if (!ok_s) return;
  const int c8 = p.C / 8;
  const long long total = p.voxels * c8 * p.N;
  for (long long i = (long long)blockIdx.x * HALO_THREADS + threadIdx.x; i < total;
       i += (long long)gridDim.x * HALO_THREADS) {
    const long long n = i / (p.voxels * c8);
    const long long r = i - n * p.voxels * c8;
    const long long v = r / c8;
    const int o = (int)(r - v * c8) * 8;
    uint4* d = reinterpret_cast<uint4*>(p.dst + n * p.dst_stride + v * p.C + o);
    const uint4 s = *reinterpret_cast<const uint4*>(p.slab + n * p.slab_stride + v * p.slab_ld + p.c_off + o);
    uint4 a = *d;
    __nv_bfloat162* ah = reinterpret_cast<__nv_bfloat162*>(&a);
    const __nv_bfloat162* sh = reinterpret_cast<const __nv_bfloat162*>(&s);
#pragma unroll
    for (int j = 0; j < 4; ++j) ah[j] = __hadd2(ah[j], sh[j]);
    *d = a;
  }
}

}  // namespace sb

using namespace sb;

// copies: ncopies x {src, dst, src_stride_bytes, dst_stride_bytes, plane_bytes, flag} as 6 int64 each
extern "C" int sb_halo_push(const long long* copies, int ncopies, int N, unsigned epoch, uint32_t* counter,
                            cudaStream_t stream) {
  if (ncopies < 1 || ncopies > HALO_MAX_COPIES) return SB_ERR_SHAPE;
  HaloPushParams p;
  memset(&p, 0, sizeof(p));
  long long most = 0;
  for (int k = 0; k < ncopies; ++k) {
    const long long* c = copies + 6 * k;
    if ((c[0] | c[1] | c[2] | c[3] | c[4]) & 15) return SB_ERR_ALIGN;
    p.c[k].src = (const uint4*)c[0];
    p.c[k].dst = (uint4*)c[1];
    p.c[k].src_stride = c[2] / 16;
    p.c[k].dst_stride = c[3] / 16;
    p.c[k].plane = c[4] / 16;
    p.c[k].flag = (uint32_t*)c[5];
    if (p.c[k].plane * N > most) most = p.c[k].plane * N;
  }
  p.ncopies = ncopies; p.N = N; p.epoch = epoch; p.counter = counter;
  long long blocks = (most + HALO_THREADS - 1) / HALO_THREADS;
  if (blocks > 64) blocks = 64;  // a few SMs are enough for a slab; the rest keep computing
  if (blocks < 1) blocks = 1;
  halo_push_kernel<<<(unsigned)blocks, HALO_THREADS, 0, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_halo_accum(void* dst, const void* slab, long long dst_stride, long long slab_stride,
                             long long voxels, int C, int slab_ld, int c_off, int N, const uint32_t* flag,
                             unsigned epoch, double wait_seconds, uint32_t* status, cudaStream_t stream) {
  if (C % 8 || slab_ld % 8 || c_off % 8) return SB_ERR_SHAPE;
  HaloAccumParams p;
  p.dst = (__nv_bfloat16*)dst; p.slab = (const __nv_bfloat16*)slab;
  p.dst_stride = dst_stride; p.slab_stride = slab_stride; p.voxels = voxels;
  p.C = C; p.slab_ld = slab_ld; p.c_off = c_off; p.N = N;
  p.flag = flag; p.epoch = epoch; p.wait_ticks = (long long)(wait_seconds * 1.8e9); p.status = status;
  long long blocks = (voxels * (C / 8) * N + HALO_THREADS - 1) / HALO_THREADS;
  if (blocks > 64) blocks = 64;
  if (blocks < 1) blocks = 1;
  halo_accum_kernel<<<(unsigned)blocks, HALO_THREADS, 0, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
