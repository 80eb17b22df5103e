// Peer memory over NVLink: allocation + CUDA IPC plumbing, and the fused
// gradient all-reduce that runs entirely on peer loads / stores.
//
// grad_allreduce_kernel (two-shot, deterministic):
//   phase 0  cross-GPU barrier: every rank publishes "my gradients are ready"
//            (st.release.sys of the epoch into each peer's flag row) and waits,
//            bounded, until every peer said the same;
//   phase 1  reduce-scatter by P2P LOADS: rank r sums chunk r of every peer's
//            buffer in rank order (fixed order => bitwise reproducible) and
//            writes the sum, times `scale`, into its own chunk r;
//   phase 2  all-gather by P2P STORES: rank r pushes its reduced chunk r into
//            every peer's chunk r (a region only rank r ever touches);
//   phase 3  the last CTA publishes "my pushes landed" and waits for every
//            peer's, so the next kernel on the stream sees complete data.
// No TMA, no multicast: plain 16-byte vector loads/stores through NVSwitch.
// Every wait is bounded; on expiry the kernel records the site in the status
// word, skips the dependent work and returns.
//
// Role of the reference: the DDP reducer behind DistConvDDP (ScaFFold/worker.py:81-97).
#include "common.cuh"
#include "host_api.h"

namespace sb {

constexpr int AR_MAX_RANKS = 8;
constexpr int AR_THREADS = 256;  // small CTAs co-reside with the persistent convolution CTAs when the reduction overlaps backward

struct AllReduceParams {
  float* bufs[AR_MAX_RANKS];        // every rank's gradient buffer (own entry = local pointer)
  uint32_t* flags[AR_MAX_RANKS];    // every rank's flag block: [2][AR_MAX_RANKS] epochs + [1] CTA counter
  int rank, world;
  long long offset, count;          // element range of this call inside the buffers
  uint32_t epoch;
  float scale;
  uint32_t* status;
  long long wait_ticks;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// waits until own_flags[slot][peer] >= epoch for every peer; returns false on timeout
__device__ __forceinline__ bool wait_peers(const AllReduceParams& p, int rank, int slot, uint32_t site) {
  bool ok = true;
  if (threadIdx.x < p.world) {
    const uint32_t* f = p.flags[rank] + slot * AR_MAX_RANKS + threadIdx.x;
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(f) - p.epoch) < 0) {
      if (clock64() - t0 > p.wait_ticks) {
        report(p.status, ST_FLAG_TIMEOUT, site, threadIdx.x, p.epoch);
        ok = false;
        break;
      }
      __nanosleep(64);
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// The work of one rank's grid: `bid` of `nblocks` CTAs acting as rank `rank`.
__device__ __forceinline__ void allreduce_body(const AllReduceParams& p, const int rank, const unsigned bid,
                                               const unsigned nblocks) {
  // phase 0: one CTA announces, every CTA waits on the (local) flag row
  if (bid == 0 && threadIdx.x < p.world)
    st_release_sys(p.flags[threadIdx.x] + 0 * AR_MAX_RANKS + rank, p.epoch);
  bool ok = wait_peers(p, rank, 0, 41);

  if (ok) {
    const long long per = ((p.count + p.world - 1) / p.world + 3) & ~3LL;  // chunk, multiple of 4 elements
    const long long c0 = p.offset + (long long)rank * per;
    long long c1 = c0 + per;
    if (c1 > p.offset + p.count) c1 = p.offset + p.count;
    const long long n4 = c1 > c0 ? (c1 - c0) / 4 : 0;
    const long long tail0 = c0 + n4 * 4;
    // phase 1 + 2 fused per element: sum over peers in rank order, scale, store to every rank
    // four independent 16-byte lanes per thread keep enough bytes in flight to cover the NVLink latency
    constexpr int U = 4;
    const long long stride = (long long)nblocks * AR_THREADS;
    for (long long i0 = (long long)bid * AR_THREADS + threadIdx.x; i0 < n4; i0 += stride * U) {
      float4 acc[U];
#pragma unroll
      for (int u = 0; u < U; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < AR_MAX_RANKS; ++r) {
        if (r < p.world) {
          float4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const long long i = i0 + u * stride;
            v[u] = i < n4 ? __ldcs(reinterpret_cast<const float4*>(p.bufs[r] + c0 + i * 4))
                          : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < n4) {
          float4 a = acc[u];
          a.x *= p.scale; a.y *= p.scale; a.z *= p.scale; a.w *= p.scale;
#pragma unroll
          for (int r = 0; r < AR_MAX_RANKS; ++r)
            if (r < p.world) __stcs(reinterpret_cast<float4*>(p.bufs[r] + c0 + i * 4), a);
        }
      }
    }
    if (bid == 0) {
      for (long long e = tail0 + threadIdx.x; e < c1; e += AR_THREADS) {
        float acc = 0.f;
        for (int r = 0; r < p.world; ++r) acc += p.bufs[r][e];
        acc *= p.scale;
        for (int r = 0; r < p.world; ++r) p.bufs[r][e] = acc;
      }
    }
  }
  // phase 3: the last CTA to get here tells the peers and waits for them
  __threadfence_system();
  __syncthreads();
  __shared__ uint32_t last_s;
  uint32_t* counter = p.flags[rank] + 2 * AR_MAX_RANKS;
  if (threadIdx.x == 0) last_s = (atomicAdd(counter, 1u) == nblocks - 1) ? 1u : 0u;
  __syncthreads();
  if (last_s) {
    if (threadIdx.x == 0) *counter = 0u;
    if (threadIdx.x < p.world) st_release_sys(p.flags[threadIdx.x] + 1 * AR_MAX_RANKS + rank, p.epoch);
    wait_peers(p, rank, 1, 42);
  }
}

__global__ void __launch_bounds__(AR_THREADS, 4) grad_allreduce_kernel(const AllReduceParams p) {
  allreduce_body(p, p.rank, blockIdx.x, gridDim.x);
}

// Single-GPU emulation of a `world`-rank reduction: row y of the grid acts as rank y on that rank's
// buffers and flags (all in this GPU's memory). The rows wait on one another, so the launch is
// cooperative: every CTA is resident at once or the launch is refused.
__global__ void __launch_bounds__(AR_THREADS, 4) grad_allreduce_loopback_kernel(const AllReduceParams p) {
  allreduce_body(p, (int)blockIdx.y, blockIdx.x, gridDim.x);
}

}  // namespace sb

using namespace sb;

// --- allocation / IPC ---------------------------------------------------------------------
extern "C" int sb_peer_alloc(void** out, long long bytes) {
  if (cudaMalloc(out, (size_t)bytes) != cudaSuccess) return SB_ERR_DRIVER;
  return cudaMemset(*out, 0, (size_t)bytes) == cudaSuccess ? 0 : SB_ERR_DRIVER;
}
extern "C" int sb_peer_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : SB_ERR_DRIVER; }
extern "C" int sb_peer_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }
extern "C" int sb_peer_get_handle(void* p, void* handle_out) {
  return cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle_out, p) == cudaSuccess ? 0 : SB_ERR_DRIVER;
}
extern "C" int sb_peer_open_handle(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : SB_ERR_DRIVER;
}
extern "C" int sb_peer_close_handle(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : SB_ERR_DRIVER; }

// bufs / flags: arrays of `world` device pointers valid on this GPU
extern "C" int sb_grad_allreduce(void* const* bufs, void* const* flags, int rank, int world, long long offset,
                                 long long count, unsigned epoch, float scale, int ctas, double wait_seconds,
                                 uint32_t* status, cudaStream_t stream) {
  if (world < 1 || world > AR_MAX_RANKS || (offset & 3) != 0) return SB_ERR_SHAPE;
  AllReduceParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < world; ++r) {
    p.bufs[r] = (float*)bufs[r];
    p.flags[r] = (uint32_t*)flags[r];
  }
  p.rank = rank; p.world = world; p.offset = offset; p.count = count; p.epoch = epoch; p.scale = scale;
  p.status = status;
  p.wait_ticks = (long long)(wait_seconds * 1.8e9);
  if (ctas < 1) ctas = 592;
  grad_allreduce_kernel<<<ctas, AR_THREADS, 0, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// The same protocol with all `world` ranks emulated on ONE GPU (tests, single-GPU bring-up): bufs / flags are
// `world` distinct local allocations. One cooperative launch of ctas x world CTAs.
extern "C" int sb_grad_allreduce_loopback(void* const* bufs, void* const* flags, int world, long long offset,
                                          long long count, unsigned epoch, float scale, int ctas,
                                          double wait_seconds, uint32_t* status, cudaStream_t stream) {
  if (world < 1 || world > AR_MAX_RANKS || (offset & 3) != 0) return SB_ERR_SHAPE;
  if (ctas < 1) ctas = 16;
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SB_ERR_DRIVER;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, grad_allreduce_loopback_kernel, AR_THREADS, 0) != cudaSuccess)
    return SB_ERR_DRIVER;
  if ((long long)ctas * world > (long long)sms * per_sm) return SB_ERR_TOO_LARGE;  // could not all be resident
  AllReduceParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < world; ++r) {
    p.bufs[r] = (float*)bufs[r];
    p.flags[r] = (uint32_t*)flags[r];
  }
  p.rank = 0; p.world = world; p.offset = offset; p.count = count; p.epoch = epoch; p.scale = scale;
  p.status = status;
  p.wait_ticks = (long long)(wait_seconds * 1.8e9);
  void* args[1] = {&p};
  if (cudaLaunchCooperativeKernel((const void*)grad_allreduce_loopback_kernel, dim3((unsigned)ctas, (unsigned)world),
                                  dim3(AR_THREADS), args, 0, stream) != cudaSuccess)
    return SB_ERR_LAUNCH;
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
