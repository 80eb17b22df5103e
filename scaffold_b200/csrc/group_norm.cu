// GroupNorm (+ fused ReLU) for channels-last bf16 activations, forward and
// backward, with statistics that can span several spatial shards.
//
// Forward, two streaming passes (3 tensor-volumes of traffic):
//   gn_stats_kernel     per (split, n) CTA: Welford-style (count, mean, M2)
//                       partials for all G groups over a contiguous voxel range
//   gn_apply_kernel     every CTA merges the partials of its sample in index
//                       order (Chan's formula; deterministic), then
//                       y = relu((x - mean) * rstd * w + b), stored in bf16
// Backward, two streaming passes (5 volumes):
//   gn_bwd_partial      per (split, n): per-channel sum(dy') and sum(dy' * xhat),
//                       dy' = dy gated by the recomputed ReLU mask
//   gn_bwd_dx           merges partials, dx = rstd * (dy' w - c1 - xhat c2);
//                       CTA (0,0) also reduces dweight / dbias over samples
//
// "Peer" partial blocks: both merge steps walk `n_parts` partial buffers (this
// rank's first, then its spatial neighbours' through peer pointers), which
// makes a sharded volume normalise exactly like the unsharded one.
//
// Every thread owns 8 consecutive channels (one 16-byte vector) of a voxel, so
// all global accesses are full coalesced 16-byte vectors.
//
// Role of the reference: ScaFFold/unet/triton_group_norm.py:594-1043.
#include <atomic>

#include "common.cuh"
#include "host_api.h"

namespace sb {

constexpr int GN_THREADS = 256;
constexpr int GN_MAX_PARTS = 8;

struct GnParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* dy;
  __nv_bfloat16* y;   // forward output / backward dx
  const float* w;
  const float* b;
  float* mean;   // [N, G]
  float* rstd;   // [N, G]
  float* part;   // this rank's partials
  float* fin;    // optional: the last block of a statistics / backward-sums launch also collapses the partials here
  unsigned int* ticket;  // block counter of that hand-over (zero before the launch, reset by the last block)
  const float* parts[GN_MAX_PARTS];  // partial buffers to merge (own first)
  int n_parts;
  float* dw;     // [C]
  float* db;     // [C]
  int N, C, G;
  long long S;   // voxels per sample (local shard)
  int nsplit;
  float eps;
  int relu;
  float group_elems;  // elements per (n, g) over ALL shards = S_total * C/G
  const uint32_t* wait_flags;  // optional: peers' "statistics landed" flags (local memory)
  uint32_t wait_epoch;
  long long wait_ticks;
  uint32_t* status;
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  return o;
}

__device__ __forceinline__ void chan_merge(float& n_a, float& mean_a, float& m2_a, float n_b, float mean_b,
                                           float m2_b) {
  if (n_b == 0.f) return;
  const float n = n_a + n_b;
  const float delta = mean_b - mean_a;
  const float r = n_b / n;
  mean_a += delta * r;
  m2_a += m2_b + delta * delta * n_a * r;
  n_a = n;
}


// One warp collapses the `nsplit` partials of (n, g) with a fixed merge tree (lane-strided, then xor
// shuffles merging the lower lane first): the separate finalize kernel and the last-block tail of the
// statistics kernel run exactly this, so both give the same bits. Loads bypass L1 (the partials may
// have been written by other SMs during this launch).
__device__ __forceinline__ void stats_collapse_warp(const float* __restrict__ part, float* __restrict__ fin, int G,
                                                    int nsplit, int n, int g, int lane) {
  float gn = 0.f, gm = 0.f, g2 = 0.f;
  for (int s = lane; s < nsplit; s += 32) {
    const float* e = part + (((long long)n * nsplit + s) * G + g) * 3;
    chan_merge(gn, gm, g2, __ldcg(e), __ldcg(e + 1), __ldcg(e + 2));
  }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float on = __shfl_xor_sync(0xffffffffu, gn, o);
    const float om = __shfl_xor_sync(0xffffffffu, gm, o);
    const float o2 = __shfl_xor_sync(0xffffffffu, g2, o);
    // merge (lower lane, higher lane) in that order on both sides: bitwise identical results
    if (lane & o) {
      float an = on, am = om, a2 = o2;
      chan_merge(an, am, a2, gn, gm, g2);
      gn = an; gm = am; g2 = a2;
    } else {
      chan_merge(gn, gm, g2, on, om, o2);
    }
  }
  if (lane == 0) {
    float* dst = fin + ((long long)n * G + g) * 3;
    dst[0] = gn; dst[1] = gm; dst[2] = g2;
  }
}

__device__ __forceinline__ void bwd_collapse_warp(const float* __restrict__ part, float* __restrict__ fin, int C,
                                                  int nsplit, int n, int c, int lane) {
  float a = 0.f, b = 0.f;
  for (int s = lane; s < nsplit; s += 32) {
    const float2 e = __ldcg(reinterpret_cast<const float2*>(part + (((long long)n * nsplit + s) * C + c) * 2));
    a += e.x;
    b += e.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  if (lane == 0) {
    float* dst = fin + ((long long)n * C + c) * 2;
    dst[0] = a; dst[1] = b;
  }
}

// True in every thread of the block that finished last (all blocks' global writes are then visible to it).
__device__ __forceinline__ bool last_block_done(unsigned int* ticket) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int total = gridDim.x * gridDim.y;
    s_last = atomicAdd(ticket, 1u) == total - 1u ? 1 : 0;
  }
  __syncthreads();
  if (s_last) __threadfence();
  return s_last != 0;
}

// ----------------------------------------------------------------------------
// forward: statistics
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(GN_THREADS) gn_stats_kernel(const GnParams p) {
  __shared__ float s_n[GN_THREADS * 4], s_mean[GN_THREADS * 4], s_m2[GN_THREADS * 4];
  const int split = blockIdx.x, n = blockIdx.y;
  const int tpv = p.C / 8;            // threads per voxel
  const int vpb = GN_THREADS / tpv;   // voxels per block iteration
  const int oct = threadIdx.x % tpv;
  const int vl = threadIdx.x / tpv;
  const int cg = p.C / p.G;
  const long long chunk = (p.S + p.nsplit - 1) / p.nsplit;
  const long long v0 = (long long)split * chunk;
  const long long v1 = v0 + chunk < p.S ? v0 + chunk : p.S;
  const __nv_bfloat16* xb = p.x + (long long)n * p.S * p.C + oct * 8;

  float s[8], q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { s[i] = 0.f; q[i] = 0.f; }
  float cnt = 0.f;
  // first value of the thread is the shift: sums of (x - shift) stay small
  float shift[8];
  bool have_shift = false;
  if (vl < vpb) {
    auto body = [&](const uint4 raw) {
      float f[8];
      unpack8(raw, f);
      if (!have_shift) {
#pragma unroll
        for (int i = 0; i < 8; ++i) shift[i] = f[i];
        have_shift = true;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = f[i] - shift[i];
        s[i] += d;
        q[i] += d * d;
      }
      cnt += 1.f;
    };
    for (long long v = v0 + vl; v < v1; v += vpb) body(__ldg(reinterpret_cast<const uint4*>(xb + v * p.C)));
  }
  // per-thread (count, mean, M2) for each group it touches (ngt = max(1, 8/cg) groups)
  const int ngt = cg >= 8 ? 1 : 8 / cg;
  const int cpg = 8 / ngt;  // channels of this thread per group
  for (int gi = 0; gi < ngt; ++gi) {
    float gn = 0.f, gm = 0.f, g2 = 0.f;
    if (cnt > 0.f) {
      for (int j = 0; j < cpg; ++j) {
        const int i = gi * cpg + j;
        const float m = s[i] / cnt;
        const float m2 = fmaxf(q[i] - s[i] * m, 0.f);
        chan_merge(gn, gm, g2, cnt, m + shift[i], m2);
      }
    }
    s_n[threadIdx.x * 4 + gi] = gn;
    s_mean[threadIdx.x * 4 + gi] = gm;
    s_m2[threadIdx.x * 4 + gi] = g2;
  }
  __syncthreads();
  // one thread per group merges that group's entries in thread order
  if (threadIdx.x < p.G) {
    const int g = threadIdx.x;
    float gn = 0.f, gm = 0.f, g2 = 0.f;
    // channels of group g: [g*cg, (g+1)*cg) -> octs [g*cg/8, ...]
    const int oct0 = (g * cg) / 8;
    const int octs = cg >= 8 ? cg / 8 : 1;
    const int gi = cg >= 8 ? 0 : (g * cg % 8) / cg;
    for (int v = 0; v < vpb; ++v)
      for (int o = 0; o < octs; ++o) {
        const int t = v * tpv + oct0 + o;
        chan_merge(gn, gm, g2, s_n[t * 4 + gi], s_mean[t * 4 + gi], s_m2[t * 4 + gi]);
      }
    float* dst = p.part + (((long long)n * p.nsplit + split) * p.G + g) * 3;
    dst[0] = gn;
    dst[1] = gm;
    dst[2] = g2;
  }
  if (p.fin != nullptr && last_block_done(p.ticket)) {
    // the last block to finish collapses every (n, g): no separate finalize launch
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int o = warp; o < p.N * p.G; o += GN_THREADS / 32)
      stats_collapse_warp(p.part, p.fin, p.G, p.nsplit, o / p.G, o % p.G, lane);
    if (threadIdx.x == 0) *p.ticket = 0u;
  }
}

// Bounded wait until every peer's statistics landed; returns false (after reporting) on timeout.
__device__ __forceinline__ bool gn_wait_peers(const GnParams& p, uint32_t site) {
  if (p.wait_flags == nullptr) return true;
  int ok = 1;
  if (threadIdx.x < p.n_parts) {
    const long long t0 = clock64();
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.wait_flags + threadIdx.x) : "memory");
      if ((int)(v - p.wait_epoch) >= 0) break;
      if (clock64() - t0 > p.wait_ticks) {
        report(p.status, ST_FLAG_TIMEOUT, site, threadIdx.x, p.wait_epoch);
        ok = 0;
        break;
      }
      __nanosleep(32);
    }
  }
  return __syncthreads_and(ok) != 0;
}

// merges every partial of sample n, group g, in (part buffer, split) order
__device__ __forceinline__ void merge_group(const GnParams& p, int n, int g, float& mean, float& rstd) {
  float gn = 0.f, gm = 0.f, g2 = 0.f;
  for (int pi = 0; pi < p.n_parts; ++pi) {
    const float* base = p.parts[pi] + ((long long)n * p.nsplit * p.G + g) * 3;
    for (int s = 0; s < p.nsplit; ++s) {
      const float* e = base + (long long)s * p.G * 3;
      chan_merge(gn, gm, g2, e[0], e[1], e[2]);
    }
  }
  mean = gm;
  rstd = rsqrtf(g2 / gn + p.eps);
}

// ----------------------------------------------------------------------------
// forward: normalise + affine + ReLU
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(GN_THREADS) gn_apply_kernel(const GnParams p) {
  __shared__ float s_mean[256], s_rstd[256];
  const int n = blockIdx.y;
  if (!gn_wait_peers(p, 61)) return;
  for (int g = threadIdx.x; g < p.G; g += GN_THREADS) {
    float m, r;
    merge_group(p, n, g, m, r);
    s_mean[g] = m;
    s_rstd[g] = r;
    if (blockIdx.x == 0) {
      p.mean[n * p.G + g] = m;
      p.rstd[n * p.G + g] = r;
    }
  }
  __syncthreads();
  const int tpv = p.C / 8;
  const int vpb = GN_THREADS / tpv;
  const int oct = threadIdx.x % tpv;
  const int vl = threadIdx.x / tpv;
  if (vl >= vpb) return;
  const int cg = p.C / p.G;
  float a[8], c[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int ch = oct * 8 + i;
    const int g = ch / cg;
    a[i] = s_rstd[g] * p.w[ch];
    c[i] = p.b[ch] - s_mean[g] * a[i];
  }
  const long long base = (long long)n * p.S * p.C + oct * 8;
  auto body = [&](const uint4 raw, long long v) {
    float f[8];
    unpack8(raw, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float yv = fmaf(f[i], a[i], c[i]);
      if (p.relu) yv = yv <= 0.f ? 0.f : yv;  // NaN propagates
      f[i] = yv;
    }
    *reinterpret_cast<uint4*>(p.y + base + v * p.C) = pack8(f);
  };
  // four voxels (four 16-byte loads) in flight per thread
  const long long stride = (long long)gridDim.x * vpb;
  long long v = (long long)blockIdx.x * vpb + vl;
  for (; v + 3 * stride < p.S; v += 4 * stride) {
    uint4 r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) r[u] = __ldg(reinterpret_cast<const uint4*>(p.x + base + (v + u * stride) * p.C));
#pragma unroll
    for (int u = 0; u < 4; ++u) body(r[u], v + u * stride);
  }
  for (; v < p.S; v += stride) body(__ldg(reinterpret_cast<const uint4*>(p.x + base + v * p.C)), v);
}

// ----------------------------------------------------------------------------
// backward: per-channel partial sums
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(GN_THREADS) gn_bwd_partial_kernel(const GnParams p) {
  __shared__ float s_a[GN_THREADS * 8], s_b[GN_THREADS * 8];
  const int split = blockIdx.x, n = blockIdx.y;
  const int tpv = p.C / 8;
  const int vpb = GN_THREADS / tpv;
  const int oct = threadIdx.x % tpv;
  const int vl = threadIdx.x / tpv;
  const int cg = p.C / p.G;
  const long long chunk = (p.S + p.nsplit - 1) / p.nsplit;
  const long long v0 = (long long)split * chunk;
  const long long v1 = v0 + chunk < p.S ? v0 + chunk : p.S;
  float mu[8], rs[8], wv[8], bv[8], A[8], B[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int ch = oct * 8 + i;
    const int g = ch / cg;
    mu[i] = p.mean[n * p.G + g];
    rs[i] = p.rstd[n * p.G + g];
    wv[i] = p.w[ch];
    bv[i] = p.b[ch];
    A[i] = 0.f;
    B[i] = 0.f;
  }
  const long long base = (long long)n * p.S * p.C + oct * 8;
  if (vl < vpb) {
    auto body = [&](const uint4 rx, const uint4 rd) {
      float fx[8], fd[8];
      unpack8(rx, fx);
      unpack8(rd, fd);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = (fx[i] - mu[i]) * rs[i];
        float d = fd[i];
        if (p.relu && fmaf(xh, wv[i], bv[i]) <= 0.f) d = 0.f;
        A[i] += d;
        B[i] += d * xh;
      }
    };
    // two voxels (four 16-byte loads) in flight per thread; the summation order per thread is unchanged
    long long v = v0 + vl;
    for (; v + vpb < v1; v += 2 * vpb) {
      const uint4 rx0 = __ldg(reinterpret_cast<const uint4*>(p.x + base + v * p.C));
      const uint4 rd0 = __ldg(reinterpret_cast<const uint4*>(p.dy + base + v * p.C));
      const uint4 rx1 = __ldg(reinterpret_cast<const uint4*>(p.x + base + (v + vpb) * p.C));
      const uint4 rd1 = __ldg(reinterpret_cast<const uint4*>(p.dy + base + (v + vpb) * p.C));
      body(rx0, rd0);
      body(rx1, rd1);
    }
    for (; v < v1; v += vpb)
      body(__ldg(reinterpret_cast<const uint4*>(p.x + base + v * p.C)),
           __ldg(reinterpret_cast<const uint4*>(p.dy + base + v * p.C)));
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s_a[threadIdx.x * 8 + i] = A[i];
    s_b[threadIdx.x * 8 + i] = B[i];
  }
  __syncthreads();
  for (int ch = threadIdx.x; ch < p.C; ch += GN_THREADS) {
    const int o = ch / 8, j = ch % 8;
    float sa = 0.f, sbv = 0.f;
    for (int v = 0; v < vpb; ++v) {
      const int t = v * tpv + o;
      sa += s_a[t * 8 + j];
      sbv += s_b[t * 8 + j];
    }
    float* dst = p.part + (((long long)n * p.nsplit + split) * p.C + ch) * 2;
    dst[0] = sa;
    dst[1] = sbv;
  }
  if (p.fin != nullptr && last_block_done(p.ticket)) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int o = warp; o < p.N * p.C; o += GN_THREADS / 32)
      bwd_collapse_warp(p.part, p.fin, p.C, p.nsplit, o / p.C, o % p.C, lane);
    if (threadIdx.x == 0) *p.ticket = 0u;
  }
}

// ----------------------------------------------------------------------------
// backward: dx (+ dweight / dbias)
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(GN_THREADS) gn_bwd_dx_kernel(const GnParams p) {
  extern __shared__ float sm[];
  float* s_A = sm;              // [C] this rank's sum(dy')
  float* s_B = sm + p.C;        // [C] this rank's sum(dy' xhat)
  float* s_c1 = sm + 2 * p.C;   // [G]
  float* s_c2 = s_c1 + p.G;     // [G]
  float* s_At = s_c2 + p.G;     // [C] all shards
  float* s_Bt = s_At + p.C;
  const int n = blockIdx.y;
  const int cg = p.C / p.G;
  if (!gn_wait_peers(p, 62)) return;
  for (int ch = threadIdx.x; ch < p.C; ch += GN_THREADS) {
    float At = 0.f, Bt = 0.f, A0 = 0.f, B0 = 0.f;
    for (int pi = 0; pi < p.n_parts; ++pi) {
      const float* base = p.parts[pi] + ((long long)n * p.nsplit * p.C + ch) * 2;
      float a = 0.f, b = 0.f;
      for (int s = 0; s < p.nsplit; ++s) {
        a += base[(long long)s * p.C * 2];
        b += base[(long long)s * p.C * 2 + 1];
      }
      if (pi == 0) { A0 = a; B0 = b; }
      At += a;
      Bt += b;
    }
    s_A[ch] = A0; s_B[ch] = B0; s_At[ch] = At; s_Bt[ch] = Bt;
  }
  __syncthreads();
  for (int g = threadIdx.x; g < p.G; g += GN_THREADS) {
    float c1 = 0.f, c2 = 0.f;
    for (int j = 0; j < cg; ++j) {
      const int ch = g * cg + j;
      c1 += p.w[ch] * s_At[ch];
      c2 += p.w[ch] * s_Bt[ch];
    }
    s_c1[g] = c1 / p.group_elems;
    s_c2[g] = c2 / p.group_elems;
  }
  __syncthreads();
  // dweight / dbias: this rank's share, summed over samples in index order
  if (blockIdx.x == 0 && blockIdx.y == 0 && p.dw != nullptr) {
    for (int ch = threadIdx.x; ch < p.C; ch += GN_THREADS) {
      float a = 0.f, b = 0.f;
      for (int nn = 0; nn < p.N; ++nn) {
        const float* base = p.parts[0] + ((long long)nn * p.nsplit * p.C + ch) * 2;
        for (int s = 0; s < p.nsplit; ++s) {
          a += base[(long long)s * p.C * 2];
          b += base[(long long)s * p.C * 2 + 1];
        }
      }
      p.db[ch] = a;
      p.dw[ch] = b;
    }
  }
  const int tpv = p.C / 8;
  const int vpb = GN_THREADS / tpv;
  const int oct = threadIdx.x % tpv;
  const int vl = threadIdx.x / tpv;
  if (vl >= vpb) return;
  float mu[8], rs[8], wv[8], bv[8], c1[8], c2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int ch = oct * 8 + i;
    const int g = ch / cg;
    mu[i] = p.mean[n * p.G + g];
    rs[i] = p.rstd[n * p.G + g];
    wv[i] = p.w[ch];
    bv[i] = p.b[ch];
    c1[i] = s_c1[g];
    c2[i] = s_c2[g];
  }
  const long long base = (long long)n * p.S * p.C + oct * 8;
  auto body = [&](const uint4 rx, const uint4 rd, long long v) {
    float fx[8], fd[8];
    unpack8(rx, fx);
    unpack8(rd, fd);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float xh = (fx[i] - mu[i]) * rs[i];
      float d = fd[i];
      if (p.relu && fmaf(xh, wv[i], bv[i]) <= 0.f) d = 0.f;
      fx[i] = rs[i] * (d * wv[i] - c1[i] - xh * c2[i]);
    }
    *reinterpret_cast<uint4*>(p.y + base + v * p.C) = pack8(fx);
  };
  // two voxels (four 16-byte loads) in flight per thread
  const long long stride = (long long)gridDim.x * vpb;
  long long v = (long long)blockIdx.x * vpb + vl;
  for (; v + stride < p.S; v += 2 * stride) {
    const uint4 rx0 = __ldg(reinterpret_cast<const uint4*>(p.x + base + v * p.C));
    const uint4 rd0 = __ldg(reinterpret_cast<const uint4*>(p.dy + base + v * p.C));
    const uint4 rx1 = __ldg(reinterpret_cast<const uint4*>(p.x + base + (v + stride) * p.C));
    const uint4 rd1 = __ldg(reinterpret_cast<const uint4*>(p.dy + base + (v + stride) * p.C));
    body(rx0, rd0, v);
    body(rx1, rd1, v + stride);
  }
  for (; v < p.S; v += stride)
    body(__ldg(reinterpret_cast<const uint4*>(p.x + base + v * p.C)),
         __ldg(reinterpret_cast<const uint4*>(p.dy + base + v * p.C)), v);
}

// ----------------------------------------------------------------------------
// finalize: collapse the per-split partials of one rank into a single entry per
// (n, g) / (n, c), in parallel (one warp per output, fixed merge tree), so the
// streaming kernels start from O(1) statistics instead of walking every split.
// ----------------------------------------------------------------------------
__global__ void __launch_bounds__(GN_THREADS) gn_stats_finalize_kernel(const float* __restrict__ part,
                                                                       float* __restrict__ fin, int N, int G,
                                                                       int nsplit) {
  const int warp = (blockIdx.x * GN_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= N * G) return;
  stats_collapse_warp(part, fin, G, nsplit, warp / G, warp % G, lane);
}

// The same collapse for MANY partials per (n, g) (the per-warp partials a convolution's epilogue leaves: up to
// 16K per sample): one block per (n, g); thread t merges partials t, t + 256, ... in order, then a fixed
// shared-memory tree merges the 256 results (lower index first), so the result is deterministic.
__global__ void __launch_bounds__(GN_THREADS) gn_stats_finalize_wide_kernel(const float* __restrict__ part,
                                                                            float* __restrict__ fin, int N, int G,
                                                                            int nsplit) {
  __shared__ float s_n[GN_THREADS], s_m[GN_THREADS], s_2[GN_THREADS];
  const int n = blockIdx.x / G, g = blockIdx.x % G;
  float gn = 0.f, gm = 0.f, g2 = 0.f;
  const float* base = part + ((long long)n * nsplit * G + g) * 3;
  int s = threadIdx.x;
  // four independent loads in flight per thread; merged in index order
  for (; s + 3 * GN_THREADS < nsplit; s += 4 * GN_THREADS) {
    float e[4][3];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float* q = base + (long long)(s + u * GN_THREADS) * G * 3;
      e[u][0] = q[0]; e[u][1] = q[1]; e[u][2] = q[2];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) chan_merge(gn, gm, g2, e[u][0], e[u][1], e[u][2]);
  }
  for (; s < nsplit; s += GN_THREADS) {
    const float* q = base + (long long)s * G * 3;
    chan_merge(gn, gm, g2, q[0], q[1], q[2]);
  }
  s_n[threadIdx.x] = gn; s_m[threadIdx.x] = gm; s_2[threadIdx.x] = g2;
  __syncthreads();
  for (int o = GN_THREADS / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      float an = s_n[threadIdx.x], am = s_m[threadIdx.x], a2 = s_2[threadIdx.x];
      chan_merge(an, am, a2, s_n[threadIdx.x + o], s_m[threadIdx.x + o], s_2[threadIdx.x + o]);
      s_n[threadIdx.x] = an; s_m[threadIdx.x] = am; s_2[threadIdx.x] = a2;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    float* dst = fin + ((long long)n * G + g) * 3;
    dst[0] = s_n[0]; dst[1] = s_m[0]; dst[2] = s_2[0];
  }
}

__global__ void __launch_bounds__(GN_THREADS) gn_bwd_finalize_kernel(const float* __restrict__ part,
                                                                     float* __restrict__ fin, int N, int C,
                                                                     int nsplit) {
  const int warp = (blockIdx.x * GN_THREADS + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= N * C) return;
  bwd_collapse_warp(part, fin, C, nsplit, warp / C, warp % C, lane);
}

// Channel / group counts the kernels cover: C a multiple of 8 in [8, 2048] (one thread per channel
// octet, at most GN_THREADS octets), G dividing C, and a group either a whole number of octets or a
// divisor of one octet holding at most four groups.
static bool gn_channels_ok(int C, int G) {
  if (C < 8 || C % 8 != 0 || C > 8 * GN_THREADS || G < 1 || G > 256 || C % G != 0) return false;
  const int cg = C / G;
  if (cg < 8 ? (8 % cg != 0) : (cg % 8 != 0)) return false;
  return !(cg < 8 && 8 / cg > 4);
}

static int gn_fill(const SbGnArgs* a, GnParams& p) {
  if (!gn_channels_ok(a->C, a->G) || a->N < 1 || a->S < 1) return SB_ERR_SHAPE;
  if (a->x == nullptr || a->w == nullptr || a->b == nullptr) return SB_ERR_SHAPE;
  const int cg = a->C / a->G;
  if (a->n_parts < 1 || a->n_parts > GN_MAX_PARTS) return SB_ERR_SHAPE;
  memset(&p, 0, sizeof(p));
  p.x = (const __nv_bfloat16*)a->x;
  p.dy = (const __nv_bfloat16*)a->dy;
  p.y = (__nv_bfloat16*)a->y;
  p.w = a->w; p.b = a->b; p.mean = a->mean; p.rstd = a->rstd;
  p.part = a->part;
  p.fin = a->fin;
  for (int i = 0; i < a->n_parts; ++i) p.parts[i] = a->parts[i];
  p.n_parts = a->n_parts;
  p.dw = a->dw; p.db = a->db;
  p.N = a->N; p.C = a->C; p.G = a->G; p.S = a->S;
  p.nsplit = a->nsplit;
  p.eps = a->eps;
  p.relu = a->relu;
  p.group_elems = (float)((double)a->S_total * cg);
  p.wait_flags = a->wait_flags;
  p.wait_epoch = a->wait_epoch;
  p.wait_ticks = (long long)((a->wait_s > 0 ? a->wait_s : 2.0) * 1.8e9);
  p.status = a->status;
  return 0;
}

// Block counters of the fused finalize: launches on one stream run one after another and each leaves its counter
// at zero, so a small rotating pool is plenty. The NAME is only a handle for cudaGetSymbolAddress in host code.
static __device__ unsigned int g_gn_tickets[256];
constexpr int GN_TICKET_DEVICES = 64;
static unsigned int* g_gn_ticket_ptr[GN_TICKET_DEVICES] = {nullptr};
static std::atomic<unsigned int> g_gn_ticket_seq{0};
static unsigned int* gn_ticket() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= GN_TICKET_DEVICES) return nullptr;
  if (g_gn_ticket_ptr[dev] == nullptr) {
    unsigned int* q = nullptr;
    if (cudaGetSymbolAddress((void**)&q, g_gn_tickets) != cudaSuccess || q == nullptr) return nullptr;
    g_gn_ticket_ptr[dev] = q;
  }
  return g_gn_ticket_ptr[dev] + (g_gn_ticket_seq.fetch_add(1u) % 256u);
}

static int apply_blocks(const GnParams& p) {
  const int vpb = GN_THREADS / (p.C / 8);
  long long need = (p.S + vpb - 1) / vpb;
  long long cap = (148LL * 8 + p.N - 1) / p.N;
  long long b = need < cap ? need : cap;
  return (int)(b < 1 ? 1 : b);
}

}  // namespace sb

using namespace sb;

// 1 when the kernels cover GroupNorm over C channels in G groups, else 0 (callers then take another path)
extern "C" int sb_gn_supported(int C, int G) { return gn_channels_ok(C, G) ? 1 : 0; }

extern "C" int sb_gn_nsplit(int N, long long S, int C) {
  if (N < 1 || S < 1 || C < 8 || C / 8 > GN_THREADS) return 1;  // unsupported shapes are refused by the launchers
  const int vpb = GN_THREADS / (C / 8);
  long long maxs = (S + vpb - 1) / vpb;  // at least one row of voxels per split
  long long want = (148LL * 4 + N - 1) / N;
  long long s = want < maxs ? want : maxs;
  if (s > 1024) s = 1024;
  return (int)(s < 1 ? 1 : s);
}

extern "C" int sb_gn_stats(const SbGnArgs* a, cudaStream_t stream) {
  GnParams p;
  int rc = gn_fill(a, p);
  if (rc) return rc;
  if (p.fin != nullptr && (p.ticket = gn_ticket()) == nullptr) return SB_ERR_DRIVER;
  gn_stats_kernel<<<dim3(p.nsplit, p.N), GN_THREADS, 0, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_gn_apply(const SbGnArgs* a, cudaStream_t stream) {
  GnParams p;
  int rc = gn_fill(a, p);
  if (rc) return rc;
  gn_apply_kernel<<<dim3(apply_blocks(p), p.N), GN_THREADS, 0, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_gn_bwd_partial(const SbGnArgs* a, cudaStream_t stream) {
  GnParams p;
  int rc = gn_fill(a, p);
  if (rc) return rc;
  if (p.fin != nullptr && (p.ticket = gn_ticket()) == nullptr) return SB_ERR_DRIVER;
  gn_bwd_partial_kernel<<<dim3(p.nsplit, p.N), GN_THREADS, 0, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_gn_bwd_dx(const SbGnArgs* a, cudaStream_t stream) {
  GnParams p;
  int rc = gn_fill(a, p);
  if (rc) return rc;
  const size_t smem = (size_t)(4 * p.C + 2 * p.G) * sizeof(float);
  gn_bwd_dx_kernel<<<dim3(apply_blocks(p), p.N), GN_THREADS, smem, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}


namespace sb {
struct ShareParams {
  const float* fin;
  long long count;
  float* dst[8];
  uint32_t* flags[8];
  int world;
  uint32_t epoch;
};
// one CTA: copy the (tiny) statistics block into every rank's landing slot, then raise the flags
__global__ void __launch_bounds__(GN_THREADS) gn_share_kernel(const ShareParams p) {
  for (int r = 0; r < p.world; ++r)
    for (long long i = threadIdx.x; i < p.count; i += GN_THREADS) p.dst[r][i] = p.fin[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.world)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[threadIdx.x]), "r"(p.epoch) : "memory");
}
}  // namespace sb

extern "C" int sb_gn_share(const float* fin, long long count, void* const* dst, void* const* flags, int world,
                           unsigned epoch, cudaStream_t stream) {
  if (world < 1 || world > 8) return SB_ERR_SHAPE;
  ShareParams p;
  memset(&p, 0, sizeof(p));
  p.fin = fin; p.count = count; p.world = world; p.epoch = epoch;
  for (int r = 0; r < world; ++r) { p.dst[r] = (float*)dst[r]; p.flags[r] = (uint32_t*)flags[r]; }
  gn_share_kernel<<<1, GN_THREADS, 0, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// fin: [N][G][3] (stats) / [N][C][2] (bwd) -- the single-split form the apply / dx kernels merge
extern "C" int sb_gn_stats_finalize(const float* part, float* fin, int N, int G, int nsplit, cudaStream_t stream) {
  const int warps = N * G;
  if (nsplit > 1024) {  // a warp per output would walk hundreds of partials per lane: a block per output instead
    gn_stats_finalize_wide_kernel<<<warps, GN_THREADS, 0, stream>>>(part, fin, N, G, nsplit);
    sb_count_launch(1);
    return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
  }
  gn_stats_finalize_kernel<<<(warps * 32 + GN_THREADS - 1) / GN_THREADS, GN_THREADS, 0, stream>>>(part, fin, N, G, nsplit);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_gn_bwd_finalize(const float* part, float* fin, int N, int C, int nsplit, cudaStream_t stream) {
  const int warps = N * C;
  gn_bwd_finalize_kernel<<<(warps * 32 + GN_THREADS - 1) / GN_THREADS, GN_THREADS, 0, stream>>>(part, fin, N, C, nsplit);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

// ----------------------------------------------------------------------------
// Allocation-free forward (declared in no_alloc.h)
// ----------------------------------------------------------------------------
#include "no_alloc.h"

namespace sb {
// Scratch of the allocation-free entry point: partial statistics, then the per-sample
// finals, then (when the caller passes none) mean / rstd. In host code this NAME is only a
// handle for cudaGetSymbolAddress; kernels get the resolved device address.
static __device__ __align__(256) float g_gn_noalloc_scratch[SB_GN_NOALLOC_SCRATCH_FLOATS + 2 * 256 * 64];
constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_gn_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace sb

extern "C" int sb_gn_forward_noalloc(const void* x, void* y, const float* w, const float* b, float* mean,
                                     float* rstd, int N, long long S, int C, int G, float eps, int relu,
                                     cudaStream_t stream) {
  if (N < 1 || N > 64 || S < 1 || !gn_channels_ok(C, G)) return SB_ERR_SHAPE;
  if (x == nullptr || y == nullptr || w == nullptr || b == nullptr) return SB_ERR_SHAPE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return SB_ERR_DRIVER;
  if (g_gn_noalloc_ptr[dev] == nullptr) {
    // once per device, with that device current: the symbol's address on THIS device
    float* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_gn_noalloc_scratch) != cudaSuccess || p == nullptr) return SB_ERR_DRIVER;
    g_gn_noalloc_ptr[dev] = p;
  }
  float* scratch = g_gn_noalloc_ptr[dev];
  const int nsplit = sb_gn_nsplit(N, S, C);
  const long long part_floats = (long long)N * nsplit * G * 3;
  const long long fin_floats = (long long)N * G * 3;
  if (part_floats + fin_floats > SB_GN_NOALLOC_SCRATCH_FLOATS) return SB_ERR_TOO_LARGE;
  float* part = scratch;
  float* fin = scratch + part_floats;
  float* tail = scratch + SB_GN_NOALLOC_SCRATCH_FLOATS;  // room for mean / rstd when the caller wants neither
  SbGnArgs a;
  memset(&a, 0, sizeof(a));
  a.x = x; a.y = y; a.w = w; a.b = b;
  a.mean = mean ? mean : tail;
  a.rstd = rstd ? rstd : tail + 256 * 64;
  a.N = N; a.C = C; a.G = G; a.S = S; a.S_total = S;
  a.eps = eps; a.relu = relu;
  a.part = part;
  a.parts[0] = part;
  a.n_parts = 1;
  a.nsplit = nsplit;
  a.fin = fin;  // the statistics launch collapses its own partials (last block)
  int rc = sb_gn_stats(&a, stream);
  if (rc) return rc;
  a.fin = nullptr;
  a.parts[0] = fin;
  a.nsplit = 1;
  return sb_gn_apply(&a, stream);
}
