// Weight gradient of the 3-D convolutions on Blackwell tensor cores (sm_100a).
//
//   dW[tap][m][n] = sum_voxels  P[voxel, m] * Q[voxel + off(tap), n]
//
// The reduction axis is the voxel axis, so both operands sit in memory with
// the GEMM's M / N index contiguous (channels) and K strided: they are fed to
// tcgen05.mma as MN-major shared-memory tiles straight out of 5-D TMA box
// loads (one 128-byte row of 64 channels per voxel); no transpose pass exists.
// With rows ordered h-fastest (8 per swizzle atom) a shift along w is a shift
// of the start address by one atom, so one halo'd box of Q serves the three kw
// taps, which accumulate into three TMEM accumulators.
//
// Split-K is deterministic: the voxel blocks are cut into `splits` contiguous
// ranges, every CTA writes its fp32 partial to a workspace slice, and
// wgrad_reduce_kernel adds the slices in index order while permuting into the
// parameter's own layout ([Cout][Cin][kd][kh][kw], or [Cin][Cout][2][2][2] for
// the transposed convolution).
//
// Role of the reference: triton_conv3d/reduce_gemm.py:137-435 and
// triton_conv3d/transposed.py:1073-1166.
#include "common.cuh"
#include "host_api.h"

namespace sb {

int make_map_bf16(CUtensorMap* m, const void* base, int rank, const long long* dims, const long long* strides,
                  const int* box, int rowb);

constexpr int WG_MAX_STAGES = 6;

struct WgradParams {
  CUtensorMap mapM[2];
  CUtensorMap mapN[8];
  int CBm, CBn;          // channels per TMA box on each side (16/32/64)
  int m_boxes, n_boxes;  // boxes per tile
  int MT, NT;            // channels per tile on each side
  int umma_m;            // 64 or 128
  int KWS, n_outer, TW, KV;  // accumulators per CTA, outer taps, brick width, voxels per block
  int flip;              // accumulator j holds tap (KWS-1-j)
  int N, D, H, W, tiles_h, tiles_w, nblocks;
  int m_tiles, n_tiles, m_tiles0, n_tiles0;  // tiles in total / in the first source of that side
  int splits, blocks_per_split;
  int stages, stage_bytes, m_bytes, boxm_bytes, boxn_bytes, tx_bytes;
  int m_off_d, m_off_h, m_off_w;  // added to the M-side box origin (halo'd x on the M side)
  signed char o_map[16], o_dd[16], o_dh[16], o_dw[16];
  int Mtot, Ntot, T;  // workspace extents: ws[split][T][Mtot][Ntot]
  float* ws;
  uint32_t* status;
};

__global__ void __launch_bounds__(192, 1) wgrad_kernel(const __grid_constant__ WgradParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[WG_MAX_STAGES];
  __shared__ uint64_t empty_bar[WG_MAX_STAGES];
  __shared__ uint64_t done_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  volatile uint32_t* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&done_bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  int t = blockIdx.x;
  const int o = t % p.n_outer; t /= p.n_outer;
  const int mt = t % p.m_tiles; t /= p.m_tiles;
  const int nt = t % p.n_tiles; t /= p.n_tiles;
  const int split = t;
  const int blk_begin = split * p.blocks_per_split;
  int blk_end = blk_begin + p.blocks_per_split;
  if (blk_end > p.nblocks) blk_end = p.nblocks;
  const int nblk = blk_end > blk_begin ? blk_end - blk_begin : 0;

  if (warp == 0) {
    if (lane == 0) {
      const int msrc = mt >= p.m_tiles0 ? 1 : 0;
      const int mc0 = (msrc ? mt - p.m_tiles0 : mt) * p.MT;
      const int nsrc = nt >= p.n_tiles0 ? 1 : 0;
      const int nc0 = (nsrc ? nt - p.n_tiles0 : nt) * p.NT;
      const CUtensorMap* mm = &p.mapM[msrc];
      const CUtensorMap* mn = &p.mapN[p.o_map[o] + nsrc];
      tma_prefetch_desc(mm);
      tma_prefetch_desc(mn);
      for (int i = 0; i < nblk; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (i / p.stages) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, p.status, 11)) break;
        int b = blk_begin + i;
        const int wt = b % p.tiles_w; b /= p.tiles_w;
        const int ht = b % p.tiles_h; b /= p.tiles_h;
        const int d = b % p.D; b /= p.D;
        const int n = b;
        const int h0 = ht * 8, w0 = wt * p.TW;
        uint8_t* sm = smem + (size_t)s * p.stage_bytes;
        uint8_t* sn = sm + p.m_bytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)p.tx_bytes);
        for (int j = 0; j < p.m_boxes; ++j)
          tma_load_5d(sm + (size_t)j * p.boxm_bytes, mm, &full_bar[s], mc0 + j * p.CBm, h0 + p.m_off_h,
                      w0 + p.m_off_w, d + p.m_off_d, n);
        for (int j = 0; j < p.n_boxes; ++j)
          tma_load_5d(sn + (size_t)j * p.boxn_bytes, mn, &full_bar[s], nc0 + j * p.CBn, h0 + p.o_dh[o],
                      w0 + p.o_dw[o], d + p.o_dd[o], n);
      }
    }
  } else if (warp == 1) {
    // warp-uniform loop, one elected lane issues (descriptor arithmetic stays in uniform registers)
    {
      const bool leader = elect_one();
      const uint32_t idesc = make_idesc_bf16(p.umma_m, p.NT, 1, 1);
      const uint32_t rowm = p.CBm * 2, rown = p.CBn * 2;
      // MN-major: LBO = distance between channel blocks, SBO = distance between 8-voxel groups
      const uint32_t lbom = p.m_boxes > 1 ? (uint32_t)p.boxm_bytes : 0u;
      const uint32_t lbon = p.n_boxes > 1 ? (uint32_t)p.boxn_bytes : 0u;
      const uint32_t m_hi = desc_hi(8u * rowm, swizzle_code_for(rowm));
      const uint32_t n_hi = desc_hi(8u * rown, swizzle_code_for(rown));
      const uint32_t m_step = (16u * rowm) >> 4, n_step = (16u * rown) >> 4, n_shift = (8u * rown) >> 4;
      const int ksteps = p.KV / 16;
      const uint32_t s0 = smem_u32(smem);
      uint32_t stage = 0, sph = 0;
      bool ok = true;
      for (int i = 0; i < nblk && ok; ++i) {
        if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], sph, abort_flag, p.status, 12))) { ok = false; break; }
        tc_fence_after();
        const uint32_t sm = s0 + stage * (uint32_t)p.stage_bytes;
        const uint32_t m_lo = desc_lo(sm, lbom), n_lo = desc_lo(sm + p.m_bytes, lbon);
        if (leader) {
          for (int kw = 0; kw < p.KWS; ++kw)
            for (int k = 0; k < ksteps; ++k)
              tc_mma_bf16_pred(tmem_base + kw * p.NT, m_lo + k * m_step, m_hi, n_lo + kw * n_shift + k * n_step, n_hi,
                               idesc, (i | k) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == (uint32_t)p.stages) { stage = 0; sph ^= 1u; }
      }
      if (ok && leader) tc_commit(&done_bar);
    }
  } else {
    const int q = warp & 3;
    bool ok = true;
    if (nblk > 0) ok = mbar_wait(&done_bar, 0, abort_flag, p.status, 13);
    tc_fence_after();
    if (ok) {
      const int row = p.umma_m == 128 ? q * 32 + lane : q * 16 + lane;
      const bool valid = row < p.MT && (p.umma_m == 128 || lane < 16);
      const int msrc_off = mt * p.MT;  // tiles of both sources are laid out back to back
      const int nsrc_off = nt * p.NT;
      for (int j = 0; j < p.KWS; ++j) {
        const int tap = o * p.KWS + (p.flip ? p.KWS - 1 - j : j);
        float* dst = p.ws + (((size_t)split * p.T + tap) * p.Mtot + msrc_off + row) * p.Ntot + nsrc_off;
        for (int c0 = 0; c0 < p.NT; c0 += 32) {
          uint32_t v[32];
          if (nblk > 0) {
            if (p.NT - c0 >= 32) {
              tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + j * p.NT + c0, v);
            } else {
              uint32_t v16[16];
              tmem_ld_32x16(tmem_base + ((uint32_t)(q * 32) << 16) + j * p.NT + c0, v16);
#pragma unroll
              for (int e = 0; e < 16; ++e) { v[e] = v16[e]; v[16 + e] = 0u; }
            }
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0u;
          }
          if (valid) {
            const int ncol = p.NT - c0 >= 32 ? 32 : p.NT - c0;
            for (int e = 0; e < ncol; e += 4) {
              float4 f = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]),
                                     __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
              *reinterpret_cast<float4*>(dst + c0 + e) = f;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// dw (+)= sum over splits, permuted into the parameter layout.
//   mode 0: conv,  M side = gy (m = co, n = ci)   dw[co][ci][tap]
//   mode 1: conv,  M side = x  (m = ci, n = co)   dw[co][ci][tap]
//   mode 2: convT, M side = x  (m = ci, n = kw*cout+co), T = 4 -> dw[ci][co][kd][kh][kw]
struct ReduceParams {
  const float* ws;
  float* dw;
  int splits, T, Mtot, Ntot;
  int mode, cout, cin, taps;
  int accumulate;
  int tap_swap;  // 3x3x3: destination tap order differs from the workspace's (0 none, 1 kd <-> kh, 2 kd <-> kw)
  long long total;
};

__device__ __forceinline__ int wg_swap_tap(int tap, int mode) {
  if (mode == 0) return tap;
  const int kd = tap / 9, kh = (tap / 3) % 3, kw = tap % 3;
  return mode == 1 ? (kh * 9 + kd * 3 + kw) : (kw * 9 + kh * 3 + kd);
}

__global__ void wgrad_reduce_kernel(const ReduceParams p) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.total) return;
  int tap, m, n;
  if (p.mode == 2) {
    // dw[ci][co][kd][kh][kw]
    const int t8 = (int)(idx % 8);
    const int co = (int)((idx / 8) % p.cout);
    const int ci = (int)(idx / (8LL * p.cout));
    const int kd = t8 >> 2, kh = (t8 >> 1) & 1, kw = t8 & 1;
    tap = kd * 2 + kh;
    m = ci;
    n = kw * p.cout + co;
  } else {
    tap = (int)(idx % p.taps);
    if (p.taps == 27) tap = wg_swap_tap(tap, p.tap_swap);  // idx walks the parameter's order; ws holds the kernels'
    const int ci = (int)((idx / p.taps) % p.cin);
    const int co = (int)(idx / ((long long)p.taps * p.cin));
    if (p.mode == 0) { m = co; n = ci; } else { m = ci; n = co; }
  }
  const size_t slice = (size_t)p.T * p.Mtot * p.Ntot;
  const float* src = p.ws + ((size_t)tap * p.Mtot + m) * p.Ntot + n;
  float acc = 0.f;
  for (int s = 0; s < p.splits; ++s) acc += src[(size_t)s * slice];
  if (p.accumulate) acc += p.dw[idx];
  p.dw[idx] = acc;
}

// Same reduction for 3x3x3 weights with the output channel on the workspace's M side (mode 0), through a
// shared-memory transpose: one block owns (co, CT input channels), CT = 128 when cin allows (else 64 or 32).
// It reads 27 runs of CT consecutive floats per split as 16-byte vectors, four in flight per thread (summed in
// split order), and writes the CT x 27 floats that are contiguous in dw[co][ci][tap] as 16-byte vectors.
constexpr int RT_MAX_CT = 128;
// MANY: the layer has at least four splits (small weights, few blocks): four splits per trip, 16 loads in flight.
template <bool MANY>
__global__ void __launch_bounds__(256) wgrad_reduce_t_kernel(const ReduceParams p, const int CT) {
  __shared__ float t[27][RT_MAX_CT + 1];
  const int co = blockIdx.y, ci0 = blockIdx.x * CT;
  const size_t slice = (size_t)p.T * p.Mtot * p.Ntot;
  const int v_per_run = CT / 4, nvec = 27 * v_per_run;
  for (int e0 = threadIdx.x; e0 < nvec; e0 += 4 * 256) {
    float4 acc[4];
    int tap[4], c4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = e0 + u * 256;
      tap[u] = e / v_per_run;
      c4[u] = (e - tap[u] * v_per_run) * 4;
      acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if constexpr (MANY) {
      // Layers with small weights have many splits and few blocks: four splits per trip keep 16 loads in flight
      // per thread; the sums are still taken in split order.
      const float* base[4];
      bool live[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        live[u] = e0 + u * 256 < nvec;
        base[u] = p.ws + ((size_t)tap[u] * p.Mtot + co) * p.Ntot + ci0 + c4[u];
      }
      int sp = 0;
      for (; sp + 4 <= p.splits; sp += 4) {
        float4 v[4][4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            v[k][u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (live[u]) v[k][u] = __ldcs(reinterpret_cast<const float4*>(base[u] + (size_t)(sp + k) * slice));
          }
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            acc[u].x += v[k][u].x; acc[u].y += v[k][u].y; acc[u].z += v[k][u].z; acc[u].w += v[k][u].w;
          }
      }
      for (; sp < p.splits; ++sp) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (live[u]) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(base[u] + (size_t)sp * slice));
            acc[u].x += v.x; acc[u].y += v.y; acc[u].z += v.z; acc[u].w += v.w;
          }
        }
      }
    } else {
      for (int sp = 0; sp < p.splits; ++sp) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (e0 + u * 256 < nvec)
            v[u] = __ldcs(reinterpret_cast<const float4*>(p.ws + (size_t)sp * slice +
                                                          ((size_t)tap[u] * p.Mtot + co) * p.Ntot + ci0 + c4[u]));
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (e0 + u * 256 < nvec) {
        t[tap[u]][c4[u]] = acc[u].x; t[tap[u]][c4[u] + 1] = acc[u].y;
        t[tap[u]][c4[u] + 2] = acc[u].z; t[tap[u]][c4[u] + 3] = acc[u].w;
      }
    }
  }
  __syncthreads();
  float* dst = p.dw + ((size_t)co * p.cin + ci0) * 27;  // 16-byte aligned: (co * cin + ci0) is a multiple of 4
  const int nout4 = CT * 27 / 4;
  for (int q = threadIdx.x; q < nout4; q += 256) {
    float o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int e = q * 4 + k;
      const int c = e / 27, tp = wg_swap_tap(e - c * 27, p.tap_swap);
      o[k] = t[tp][c];
    }
    float4 v = make_float4(o[0], o[1], o[2], o[3]);
    float4* d4 = reinterpret_cast<float4*>(dst) + q;
    if (p.accumulate) {
      const float4 old = *d4;
      v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
    }
    *d4 = v;
  }
}

static int g_wg_smem = 0, g_wg_sms = 0;
static int wg_setup() {
  if (g_wg_smem) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SB_ERR_DRIVER;
  int lim = 0, sms = 0;
  cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaFuncSetAttribute(wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim - 2048) != cudaSuccess)
    return SB_ERR_DRIVER;
  g_wg_smem = lim - 2048;
  g_wg_sms = sms;
  return 0;
}

static int cdiv(int a, int b) { return (a + b - 1) / b; }
static int box_c(int c) { return c % 64 == 0 ? 64 : c % 32 == 0 ? 32 : 16; }

struct Plan {
  WgradParams p;
  ReduceParams r;
};

// Fills the plan (no tensor maps when `maps` is false: used to size the workspace).
static int build_plan(const SbWgradArgs* a, Plan& pl, bool maps) {
  WgradParams& p = pl.p;
  memset(&pl, 0, sizeof(pl));
  const int xc = a->x_c[0] + a->x_c[1];
  const int gc = a->gy_c;
  const bool convT = a->ksize == 2;
  if (!(a->ksize == 1 || a->ksize == 2 || a->ksize == 3)) return SB_ERR_SHAPE;
  if (xc % 16 || gc % 16) return SB_ERR_SHAPE;
  p.N = a->N; p.D = a->D; p.H = a->H; p.W = a->W;
  // which tensor sits on the M side (needs >= 64 channels to fill the MMA rows)
  bool m_is_x;
  if (convT) m_is_x = true;
  else if (gc >= 128) m_is_x = false;
  else if (xc >= 128) m_is_x = true;
  else m_is_x = gc < 64 && xc >= 64;
  if (m_is_x && a->x_c[1] > 0 && (a->x_c[0] % 64 != 0)) return SB_ERR_SHAPE;
  const int mc = m_is_x ? xc : gc;
  const int nc_full = convT ? 2 * gc : (m_is_x ? gc : xc);
  // tiles
  const int m_first = m_is_x ? a->x_c[0] : gc;
  p.MT = (m_first % 128 == 0 && (mc - m_first) % 128 == 0) ? 128 : (m_first % 64 == 0 ? 64 : m_first);
  if (p.MT < 64 && mc != p.MT) return SB_ERR_SHAPE;
  p.CBm = box_c(p.MT);
  p.m_boxes = p.MT / p.CBm;
  p.umma_m = p.MT > 64 ? 128 : 64;
  const int n_first = convT ? nc_full : (m_is_x ? gc : a->x_c[0]);
  p.NT = (n_first % 128 == 0 && (nc_full - n_first) % 128 == 0) ? 128
         : (n_first % 64 == 0 && (nc_full - n_first) % 64 == 0) ? 64 : n_first;
  if (p.NT > 128 || p.NT % 16) return SB_ERR_SHAPE;
  if (p.NT < 64 && nc_full != p.NT) return SB_ERR_SHAPE;
  p.CBn = box_c(p.NT);
  p.n_boxes = p.NT / p.CBn;
  p.m_tiles = mc / p.MT;
  p.m_tiles0 = m_first / p.MT;
  p.n_tiles = nc_full / p.NT;
  p.n_tiles0 = n_first / p.NT;
  // voxel blocks: 8 h x TW w
  p.TW = a->W >= 16 ? 16 : (a->W >= 8 ? 8 : (a->W >= 4 ? 4 : 2));
  p.KV = 8 * p.TW;
  p.tiles_h = cdiv(a->H, 8);
  p.tiles_w = cdiv(a->W, p.TW);
  p.nblocks = a->N * a->D * p.tiles_h * p.tiles_w;
  p.KWS = a->ksize == 3 ? 3 : 1;
  p.n_outer = a->ksize == 3 ? 9 : (convT ? 4 : 1);
  p.T = a->ksize == 3 ? 27 : (convT ? 4 : 1);
  p.flip = (!convT && m_is_x) ? 1 : 0;  // shifted tensor is gy: accumulator j <-> kw = 2-j
  const int sign = p.flip ? -1 : 1;
  for (int o = 0; o < p.n_outer; ++o) {
    if (a->ksize == 3) {
      const int kd = o / 3, kh = o % 3;
      p.o_map[o] = 0;
      p.o_dd[o] = (signed char)(sign * (kd - 1));
      p.o_dh[o] = (signed char)(sign * (kh - 1));
      p.o_dw[o] = -1;
    } else if (convT) {
      p.o_map[o] = (signed char)o;
    }
  }
  p.Mtot = mc;
  p.Ntot = nc_full;
  const int base_ctas = p.n_outer * p.m_tiles * p.n_tiles;
  int sms = g_wg_sms > 0 ? g_wg_sms : 148;
  int splits = a->splits > 0 ? a->splits : (sms + base_ctas - 1) / base_ctas;
  if (splits > p.nblocks) splits = p.nblocks;
  if (splits < 1) splits = 1;
  p.blocks_per_split = cdiv(p.nblocks, splits);
  p.splits = cdiv(p.nblocks, p.blocks_per_split);
  // shared memory
  p.boxm_bytes = p.KV * p.CBm * 2;
  const int rows_n = 8 * (p.TW + p.KWS - 1);
  p.boxn_bytes = rows_n * p.CBn * 2;
  p.m_bytes = ((p.m_boxes * p.boxm_bytes + 1023) / 1024) * 1024;
  int n_bytes = ((p.n_boxes * p.boxn_bytes + 1023) / 1024) * 1024;
  p.stage_bytes = p.m_bytes + n_bytes;
  p.tx_bytes = p.m_boxes * p.boxm_bytes + p.n_boxes * p.boxn_bytes;
  // reduce
  ReduceParams& r = pl.r;
  r.splits = p.splits; r.T = p.T; r.Mtot = p.Mtot; r.Ntot = p.Ntot;
  r.mode = convT ? 2 : (m_is_x ? 1 : 0);
  r.accumulate = a->accumulate;
  if (!maps) return 0;

  int st = (g_wg_smem - 1024) / p.stage_bytes;
  if (st > WG_MAX_STAGES) st = WG_MAX_STAGES;
  if (st < 2) return SB_ERR_SHAPE;
  p.stages = st;
  int rc;
  // M side maps
  auto act_map = [&](CUtensorMap* m, const void* base, int c, long long ld, int cb, int box_w) {
    // x may carry a halo (its own extents); gy always lives on the (N, D, H, W) grid
    const bool is_x = base == a->x[0] || (a->x[1] != nullptr && base == a->x[1]);
    const long long D = is_x && a->xin_d ? a->xin_d : a->D, H = is_x && a->xin_h ? a->xin_h : a->H,
                    W = is_x && a->xin_w ? a->xin_w : a->W;
    long long dims[5] = {c, H, W, D, a->N};
    long long str[5] = {1, W * ld, ld, H * W * ld, D * H * W * ld};
    int box[5] = {cb, 8, box_w, 1, 1};
    return make_map_bf16(m, base, 5, dims, str, box, cb * 2);
  };
  if (!convT) {
    if (m_is_x) {
      p.m_off_d = a->xoff_d; p.m_off_h = a->xoff_h; p.m_off_w = a->xoff_w;
    } else {
      for (int o = 0; o < p.n_outer; ++o) {
        p.o_dd[o] = (signed char)(p.o_dd[o] + a->xoff_d);
        p.o_dh[o] = (signed char)(p.o_dh[o] + a->xoff_h);
        p.o_dw[o] = (signed char)(p.o_dw[o] + a->xoff_w);
      }
    }
  }
  if (m_is_x) {
    rc = act_map(&p.mapM[0], a->x[0], a->x_c[0], a->x_ld[0], p.CBm, p.TW);
    if (rc) return rc;
    if (a->x_c[1] > 0) {
      rc = act_map(&p.mapM[1], a->x[1], a->x_c[1], a->x_ld[1], p.CBm, p.TW);
      if (rc) return rc;
    } else p.mapM[1] = p.mapM[0];
  } else {
    rc = act_map(&p.mapM[0], a->gy, gc, a->gy_ld, p.CBm, p.TW);
    if (rc) return rc;
    p.mapM[1] = p.mapM[0];
  }
  // N side maps
  if (convT) {
    const long long C = a->gy_ld;
    if (C != gc) return SB_ERR_SHAPE;
    const long long W2 = 2LL * a->W, H2 = 2LL * a->H, D2 = 2LL * a->D;
    for (int o = 0; o < 4; ++o) {
      const int kd = o >> 1, kh = o & 1;
      const __nv_bfloat16* base = (const __nv_bfloat16*)a->gy + ((long long)kd * H2 + kh) * W2 * C;
      long long dims[5] = {2 * gc, a->H, a->W, a->D, a->N};
      long long str[5] = {1, 2 * W2 * C, 2 * C, 2 * H2 * W2 * C, D2 * H2 * W2 * C};
      int box[5] = {p.CBn, 8, p.TW, 1, 1};
      rc = make_map_bf16(&p.mapN[o], base, 5, dims, str, box, p.CBn * 2);
      if (rc) return rc;
    }
    for (int o = 4; o < 8; ++o) p.mapN[o] = p.mapN[0];
  } else if (m_is_x) {
    rc = act_map(&p.mapN[0], a->gy, gc, a->gy_ld, p.CBn, p.TW + p.KWS - 1);
    if (rc) return rc;
    for (int o = 1; o < 8; ++o) p.mapN[o] = p.mapN[0];
  } else {
    rc = act_map(&p.mapN[0], a->x[0], a->x_c[0], a->x_ld[0], p.CBn, p.TW + p.KWS - 1);
    if (rc) return rc;
    if (a->x_c[1] > 0) {
      rc = act_map(&p.mapN[1], a->x[1], a->x_c[1], a->x_ld[1], p.CBn, p.TW + p.KWS - 1);
      if (rc) return rc;
    } else p.mapN[1] = p.mapN[0];
    for (int o = 2; o < 8; ++o) p.mapN[o] = p.mapN[0];
  }
  return 0;
}

}  // namespace sb

using namespace sb;

namespace sb {
long long wgrad_plane_workspace(const SbWgradArgs* a);
int wgrad_plane_launch(const SbWgradArgs* a, cudaStream_t stream, int* splits_out);
}

// a->splits < 0 forces the generic kernel (tests); >= 0 prefers the plane kernel when eligible
extern "C" long long sb_conv_wgrad_workspace(const SbWgradArgs* a) {
  if (a->splits >= 0) {
    const long long w = wgrad_plane_workspace(a);
    if (w >= 0) return w;
  }
  Plan pl;
  wg_setup();
  SbWgradArgs generic = *a;
  if (generic.splits < 0) generic.splits = -generic.splits - 1;
  if (build_plan(&generic, pl, false)) return -1;
  return (long long)pl.p.splits * pl.p.T * pl.p.Mtot * pl.p.Ntot;
}

// real (unpadded) channel counts of the parameter are passed in dw_cout/dw_cin
static int run_reduce(const SbWgradArgs* a, ReduceParams& r, cudaStream_t stream) {
  r.ws = a->workspace;
  r.dw = a->dw;
  r.cout = a->dw_cout;
  r.cin = a->dw_cin;
  r.taps = a->ksize == 3 ? 27 : (a->ksize == 2 ? 8 : 1);
  r.tap_swap = a->ksize == 3 ? a->tap_swap : 0;
  if (r.tap_swap < 0 || r.tap_swap > 2) return SB_ERR_SHAPE;
  r.total = (long long)r.cout * r.cin * r.taps;
  const int threads = 256;
  const long long blocks = (r.total + threads - 1) / threads;
  if (r.mode == 0 && r.taps == 27 && r.cin % 32 == 0 && r.cout <= 65535 && r.Ntot % 4 == 0 &&
      (reinterpret_cast<uintptr_t>(r.dw) & 15) == 0 && (reinterpret_cast<uintptr_t>(r.ws) & 15) == 0) {
    // the widest input-channel tile that still leaves about two blocks per SM (small weights: narrower tiles)
    int ct = r.cin % 128 == 0 ? 128 : (r.cin % 64 == 0 ? 64 : 32);
    while (ct > 32 && (long long)(r.cin / ct) * r.cout < 296) ct /= 2;
    if (r.splits >= 4) wgrad_reduce_t_kernel<true><<<dim3(r.cin / ct, r.cout), threads, 0, stream>>>(r, ct);
    else wgrad_reduce_t_kernel<false><<<dim3(r.cin / ct, r.cout), threads, 0, stream>>>(r, ct);
  } else
    wgrad_reduce_kernel<<<(unsigned)blocks, threads, 0, stream>>>(r);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_conv_wgrad(const SbWgradArgs* a, cudaStream_t stream) {
  int rc;
  if (a->splits >= 0) {
    int splits = 0;
    rc = wgrad_plane_launch(a, stream, &splits);
    if (rc > 0) return rc;
    if (rc == 0) {
      ReduceParams r;
      memset(&r, 0, sizeof(r));
      r.splits = splits; r.T = 27; r.Mtot = a->gy_c; r.Ntot = a->x_c[0] + a->x_c[1];
      r.mode = 0;
      r.accumulate = a->accumulate;
      return run_reduce(a, r, stream);
    }
  }
  if (a->xhalo[0][0] || a->xhalo[0][1]) return SB_ERR_SHAPE;  // slab halos: plane kernel only
  rc = wg_setup();
  if (rc) return rc;
  Plan pl;
  SbWgradArgs generic = *a;
  if (generic.splits < 0) generic.splits = -generic.splits - 1;  // -1 -> automatic, -(k+1) -> k splits
  a = &generic;
  rc = build_plan(a, pl, true);
  if (rc) return rc;
  WgradParams& p = pl.p;
  const long long need = (long long)p.splits * p.T * p.Mtot * p.Ntot;
  if (need > a->workspace_elems) return SB_ERR_TOO_LARGE;
  p.ws = a->workspace;
  p.status = a->status;
  const int grid = p.n_outer * p.m_tiles * p.n_tiles * p.splits;
  const size_t smem = (size_t)p.stages * p.stage_bytes + 1024;
  wgrad_kernel<<<grid, 192, smem, stream>>>(p);
  sb_count_launch(1);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  return run_reduce(a, pl.r, stream);
}
