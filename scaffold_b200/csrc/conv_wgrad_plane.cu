// Weight gradient of the 3x3x3 convolution, high-reuse variant (sm_100a).
//
//   dW[kd,kh,kw][co][ci] = sum_v gy[v, co] * x[v + (kd-1, kh-1, kw-1), ci]
//
// A CTA owns one kd, 64 (or 32) output channels, up to 64 input channels and a
// contiguous range of 8(h) x TW(w) voxel blocks. Per block it loads ONE box of
// gy (10 h x TW w rows) and ONE box of x (10 h x (TW+2) w rows, plane d+kd-1),
// both straight from NDHWC memory as MN-major operands (voxel = K). Because
// rows are h-fastest and the swizzle is a function of the absolute address,
// shifted views of a box are just other start addresses, and the
// descriptor's "leading" stride can step between shifted views:
//   * M = 2 x 64 rows: gy at h-shift 0 and at h-shift +1 (leading stride 1 row)
//   * N = 3 x CN cols: x at w-shift -1, 0, +1 (leading stride one w column)
// so ONE 128 x 192 x 16 tcgen05.mma accumulates six taps. Two accumulators (x
// at h-shift 0 and +1) cover the nine (kh,kw) taps of the CTA's kd:
//   acc0: rows 0-63 -> kh=1, rows 64-127 -> kh=0     acc1: rows 0-63 -> kh=2
// (rows 64-127 of acc1 repeat kh=1 and are dropped). The h-shifted copy of gy
// never sees output row 0, but that row only pairs with x at h=-1, which is
// zero padding, so nothing is lost.
//
// Partials go to the same workspace layout as the generic kernel,
// ws[split][tap][co][ci], and are reduced in index order by wgrad_reduce_kernel.
//
// Role of the reference: triton_conv3d/reduce_gemm.py:137-435.
#include "common.cuh"
#include "host_api.h"

namespace sb {

int make_map_bf16(CUtensorMap* m, const void* base, int rank, const long long* dims, const long long* strides,
                  const int* box, int rowb);

constexpr int WP_MAX_STAGES = 6;
constexpr int WP_RH = 10;

struct WgradPlaneParams {
  CUtensorMap mapG;     // gy
  CUtensorMap mapX[2];  // x sources
  int CM, CN;           // channels per tile on each side (CM: 64/32, CN: 16/32/64)
  int TW, KV;           // brick width, voxels per block
  int N, D, H, W, tiles_h, tiles_w, nblocks;
  int m_tiles, n_tiles, n_tiles0;
  int splits, blocks_per_split;
  int stages, stage_bytes, g_bytes, g_tx, x_tx;
  int Mtot, Ntot;
  int xoff_d, xoff_h, xoff_w;
  CUtensorMap mapXh[4];  // depth-halo slabs of x: [source * 2 + face]
  int xh_has[2], xin_D;
  int h_origin;  // first block row starts here (-1 when x carries an h halo, see wp_plan)
  float* ws;
  uint32_t* status;
};

__global__ void __launch_bounds__(192, 1) wgrad_plane_kernel(const __grid_constant__ WgradPlaneParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[WP_MAX_STAGES];
  __shared__ uint64_t empty_bar[WP_MAX_STAGES];
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
  const int kd = t % 3; t /= 3;
  const int mt = t % p.m_tiles; t /= p.m_tiles;
  const int nt = t % p.n_tiles; t /= p.n_tiles;
  const int split = t;
  const int blk_begin = split * p.blocks_per_split;
  int blk_end = blk_begin + p.blocks_per_split;
  if (blk_end > p.nblocks) blk_end = p.nblocks;
  const int nblk = blk_end > blk_begin ? blk_end - blk_begin : 0;
  const int rowm = p.CM * 2, rown = p.CN * 2;
  const int umma_m = 2 * p.CM;

  if (warp == 0) {
    if (lane == 0) {
      const int nsrc = nt >= p.n_tiles0 ? 1 : 0;
      const int nc0 = (nsrc ? nt - p.n_tiles0 : nt) * p.CN;
      const CUtensorMap* mx = &p.mapX[nsrc];
      tma_prefetch_desc(&p.mapG);
      tma_prefetch_desc(mx);
      for (int i = 0; i < nblk; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (i / p.stages) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, p.status, 31)) break;
        int b = blk_begin + i;
        const int wt = b % p.tiles_w; b /= p.tiles_w;
        const int ht = b % p.tiles_h; b /= p.tiles_h;
        const int d = b % p.D; b /= p.D;
        const int n = b;
        const int h0 = ht * 8 + p.h_origin, w0 = wt * p.TW;
        uint8_t* sg = smem + (size_t)s * p.stage_bytes;
        uint8_t* sx = sg + p.g_bytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)(p.g_tx + p.x_tx));
        tma_load_5d(sg, &p.mapG, &full_bar[s], mt * p.CM, h0, w0, d, n);
        const int dz = d + kd - 1 + p.xoff_d;
        const int face = dz < 0 ? 0 : (dz >= p.xin_D ? 1 : -1);
        if (face >= 0 && p.xh_has[face])
          tma_load_5d(sx, &p.mapXh[nsrc * 2 + face], &full_bar[s], nc0, h0 + p.xoff_h, w0 - 1 + p.xoff_w, 0, n);
        else
          tma_load_5d(sx, mx, &full_bar[s], nc0, h0 + p.xoff_h, w0 - 1 + p.xoff_w, dz, n);
      }
    }
  } else if (warp == 1) {
    // warp-uniform loop, one elected lane issues
    const bool leader = elect_one();
    const uint32_t idesc = make_idesc_bf16(umma_m, 3 * p.CN, 1, 1);
    const uint32_t g_hi = desc_hi((uint32_t)WP_RH * rowm, swizzle_code_for(rowm));
    const uint32_t x_hi = desc_hi((uint32_t)WP_RH * rown, swizzle_code_for(rown));
    const uint32_t g_step = (2u * WP_RH * rowm) >> 4;  // 16 voxels = two w columns
    const uint32_t x_step = (2u * WP_RH * rown) >> 4;
    const uint32_t x_hshift = (uint32_t)rown >> 4;
    const int ksteps = p.KV / 16;
    const uint32_t s0 = smem_u32(smem);
    bool ok = true;
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < nblk && ok; ++i) {
      if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], ph, abort_flag, p.status, 32))) { ok = false; break; }
      tc_fence_after();
      const uint32_t sg = s0 + (uint32_t)s * p.stage_bytes;
      const uint32_t g_lo = desc_lo(sg, (uint32_t)rowm);                        // M blocks: 1 row apart
      const uint32_t x_lo = desc_lo(sg + p.g_bytes, (uint32_t)WP_RH * rown);    // N blocks: 1 w column apart
      for (int k = 0; k < ksteps; ++k) {
        if (leader) {
          const uint32_t acc_flag = (i | k) != 0 ? 1u : 0u;
          tc_mma_bf16_pred(tmem_base, g_lo + k * g_step, g_hi, x_lo + k * x_step, x_hi, idesc, acc_flag);
          tc_mma_bf16_pred(tmem_base + 256u, g_lo + k * g_step, g_hi, x_lo + k * x_step + x_hshift, x_hi, idesc,
                           acc_flag);
        }
      }
      if (leader) tc_commit(&empty_bar[s]);
      __syncwarp();
      if (++s == p.stages) { s = 0; ph ^= 1u; }
    }
    if (ok && leader) tc_commit(&done_bar);
  } else {
    const int q = warp & 3;
    bool ok = true;
    if (nblk > 0) ok = mbar_wait(&done_bar, 0, abort_flag, p.status, 33);
    tc_fence_after();
    if (ok) {
      int m;
      bool rowvalid;
      if (umma_m == 128) { m = q * 32 + lane; rowvalid = true; }
      else { m = q * 16 + lane; rowvalid = lane < 16; }
      const int blk_i = m / p.CM;   // 0: gy unshifted, 1: gy shifted by +1 in h
      const int co = mt * p.CM + (m % p.CM);
      for (int a = 0; a < 2; ++a) {
        const int kh = a == 0 ? (blk_i == 0 ? 1 : 0) : 2;
        const bool use = rowvalid && !(a == 1 && blk_i == 1);
        for (int j = 0; j < 3; ++j) {
          const int tap = (kd * 3 + kh) * 3 + j;
          float* dst = p.ws + (((size_t)split * 27 + tap) * p.Mtot + co) * p.Ntot + (size_t)nt * p.CN;
          for (int c0 = 0; c0 < p.CN; c0 += 16) {
            uint32_t v[16];
            if (nblk > 0) {
              tmem_ld_32x16(tmem_base + ((uint32_t)(q * 32) << 16) + a * 256u + j * p.CN + c0, v);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int e = 0; e < 16; ++e) v[e] = 0u;
            }
            if (use) {
#pragma unroll
              for (int e = 0; e < 16; e += 4) {
                float4 f = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]),
                                       __uint_as_float(v[e + 3]));
                *reinterpret_cast<float4*>(dst + c0 + e) = f;
              }
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

}  // namespace sb

namespace sb {

static int g_wp_smem = 0, g_wp_sms = 0;
static int wp_setup() {
  if (g_wp_smem) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SB_ERR_DRIVER;
  int lim = 0, sms = 0;
  cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaFuncSetAttribute(wgrad_plane_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim - 2048) !=
      cudaSuccess)
    return SB_ERR_DRIVER;
  g_wp_smem = lim - 2048;
  g_wp_sms = sms;
  return 0;
}

static int cdiv_wp(int a, int b) { return (a + b - 1) / b; }

// Fills everything but the tensor maps. Returns -1 when the shape is not eligible.
static int wp_plan(const SbWgradArgs* a, WgradPlaneParams& p) {
  memset(&p, 0, sizeof(p));
  if (a->ksize != 3 || a->H < 8 || a->W < 8) return -1;
  const int gc = a->gy_c, xc = a->x_c[0] + a->x_c[1];
  if (gc % 32 != 0) return -1;
  p.CM = gc % 64 == 0 ? 64 : 32;
  // input-channel tile: the largest of 64/32/16 dividing every source
  int cn = 64;
  while (cn > 16 && (a->x_c[0] % cn != 0 || xc % cn != 0)) cn /= 2;
  if (a->x_c[0] % cn != 0 || xc % cn != 0) return -1;
  p.CN = cn;
  p.N = a->N; p.D = a->D; p.H = a->H; p.W = a->W;
  p.TW = a->W >= 16 ? 16 : 8;
  p.KV = 8 * p.TW;
  // The h-shifted copy of gy never covers output row 0; that is harmless when x[-1] is zero padding, but
  // with an h halo in x the row is real data, so the blocks then start one row early (gy row -1 reads zero).
  p.h_origin = a->xoff_h != 0 ? -1 : 0;
  p.tiles_h = cdiv_wp(a->H - p.h_origin, 8);
  p.tiles_w = cdiv_wp(a->W, p.TW);
  p.nblocks = a->N * a->D * p.tiles_h * p.tiles_w;
  p.m_tiles = gc / p.CM;
  p.n_tiles = xc / cn;
  p.n_tiles0 = a->x_c[0] / cn;
  p.Mtot = gc;
  p.Ntot = xc;
  const int base = 3 * p.m_tiles * p.n_tiles;
  const int sms = g_wp_sms > 0 ? g_wp_sms : 148;
  int splits = a->splits;
  if (splits <= 0) {
    // Split count by a small cost model (clock ticks): waves x (blocks per CTA x MMA time per block + epilogue)
    // + ordered reduce of the partial buffers. It avoids a nearly empty last wave (e.g. 192 CTAs on 148 SMs).
    const double block_clk = (p.KV / 16) * 2.0 * 96.0;
    const double epi_clk = 6000.0;
    const double reduce_clk = 27.0 * gc * xc * 4.0 / 3400.0;
    double best = 0.0;
    splits = 1;
    const int sp_max = 2 * sms / base + 1 > 16 ? 2 * sms / base + 1 : 16;
    for (int sp = 1; sp <= sp_max && sp <= p.nblocks; ++sp) {
      const int per = cdiv_wp(p.nblocks, sp);
      const int eff = cdiv_wp(p.nblocks, per);
      const int waves = cdiv_wp(base * eff, sms);
      const double cost = waves * (per * block_clk + epi_clk) + (eff > 1 ? eff * reduce_clk : 0.0);
      if (sp == 1 || cost < best) { best = cost; splits = eff; }
    }
  }
  if (splits < 1) splits = 1;
  if (splits > p.nblocks) splits = p.nblocks;
  p.blocks_per_split = cdiv_wp(p.nblocks, splits);
  p.splits = cdiv_wp(p.nblocks, p.blocks_per_split);
  p.g_tx = WP_RH * p.TW * p.CM * 2;
  p.x_tx = WP_RH * (p.TW + 2) * cn * 2;
  p.g_bytes = ((p.g_tx + 1023) / 1024) * 1024;
  p.stage_bytes = p.g_bytes + ((p.x_tx + 1023) / 1024) * 1024;
  return 0;
}

long long wgrad_plane_workspace(const SbWgradArgs* a) {
  WgradPlaneParams p;
  wp_setup();
  if (wp_plan(a, p) != 0) return -1;
  return (long long)p.splits * 27 * p.Mtot * p.Ntot;
}

// Returns -1 when ineligible; otherwise launches the main kernel and reports the split count.
int wgrad_plane_launch(const SbWgradArgs* a, cudaStream_t stream, int* splits_out) {
  int rc = wp_setup();
  if (rc) return rc;
  WgradPlaneParams p;
  if (wp_plan(a, p) != 0) return -1;
  const long long need = (long long)p.splits * 27 * p.Mtot * p.Ntot;
  if (need > a->workspace_elems) return SB_ERR_TOO_LARGE;
  int st = (g_wp_smem - 1024) / p.stage_bytes;
  if (st > WP_MAX_STAGES) st = WP_MAX_STAGES;
  if (st < 2) return -1;
  p.stages = st;
  auto act_map = [&](CUtensorMap* m, const void* base, int c, long long ld, int cb, int box_w, bool is_x) {
    const long long D = is_x && a->xin_d ? a->xin_d : a->D, H = is_x && a->xin_h ? a->xin_h : a->H,
                    W = is_x && a->xin_w ? a->xin_w : a->W;
    long long dims[5] = {c, H, W, D, a->N};
    long long str[5] = {1, W * ld, ld, H * W * ld, D * H * W * ld};
    int box[5] = {cb, WP_RH, box_w, 1, 1};
    return make_map_bf16(m, base, 5, dims, str, box, cb * 2);
  };
  p.xoff_d = a->xoff_d; p.xoff_h = a->xoff_h; p.xoff_w = a->xoff_w;
  p.xin_D = a->xin_d ? a->xin_d : a->D;
  for (int f = 0; f < 2; ++f) p.xh_has[f] = a->xhalo[0][f] != nullptr ? 1 : 0;
  rc = act_map(&p.mapG, a->gy, a->gy_c, a->gy_ld, p.CM, p.TW, false);
  if (rc) return rc;
  rc = act_map(&p.mapX[0], a->x[0], a->x_c[0], a->x_ld[0], p.CN, p.TW + 2, true);
  if (rc) return rc;
  if (a->x_c[1] > 0) {
    rc = act_map(&p.mapX[1], a->x[1], a->x_c[1], a->x_ld[1], p.CN, p.TW + 2, true);
    if (rc) return rc;
  } else {
    p.mapX[1] = p.mapX[0];
  }
  for (int s = 0; s < 2; ++s)
    for (int f = 0; f < 2; ++f) {
      if (a->x_c[s] > 0 && a->xhalo[s][f] != nullptr) {
        const long long C = a->x_c[s];
        const long long H = a->xin_h ? a->xin_h : a->H, W = a->xin_w ? a->xin_w : a->W;
        long long dims[5] = {C, H, W, 1, a->N};
        long long str[5] = {1, W * C, C, H * W * C, H * W * C};
        int box[5] = {p.CN, WP_RH, p.TW + 2, 1, 1};
        rc = make_map_bf16(&p.mapXh[s * 2 + f], a->xhalo[s][f], 5, dims, str, box, p.CN * 2);
        if (rc) return rc;
      } else {
        p.mapXh[s * 2 + f] = p.mapX[0];
      }
    }
  p.ws = a->workspace;
  p.status = a->status;
  const int grid = 3 * p.m_tiles * p.n_tiles * p.splits;
  const size_t smem = (size_t)p.stages * p.stage_bytes + 1024;
  wgrad_plane_kernel<<<grid, 192, smem, stream>>>(p);
  sb_count_launch(1);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  *splits_out = p.splits;
  return 0;
}

}  // namespace sb
