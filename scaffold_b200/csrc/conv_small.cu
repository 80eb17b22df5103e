// 3x3x3 convolution on 8 x 8 planes (the U-Net bottleneck): one CTA per (sample, 128 output channels, slice of
// the input channels).
//
// An 8 x 8 plane gives only 64 rows, and the generic kernel's 128-voxel tiles re-read the 56 MB of bottleneck
// weights once per tile while filling 64 of 148 SMs. Here the whole sample is the tile: per 16-channel block and
// kw, ONE TMA box brings planes -1 .. D with an h halo (rows h-fastest: 10 h x 8 w = 80 rows per plane, shifted by
// kw - 1 in w, zero-filled outside), and every (kd, kh) tap of every pair of output planes reads it in place:
// two adjacent planes are 16 groups of 8 rows at one uniform stride (10 rows), so a pair of planes is a legal
// M = 128 operand whose start address moves by kd planes and kh rows. D/2 accumulators (128 columns each) fill TMEM.
// Weights: the nine (kd, kh) taps of one kw arrive as one box of the (kd,kh,kw)-ordered pack (the tap axis is
// viewed as kw x (kd,kh)). The input-channel blocks are split over CTAs; partial sums go to an fp32 workspace and a
// second kernel adds them in split order (deterministic), adds the bias and writes bf16.
//
// Role of the reference: the same layers run triton_conv3d/gather_gemm.py:112-341 (forward) and
// bwd_data.py:275-363 on MI300A; on NVIDIA its adapters fall back to cuDNN.
#include "common.cuh"
#include "host_api.h"

namespace sb {

int make_map_bf16(CUtensorMap* m, const void* base, int rank, const long long* dims, const long long* strides,
                  const int* box, int rowb);

constexpr int SM_BK = 16, SM_ROWB = 32, SM_BN = 128, SM_STAGES = 3;
constexpr int SM_PLANE_ROWS = 80;  // 10 h x 8 w

struct SmallParams {
  CUtensorMap mapA, mapB;
  int N, D, cblks, splits, cb_per_split, tiles_co, cout_pad;
  int a_bytes, stage_bytes, tx_bytes;
  float* ws;
  uint32_t* status;
};

__global__ void __launch_bounds__(192, 1) conv_small_kernel(const __grid_constant__ SmallParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[SM_STAGES], empty_bar[SM_STAGES], done_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  volatile uint32_t* abort_flag = &abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  int t = blockIdx.x;
  const int co_t = t % p.tiles_co; t /= p.tiles_co;
  const int split = t % p.splits; t /= p.splits;
  const int n = t;
  const int cb0 = split * p.cb_per_split;
  const int cb1 = min(p.cblks, cb0 + p.cb_per_split);
  const int nsteps = (cb1 - cb0) * 3;  // (channel block, kw)
  const int ntile = p.D / 2;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < SM_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&done_bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&p.mapA);
      tma_prefetch_desc(&p.mapB);
      for (int i = 0; i < nsteps; ++i) {
        const int s = i % SM_STAGES;
        const uint32_t ph = (i / SM_STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, p.status, 81)) break;
        const int cb = cb0 + i / 3, kw = i % 3;
        uint8_t* sa = smem + (size_t)s * p.stage_bytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)p.tx_bytes);
        tma_load_5d(sa, &p.mapA, &full_bar[s], cb * SM_BK, -1, kw - 1, -1, n);
        tma_load_4d(sa + p.a_bytes, &p.mapB, &full_bar[s], cb * SM_BK, co_t * SM_BN, kw, 0);
      }
    }
  } else if (warp == 1) {
    const bool leader = elect_one();
    const uint32_t idesc = make_idesc_bf16(128, SM_BN, 0, 0);
    const uint32_t swz = swizzle_code_for(SM_ROWB);
    const uint32_t a_hi = desc_hi(10u * SM_ROWB, swz);  // 8-row groups one w column (10 rows) apart
    const uint32_t b_hi = desc_hi(8u * SM_ROWB, swz);
    const uint32_t s0 = smem_u32(smem);
    const uint32_t plane_step = ((uint32_t)SM_PLANE_ROWS * SM_ROWB) >> 4;
    const uint32_t tap_step = ((uint32_t)SM_BN * SM_ROWB) >> 4;
    bool ok = true;
    for (int i = 0; i < nsteps && ok; ++i) {
      const int s = i % SM_STAGES;
      const uint32_t ph = (i / SM_STAGES) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], ph, abort_flag, p.status, 82))) { ok = false; break; }
      tc_fence_after();
      const uint32_t a_lo0 = desc_lo(s0 + (uint32_t)s * p.stage_bytes, 16u);
      const uint32_t b_lo0 = desc_lo(s0 + (uint32_t)s * p.stage_bytes + p.a_bytes, 16u);
#pragma unroll
      for (int tap = 0; tap < 9; ++tap) {
        const int kd = tap / 3, kh = tap - kd * 3;
        const uint32_t b_lo = b_lo0 + (uint32_t)tap * tap_step;
        for (int tl = 0; tl < ntile; ++tl) {
          // output planes 2 tl, 2 tl + 1 read box planes 2 tl + kd, 2 tl + kd + 1 (box plane 0 is d = -1)
          const uint32_t a_lo = a_lo0 + (uint32_t)(2 * tl + kd) * plane_step + (uint32_t)kh * (SM_ROWB >> 4);
          if (leader) tc_mma_bf16_pred(tmem_base + tl * SM_BN, a_lo, a_hi, b_lo, b_hi, idesc, (i | tap) != 0 ? 1u : 0u);
        }
      }
      if (leader) tc_commit(&empty_bar[s]);
      __syncwarp();
    }
    if (ok && leader) tc_commit(&done_bar);
    __syncwarp();
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int g = row >> 3, h = row & 7;
    bool ok = nsteps > 0 ? mbar_wait(&done_bar, 0, abort_flag, p.status, 83) : true;
    tc_fence_after();
    if (ok) {
      for (int tl = 0; tl < ntile; ++tl) {
        const int d = 2 * tl + (g >> 3), w = g & 7;
        const long long vox = ((long long)d * 8 + h) * 8 + w;
        float* dst = p.ws + ((((long long)split * p.N + n) * p.D * 64 + vox) * p.cout_pad + co_t * SM_BN);
        const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + tl * SM_BN;
        for (int c0 = 0; c0 < SM_BN; c0 += 32) {
          uint32_t v[32];
          if (nsteps > 0) {
            tmem_ld_32x32(tbase + c0, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0u;
          }
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            *reinterpret_cast<uint4*>(dst + c0 + e) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
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

// out[v][c] = bf16(bias[c] + sum_s ws[s][v][c]), channels routed to up to two destinations
struct SmallReduceParams {
  const float* ws;
  long long rows;  // N * D * 64 voxels
  int splits, cout_pad;
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  int width0, width1, ld0, ld1;
  const float* bias;
};

__global__ void __launch_bounds__(256) conv_small_reduce_kernel(const SmallReduceParams p) {
  const int oct_per_row = p.cout_pad / 8;
  const long long total = p.rows * oct_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long v = i / oct_per_row;
    const int col = (int)(i - v * oct_per_row) * 8;
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float4* src = reinterpret_cast<const float4*>(p.ws + ((long long)s * p.rows + v) * p.cout_pad + col);
      const float4 a = src[0], b = src[1];
      f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
      f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
    }
    __nv_bfloat16* dst = nullptr;
    if (col < p.width0) {
      dst = p.out0 + v * p.ld0 + col;
      if (p.bias) {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += p.bias[col + e];
      }
    } else if (col - p.width0 < p.width1) {
      dst = p.out1 + v * p.ld1 + (col - p.width0);
    }
    if (dst) {
      uint4 o;
      o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
      o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
      *reinterpret_cast<uint4*>(dst) = o;
    }
  }
}

static int g_sm_sms = 0, g_sm_smem = 0;
static int small_setup() {
  if (g_sm_sms) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SB_ERR_DRIVER;
  int lim = 0, sms = 0;
  cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaFuncSetAttribute(conv_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim - 2048) != cudaSuccess)
    return SB_ERR_DRIVER;
  g_sm_smem = lim - 2048;
  g_sm_sms = sms;
  return 0;
}

static bool small_eligible(const SbConvArgs* a) {
  if (a->ksize != 3 || a->H != 8 || a->W != 8 || a->D < 2 || a->D > 8 || (a->D & 1)) return false;
  if (a->src_c[1] > 0 || a->src_c[0] % SM_BK != 0 || a->cout_pad % SM_BN != 0 || a->wpack == nullptr) return false;
  if (a->off_d || a->off_h || a->off_w) return false;
  if ((a->in_d && a->in_d != a->D) || (a->in_h && a->in_h != a->H) || (a->in_w && a->in_w != a->W)) return false;
  if (a->halo_land[0][0] || a->halo_land[0][1] || a->slab_out[0]) return false;
  return true;
}

static int small_splits(const SbConvArgs* a, int sms) {
  const int cblks = a->src_c[0] / SM_BK;
  const int base = a->N * (a->cout_pad / SM_BN);
  int splits = sms / base;  // one wave: at most one CTA per SM
  if (splits > cblks) splits = cblks;
  if (splits < 1) splits = 1;
  // no empty split: splits * ceil(cblks / splits) may overshoot cblks by less than one slice
  const int per = (cblks + splits - 1) / splits;
  return (cblks + per - 1) / per;
}

long long conv_small_workspace(const SbConvArgs* a) {
  if (!small_eligible(a)) return 0;
  if (small_setup()) return 0;
  return (long long)small_splits(a, g_sm_sms) * a->N * a->D * 64 * a->cout_pad;
}

// Returns -1 when the call is not eligible or no workspace was given.
int conv_small_launch(const SbConvArgs* a, cudaStream_t stream) {
  if (!small_eligible(a)) return -1;
  int rc = small_setup();
  if (rc) return rc;
  SmallParams p;
  memset(&p, 0, sizeof(p));
  p.N = a->N; p.D = a->D;
  p.cblks = a->src_c[0] / SM_BK;
  p.splits = small_splits(a, g_sm_sms);
  p.cb_per_split = (p.cblks + p.splits - 1) / p.splits;
  p.tiles_co = a->cout_pad / SM_BN;
  p.cout_pad = a->cout_pad;
  const long long need = (long long)p.splits * a->N * a->D * 64 * a->cout_pad;
  if (a->workspace == nullptr || a->workspace_elems < need) return -1;
  p.ws = a->workspace;
  p.status = a->status;
  const int planes = a->D + 2;
  p.a_bytes = ((planes * SM_PLANE_ROWS * SM_ROWB + 1023) / 1024) * 1024;
  const int b_bytes = 9 * SM_BN * SM_ROWB;
  p.stage_bytes = p.a_bytes + b_bytes;
  p.tx_bytes = planes * SM_PLANE_ROWS * SM_ROWB + b_bytes;
  if (SM_STAGES * p.stage_bytes + 1024 > g_sm_smem) return -1;
  {
    const long long C = a->src_ld[0];
    long long dims[5] = {a->src_c[0], a->H, a->W, a->D, a->N};
    long long str[5] = {1, (long long)a->W * C, C, (long long)a->H * a->W * C, (long long)a->D * a->H * a->W * C};
    int box[5] = {SM_BK, 10, 8, planes, 1};
    rc = make_map_bf16(&p.mapA, a->src[0], 5, dims, str, box, SM_ROWB);
    if (rc) return rc;
  }
  {
    const long long K = a->src_c[0];
    long long dims[4] = {K, a->cout_pad, 3, 9};
    long long str[4] = {1, K, (long long)a->cout_pad * K, 3LL * a->cout_pad * K};
    int box[4] = {SM_BK, SM_BN, 1, 9};
    rc = make_map_bf16(&p.mapB, a->wpack, 4, dims, str, box, SM_ROWB);
    if (rc) return rc;
  }
  const int grid = a->N * p.splits * p.tiles_co;
  const size_t smem = (size_t)SM_STAGES * p.stage_bytes + 1024;
  conv_small_kernel<<<grid, 192, smem, stream>>>(p);
  if (cudaGetLastError() != cudaSuccess) return SB_ERR_LAUNCH;
  SmallReduceParams r;
  memset(&r, 0, sizeof(r));
  r.ws = p.ws;
  r.rows = (long long)a->N * a->D * 64;
  r.splits = p.splits;
  r.cout_pad = a->cout_pad;
  r.out0 = (__nv_bfloat16*)a->dst[0];
  r.out1 = (__nv_bfloat16*)a->dst[1];
  r.width0 = a->dst_c[0];
  r.width1 = a->dst[1] ? a->dst_c[1] : 0;
  r.ld0 = a->dst_ld[0];
  r.ld1 = a->dst_ld[1];
  if (r.width0 % 8 || r.width1 % 8 || r.ld0 % 8 || r.ld1 % 8) return SB_ERR_SHAPE;
  r.bias = a->bias;
  const long long total = r.rows * (a->cout_pad / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  conv_small_reduce_kernel<<<(int)blocks, 256, 0, stream>>>(r);
  sb_count_launch(2);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb
