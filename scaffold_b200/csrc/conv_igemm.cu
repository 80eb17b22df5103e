// Implicit-GEMM 3-D convolution on Blackwell tensor cores (sm_100a).
//
//   Y[voxel, co] = sum_{tap, ci} X[voxel + off(tap), ci] * Wp[tap][co][ci]
//
// Activations are NDHWC bf16. One CTA tile is 128 output voxels (a small brick
// h x w x d x n, h fastest) by BN output channels. Per K step the producer warp
// issues ONE 5-D TMA box load of the (shifted) input brick and one 3-D box load
// of the packed weights; TMA out-of-bounds zero fill is the convolution's zero
// padding, so no im2col buffer and no padded copy of the activation exists.
// A single elected thread issues tcgen05.mma into a TMEM accumulator
// (double-buffered, so the epilogue of tile i overlaps the main loop of tile
// i+1); four epilogue warps read TMEM with tcgen05.ld and store bf16.
//
// W-shift reuse: with rows ordered h-fastest and 8 rows per swizzle atom, a
// shift of the input by one voxel along w is a shift of the shared-memory start
// address by exactly one atom. One halo'd box (8 h x (TW+2) w) therefore serves
// the three kw taps of a 3x3x3 filter: 9 activation loads per channel block
// instead of 27.
//
// The same kernel serves forward, backward-data (weights packed transposed and
// tap-flipped by the caller), the k2s2 transposed convolution (forward: one
// tap, N = 8*Cout columns scattered to the 2x upsampled grid; backward-data:
// four strided views of the gradient, one per (kd,kh)), reading up to two
// channel-concatenated sources (the U-Net skip concat is never materialised)
// and writing up to two channel-split destinations.
//
// Role of the reference: triton_conv3d/gather_gemm.py:112-341 (forward),
// triton_conv3d/bwd_data.py:275-363, triton_conv3d/transposed.py:135-319.
#include "common.cuh"
#include "host_api.h"

namespace sb {

constexpr int MAX_STAGES = 8;
constexpr int MAX_OUTER = 32;

struct IgemmParams {
  CUtensorMap mapA[8];
  CUtensorMap mapB;
  int TH, TW, TD, TN;
  int KWS, KHS, n_outer, BK, BN;
  int stages, stage_bytes, a_bytes, b_bytes, tx_bytes;  // a_bytes: offset of B inside a stage
  int N, D, H, W;  // output voxel grid (== the grid the tile bricks walk)
  int tiles_h, tiles_w, tiles_d, tiles_n, tiles_co, num_tiles;
  int cblks, cblks0;  // channel blocks in total / in the first source
  int maps_per_tap;   // stride of the tap's map index (2 when two sources)
  signed char tap_map[MAX_OUTER];
  signed char tap_dh[MAX_OUTER], tap_dw[MAX_OUTER], tap_dd[MAX_OUTER];
  // epilogue
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  int width0, width1;  // stored channels per destination
  int ld0, ld1;        // channel stride (elements per voxel) per destination
  const float* bias;
  int scatter;  // 1: columns are (tap8, co) of a k2s2 transposed conv
  int sc_cout;
  uint32_t* status;
};

__global__ void __launch_bounds__(192, 2) igemm_kernel(const __grid_constant__ IgemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[MAX_STAGES];
  __shared__ uint64_t empty_bar[MAX_STAGES];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  volatile uint32_t* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rowb = p.BK * 2;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  const int kiters = p.n_outer * p.cblks;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      for (int i = 0; i < 8; ++i) tma_prefetch_desc(&p.mapA[i]);
      tma_prefetch_desc(&p.mapB);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        int t = tile;
        const int co_t = t % p.tiles_co; t /= p.tiles_co;
        const int w_t = t % p.tiles_w; t /= p.tiles_w;
        const int h_t = t % p.tiles_h; t /= p.tiles_h;
        const int d_t = t % p.tiles_d; t /= p.tiles_d;
        const int n_t = t;
        const int h0 = h_t * p.TH, w0 = w_t * p.TW, d0 = d_t * p.TD, n0 = n_t * p.TN;
        const int co0 = co_t * p.BN;
        for (int o = 0; o < p.n_outer && ok; ++o) {
          for (int cb = 0; cb < p.cblks; ++cb, ++it) {
            const int s = it % p.stages;
            const uint32_t ph = (it / p.stages) & 1u;
            if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
            uint8_t* sa = smem + (size_t)s * p.stage_bytes;
            uint8_t* sbm = sa + p.a_bytes;
            mbar_expect_tx(&full_bar[s], (uint32_t)p.tx_bytes);
            const int second = cb >= p.cblks0 ? 1 : 0;
            const int mi = p.tap_map[o] + second;
            const int c = (second ? cb - p.cblks0 : cb) * p.BK;
            tma_load_5d(sa, &p.mapA[mi], &full_bar[s], c, h0 + p.tap_dh[o], w0 + p.tap_dw[o],
                        d0 + p.tap_dd[o], n0);
            tma_load_3d(sbm, &p.mapB, &full_bar[s], cb * p.BK, co0, o * p.KWS * p.KHS);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // Warp-uniform control flow (wait results are voted on) keeps the descriptor arithmetic in
    // uniform registers; one elected lane issues. Descriptors are (lo, hi) words: a new operand
    // address is one add.
    {
      const bool leader = elect_one();
      const uint32_t idesc = make_idesc_bf16(128, p.BN, 0, 0);
      const uint32_t swz = swizzle_code_for(rowb);
      const int rh = p.TH + p.KHS - 1;             // rows per w column of the A box
      // 8-row groups are contiguous unless the box carries an h halo (then one w step apart)
      const uint32_t a_hi = desc_hi((uint32_t)(p.KHS > 1 ? rh : 8) * rowb, swz);
      const uint32_t b_hi = desc_hi(8u * rowb, swz);
      const uint32_t b_shift = ((uint32_t)p.BN * rowb) >> 4;
      const uint32_t a_wstep = ((uint32_t)(p.KHS > 1 ? rh : p.TH) * rowb) >> 4;
      const uint32_t a_hstep = (uint32_t)rowb >> 4;
      const int ksteps = p.BK / 16;
      const uint32_t s0 = smem_u32(smem);
      uint32_t stage = 0, sph = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++tcount) {
        const uint32_t buf = tcount & 1u;
        const uint32_t bph = (tcount >> 1) & 1u;
        if (!__all_sync(0xffffffffu, mbar_wait(&tempty_bar[buf], bph ^ 1u, abort_flag, p.status, 2))) { ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * 128u;
        for (int ki = 0; ki < kiters; ++ki) {
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], sph, abort_flag, p.status, 3))) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = s0 + stage * (uint32_t)p.stage_bytes;
          const uint32_t a_lo0 = desc_lo(sa, 16u);
          const uint32_t b_lo0 = desc_lo(sa + p.a_bytes, 16u);
          for (int kh = 0; kh < p.KHS; ++kh) {
            for (int kw = 0; kw < p.KWS; ++kw) {
              const uint32_t a_lo = a_lo0 + kw * a_wstep + kh * a_hstep;
              const uint32_t b_lo = b_lo0 + (uint32_t)(kh * p.KWS + kw) * b_shift;
              if (leader) {
                for (int k = 0; k < ksteps; ++k)
                  tc_mma_bf16_pred(acc, a_lo + 2u * k, a_hi, b_lo + 2u * k, b_hi, idesc,
                                   (ki | kh | kw | k) != 0 ? 1u : 0u);
              }
            }
          }
          if (leader) tc_commit(&empty_bar[stage]);
          __syncwarp();
          if (++stage == (uint32_t)p.stages) { stage = 0; sph ^= 1u; }
        }
        if (ok && leader) tc_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int rh = row % p.TH;
    const int rw = (row / p.TH) % p.TW;
    const int rd = (row / (p.TH * p.TW)) % p.TD;
    const int rn = row / (p.TH * p.TW * p.TD);
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++tcount) {
      const uint32_t buf = tcount & 1u;
      const uint32_t bph = (tcount >> 1) & 1u;
      if (!mbar_wait(&tfull_bar[buf], bph, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      int t = tile;
      const int co_t = t % p.tiles_co; t /= p.tiles_co;
      const int w_t = t % p.tiles_w; t /= p.tiles_w;
      const int h_t = t % p.tiles_h; t /= p.tiles_h;
      const int d_t = t % p.tiles_d; t /= p.tiles_d;
      const int n_t = t;
      const int h = h_t * p.TH + rh, w = w_t * p.TW + rw, d = d_t * p.TD + rd, n = n_t * p.TN + rn;
      const bool valid = (rn < p.TN) && h < p.H && w < p.W && d < p.D && n < p.N;
      const long long vox = (((long long)n * p.D + d) * p.H + h) * p.W + w;
      const int co0 = co_t * p.BN;
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 128u;
      const int nchunk = (p.BN + 31) / 32;
      for (int ch = 0; ch < nchunk; ++ch) {
        uint32_t v[32];
        if (p.BN >= 32) {
          tmem_ld_32x32(tbase + ch * 32, v);
        } else {
          uint32_t v16[16];
          tmem_ld_32x16(tbase, v16);
#pragma unroll
          for (int j = 0; j < 16; ++j) { v[j] = v16[j]; v[16 + j] = 0u; }
        }
        tmem_ld_wait();
        if (valid) {
          const int ngroups = p.BN >= 32 ? 4 : 2;
#pragma unroll
          for (int g2 = 0; g2 < 2; ++g2) {
            if (g2 * 2 >= ngroups) break;
            // two groups of 8 channels; they share a destination row when the split points are multiples of 16
            uint4 o[2];
            __nv_bfloat16* dst[2] = {nullptr, nullptr};
#pragma unroll
            for (int gi = 0; gi < 2; ++gi) {
              const int g = g2 * 2 + gi;
              const int col = co0 + ch * 32 + g * 8;
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[g * 8 + j]);
              if (p.scatter) {
                const int tap = col / p.sc_cout;
                const int co = col - tap * p.sc_cout;
                if (tap < 8) {
                  const int kd = tap >> 2, kh = (tap >> 1) & 1, kw = tap & 1;
                  const long long ov =
                      (((long long)n * (2 * p.D) + (2 * d + kd)) * (2 * p.H) + (2 * h + kh)) * (2 * p.W) +
                      (2 * w + kw);
                  dst[gi] = p.out0 + ov * p.ld0 + co;
                  if (p.bias) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] += p.bias[co + j];
                  }
                }
              } else if (col < p.width0) {
                dst[gi] = p.out0 + vox * p.ld0 + col;
                if (p.bias) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) f[j] += p.bias[col + j];
                }
              } else if (col - p.width0 < p.width1) {
                dst[gi] = p.out1 + vox * p.ld1 + (col - p.width0);
              }
              o[gi].x = pack_bf16x2(f[0], f[1]);
              o[gi].y = pack_bf16x2(f[2], f[3]);
              o[gi].z = pack_bf16x2(f[4], f[5]);
              o[gi].w = pack_bf16x2(f[6], f[7]);
            }
            if (dst[0] && dst[1] == dst[0] + 8 && (reinterpret_cast<uintptr_t>(dst[0]) & 31) == 0) {
              st_global_v8(dst[0], o[0], o[1]);
            } else {
              if (dst[0]) *reinterpret_cast<uint4*>(dst[0]) = o[0];
              if (dst[1]) *reinterpret_cast<uint4*>(dst[1]) = o[1];
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
  }

  // ------------------------------- teardown ---------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // copies may still be in flight towards this CTA's shared memory: give
    // them a bounded grace period before the CTA (and its TMEM) goes away
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// ---------------------------------------------------------------------------
// Host side: tensor maps and launch plans
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

static CUtensorMapSwizzle swz_enum(int rowb) {
  return rowb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                     : rowb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
}

// bf16 tensor map; dims/strides fastest first, strides in ELEMENTS (stride[0] is implicit 1)
int make_map_bf16(CUtensorMap* m, const void* base, int rank, const long long* dims, const long long* strides,
                  const int* box, int rowb) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return SB_ERR_DRIVER;
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = (cuuint64_t)dims[i];
    bx[i] = (cuuint32_t)box[i];
    es[i] = 1;
    if (i > 0) gstr[i - 1] = (cuuint64_t)strides[i] * 2ull;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return SB_ERR_ALIGN;
  for (int i = 0; i + 1 < rank; ++i)
    if (gstr[i] % 16 != 0) return SB_ERR_ALIGN;
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr,
                   bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz_enum(rowb), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : SB_ERR_TENSORMAP;
}

static int pow2_floor(int v) {
  int p = 1;
  while (p * 2 <= v) p *= 2;
  return p;
}
static int cdiv(int a, int b) { return (a + b - 1) / b; }

static int g_smem_limit = 0;
static int g_sm_count = 0;
static int device_setup() {
  if (g_smem_limit) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SB_ERR_DRIVER;
  int lim = 0, sms = 0;
  cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaFuncSetAttribute(igemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim - 2048) != cudaSuccess)
    return SB_ERR_DRIVER;
  g_smem_limit = lim - 2048;
  g_sm_count = sms;
  return 0;
}

// Choose the voxel brick and finish the geometry common to all plans.
static void choose_brick(IgemmParams& p, bool shift) {
  p.KHS = 1;
  if (shift) {
    p.TH = 8; p.TW = 16; p.TD = 1; p.TN = 1; p.KWS = 3;
  } else {
    p.KWS = 1;
    p.TH = p.H >= 8 ? 8 : pow2_floor(p.H);
    int rem = 128 / p.TH;
    p.TW = p.W >= rem ? rem : pow2_floor(p.W);
    if (p.TW > 16) p.TW = 16;
    rem = 128 / (p.TH * p.TW);
    p.TD = p.D >= rem ? rem : pow2_floor(p.D);
    rem = 128 / (p.TH * p.TW * p.TD);
    p.TN = p.N >= rem ? rem : pow2_floor(p.N);
  }
  p.tiles_h = cdiv(p.H, p.TH);
  p.tiles_w = cdiv(p.W, p.TW);
  p.tiles_d = cdiv(p.D, p.TD);
  p.tiles_n = cdiv(p.N, p.TN);
}

static int finish_and_launch(IgemmParams& p, int cout_rows, cudaStream_t stream) {
  const int rowb = p.BK * 2;
  const int rows_a = (p.TH + p.KHS - 1) * (p.TW + p.KWS - 1) * p.TD * p.TN;
  // the MMA always reads 128 rows starting at an offset of up to (KWS-1)*TH rows
  const int rows_alloc = rows_a > 128 + (p.KWS - 1) * p.TH ? rows_a : 128 + (p.KWS - 1) * p.TH;
  p.a_bytes = ((rows_alloc * rowb + 1023) / 1024) * 1024;
  p.b_bytes = p.KWS * p.KHS * p.BN * rowb;
  p.stage_bytes = ((p.a_bytes + p.b_bytes + 1023) / 1024) * 1024;
  // Two CTAs per SM when there are tiles for them and three stages fit in half the shared memory: the second
  // CTA's MMAs and epilogue fill the first one's waits (each CTA allocates 256 of the 512 TMEM columns).
  p.tiles_co = cdiv(cout_rows, p.BN);
  p.num_tiles = p.tiles_co * p.tiles_w * p.tiles_h * p.tiles_d * p.tiles_n;
  const int half = g_smem_limit / 2 - 2048;
  const bool dual = p.num_tiles > g_sm_count && (half - 1024) / p.stage_bytes >= 3;
  int st = ((dual ? half : g_smem_limit) - 1024) / p.stage_bytes;
  if (st > MAX_STAGES) st = MAX_STAGES;
  if (st < 2) return SB_ERR_SHAPE;
  p.stages = st;
  // expected transaction bytes are what the two boxes really deliver
  p.tx_bytes = rows_a * rowb + p.b_bytes;
  const IgemmParams& q = p;
  const int slots = dual ? 2 * g_sm_count : g_sm_count;
  int grid = q.num_tiles < slots ? q.num_tiles : slots;
  const size_t smem = (size_t)q.stages * q.stage_bytes + 1024;
  igemm_kernel<<<grid, 192, smem, stream>>>(q);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb

using namespace sb;

// Stride-1 "same" convolution, k in {1,3}; also backward-data when the caller
// packs the weights transposed and tap-flipped.
namespace sb {
int conv_plane_launch(const SbConvArgs* a, cudaStream_t stream);
int conv_plane2_launch(const SbConvArgs* a, cudaStream_t stream);
int conv_plane2_gn_splits(const SbConvArgs* a);
int conv_plane3_launch(const SbConvArgs* a, cudaStream_t stream);
int conv_plane3_gn_splits(const SbConvArgs* a);
int conv_small_launch(const SbConvArgs* a, cudaStream_t stream);
long long conv_small_workspace(const SbConvArgs* a);
}

// fp32 scratch elements sb_conv_fwd wants for this call (0: none)
static bool automatic(const SbConvArgs* a) { return a->force_plain == 0 || a->force_plain == 4; }

extern "C" long long sb_conv_fwd_workspace(const SbConvArgs* a) {
  return automatic(a) ? conv_small_workspace(a) : 0;
}

static bool pair_first(const SbConvArgs* a) { return a->force_plain == 0 && a->wpack_kd == nullptr; }

extern "C" int sb_conv_gn_splits(const SbConvArgs* a) {
  if (!automatic(a)) return 0;
  if (pair_first(a)) {
    const int s2 = conv_plane2_gn_splits(a);
    if (s2 > 0) return s2;
  }
  return conv_plane3_gn_splits(a);
}

// force_plain: 0 = automatic (8 x 8 plane kernel; the two-SM pair kernel for wide outputs given tap-ordered
// weights only; kd-fused or plane-walk kernel when the shape is eligible; else this file's generic kernel),
// 1 = generic kernel one tap per load, 2 = generic kernel with the w-shift reuse, 3 = generic kernel with the
// (h, w)-shift reuse, 4 = automatic without the pair kernel.
extern "C" int sb_conv_fwd(const SbConvArgs* a, cudaStream_t stream) {
  if (automatic(a)) {
    const int sm = conv_small_launch(a, stream);
    if (sm >= 0) return sm;
    // with a partial-statistics buffer only when the pair kernel is the one that sized it (sb_conv_gn_splits)
    if (pair_first(a) && (a->gn_part == nullptr || conv_plane2_gn_splits(a) > 0)) {
      const int p2 = conv_plane2_launch(a, stream);
      if (p2 >= 0) return p2;
    }
    const int p3 = conv_plane3_launch(a, stream);
    if (p3 >= 0) return p3;
    if (a->gn_part != nullptr) return SB_ERR_SHAPE;  // statistics come from the kd-fused kernel only
    if (a->wpack == nullptr) return SB_ERR_SHAPE;  // only the kd-ordered weights were given
    const int prc = conv_plane_launch(a, stream);
    if (prc >= 0) return prc;
  }
  if (a->wpack == nullptr) return SB_ERR_SHAPE;
  if (a->halo_land[0][0] || a->halo_land[0][1] || a->slab_out[0]) return SB_ERR_SHAPE;  // plane-walk kernel only
  int rc = device_setup();
  if (rc) return rc;
  IgemmParams p;
  memset(&p, 0, sizeof(p));
  const int cin_tot = a->src_c[0] + a->src_c[1];
  const int nsrc = a->src_c[1] > 0 ? 2 : 1;
  int bk = 64;
  while (bk > 16 && (a->src_c[0] % bk != 0 || cin_tot % bk != 0)) bk /= 2;
  if (a->src_c[0] % bk != 0 || cin_tot % bk != 0) return SB_ERR_SHAPE;
  p.BK = bk;
  p.BN = a->cout_pad >= 128 ? 128 : a->cout_pad;
  if (p.BN % 16 != 0 || a->cout_pad % p.BN != 0) return SB_ERR_SHAPE;
  if (a->ksize != 1 && a->ksize != 3) return SB_ERR_SHAPE;
  p.N = a->N; p.D = a->D; p.H = a->H; p.W = a->W;
  const bool can_shift = a->ksize == 3 && a->W >= 16 && a->H >= 8;
  const bool shift = can_shift && a->force_plain != 1;
  choose_brick(p, shift);
  if (shift && a->force_plain == 3) p.KHS = 3;
  const int taps = a->ksize * a->ksize * a->ksize;
  p.n_outer = taps / (p.KWS * p.KHS);
  p.maps_per_tap = nsrc;
  const int half = a->ksize / 2;
  for (int o = 0; o < p.n_outer; ++o) {
    const int t0 = o * p.KWS * p.KHS;  // taps ordered (kd, kh, kw), kw fastest
    const int kd = t0 / (a->ksize * a->ksize), kh = (t0 / a->ksize) % a->ksize, kw = t0 % a->ksize;
    p.tap_map[o] = 0;
    p.tap_dd[o] = (signed char)(kd - half + a->off_d);
    p.tap_dh[o] = (signed char)(kh - half + a->off_h);
    p.tap_dw[o] = (signed char)(kw - half + a->off_w);  // shift mode: kw == 0 -> -1, the box is TW+2 wide
  }
  p.cblks0 = a->src_c[0] / bk;
  p.cblks = cin_tot / bk;
  const int rowb = bk * 2;
  for (int s = 0; s < nsrc; ++s) {
    const long long C = a->src_ld[s];
    const long long iD = a->in_d ? a->in_d : a->D, iH = a->in_h ? a->in_h : a->H, iW = a->in_w ? a->in_w : a->W;
    long long dims[5] = {a->src_c[s], iH, iW, iD, a->N};
    long long str[5] = {1, iW * C, C, iH * iW * C, iD * iH * iW * C};
    int box[5] = {bk, p.TH + p.KHS - 1, p.TW + p.KWS - 1, p.TD, p.TN};
    rc = make_map_bf16(&p.mapA[s], a->src[s], 5, dims, str, box, rowb);
    if (rc) return rc;
  }
  for (int s = nsrc; s < 8; ++s) p.mapA[s] = p.mapA[0];
  {
    long long dims[3] = {cin_tot, a->cout_pad, taps};
    long long str[3] = {1, cin_tot, (long long)a->cout_pad * cin_tot};
    int box[3] = {bk, p.BN, p.KWS * p.KHS};
    rc = make_map_bf16(&p.mapB, a->wpack, 3, dims, str, box, rowb);
    if (rc) return rc;
  }
  p.out0 = (__nv_bfloat16*)a->dst[0];
  p.out1 = (__nv_bfloat16*)a->dst[1];
  p.width0 = a->dst_c[0];
  p.width1 = a->dst[1] ? a->dst_c[1] : 0;
  p.ld0 = a->dst_ld[0];
  p.ld1 = a->dst_ld[1];
  if (p.width0 % 8 || p.width1 % 8 || p.ld0 % 8 || p.ld1 % 8) return SB_ERR_SHAPE;
  p.bias = a->bias;
  p.scatter = 0;
  p.sc_cout = 1;
  p.status = a->status;
  return finish_and_launch(p, a->cout_pad, stream);
}

// k=2, s=2 transposed convolution, forward: pointwise GEMM with N = 8*Cout
// columns (tap-major) scattered to the upsampled grid, bias fused.
extern "C" int sb_convT_fwd(const SbConvTArgs* a, cudaStream_t stream) {
  int rc = device_setup();
  if (rc) return rc;
  IgemmParams p;
  memset(&p, 0, sizeof(p));
  int bk = 64;
  while (bk > 16 && a->cin % bk != 0) bk /= 2;
  if (a->cin % bk != 0 || a->cout % 8 != 0) return SB_ERR_SHAPE;
  const int ncols = 8 * a->cout;
  p.BK = bk;
  p.BN = ncols >= 128 ? 128 : ncols;
  if (ncols % p.BN != 0) return SB_ERR_SHAPE;
  p.N = a->N; p.D = a->D; p.H = a->H; p.W = a->W;  // input grid
  choose_brick(p, false);
  p.n_outer = 1;
  p.maps_per_tap = 1;
  p.cblks0 = p.cblks = a->cin / bk;
  const int rowb = bk * 2;
  {
    const long long C = a->src_ld;
    long long dims[5] = {a->cin, a->H, a->W, a->D, a->N};
    long long str[5] = {1, (long long)a->W * C, C, (long long)a->H * a->W * C, (long long)a->D * a->H * a->W * C};
    int box[5] = {bk, p.TH, p.TW, p.TD, p.TN};
    rc = make_map_bf16(&p.mapA[0], a->src, 5, dims, str, box, rowb);
    if (rc) return rc;
    for (int s = 1; s < 8; ++s) p.mapA[s] = p.mapA[0];
  }
  {
    long long dims[3] = {a->cin, ncols, 1};
    long long str[3] = {1, a->cin, (long long)ncols * a->cin};
    int box[3] = {bk, p.BN, 1};
    rc = make_map_bf16(&p.mapB, a->wpack, 3, dims, str, box, rowb);
    if (rc) return rc;
  }
  p.out0 = (__nv_bfloat16*)a->dst;
  p.width0 = a->cout;
  p.ld0 = a->dst_ld;
  p.bias = a->bias;
  p.scatter = 1;
  p.sc_cout = a->cout;
  p.status = a->status;
  return finish_and_launch(p, ncols, stream);
}

// k=2, s=2 transposed convolution, backward-data: gx[v, ci] = sum_{tap,co}
// gy[2v+tap, co] * W[ci, co, tap]. The gradient is read through four strided
// views (one per (kd,kh)); kw is folded into the channel axis (2*Cout wide).
extern "C" int sb_convT_dgrad(const SbConvTArgs* a, cudaStream_t stream) {
  int rc = device_setup();
  if (rc) return rc;
  IgemmParams p;
  memset(&p, 0, sizeof(p));
  // here: src = gy [N, 2D, 2H, 2W, cout], dst = gx [N, D, H, W, cin]; a->cout is the
  // channel count of gy, a->cin the channel count of gx; wpack = [4][cin_pad][2*cout]
  const int kc = 2 * a->cout;
  int bk = 64;
  while (bk > 16 && kc % bk != 0) bk /= 2;
  if (kc % bk != 0 || a->cin % 8 != 0) return SB_ERR_SHAPE;
  const int rows = a->wrows;
  p.BK = bk;
  p.BN = rows >= 128 ? 128 : rows;
  if (p.BN % 16 != 0 || rows % p.BN != 0) return SB_ERR_SHAPE;
  p.N = a->N; p.D = a->D; p.H = a->H; p.W = a->W;  // gx grid
  choose_brick(p, false);
  p.n_outer = 4;
  p.maps_per_tap = 1;
  p.cblks0 = p.cblks = kc / bk;
  const int rowb = bk * 2;
  const long long C = a->src_ld;  // channel stride of gy
  const long long W2 = 2LL * a->W, H2 = 2LL * a->H, D2 = 2LL * a->D;
  for (int o = 0; o < 4; ++o) {
    const int kd = o >> 1, kh = o & 1;
    const __nv_bfloat16* base = (const __nv_bfloat16*)a->src + ((long long)kd * H2 + kh) * W2 * C;
    // when ld == cout the pair (kw, co) is one contiguous run of 2*cout elements
    if (C != a->cout) return SB_ERR_SHAPE;
    long long dims[5] = {kc, a->H, a->W, a->D, a->N};
    long long str[5] = {1, 2 * W2 * C, 2 * C, 2 * H2 * W2 * C, D2 * H2 * W2 * C};
    int box[5] = {bk, p.TH, p.TW, p.TD, p.TN};
    rc = make_map_bf16(&p.mapA[o], base, 5, dims, str, box, rowb);
    if (rc) return rc;
    p.tap_map[o] = (signed char)o;
  }
  for (int s = 4; s < 8; ++s) p.mapA[s] = p.mapA[0];
  {
    long long dims[3] = {kc, rows, 4};
    long long str[3] = {1, kc, (long long)rows * kc};
    int box[3] = {bk, p.BN, 1};
    rc = make_map_bf16(&p.mapB, a->wpack, 3, dims, str, box, rowb);
    if (rc) return rc;
  }
  p.out0 = (__nv_bfloat16*)a->dst;
  p.width0 = a->cin;
  p.ld0 = a->dst_ld;
  p.scatter = 0;
  p.sc_cout = 1;
  p.status = a->status;
  return finish_and_launch(p, rows, stream);
}
