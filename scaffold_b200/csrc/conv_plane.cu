// "Plane-walk" 3x3x3 convolution on Blackwell tensor cores (sm_100a): the
// high-reuse variant of the implicit GEMM for volumes at least 8 x 16 in (h, w).
//
// A CTA job is an 8(h) x 16(w) output column, TD consecutive d planes deep, by
// BN output channels. Shared memory holds two rings:
//   * activation PLANES: one 5-D TMA box (BK channels x 10 h x 18 w) per input
//     plane and channel block. Rows are ordered h-fastest, so the operand of
//     tap (kh, kw) is the same box read from a start address shifted by
//     (kw * 10 + kh) rows with a stride of 10 rows between 8-row groups: one
//     box feeds all 9 in-plane taps, and each plane feeds up to three output
//     planes (kd). The shared-memory swizzle is a function of the absolute
//     address, so a row-shifted start needs no re-layout.
//   * weight TAPS: one (BK x BN) box per tap, each used by all TD planes.
// Per 128 x BN x (27*BK) tile this moves ~(TD+2)/TD * 23 KB of activations and
// 27*BN*BK*2/TD bytes of weights, against 27 * (16 + BN*BK*2/1024) KB for a
// tap-at-a-time implicit GEMM.
//
// Warp roles: 0 = plane producer, 1 = tap producer, 2 = MMA issuer (one
// thread), 3..6 = epilogue (TMEM -> registers -> bf16 global). Accumulators
// live in TMEM (TD x BN columns, double-buffered when they fit). Every wait is
// bounded and reports to the status word.
//
// Role of the reference: triton_conv3d/gather_gemm.py:112-341 (forward) and
// triton_conv3d/bwd_data.py:275-363 (backward-data, via flipped/transposed packing).
#include "common.cuh"
#include "host_api.h"

namespace sb {

int make_map_bf16(CUtensorMap* m, const void* base, int rank, const long long* dims, const long long* strides,
                  const int* box, int rowb);

constexpr int PL_MAX_A = 8;
constexpr int PL_MAX_B = 16;
constexpr int PL_RH = 10;  // rows per w column of a plane box (8 + halo)
constexpr int PL_RW = 18;  // w columns of a plane box (16 + halo)

struct PlaneParams {
  CUtensorMap mapA[2];
  CUtensorMap mapB;
  int BK, BN, TD;
  int a_slots, b_slots, a_slot_bytes, b_slot_bytes, a_tx, b_tx;
  int n_bufs;
  int N, D, H, W;
  int tiles_h, tiles_w, groups_d, tiles_co, num_jobs;
  int cblks, cblks0;
  int off_d, off_h, off_w;  // position of output voxel 0 inside the (possibly halo'd) sources
  // fused depth halo: landing slabs of the neighbours' boundary planes, guarded by flag words
  CUtensorMap mapHalo[4];  // [source * 2 + face]
  int halo_has[2], in_D;
  const uint32_t* halo_flag[2];
  uint32_t halo_epoch;
  long long halo_wait_ticks;
  // backward-data with halo: output planes 0 and D-1 go to slabs
  __nv_bfloat16* slab_out[2];
  int slab_ld, slab_mode;
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  int width0, width1, ld0, ld1;
  const float* bias;
  uint32_t* status;
};

struct JobCoord {
  int co0, h0, w0, d0, n;
};

__device__ __forceinline__ JobCoord decode_job(const PlaneParams& p, int job) {
  JobCoord j;
  int t = job;
  j.co0 = (t % p.tiles_co) * p.BN; t /= p.tiles_co;
  j.w0 = (t % p.tiles_w) * 16; t /= p.tiles_w;
  j.h0 = (t % p.tiles_h) * 8; t /= p.tiles_h;
  j.d0 = (t % p.groups_d) * p.TD; t /= p.groups_d;
  j.n = t;
  return j;
}

template <int TD, int KSTEPS>
__global__ void __launch_bounds__(224, 1) conv_plane_kernel(const __grid_constant__ PlaneParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_b = smem + (size_t)p.a_slots * p.a_slot_bytes;
  __shared__ uint64_t a_full[PL_MAX_A], a_empty[PL_MAX_A];
  __shared__ uint64_t b_full[PL_MAX_B], b_empty[PL_MAX_B];
  __shared__ uint64_t tfull[2];
  __shared__ uint64_t tempty[8];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  volatile uint32_t* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int BK = KSTEPS * 16;
  constexpr int rowb = BK * 2;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < p.a_slots; ++s) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
    for (int s = 0; s < p.b_slots; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
    for (int b = 0; b < 2; ++b) mbar_init(&tfull[b], 1);
    for (int a = 0; a < 8; ++a) mbar_init(&tempty[a], 4);
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
  constexpr int planes = TD + 2;

  if (warp == 0) {
    // --------------------------- activation planes ---------------------------
    if (lane == 0) {
      tma_prefetch_desc(&p.mapA[0]);
      tma_prefetch_desc(&p.mapA[1]);
      uint32_t it = 0;
      bool ok = true;
      bool halo_ready[2] = {false, false};
      for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x) {
        const JobCoord jc = decode_job(p, job);
        for (int cb = 0; cb < p.cblks && ok; ++cb) {
          const int second = cb >= p.cblks0 ? 1 : 0;
          const int c = (second ? cb - p.cblks0 : cb) * BK;
          for (int j = 0; j < planes; ++j, ++it) {
            const int s = it % p.a_slots;
            const uint32_t ph = (it / p.a_slots) & 1u;
            if (!mbar_wait(&a_empty[s], ph ^ 1u, abort_flag, p.status, 21)) { ok = false; break; }
            const int dz = jc.d0 - 1 + j + p.off_d;
            const int face = dz < 0 ? 0 : (dz >= p.in_D ? 1 : -1);
            if (face >= 0 && p.halo_has[face]) {
              // a neighbour's boundary plane: wait (bounded) until its push landed, then read it locally
              if (!halo_ready[face]) {
                if (p.halo_flag[face] != nullptr) {
                  const long long t0 = clock64();
                  uint32_t v;
                  while (true) {
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.halo_flag[face]) : "memory");
                    if ((int)(v - p.halo_epoch) >= 0) break;
                    if (*abort_flag || clock64() - t0 > p.halo_wait_ticks) {
                      *abort_flag = 1u;
                      report(p.status, ST_FLAG_TIMEOUT, 27, blockIdx.x, face);
                      ok = false;
                      break;
                    }
                    __nanosleep(32);
                  }
                  if (!ok) break;
                  asm volatile("fence.proxy.async;" ::: "memory");
                }
                halo_ready[face] = true;
              }
              mbar_expect_tx(&a_full[s], (uint32_t)p.a_tx);
              tma_load_5d(smem + (size_t)s * p.a_slot_bytes, &p.mapHalo[second * 2 + face], &a_full[s], c,
                          jc.h0 - 1 + p.off_h, jc.w0 - 1 + p.off_w, 0, jc.n);
            } else {
              mbar_expect_tx(&a_full[s], (uint32_t)p.a_tx);
              tma_load_5d(smem + (size_t)s * p.a_slot_bytes, &p.mapA[second], &a_full[s], c, jc.h0 - 1 + p.off_h,
                          jc.w0 - 1 + p.off_w, dz, jc.n);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ weight taps ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&p.mapB);
      uint32_t it = 0;
      bool ok = true;
      for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x) {
        const JobCoord jc = decode_job(p, job);
        for (int cb = 0; cb < p.cblks && ok; ++cb) {
          for (int tap = 0; tap < 27; ++tap, ++it) {
            const int s = it % p.b_slots;
            const uint32_t ph = (it / p.b_slots) & 1u;
            if (!mbar_wait(&b_empty[s], ph ^ 1u, abort_flag, p.status, 22)) { ok = false; break; }
            mbar_expect_tx(&b_full[s], (uint32_t)p.b_tx);
            tma_load_3d(smem_b + (size_t)s * p.b_slot_bytes, &p.mapB, &b_full[s], cb * BK, jc.co0, tap);
          }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------- MMA issuer -------------------------------
    // The whole warp runs this loop with warp-uniform control flow (every wait result is
    // voted on), so descriptor arithmetic stays in uniform registers; one elected lane
    // issues the tcgen05 instructions. Descriptors are kept as (lo, hi) words so that a
    // new operand address is one integer add; all plane / k loops are unrolled.
    {
      const bool leader = elect_one();
      const uint32_t idesc = make_idesc_bf16(128, p.BN, 0, 0);
      const uint32_t swz = swizzle_code_for(rowb);
      const uint32_t a_hi = desc_hi((uint32_t)PL_RH * rowb, swz);
      const uint32_t b_hi = desc_hi(8u * rowb, swz);
      const uint32_t sa0 = smem_u32(smem), sb0 = smem_u32(smem_b);
      uint32_t a_slot = 0, a_par = 0, b_slot = 0, b_par = 0, jcount = 0;
      uint32_t acc_uses[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      bool ok = true;
      for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x, ++jcount) {
        const uint32_t buf = jcount % p.n_bufs;
        for (int cb = 0; cb < p.cblks && ok; ++cb) {
          uint32_t pl_lo[planes], pl_slot[planes], pl_par[planes];
#pragma unroll
          for (int j = 0; j < planes; ++j) {
            uint32_t sidx = a_slot + j, par = a_par;
            if (sidx >= (uint32_t)p.a_slots) { sidx -= p.a_slots; par ^= 1u; }
            pl_slot[j] = sidx;
            pl_par[j] = par;
            pl_lo[j] = desc_lo(sa0 + sidx * p.a_slot_bytes, 16u);
          }
          int waited = 0;  // planes of this (job, cb) whose arrival has been observed
#pragma unroll
          for (int kd = 0; kd < 3; ++kd) {
            for (int khw = 0; khw < 9 && ok; ++khw) {
              const int kh = khw / 3, kw = khw - kh * 3;
              if (!__all_sync(0xffffffffu, mbar_wait(&b_full[b_slot], b_par, abort_flag, p.status, 23))) { ok = false; break; }
              tc_fence_after();
              const uint32_t b_lo = desc_lo(sb0 + b_slot * p.b_slot_bytes, 16u);
              const uint32_t tap_off = ((uint32_t)(kw * PL_RH + kh) * rowb) >> 4;
              const bool first = kd == 0 && (cb | khw) == 0;
#pragma unroll
              for (int t = 0; t < TD; ++t) {
                const int j = t + kd;
                if (j >= waited) {
                  if (!__all_sync(0xffffffffu, mbar_wait(&a_full[pl_slot[j]], pl_par[j], abort_flag, p.status, 24))) { ok = false; break; }
                  tc_fence_after();
                  waited = j + 1;
                }
                const uint32_t acc_i = buf * TD + t;
                if (kd == 0 && first) {
                  const uint32_t u = acc_uses[acc_i]++;
                  if (!__all_sync(0xffffffffu, mbar_wait(&tempty[acc_i], (u & 1u) ^ 1u, abort_flag, p.status, 25))) { ok = false; break; }
                  tc_fence_after();
                }
                const uint32_t a_lo = pl_lo[j] + tap_off;
                const uint32_t acc = tmem_base + acc_i * p.BN;
#pragma unroll
                for (int k = 0; k < KSTEPS; ++k) {
                  if (leader) {
                    if (kd == 0 && k == 0)
                      tc_mma_bf16_pred(acc, a_lo, a_hi, b_lo, b_hi, idesc, first ? 0u : 1u);
                    else
                      tc_mma_bf16_acc(acc, a_lo + 2u * k, a_hi, b_lo + 2u * k, b_hi, idesc);
                  }
                }
              }
              if (!ok) break;
              if (leader) tc_commit(&b_empty[b_slot]);
              __syncwarp();
              if (++b_slot == (uint32_t)p.b_slots) { b_slot = 0; b_par ^= 1u; }
            }
            if (!ok) break;
            // planes that no later phase of this (job, cb) reads
            if (kd < 2) {
              if (leader) tc_commit(&a_empty[pl_slot[kd]]);
            } else {
#pragma unroll
              for (int j = 2; j < planes; ++j)
                if (leader) tc_commit(&a_empty[pl_slot[j]]);
            }
          }
          a_slot += planes;
          while (a_slot >= (uint32_t)p.a_slots) { a_slot -= p.a_slots; a_par ^= 1u; }
        }
        if (ok && leader) tc_commit(&tfull[buf]);
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int rh = row & 7, rw = row >> 3;
    uint32_t jcount = 0;
    bool ok = true;
    for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x, ++jcount) {
      const uint32_t buf = jcount % p.n_bufs;
      const uint32_t use = jcount / p.n_bufs;
      if (!mbar_wait(&tfull[buf], use & 1u, abort_flag, p.status, 26)) { ok = false; break; }
      tc_fence_after();
      const JobCoord jc = decode_job(p, job);
      const int h = jc.h0 + rh, w = jc.w0 + rw;
      for (int t = 0; t < TD; ++t) {
        const int d = jc.d0 + t;
        const bool valid = h < p.H && w < p.W && d < p.D;
        long long vox = (((long long)jc.n * p.D + d) * p.H + h) * p.W + w;
        __nv_bfloat16* slab = nullptr;
        if (p.slab_mode) {
          // output grid = D+2 planes: the two outermost are the halo's gradient and live in slabs
          if (d == 0) slab = p.slab_out[0];
          else if (d == p.D - 1) slab = p.slab_out[1];
          if (slab) vox = ((long long)jc.n * p.H + h) * p.W + w;
          else vox = (((long long)jc.n * (p.D - 2) + (d - 1)) * p.H + h) * p.W + w;
        }
        const uint32_t acc_i = buf * TD + t;
        const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + acc_i * p.BN;
        const int nchunk = (p.BN + 31) / 32;
        for (int ch = 0; ch < nchunk; ++ch) {
          uint32_t v[32];
          if (p.BN >= 32) {
            tmem_ld_32x32(tbase + ch * 32, v);
          } else {
            uint32_t v16[16];
            tmem_ld_32x16(tbase, v16);
#pragma unroll
            for (int e = 0; e < 16; ++e) { v[e] = v16[e]; v[16 + e] = 0u; }
          }
          tmem_ld_wait();
          if (valid) {
            const int ngroups = p.BN >= 32 ? 4 : 2;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (g >= ngroups) break;
              const int col = jc.co0 + ch * 32 + g * 8;
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[g * 8 + e]);
              __nv_bfloat16* dst = nullptr;
              if (slab) {
                if (col < p.width0 + p.width1) dst = slab + vox * p.slab_ld + col;
              } else if (col < p.width0) {
                dst = p.out0 + vox * p.ld0 + col;
                if (p.bias) {
#pragma unroll
                  for (int e = 0; e < 8; ++e) f[e] += p.bias[col + e];
                }
              } else if (col - p.width0 < p.width1) {
                dst = p.out1 + vox * p.ld1 + (col - p.width0);
              }
              if (dst) {
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]);
                o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]);
                o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(dst) = o;
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc_i]);
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

static int g_pl_smem = 0, g_pl_sms = 0;
static int pl_setup() {
  if (g_pl_smem) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SB_ERR_DRIVER;
  int lim = 0, sms = 0;
  cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const void* fns[9] = {
      (const void*)conv_plane_kernel<1, 1>, (const void*)conv_plane_kernel<1, 2>, (const void*)conv_plane_kernel<1, 4>,
      (const void*)conv_plane_kernel<2, 1>, (const void*)conv_plane_kernel<2, 2>, (const void*)conv_plane_kernel<2, 4>,
      (const void*)conv_plane_kernel<4, 1>, (const void*)conv_plane_kernel<4, 2>, (const void*)conv_plane_kernel<4, 4>};
  for (int i = 0; i < 9; ++i)
    if (cudaFuncSetAttribute(fns[i], cudaFuncAttributeMaxDynamicSharedMemorySize, lim - 2048) != cudaSuccess)
      return SB_ERR_DRIVER;
  g_pl_smem = lim - 2048;
  g_pl_sms = sms;
  return 0;
}

static int cdiv_pl(int a, int b) { return (a + b - 1) / b; }

// Returns -1 when the shape is not eligible (the caller then uses the generic kernel).
int conv_plane_launch(const SbConvArgs* a, cudaStream_t stream) {
  if (a->ksize != 3 || a->W < 16 || a->H < 8) return -1;
  int rc = pl_setup();
  if (rc) return rc;
  PlaneParams p;
  memset(&p, 0, sizeof(p));
  const int cin_tot = a->src_c[0] + a->src_c[1];
  const int nsrc = a->src_c[1] > 0 ? 2 : 1;
  int bk = 64;
  while (bk > 16 && (a->src_c[0] % bk != 0 || cin_tot % bk != 0)) bk /= 2;
  if (a->src_c[0] % bk != 0 || cin_tot % bk != 0) return SB_ERR_SHAPE;
  p.BK = bk;
  p.BN = a->cout_pad >= 128 ? 128 : a->cout_pad;
  if (p.BN % 16 != 0 || a->cout_pad % p.BN != 0) return SB_ERR_SHAPE;
  p.N = a->N; p.D = a->D; p.H = a->H; p.W = a->W;
  p.tiles_h = cdiv_pl(a->H, 8);
  p.tiles_w = cdiv_pl(a->W, 16);
  p.tiles_co = a->cout_pad / p.BN;
  const int rowb = bk * 2;
  p.a_tx = PL_RH * PL_RW * rowb;
  p.a_slot_bytes = ((p.a_tx + 1023) / 1024) * 1024;
  p.b_tx = p.BN * rowb;
  p.b_slot_bytes = ((p.b_tx + 1023) / 1024) * 1024;
  const int max_acc = 512 / p.BN;
  // depth of the job: as deep as keeps >= 2 jobs per SM, fits TMEM and leaves >= 3 weight slots
  int td = 4;
  for (;; td /= 2) {
    const long long jobs = (long long)a->N * cdiv_pl(a->D, td) * p.tiles_h * p.tiles_w * p.tiles_co;
    const int a_need = (td + 2) * p.a_slot_bytes + 3 * p.b_slot_bytes;
    if (td == 1) break;
    if (td <= max_acc && td <= a->D && jobs >= 2LL * g_pl_sms && a_need <= g_pl_smem - 1024) break;
  }
  p.TD = td;
  p.n_bufs = max_acc / td >= 2 ? 2 : 1;
  p.groups_d = cdiv_pl(a->D, td);
  p.num_jobs = a->N * p.groups_d * p.tiles_h * p.tiles_w * p.tiles_co;
  const int budget = g_pl_smem - 1024;
  int a_slots = td + 3;
  while (a_slots > td + 1 && a_slots * p.a_slot_bytes + 3 * p.b_slot_bytes > budget) --a_slots;
  if (a_slots > PL_MAX_A) a_slots = PL_MAX_A;
  if (a_slots < td + 2 && a_slots * p.a_slot_bytes + 3 * p.b_slot_bytes > budget) return SB_ERR_SHAPE;
  int b_slots = (budget - a_slots * p.a_slot_bytes) / p.b_slot_bytes;
  if (b_slots > PL_MAX_B) b_slots = PL_MAX_B;
  if (b_slots < 2) return SB_ERR_SHAPE;
  p.a_slots = a_slots;
  p.b_slots = b_slots;
  p.cblks0 = a->src_c[0] / bk;
  p.cblks = cin_tot / bk;
  for (int s = 0; s < nsrc; ++s) {
    const long long C = a->src_ld[s];
    const long long iD = a->in_d ? a->in_d : a->D, iH = a->in_h ? a->in_h : a->H, iW = a->in_w ? a->in_w : a->W;
    long long dims[5] = {a->src_c[s], iH, iW, iD, a->N};
    long long str[5] = {1, iW * C, C, iH * iW * C, iD * iH * iW * C};
    int box[5] = {bk, PL_RH, PL_RW, 1, 1};
    rc = make_map_bf16(&p.mapA[s], a->src[s], 5, dims, str, box, rowb);
    if (rc) return rc;
  }
  if (nsrc == 1) p.mapA[1] = p.mapA[0];
  {
    long long dims[3] = {cin_tot, a->cout_pad, 27};
    long long str[3] = {1, cin_tot, (long long)a->cout_pad * cin_tot};
    int box[3] = {bk, p.BN, 1};
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
  p.status = a->status;
  p.off_d = a->off_d; p.off_h = a->off_h; p.off_w = a->off_w;
  p.in_D = a->in_d ? a->in_d : a->D;
  for (int f = 0; f < 2; ++f) {
    p.halo_has[f] = a->halo_land[0][f] != nullptr ? 1 : 0;
    p.halo_flag[f] = a->halo_flag[f];
    for (int s = 0; s < 2; ++s) {
      const int idx = s * 2 + f;
      if (s < nsrc && a->halo_land[s][f] != nullptr) {
        const long long C = a->src_c[s];
        const long long iH = a->in_h ? a->in_h : a->H, iW = a->in_w ? a->in_w : a->W;
        long long dims[5] = {C, iH, iW, 1, a->N};
        long long str[5] = {1, iW * C, C, iH * iW * C, iH * iW * C};
        int box[5] = {bk, PL_RH, PL_RW, 1, 1};
        rc = make_map_bf16(&p.mapHalo[idx], a->halo_land[s][f], 5, dims, str, box, rowb);
        if (rc) return rc;
      } else {
        p.mapHalo[idx] = p.mapA[0];
      }
    }
  }
  p.halo_epoch = a->halo_epoch;
  p.halo_wait_ticks = (long long)((a->halo_wait_s > 0 ? a->halo_wait_s : 2.0) * 1.8e9);
  p.slab_mode = a->slab_out[0] != nullptr ? 1 : 0;
  p.slab_out[0] = (__nv_bfloat16*)a->slab_out[0];
  p.slab_out[1] = (__nv_bfloat16*)a->slab_out[1];
  p.slab_ld = a->slab_ld;
  if (p.slab_mode && (p.slab_ld % 8 != 0 || a->D < 3)) return SB_ERR_SHAPE;
  const int grid = p.num_jobs < g_pl_sms ? p.num_jobs : g_pl_sms;
  const size_t smem = (size_t)p.a_slots * p.a_slot_bytes + (size_t)p.b_slots * p.b_slot_bytes + 1024;
#define SB_PL_LAUNCH(TD_, KS_) conv_plane_kernel<TD_, KS_><<<grid, 224, smem, stream>>>(p)
  const int ks = bk / 16;
  if (td == 4) { if (ks == 4) SB_PL_LAUNCH(4, 4); else if (ks == 2) SB_PL_LAUNCH(4, 2); else SB_PL_LAUNCH(4, 1); }
  else if (td == 2) { if (ks == 4) SB_PL_LAUNCH(2, 4); else if (ks == 2) SB_PL_LAUNCH(2, 2); else SB_PL_LAUNCH(2, 1); }
  else { if (ks == 4) SB_PL_LAUNCH(1, 4); else if (ks == 2) SB_PL_LAUNCH(1, 2); else SB_PL_LAUNCH(1, 1); }
#undef SB_PL_LAUNCH
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb
