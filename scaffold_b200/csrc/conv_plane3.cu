// Plane-walk 3x3x3 convolution, kd-fused variant for narrow outputs (BN <= 64 channels per tile).
//
// With 64 output channels a 128 x 64 x 16 MMA re-reads its 4 KB activation tile from shared memory
// for only 32 tensor-core cycles of work: operand delivery, not math, is the limit. The same
// activation tile (input plane j, in-plane shift (kh,kw)) is needed by up to three output planes
// t = j - kd. This variant issues those as ONE MMA: the weight taps kd = 2,1,0 of a (kh,kw) pair sit
// back to back in shared memory (N = 3 x BN rows) and the accumulators of consecutive output planes
// sit back to back in TMEM, so D = acc[t_lo .. t_hi] is one N <= 192 column range. Activation reads
// per unit of math halve.
//
// All planes of a (job, channel block) stay resident while the nine (kh,kw) pairs run, so plane SETS
// are double-buffered; to make two sets fit, channel blocks are 32 wide (64-byte rows, 64B swizzle).
// Weight taps arrive as [kh][kw][2-kd] boxes of three taps.
//
// Everything else (row-shifted descriptors, TMA zero padding, warp roles, bounded waits, epilogue)
// is as in conv_plane.cu.
#include "common.cuh"
#include "host_api.h"

namespace sb {

int make_map_bf16(CUtensorMap* m, const void* base, int rank, const long long* dims, const long long* strides,
                  const int* box, int rowb);

constexpr int P3_BK = 32;
constexpr int P3_ROWB = 64;
constexpr int P3_RH = 10, P3_RW = 18;
constexpr int P3_MAX_B = 8;

struct Plane3Params {
  CUtensorMap mapA[2];
  CUtensorMap mapB;
  int BN, TD;
  int b_slots, a_slot_bytes, b_slot_bytes, a_tx, b_tx;
  int N, D, H, W;
  int tiles_h, tiles_w, groups_d, tiles_co, num_jobs;
  int cblks, cblks0;
  int off_d, off_h, off_w;
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  int width0, width1, ld0, ld1;
  const float* bias;
  uint32_t* status;
  unsigned long long* stall;  // optional stall counters (clock ticks summed over CTAs), null = off
};

struct P3Job { int co0, h0, w0, d0, n; };
__device__ __forceinline__ P3Job p3_decode(const Plane3Params& p, int job) {
  P3Job j;
  int t = job;
  j.co0 = (t % p.tiles_co) * p.BN; t /= p.tiles_co;
  j.w0 = (t % p.tiles_w) * 16; t /= p.tiles_w;
  j.h0 = (t % p.tiles_h) * 8; t /= p.tiles_h;
  j.d0 = (t % p.groups_d) * p.TD; t /= p.groups_d;
  j.n = t;
  return j;
}

template <int TD>
__global__ void __launch_bounds__(224, 1) conv_plane3_kernel(const __grid_constant__ Plane3Params p) {
  constexpr int planes = TD + 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_b = smem + (size_t)2 * planes * p.a_slot_bytes;
  __shared__ uint64_t a_full[2 * planes];
  __shared__ uint64_t set_empty[2];
  __shared__ uint64_t b_full[P3_MAX_B], b_empty[P3_MAX_B];
  __shared__ uint64_t tfull[2];
  __shared__ uint64_t tempty[8];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  volatile uint32_t* abort_flag = &abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < 2 * planes; ++s) mbar_init(&a_full[s], 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&set_empty[s], 1); mbar_init(&tfull[s], 1); }
    for (int s = 0; s < p.b_slots; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
    for (int a = 0; a < 8; ++a) mbar_init(&tempty[a], 4);
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------- activation plane sets -------------------------
    if (lane == 0) {
      tma_prefetch_desc(&p.mapA[0]);
      tma_prefetch_desc(&p.mapA[1]);
      uint32_t uses = 0;
      bool ok = true;
      for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x) {
        const P3Job jc = p3_decode(p, job);
        for (int cb = 0; cb < p.cblks && ok; ++cb, ++uses) {
          const uint32_t set = uses & 1u, ph = (uses >> 1) & 1u;
          if (!mbar_wait(&set_empty[set], ph ^ 1u, abort_flag, p.status, 71)) { ok = false; break; }
          const int second = cb >= p.cblks0 ? 1 : 0;
          const int c = (second ? cb - p.cblks0 : cb) * P3_BK;
          for (int j = 0; j < planes; ++j) {
            const int s = set * planes + j;
            mbar_expect_tx(&a_full[s], (uint32_t)p.a_tx);
            tma_load_5d(smem + (size_t)s * p.a_slot_bytes, &p.mapA[second], &a_full[s], c, jc.h0 - 1 + p.off_h,
                        jc.w0 - 1 + p.off_w, jc.d0 - 1 + j + p.off_d, jc.n);
          }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------- weight taps: three (kd) per box ---------------------
    if (lane == 0) {
      tma_prefetch_desc(&p.mapB);
      uint32_t it = 0;
      bool ok = true;
      for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x) {
        const P3Job jc = p3_decode(p, job);
        for (int cb = 0; cb < p.cblks && ok; ++cb) {
          for (int khw = 0; khw < 9; ++khw, ++it) {
            const int s = it % p.b_slots;
            const uint32_t ph = (it / p.b_slots) & 1u;
            if (!mbar_wait(&b_empty[s], ph ^ 1u, abort_flag, p.status, 72)) { ok = false; break; }
            mbar_expect_tx(&b_full[s], (uint32_t)p.b_tx);
            tma_load_3d(smem_b + (size_t)s * p.b_slot_bytes, &p.mapB, &b_full[s], cb * P3_BK, jc.co0, khw * 3);
          }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------- MMA issuer -------------------------------
    // Measured on this part: one thread can keep the tensor pipe full only if nothing but integer
    // adds sits between consecutive tcgen05.mma (the pipe accepts about one instruction ahead), and
    // a 128 x N x 16 MMA costs max(N/2, 32 + N/4) cycles. So all waits are hoisted out of the MMA
    // runs: accumulators at job start, planes at channel-block start, weights once per (kh, kw).
    const bool leader = elect_one();
    const uint32_t swz = swizzle_code_for(P3_ROWB);
    const uint32_t a_hi = desc_hi((uint32_t)P3_RH * P3_ROWB, swz);
    const uint32_t b_hi = desc_hi(8u * P3_ROWB, swz);
    uint32_t idesc[4];
#pragma unroll
    for (int n = 1; n <= 3; ++n) idesc[n] = make_idesc_bf16(128, n * p.BN, 0, 0);
    const uint32_t sa0 = smem_u32(smem), sb0 = smem_u32(smem_b);
    const uint32_t b_tap = ((uint32_t)p.BN * P3_ROWB) >> 4;  // one tap's rows, in descriptor units
    uint32_t uses = 0, b_slot = 0, b_par = 0, jcount = 0;
    bool ok = true;
    long long st_b = 0, st_a = 0, st_t = 0;
    const long long st_begin = clock64();
#define P3_TIMED(counter, expr) \
  [&]() { const long long c0_ = p.stall ? clock64() : 0; const bool r_ = (expr); if (p.stall) counter += clock64() - c0_; return r_; }()
    for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x, ++jcount) {
      const uint32_t buf = jcount & 1u, buf_par = ((jcount >> 1) & 1u) ^ 1u;
      for (int t = 0; t < TD; ++t)
        if (!P3_TIMED(st_t, __all_sync(0xffffffffu, mbar_wait(&tempty[buf * TD + t], buf_par, abort_flag, p.status, 75)))) { ok = false; break; }
      if (!ok) break;
      const uint32_t acc0 = tmem_base + buf * TD * p.BN;
      for (int cb = 0; cb < p.cblks && ok; ++cb, ++uses) {
        const uint32_t set = uses & 1u, sph = (uses >> 1) & 1u;
        for (int j = 0; j < planes; ++j)
          if (!P3_TIMED(st_a, __all_sync(0xffffffffu, mbar_wait(&a_full[set * planes + j], sph, abort_flag, p.status, 74)))) { ok = false; break; }
        if (!ok) break;
        const uint32_t a_set = desc_lo(sa0 + set * planes * (uint32_t)p.a_slot_bytes, 16u);
        const uint32_t a_step = (uint32_t)p.a_slot_bytes >> 4;
        for (int khw = 0; khw < 9; ++khw) {
          const int kh = khw / 3, kw = khw - kh * 3;
          if (!P3_TIMED(st_b, __all_sync(0xffffffffu, mbar_wait(&b_full[b_slot], b_par, abort_flag, p.status, 73)))) { ok = false; break; }
          tc_fence_after();
          const uint32_t b_lo0 = desc_lo(sb0 + b_slot * (uint32_t)p.b_slot_bytes, 16u);
          const uint32_t a_tap = a_set + (((uint32_t)(kw * P3_RH + kh) * P3_ROWB) >> 4);
          if ((cb | khw) == 0) {
            // first touch of each accumulator overwrites: one N = BN MMA per (input plane, output plane)
#pragma unroll
            for (int j = 0; j < planes; ++j) {
#pragma unroll
              for (int t = (j - 2 > 0 ? j - 2 : 0); t <= (j < TD - 1 ? j : TD - 1); ++t) {
                if (leader) {
#pragma unroll
                  for (int k = 0; k < 2; ++k)
                    tc_mma_bf16_pred(acc0 + t * p.BN, a_tap + j * a_step + 2u * k, a_hi,
                                     b_lo0 + (uint32_t)(2 - (j - t)) * b_tap + 2u * k, b_hi, idesc[1],
                                     (t == j && k == 0) ? 0u : 1u);
                }
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < planes; ++j) {
              const int t_lo = j - 2 > 0 ? j - 2 : 0;
              const int t_hi = j < TD - 1 ? j : TD - 1;
              if (leader) {
#pragma unroll
                for (int k = 0; k < 2; ++k)
                  tc_mma_bf16_acc(acc0 + t_lo * p.BN, a_tap + j * a_step + 2u * k, a_hi,
                                  b_lo0 + (uint32_t)(2 - (j - t_lo)) * b_tap + 2u * k, b_hi, idesc[t_hi - t_lo + 1]);
              }
            }
          }
          if (leader) tc_commit(&b_empty[b_slot]);
          __syncwarp();
          if (++b_slot == (uint32_t)p.b_slots) { b_slot = 0; b_par ^= 1u; }
        }
        if (!ok) break;
        if (leader) tc_commit(&set_empty[set]);
        __syncwarp();
      }
      if (ok && leader) tc_commit(&tfull[buf]);
      __syncwarp();
    }
#undef P3_TIMED
    if (p.stall && lane == 0) {
      atomicAdd(&p.stall[0], (unsigned long long)(clock64() - st_begin));
      atomicAdd(&p.stall[1], (unsigned long long)st_b);
      atomicAdd(&p.stall[2], (unsigned long long)st_a);
      atomicAdd(&p.stall[3], (unsigned long long)st_t);
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int rh = row & 7, rw = row >> 3;
    uint32_t jcount = 0;
    bool ok = true;
    long long st_f = 0;
    const long long ep_begin = clock64();
    for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x, ++jcount) {
      const uint32_t buf = jcount & 1u, use = jcount >> 1;
      const long long c0 = p.stall ? clock64() : 0;
      if (!mbar_wait(&tfull[buf], use & 1u, abort_flag, p.status, 76)) { ok = false; break; }
      if (p.stall) st_f += clock64() - c0;
      tc_fence_after();
      const P3Job jc = p3_decode(p, job);
      const int h = jc.h0 + rh, w = jc.w0 + rw;
      for (int t = 0; t < TD; ++t) {
        const int d = jc.d0 + t;
        const bool valid = h < p.H && w < p.W && d < p.D;
        const long long vox = (((long long)jc.n * p.D + d) * p.H + h) * p.W + w;
        const uint32_t acc_i = buf * TD + t;
        const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + acc_i * p.BN;
        for (int c0 = 0; c0 < p.BN; c0 += 16) {
          uint32_t v[16];
          tmem_ld_32x16(tbase + c0, v);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              const int col = jc.co0 + c0 + g * 8;
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[g * 8 + e]);
              __nv_bfloat16* dst = nullptr;
              if (col < p.width0) {
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
                o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
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
    if (p.stall && threadIdx.x == 96) {
      atomicAdd(&p.stall[4], (unsigned long long)(clock64() - ep_begin));
      atomicAdd(&p.stall[5], (unsigned long long)st_f);
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

static int g_p3_smem = 0, g_p3_sms = 0;
static unsigned long long* g_p3_stall = nullptr;
static int p3_setup() {
  if (g_p3_smem) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SB_ERR_DRIVER;
  int lim = 0, sms = 0;
  cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const void* fns[3] = {(const void*)conv_plane3_kernel<1>, (const void*)conv_plane3_kernel<2>,
                        (const void*)conv_plane3_kernel<4>};
  for (int i = 0; i < 3; ++i)
    if (cudaFuncSetAttribute(fns[i], cudaFuncAttributeMaxDynamicSharedMemorySize, lim - 2048) != cudaSuccess)
      return SB_ERR_DRIVER;
  g_p3_smem = lim - 2048;
  g_p3_sms = sms;
  return 0;
}

static int cdiv_p3(int a, int b) { return (a + b - 1) / b; }

// Returns -1 when the call is not eligible (no kd-grouped weights, wide outputs, channel counts that
// are not multiples of 32, halo or slab operands); the caller then uses the plane-walk kernel.
int conv_plane3_launch(const SbConvArgs* a, cudaStream_t stream) {
  if (a->ksize != 3 || a->W < 16 || a->H < 8 || a->wpack_kd == nullptr) return -1;
  if (a->cout_pad > 64 || a->cout_pad % 16 != 0) return -1;
  const int cin_tot = a->src_c[0] + a->src_c[1];
  if (a->src_c[0] % P3_BK != 0 || cin_tot % P3_BK != 0) return -1;
  if (a->halo_land[0][0] || a->halo_land[0][1] || a->slab_out[0]) return -1;
  int rc = p3_setup();
  if (rc) return rc;
  Plane3Params p;
  memset(&p, 0, sizeof(p));
  const int nsrc = a->src_c[1] > 0 ? 2 : 1;
  p.BN = a->cout_pad;
  p.N = a->N; p.D = a->D; p.H = a->H; p.W = a->W;
  p.tiles_h = cdiv_p3(a->H, 8);
  p.tiles_w = cdiv_p3(a->W, 16);
  p.tiles_co = 1;
  p.a_tx = P3_RH * P3_RW * P3_ROWB;
  p.a_slot_bytes = ((p.a_tx + 1023) / 1024) * 1024;
  p.b_tx = 3 * p.BN * P3_ROWB;
  p.b_slot_bytes = ((p.b_tx + 1023) / 1024) * 1024;
  int td = 4;
  for (; td > 1; td /= 2) {
    const long long jobs = (long long)a->N * cdiv_p3(a->D, td) * p.tiles_h * p.tiles_w;
    if (td <= a->D && 2 * td * p.BN <= 512 && jobs >= 2LL * g_p3_sms) break;
  }
  p.TD = td;
  p.groups_d = cdiv_p3(a->D, td);
  p.num_jobs = a->N * p.groups_d * p.tiles_h * p.tiles_w;
  const int budget = g_p3_smem - 1024;
  const int a_bytes = 2 * (td + 2) * p.a_slot_bytes;
  int b_slots = (budget - a_bytes) / p.b_slot_bytes;
  if (b_slots > P3_MAX_B) b_slots = P3_MAX_B;
  if (b_slots < 2) return -1;
  p.b_slots = b_slots;
  p.cblks0 = a->src_c[0] / P3_BK;
  p.cblks = cin_tot / P3_BK;
  for (int s = 0; s < nsrc; ++s) {
    const long long C = a->src_ld[s];
    const long long iD = a->in_d ? a->in_d : a->D, iH = a->in_h ? a->in_h : a->H, iW = a->in_w ? a->in_w : a->W;
    long long dims[5] = {a->src_c[s], iH, iW, iD, a->N};
    long long str[5] = {1, iW * C, C, iH * iW * C, iD * iH * iW * C};
    int box[5] = {P3_BK, P3_RH, P3_RW, 1, 1};
    rc = make_map_bf16(&p.mapA[s], a->src[s], 5, dims, str, box, P3_ROWB);
    if (rc) return rc;
  }
  if (nsrc == 1) p.mapA[1] = p.mapA[0];
  {
    long long dims[3] = {cin_tot, a->cout_pad, 27};
    long long str[3] = {1, cin_tot, (long long)a->cout_pad * cin_tot};
    int box[3] = {P3_BK, p.BN, 3};
    rc = make_map_bf16(&p.mapB, a->wpack_kd, 3, dims, str, box, P3_ROWB);
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
  p.stall = g_p3_stall;
  p.off_d = a->off_d; p.off_h = a->off_h; p.off_w = a->off_w;
  const int grid = p.num_jobs < g_p3_sms ? p.num_jobs : g_p3_sms;
  const size_t smem = (size_t)a_bytes + (size_t)p.b_slots * p.b_slot_bytes + 1024;
  if (td == 4) conv_plane3_kernel<4><<<grid, 224, smem, stream>>>(p);
  else if (td == 2) conv_plane3_kernel<2><<<grid, 224, smem, stream>>>(p);
  else conv_plane3_kernel<1><<<grid, 224, smem, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb

// Performance diagnostic: while a device buffer of 8 counters is set, every kd-fused launch adds, summed over
// CTAs in clock ticks, [0] MMA-warp loop time, [1] its wait for weights, [2] for activation planes, [3] for a
// free accumulator, [4] epilogue-warp loop time, [5] its wait for a finished accumulator. Null switches it off.
extern "C" void sb_conv_stall_counters(unsigned long long* buf) { sb::g_p3_stall = buf; }
