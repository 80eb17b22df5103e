// Plane-walk 3x3x3 convolution, kd-fused variant: output channels in tiles of BN <= 64.
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
  CUtensorMap mapHalo[4];  // [source * 2 + face]: landing slabs of the depth neighbours' boundary planes
  int BN, TD;
  int bgroup;  // (kh,kw) pairs per weight box: 1, or 3 (a whole kh row, fewer waits) when shared memory allows
  int nsets, nbufs, tmem_cols;  // plane sets / accumulator buffers per CTA (1 when two CTAs share an SM)
  int b_slots, a_slot_bytes, b_slot_bytes, a_tx, b_tx;
  int N, D, H, W;
  int tiles_h, tiles_w, groups_d, tiles_co, num_jobs;
  int cblks, cblks0;
  int off_d, off_h, off_w;
  int in_D;
  int halo_has[2];
  const unsigned* halo_flag[2];
  unsigned halo_epoch;
  long long halo_wait_ticks;
  int slab_mode;
  __nv_bfloat16* slab_out[2];
  int slab_ld;
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  int width0, width1, ld0, ld1;
  int wide;  // widths and strides are multiples of 16 channels: 32-byte stores
  const float* bias;
  uint32_t* status;
  unsigned long long* stall;  // optional stall counters (clock ticks summed over CTAs), null = off
  float* gn_part;   // optional GroupNorm partials of the output: [N][jobs per sample and channel tile][G][3]
  int gn_groups;    // G
  int gn_cg;        // channels per group (4 .. BN, divides BN)
  int gn_splits;    // groups_d * tiles_h * tiles_w * 4 (one partial per epilogue warp)
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

// STATS: the epilogue also writes GroupNorm partials (forward passes only; the variant without them keeps the
// register count low enough for small co-resident kernels, e.g. the overlapped gradient reduction, during backward)
template <int TD, bool STATS>
__global__ void __launch_bounds__(224, 2) conv_plane3_kernel(const __grid_constant__ Plane3Params p) {
  constexpr int planes = TD + 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_b = smem + (size_t)p.nsets * planes * p.a_slot_bytes;
  __shared__ uint64_t a_full[2];
  __shared__ uint64_t set_empty[2];
  __shared__ uint64_t b_full[P3_MAX_B], b_empty[P3_MAX_B];
  __shared__ uint64_t tfull[2];
  __shared__ uint64_t tempty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  __shared__ float gn_s[4][33];  // per epilogue warp: 16 x (sum, sum of squares) over 4-channel runs + voxel count
  volatile uint32_t* abort_flag = &abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < 2; ++s) { mbar_init(&a_full[s], 1); mbar_init(&set_empty[s], 1); mbar_init(&tfull[s], 1); mbar_init(&tempty[s], 4); }
    for (int s = 0; s < p.b_slots; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
    mbar_fence_init();
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, (uint32_t)p.tmem_cols); tmem_relinquish(); }
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
      bool halo_ready[2] = {false, false};
      for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x) {
        const P3Job jc = p3_decode(p, job);
        for (int cb = 0; cb < p.cblks && ok; ++cb, ++uses) {
          const uint32_t set = p.nsets == 2 ? (uses & 1u) : 0u;
          const uint32_t ph = (p.nsets == 2 ? (uses >> 1) : uses) & 1u;
          if (!mbar_wait(&set_empty[set], ph ^ 1u, abort_flag, p.status, 71)) { ok = false; break; }
          const int second = cb >= p.cblks0 ? 1 : 0;
          const int c = (second ? cb - p.cblks0 : cb) * P3_BK;
          mbar_expect_tx(&a_full[set], (uint32_t)(planes * p.a_tx));
          for (int j = 0; j < planes && ok; ++j) {
            const int s = set * planes + j;
            const int dz = jc.d0 - 1 + j + p.off_d;
            const int face = dz < 0 ? 0 : (dz >= p.in_D ? 1 : -1);
            if (face >= 0 && p.halo_has[face]) {
              // a depth neighbour's boundary plane: wait (bounded) until its push landed, then read it locally
              if (!halo_ready[face]) {
                if (p.halo_flag[face] != nullptr) {
                  const long long t0 = clock64();
                  uint32_t v;
                  while (true) {
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.halo_flag[face]) : "memory");
                    if ((int)(v - p.halo_epoch) >= 0) break;
                    if (*abort_flag || clock64() - t0 > p.halo_wait_ticks) {
                      *abort_flag = 1u;
                      report(p.status, ST_FLAG_TIMEOUT, 77, blockIdx.x, face);
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
              tma_load_5d(smem + (size_t)s * p.a_slot_bytes, &p.mapHalo[second * 2 + face], &a_full[set], c,
                          jc.h0 - 1 + p.off_h, jc.w0 - 1 + p.off_w, 0, jc.n);
            } else {
              tma_load_5d(smem + (size_t)s * p.a_slot_bytes, &p.mapA[second], &a_full[set], c, jc.h0 - 1 + p.off_h,
                          jc.w0 - 1 + p.off_w, dz, jc.n);
            }
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
          for (int khw = 0; khw < 9; khw += p.bgroup, ++it) {
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
    // Measured on this part: one thread keeps the tensor pipe full only if nothing but integer adds
    // sits between consecutive tcgen05.mma (the pipe accepts about one instruction ahead), and a
    // 128 x N x 16 MMA costs max(N/2, 32 + N/4) cycles. So no wait sits in front of an MMA run: the
    // operands of step g+1 (weights; at a channel-block change the plane set; at a job change the
    // accumulators) are awaited in the middle of step g, behind the N = 192 MMAs already queued.
    const bool leader = elect_one();
    const uint32_t swz = swizzle_code_for(P3_ROWB);
    const uint32_t a_hi = desc_hi((uint32_t)P3_RH * P3_ROWB, swz);
    const uint32_t b_hi = desc_hi(8u * P3_ROWB, swz);
    uint32_t idesc[4];
#pragma unroll
    for (int n = 1; n <= 3; ++n) idesc[n] = make_idesc_bf16(128, n * p.BN, 0, 0);
    const uint32_t sa0 = smem_u32(smem), sb0 = smem_u32(smem_b);
    const uint32_t b_tap = ((uint32_t)p.BN * P3_ROWB) >> 4;  // one tap's rows, in descriptor units
    const uint32_t a_step = (uint32_t)p.a_slot_bytes >> 4;
    uint32_t uses = 0, b_slot = 0, b_par = 0, jcount = 0;
    bool ok = true;
    long long st_b = 0, st_a = 0, st_t = 0;
    const long long st_begin = clock64();
#define P3_TIMED(counter, expr) \
  [&]() { const long long c0_ = p.stall ? clock64() : 0; const bool r_ = (expr); if (p.stall) counter += clock64() - c0_; return r_; }()
#define P3_WAIT(counter, bar, par, site) P3_TIMED(counter, __all_sync(0xffffffffu, mbar_wait(bar, par, abort_flag, p.status, site)))
    // With one plane set / one accumulator buffer (two CTAs per SM hide each other's gaps) the
    // next set or buffer is the current one: it can only be awaited after this step's commit.
    const bool sets2 = p.nsets == 2, bufs2 = p.nbufs == 2;
    if (blockIdx.x < p.num_jobs) ok = P3_WAIT(st_b, &b_full[0], 0u, 73);
    for (int job = blockIdx.x; job < p.num_jobs && ok; job += gridDim.x, ++jcount) {
      const uint32_t buf = bufs2 ? (jcount & 1u) : 0u;
      const bool last_job = job + (int)gridDim.x >= p.num_jobs;
      const uint32_t acc0 = tmem_base + buf * TD * p.BN;
      if (!bufs2 || jcount == 0) {
        if (!P3_WAIT(st_t, &tempty[buf], ((bufs2 ? (jcount >> 1) : jcount) & 1u) ^ 1u, 75)) { ok = false; break; }
      }
      for (int cb = 0; cb < p.cblks && ok; ++cb, ++uses) {
        const uint32_t set = sets2 ? (uses & 1u) : 0u;
        const bool last_cb = cb + 1 == p.cblks;
        if (!sets2 || uses == 0) {
          if (!P3_WAIT(st_a, &a_full[set], (sets2 ? (uses >> 1) : uses) & 1u, 74)) { ok = false; break; }
        }
        const uint32_t a_set = desc_lo(sa0 + set * planes * (uint32_t)p.a_slot_bytes, 16u);
        for (int khw = 0; khw < 9; ++khw) {
          const int kh = khw / 3, kw = khw - kh * 3;
          tc_fence_after();
          const int sub = p.bgroup == 3 ? kw : 0;             // position of this (kh,kw) pair inside its weight box
          const bool box_done = p.bgroup == 3 ? kw == 2 : true;  // last pair of the box: the next step reads a new slot
          const uint32_t b_lo0 = desc_lo(sb0 + b_slot * (uint32_t)p.b_slot_bytes, 16u) + (uint32_t)sub * 3u * b_tap;
          const uint32_t a_tap = a_set + (((uint32_t)(kw * P3_RH + kh) * P3_ROWB) >> 4);
          const bool first = (cb | khw) == 0;
          uint32_t nb_slot = b_slot + 1, nb_par = b_par;
          if (nb_slot == (uint32_t)p.b_slots) { nb_slot = 0; nb_par ^= 1u; }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (first) {
              // first touch of each accumulator overwrites: one N = BN MMA per (input plane, output plane)
#pragma unroll
              for (int j = half * (planes / 2); j < (half ? planes : planes / 2); ++j) {
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
              for (int j = half * (planes / 2); j < (half ? planes : planes / 2); ++j) {
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
            if (half == 0) {
              // look ahead: what the next step reads
              const bool more = !(last_job && last_cb && khw == 8);
              if (more) {
                if (box_done && !P3_WAIT(st_b, &b_full[nb_slot], nb_par, 73)) { ok = false; break; }
                if (khw == 8) {
                  const uint32_t nu = uses + 1;
                  if (sets2 && !P3_WAIT(st_a, &a_full[nu & 1u], (nu >> 1) & 1u, 74)) { ok = false; break; }
                  if (last_cb && bufs2) {
                    const uint32_t nj = jcount + 1;
                    if (!P3_WAIT(st_t, &tempty[nj & 1u], ((nj >> 1) & 1u) ^ 1u, 75)) { ok = false; break; }
                  }
                }
              }
            }
          }
          if (!ok) break;
          if (leader) {
            if (box_done) tc_commit(&b_empty[b_slot]);
            if (khw == 8) {
              tc_commit(&set_empty[set]);
              if (last_cb) tc_commit(&tfull[buf]);
            }
          }
          __syncwarp();
          if (box_done) {
            b_slot = nb_slot;
            b_par = nb_par;
          }
        }
      }
    }
#undef P3_WAIT
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
      const uint32_t buf = p.nbufs == 2 ? (jcount & 1u) : 0u, use = p.nbufs == 2 ? (jcount >> 1) : jcount;
      const long long c0 = p.stall ? clock64() : 0;
      if (!mbar_wait(&tfull[buf], use & 1u, abort_flag, p.status, 76)) { ok = false; break; }
      if (p.stall) st_f += clock64() - c0;
      tc_fence_after();
      const P3Job jc = p3_decode(p, job);
      const int h = jc.h0 + rh, w = jc.w0 + rw;
      // GroupNorm statistics of what this job stores (optional): per thread, sums over runs of 4 channels
      float gsum[16], gsq[16];
      float gcnt = 0.f;
      constexpr bool stats = STATS;
      if (stats) {
#pragma unroll
        for (int i = 0; i < 16; ++i) { gsum[i] = 0.f; gsq[i] = 0.f; }
      }
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
        if (stats && valid) gcnt += 1.f;
#pragma unroll
        for (int ci = 0; ci < 4; ++ci) {
          const int c0 = ci * 16;
          if (c0 >= p.BN) break;
          uint32_t v[16];
          tmem_ld_32x16(tbase + c0, v);
          tmem_ld_wait();
          if (valid) {
            const int col0 = jc.co0 + c0;
            uint4 o[2];
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[g * 8 + e]);
              if (p.bias && !slab && col0 + g * 8 < p.width0) {
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] += p.bias[col0 + g * 8 + e];
              }
              o[g].x = pack_bf16x2(f[0], f[1]); o[g].y = pack_bf16x2(f[2], f[3]);
              o[g].z = pack_bf16x2(f[4], f[5]); o[g].w = pack_bf16x2(f[6], f[7]);
              if (stats) {
                // the values as stored (bf16-rounded): the statistics must describe the tensor the next pass reads
                const uint32_t w4[4] = {o[g].x, o[g].y, o[g].z, o[g].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float lo = __uint_as_float(w4[e] << 16), hi = __uint_as_float(w4[e] & 0xffff0000u);
                  const int run = ci * 4 + g * 2 + (e >> 1);
                  gsum[run] += lo + hi;
                  gsq[run] += lo * lo + hi * hi;
                }
              }
            }
            if (slab) {
              if (col0 < p.width0 + p.width1) {
                if (p.wide) st_global_v8(slab + vox * p.slab_ld + col0, o[0], o[1]);
                else {
                  *reinterpret_cast<uint4*>(slab + vox * p.slab_ld + col0) = o[0];
                  if (col0 + 8 < p.width0 + p.width1) *reinterpret_cast<uint4*>(slab + vox * p.slab_ld + col0 + 8) = o[1];
                }
              }
            } else if (p.wide) {
              // destinations split at a multiple of 16 channels: one 32-byte store per 16 channels
              if (col0 < p.width0) st_global_v8(p.out0 + vox * p.ld0 + col0, o[0], o[1]);
              else if (col0 - p.width0 < p.width1) st_global_v8(p.out1 + vox * p.ld1 + (col0 - p.width0), o[0], o[1]);
            } else {
#pragma unroll
              for (int g = 0; g < 2; ++g) {
                const int col = col0 + g * 8;
                if (col < p.width0) *reinterpret_cast<uint4*>(p.out0 + vox * p.ld0 + col) = o[g];
                else if (col - p.width0 < p.width1) *reinterpret_cast<uint4*>(p.out1 + vox * p.ld1 + (col - p.width0)) = o[g];
              }
            }
          }
        }
      }
      if (stats) {
        // warp sums; every epilogue warp owns 32 rows of the tile and writes its own partial (no cross-warp barrier)
#pragma unroll
        for (int i = 0; i < 16; ++i) {
#pragma unroll
          for (int o2 = 16; o2 > 0; o2 >>= 1) {
            gsum[i] += __shfl_xor_sync(0xffffffffu, gsum[i], o2);
            gsq[i] += __shfl_xor_sync(0xffffffffu, gsq[i], o2);
          }
        }
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) gcnt += __shfl_xor_sync(0xffffffffu, gcnt, o2);
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int i = 0; i < 16; ++i) { gn_s[q][2 * i] = gsum[i]; gn_s[q][2 * i + 1] = gsq[i]; }
          gn_s[q][32] = gcnt;
        }
        __syncwarp();
        const int groups_here = p.BN / p.gn_cg;      // groups this channel tile covers (at most 16)
        if (lane < groups_here) {
          const int runs = p.gn_cg / 4;
          float s1 = 0.f, s2 = 0.f;
          for (int r = 0; r < runs; ++r) {
            s1 += gn_s[q][2 * (lane * runs + r)];
            s2 += gn_s[q][2 * (lane * runs + r) + 1];
          }
          const float n_el = gn_s[q][32] * (float)p.gn_cg;
          const float mean = n_el > 0.f ? s1 / n_el : 0.f;
          const float m2 = n_el > 0.f ? fmaxf(s2 - s1 * mean, 0.f) : 0.f;
          const int sj = ((jc.d0 / TD * p.tiles_h + jc.h0 / 8) * p.tiles_w + jc.w0 / 16) * 4 + q;
          const int g_glob = jc.co0 / p.gn_cg + lane;
          float* dst = p.gn_part + (((long long)jc.n * p.gn_splits + sj) * p.gn_groups + g_glob) * 3;
          dst[0] = n_el; dst[1] = mean; dst[2] = m2;
        }
        __syncwarp();  // gn_s[q] is reused by this warp's next job
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
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
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
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
  const void* fns[6] = {(const void*)conv_plane3_kernel<1, false>, (const void*)conv_plane3_kernel<2, false>,
                        (const void*)conv_plane3_kernel<4, false>, (const void*)conv_plane3_kernel<1, true>,
                        (const void*)conv_plane3_kernel<2, true>, (const void*)conv_plane3_kernel<4, true>};
  for (int i = 0; i < 6; ++i)
    if (cudaFuncSetAttribute(fns[i], cudaFuncAttributeMaxDynamicSharedMemorySize, lim - 2048) != cudaSuccess)
      return SB_ERR_DRIVER;
  g_p3_smem = lim - 2048;
  g_p3_sms = sms;
  return 0;
}

static int cdiv_p3(int a, int b) { return (a + b - 1) / b; }

// Returns -1 when the call is not eligible (no kd-grouped weights, wide outputs, channel counts that
// are not multiples of 32); the caller then uses the plane-walk kernel.
// Tile shape, job depth and CTA mode of a call (everything the launch and the statistics query share).
// Returns -1 when the call is not eligible, an SB_ERR_* code on failure, 0 with `p` / `dual` filled otherwise.
static int p3_plan(const SbConvArgs* a, Plane3Params& p, bool& dual) {
  if (a->ksize != 3 || a->W < 16 || a->H < 8 || a->wpack_kd == nullptr) return -1;
  if (a->cout_pad % 16 != 0 || (a->cout_pad > 64 && a->cout_pad % 64 != 0)) return -1;
  const int cin_tot = a->src_c[0] + a->src_c[1];
  if (a->src_c[0] % P3_BK != 0 || cin_tot % P3_BK != 0) return -1;
  int rc = p3_setup();
  if (rc) return rc;
  memset(&p, 0, sizeof(p));
  p.BN = a->cout_pad > 64 ? 64 : a->cout_pad;
  p.N = a->N; p.D = a->D; p.H = a->H; p.W = a->W;
  p.tiles_h = cdiv_p3(a->H, 8);
  p.tiles_w = cdiv_p3(a->W, 16);
  p.tiles_co = a->cout_pad / p.BN;
  p.a_tx = P3_RH * P3_RW * P3_ROWB;
  p.a_slot_bytes = ((p.a_tx + 511) / 512) * 512;  // the 64-byte swizzle pattern repeats every 512 bytes
  // Deep reductions (>= 4 channel blocks) run two CTAs per SM, each with one plane set and one
  // accumulator buffer: while one CTA's issuing thread sits in a wait, a commit or the turn-around
  // between channel blocks, the other CTA's MMAs keep the tensor pipe busy (measured: a second
  // issuing stream hides these gaps). Shallow ones are faster with one CTA per SM that double-buffers
  // plane sets and accumulators (measured on 64-channel inputs).
  // The mode and the depth of a job are chosen together: last-wave fill of the CTA slots x reuse of a weight load
  // (deeper jobs) x the measured preference of the mode (two CTAs per SM gain about 7 % on deep reductions and
  // lose about as much on shallow ones). A small volume with many channels may fill 148 slots but not 296.
  const int cblks_all = cin_tot / P3_BK;
  dual = cblks_all >= 4;
  int td = 1;
  double best = 0.0;
  for (int mode = 0; mode < 2; ++mode) {
    const bool d2 = mode == 0;  // two CTAs per SM first: it wins ties
    const int m_slots = (d2 ? 2 : 1) * g_p3_sms;
    const int m_tmem = d2 ? 256 : 512, m_bufs = d2 ? 1 : 2;
    const double pref = d2 ? (cblks_all >= 4 ? 1.0 : 0.9) : (cblks_all >= 4 ? 0.93 : 1.0);
    for (int cand = 4; cand >= 1; cand /= 2) {
      if (cand > a->D || m_bufs * cand * p.BN > m_tmem) continue;
      const long long jobs = (long long)a->N * cdiv_p3(a->D, cand) * p.tiles_h * p.tiles_w * p.tiles_co;
      const long long waves = (jobs + m_slots - 1) / m_slots;
      const double score = (double)jobs / (double)(waves * m_slots) * (cand == 4 ? 1.0 : cand == 2 ? 0.93 : 0.8) * pref;
      if (score > best) { best = score; td = cand; dual = d2; }
    }
  }
  p.nsets = dual ? 1 : 2;
  p.nbufs = dual ? 1 : 2;
  p.TD = td;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.nbufs * td * p.BN) p.tmem_cols *= 2;
  p.groups_d = cdiv_p3(a->D, td);
  p.num_jobs = a->N * p.groups_d * p.tiles_h * p.tiles_w * p.tiles_co;
  return 0;
}

// GroupNorm statistics from the epilogue: one destination, no slab outputs, a group made of whole 4-channel runs
// that does not straddle channel tiles, at most 16 groups per tile.
static bool p3_gn_ok(const SbConvArgs* a, const Plane3Params& p) {
  if (a->gn_groups < 1 || a->dst[1] != nullptr || a->slab_out[0] != nullptr) return false;
  if (a->dst_c[0] != a->cout_pad || a->cout_pad % a->gn_groups != 0) return false;
  const int cg = a->cout_pad / a->gn_groups;
  return cg % 4 == 0 && cg <= p.BN && p.BN % cg == 0 && p.BN / cg <= 16;
}

int conv_plane3_gn_splits(const SbConvArgs* a) {
  Plane3Params p;
  bool dual = false;
  if (p3_plan(a, p, dual) != 0 || !p3_gn_ok(a, p)) return 0;
  return p.groups_d * p.tiles_h * p.tiles_w * 4;
}

int conv_plane3_launch(const SbConvArgs* a, cudaStream_t stream) {
  Plane3Params p;
  bool dual = false;
  int rc = p3_plan(a, p, dual);
  if (rc != 0) return rc;
  const int cin_tot = a->src_c[0] + a->src_c[1];
  const int nsrc = a->src_c[1] > 0 ? 2 : 1;
  const int td = p.TD;
  const int slots = (dual ? 2 : 1) * g_p3_sms;
  if (a->gn_part != nullptr) {
    if (!p3_gn_ok(a, p)) return SB_ERR_SHAPE;
    p.gn_part = a->gn_part;
    p.gn_groups = a->gn_groups;
    p.gn_cg = a->cout_pad / a->gn_groups;
    p.gn_splits = p.groups_d * p.tiles_h * p.tiles_w * 4;
  }
  const int budget = dual ? g_p3_smem / 2 - 2048 : g_p3_smem;  // per CTA
  const int a_bytes = p.nsets * (td + 2) * p.a_slot_bytes;
  // weight boxes of a whole kh row (nine taps) when two of them fit: a third of the waits and commits
  int b_slots = 0;
  for (p.bgroup = 3; p.bgroup >= 1; p.bgroup -= 2) {
    p.b_tx = 3 * p.bgroup * p.BN * P3_ROWB;
    p.b_slot_bytes = ((p.b_tx + 1023) / 1024) * 1024;
    b_slots = (budget - 1024 - a_bytes) / p.b_slot_bytes;
    if (b_slots >= 2) break;
  }
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
    int box[3] = {P3_BK, p.BN, 3 * p.bgroup};
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
  p.wide = (p.width0 % 16 == 0 && p.width1 % 16 == 0 && p.ld0 % 16 == 0 && p.ld1 % 16 == 0 &&
            (reinterpret_cast<uintptr_t>(p.out0) & 31) == 0 && (reinterpret_cast<uintptr_t>(p.out1) & 31) == 0) ? 1 : 0;
  p.bias = a->bias;
  p.status = a->status;
  p.stall = g_p3_stall;
  p.off_d = a->off_d; p.off_h = a->off_h; p.off_w = a->off_w;
  p.in_D = a->in_d ? a->in_d : a->D;
  for (int f = 0; f < 2; ++f) {
    p.halo_has[f] = a->halo_land[0][f] != nullptr ? 1 : 0;
    p.halo_flag[f] = a->halo_flag[f];
    for (int sidx = 0; sidx < 2; ++sidx) {
      const int idx = sidx * 2 + f;
      if (sidx < nsrc && a->halo_land[sidx][f] != nullptr) {
        const long long C = a->src_c[sidx];
        const long long iH = a->in_h ? a->in_h : a->H, iW = a->in_w ? a->in_w : a->W;
        long long dims[5] = {C, iH, iW, 1, a->N};
        long long str[5] = {1, iW * C, C, iH * iW * C, iH * iW * C};
        int box[5] = {P3_BK, P3_RH, P3_RW, 1, 1};
        rc = make_map_bf16(&p.mapHalo[idx], a->halo_land[sidx][f], 5, dims, str, box, P3_ROWB);
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
  if (p.slab_mode && (p.slab_ld % 16 != 0 || (reinterpret_cast<uintptr_t>(p.slab_out[0]) & 31) != 0 ||
                      (reinterpret_cast<uintptr_t>(p.slab_out[1]) & 31) != 0))
    p.wide = 0;
  const int grid = p.num_jobs < slots ? p.num_jobs : slots;
  const size_t smem = (size_t)a_bytes + (size_t)p.b_slots * p.b_slot_bytes + 1024;
  if (p.gn_part != nullptr) {
    if (td == 4) conv_plane3_kernel<4, true><<<grid, 224, smem, stream>>>(p);
    else if (td == 2) conv_plane3_kernel<2, true><<<grid, 224, smem, stream>>>(p);
    else conv_plane3_kernel<1, true><<<grid, 224, smem, stream>>>(p);
  } else if (td == 4) conv_plane3_kernel<4, false><<<grid, 224, smem, stream>>>(p);
  else if (td == 2) conv_plane3_kernel<2, false><<<grid, 224, smem, stream>>>(p);
  else conv_plane3_kernel<1, false><<<grid, 224, smem, stream>>>(p);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb

// Performance diagnostic: while a device buffer of 8 counters is set, every kd-fused launch adds, summed over
// CTAs in clock ticks, [0] MMA-warp loop time, [1] its wait for weights, [2] for activation planes, [3] for a
// free accumulator, [4] epilogue-warp loop time, [5] its wait for a finished accumulator. Null switches it off.
extern "C" void sb_conv_stall_counters(unsigned long long* buf) { sb::g_p3_stall = buf; }
