// Plane-walk 3x3x3 convolution for wide layers (>= 128 output channels) on a PAIR of SMs:
// a thread-block cluster of two CTAs issues tcgen05.mma.cta_group::2 with M = 256, N = BN.
//
// Why a pair: with one CTA a 128 x 128 x 16 MMA reads 4 KB of activations and 4 KB of weights
// from shared memory every 64 tensor-pipe cycles, which is the whole 128 B/clk the shared
// memory delivers, so the tensor pipe idles about a quarter of the time. In pair mode each CTA
// supplies its own 128 voxel rows (its own 8 x 16 column of the volume) and only HALF of the
// weight rows, and the tensor cores of both SMs read both halves: 4 KB + 2 KB (BN = 128) or
// 4 KB + 4 KB per 128 cycles (BN = 256), i.e. 96 or 64 B/clk per SM.
//
// Layout of the work: a pair-job is two neighbouring spatial tiles (consecutive in the linear
// (n, d-group, h-tile, w-tile) order) by BN output channels. CTA r of the cluster
//   * loads the activation planes of tile r and weight rows [r * BN/2, (r+1) * BN/2) of each tap
//     with ordinary TMA loads of this GPU's memory (cta_group::2 form, no multicast) whose
//     byte counts complete on the LEADER's (rank 0) barriers,
//   * reads back the 128 TMEM lanes that hold tile r's accumulators and stores them.
// Only the leader issues MMAs. Its tcgen05.commit arrives on the barrier at the same offset in
// both CTAs (slot release and accumulator-ready), and the peer's epilogue releases accumulators
// by a remote mbarrier arrive on the leader. Every wait is bounded and reports to the status
// word; a CTA leaves only after a cluster barrier, so no arrive can land in a CTA that is gone.
//
// Features are those of the single-CTA plane kernel: two concatenated sources, the fused depth
// halo (landing slabs + flag words), slab outputs for backward-data; the forward instantiation
// can also leave GroupNorm partial statistics of what it stores (one partial per epilogue warp).
// Tile width (128 / 256) and job depth come from a cost model fitted to measurements (p2_choose).
// Role of the reference: triton_conv3d/gather_gemm.py:112-341 and bwd_data.py:275-363.
#include "common.cuh"
#include "host_api.h"

namespace sb {

int make_map_bf16(CUtensorMap* m, const void* base, int rank, const long long* dims, const long long* strides,
                  const int* box, int rowb);

constexpr int P2_MAX_A = 8;
constexpr int P2_MAX_B = 16;
constexpr int P2_RH = 10;
constexpr int P2_RW = 18;
constexpr int P2_BK = 64;
constexpr int P2_KSTEPS = P2_BK / 16;
constexpr int P2_ROWB = P2_BK * 2;

struct Plane2Params {
  CUtensorMap mapA[2];
  CUtensorMap mapB;
  int BN, TD;
  int a_slots, b_slots, a_slot_bytes, b_slot_bytes, a_tx, b_tx;  // per CTA
  int n_bufs;
  int N, D, H, W;
  int tiles_h, tiles_w, groups_d, tiles_co, num_pair_jobs;
  int cblks, cblks0;
  int off_d, off_h, off_w;
  CUtensorMap mapHalo[4];
  int halo_has[2], in_D;
  const uint32_t* halo_flag[2];
  uint32_t halo_epoch;
  long long halo_wait_ticks;
  __nv_bfloat16* slab_out[2];
  int slab_ld, slab_mode;
  __nv_bfloat16* out0;
  __nv_bfloat16* out1;
  int width0, width1, ld0, ld1;
  const float* bias;
  uint32_t* status;
  // optional GroupNorm partials of the output: [N][gn_splits][gn_groups][3] (count, mean, M2), one per epilogue warp
  float* gn_part;
  int gn_groups, gn_cg, gn_splits;
};

struct Job2 {
  int co0, h0, w0, d0, n;
};

__device__ __forceinline__ Job2 decode_job2(const Plane2Params& p, int pj, int rank) {
  Job2 j;
  j.co0 = (pj % p.tiles_co) * p.BN;
  int t = (pj / p.tiles_co) * 2 + rank;
  j.w0 = (t % p.tiles_w) * 16; t /= p.tiles_w;
  j.h0 = (t % p.tiles_h) * 8; t /= p.tiles_h;
  j.d0 = (t % p.groups_d) * p.TD; t /= p.groups_d;
  j.n = t;  // may be N for the odd tile out: its loads read the fill value and its stores are masked
  return j;
}

// ---- cluster / pair primitives ---------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cl(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait with cluster-scope acquire (the arrivals come from the other CTA or from its copies)
__device__ __forceinline__ bool mbar_wait_cl(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                             uint32_t* status, uint32_t site) {
  if (mbar_try_wait_cl(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cl(bar, parity)) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > SB_WAIT_LIMIT_TICKS) {
        *abort_flag = 1u;
        report(status, ST_MBAR_TIMEOUT, site, blockIdx.x, parity);
        return false;
      }
    }
  }
}
// TMA loads of this CTA's own shared memory whose byte count completes on a barrier of the pair's leader
__device__ __forceinline__ void tma2_load_5d(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0,
                                             int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0,
                                             int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem2_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem2_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem2_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs of the pair once the MMAs issued so far retired.
__device__ __forceinline__ void tc2_commit_both(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void tc2_mma_bf16_acc(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                 uint32_t b_hi, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, 1, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc)
      : "memory");
}
__device__ __forceinline__ void tc2_mma_bf16_pred(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                  uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// STATS: the epilogue also leaves GroupNorm partial statistics of what it stores (forward passes that feed a
// GroupNorm; groups of 16 channels or more, i.e. whole halves of a 32-column TMEM chunk).
template <int TD, bool STATS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(224, 1)
conv_plane2_kernel(const __grid_constant__ Plane2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_b = smem + (size_t)p.a_slots * p.a_slot_bytes;
  __shared__ uint64_t a_full[P2_MAX_A], a_empty[P2_MAX_A];
  __shared__ uint64_t b_full[P2_MAX_B], b_empty[P2_MAX_B];
  __shared__ uint64_t tfull[2];
  __shared__ uint64_t tempty[8];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  __shared__ float gn_acc[4][16][2];  // per epilogue warp: (sum, sum of squares) of up to 16 groups of this job
  volatile uint32_t* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  constexpr int rowb = P2_ROWB;
  constexpr int planes = TD + 2;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < p.a_slots; ++s) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
    for (int s = 0; s < p.b_slots; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
    for (int b = 0; b < 2; ++b) mbar_init(&tfull[b], 1);
    for (int a = 0; a < 8; ++a) mbar_init(&tempty[a], 8);  // four epilogue warps in each CTA of the pair
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem2_alloc(&tmem_base_s, 512);
    tmem2_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before any copy or arrive targets them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // --------------------------- activation planes ---------------------------
    if (lane == 0) {
      tma_prefetch_desc(&p.mapA[0]);
      tma_prefetch_desc(&p.mapA[1]);
      uint32_t it = 0;
      bool ok = true;
      bool halo_ready[2] = {false, false};
      for (int pj = pair; pj < p.num_pair_jobs && ok; pj += npairs) {
        const Job2 jc = decode_job2(p, pj, (int)rank);
        for (int cb = 0; cb < p.cblks && ok; ++cb) {
          const int second = cb >= p.cblks0 ? 1 : 0;
          const int c = (second ? cb - p.cblks0 : cb) * P2_BK;
          for (int j = 0; j < planes; ++j, ++it) {
            const int s = it % p.a_slots;
            const uint32_t ph = (it / p.a_slots) & 1u;
            if (!mbar_wait_cl(&a_empty[s], ph ^ 1u, abort_flag, p.status, 71)) { ok = false; break; }
            const uint32_t full_addr = map_to_rank(smem_u32(&a_full[s]), 0);
            const int dz = jc.d0 - 1 + j + p.off_d;
            const int face = dz < 0 ? 0 : (dz >= p.in_D ? 1 : -1);
            const bool from_halo = face >= 0 && p.halo_has[face];
            if (from_halo && !halo_ready[face]) {
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
            if (rank == 0) mbar_expect_tx(&a_full[s], 2u * (uint32_t)p.a_tx);  // both CTAs' planes
            if (from_halo)
              tma2_load_5d(smem + (size_t)s * p.a_slot_bytes, &p.mapHalo[second * 2 + face], full_addr, c,
                           jc.h0 - 1 + p.off_h, jc.w0 - 1 + p.off_w, 0, jc.n);
            else
              tma2_load_5d(smem + (size_t)s * p.a_slot_bytes, &p.mapA[second], full_addr, c, jc.h0 - 1 + p.off_h,
                           jc.w0 - 1 + p.off_w, dz, jc.n);
          }
        }
      }
      // every release of a slot this CTA filled has arrived before the CTA may leave
      for (int k = 0; k < p.a_slots && ok; ++k, ++it) {
        const int s = it % p.a_slots;
        const uint32_t ph = (it / p.a_slots) & 1u;
        if (!mbar_wait_cl(&a_empty[s], ph ^ 1u, abort_flag, p.status, 78)) ok = false;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ weight taps ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&p.mapB);
      uint32_t it = 0;
      bool ok = true;
      const int half = p.BN / 2;
      for (int pj = pair; pj < p.num_pair_jobs && ok; pj += npairs) {
        const int co0 = (pj % p.tiles_co) * p.BN + (int)rank * half;
        for (int cb = 0; cb < p.cblks && ok; ++cb) {
          for (int tap = 0; tap < 27; ++tap, ++it) {
            const int s = it % p.b_slots;
            const uint32_t ph = (it / p.b_slots) & 1u;
            if (!mbar_wait_cl(&b_empty[s], ph ^ 1u, abort_flag, p.status, 72)) { ok = false; break; }
            if (rank == 0) mbar_expect_tx(&b_full[s], 2u * (uint32_t)p.b_tx);
            tma2_load_3d(smem_b + (size_t)s * p.b_slot_bytes, &p.mapB, map_to_rank(smem_u32(&b_full[s]), 0),
                         cb * P2_BK, co0, tap);
          }
        }
      }
      for (int k = 0; k < p.b_slots && ok; ++k, ++it) {
        const int s = it % p.b_slots;
        const uint32_t ph = (it / p.b_slots) & 1u;
        if (!mbar_wait_cl(&b_empty[s], ph ^ 1u, abort_flag, p.status, 79)) ok = false;
      }
    }
  } else if (warp == 2) {
    // ------------------------- MMA issuer (leader CTA only) -------------------------
    if (rank == 0) {
      const bool leader = elect_one();
      const uint32_t idesc = make_idesc_bf16(256, p.BN, 0, 0);
      const uint32_t swz = swizzle_code_for(rowb);
      const uint32_t a_hi = desc_hi((uint32_t)P2_RH * rowb, swz);
      const uint32_t b_hi = desc_hi(8u * rowb, swz);
      const uint32_t sa0 = smem_u32(smem), sb0 = smem_u32(smem_b);
      uint32_t a_slot = 0, a_par = 0, b_slot = 0, b_par = 0, jcount = 0;
      uint32_t acc_uses[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      bool ok = true;
      for (int pj = pair; pj < p.num_pair_jobs && ok; pj += npairs, ++jcount) {
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
          int waited = 0;
#pragma unroll
          for (int kd = 0; kd < 3; ++kd) {
            for (int khw = 0; khw < 9 && ok; ++khw) {
              const int kh = khw / 3, kw = khw - kh * 3;
              if (!__all_sync(0xffffffffu, mbar_wait_cl(&b_full[b_slot], b_par, abort_flag, p.status, 73))) { ok = false; break; }
              tc_fence_after();
              const uint32_t b_lo = desc_lo(sb0 + b_slot * p.b_slot_bytes, 16u);
              const uint32_t tap_off = ((uint32_t)(kw * P2_RH + kh) * rowb) >> 4;
              const bool first = kd == 0 && (cb | khw) == 0;
#pragma unroll
              for (int t = 0; t < TD; ++t) {
                const int j = t + kd;
                if (j >= waited) {
                  if (!__all_sync(0xffffffffu, mbar_wait_cl(&a_full[pl_slot[j]], pl_par[j], abort_flag, p.status, 74))) { ok = false; break; }
                  tc_fence_after();
                  waited = j + 1;
                }
                const uint32_t acc_i = buf * TD + t;
                if (kd == 0 && first) {
                  const uint32_t u = acc_uses[acc_i]++;
                  if (!__all_sync(0xffffffffu, mbar_wait_cl(&tempty[acc_i], (u & 1u) ^ 1u, abort_flag, p.status, 75))) { ok = false; break; }
                  tc_fence_after();
                }
                const uint32_t a_lo = pl_lo[j] + tap_off;
                const uint32_t acc = tmem_base + acc_i * p.BN;
#pragma unroll
                for (int k = 0; k < P2_KSTEPS; ++k) {
                  if (leader) {
                    if (kd == 0 && k == 0)
                      tc2_mma_bf16_pred(acc, a_lo, a_hi, b_lo, b_hi, idesc, first ? 0u : 1u);
                    else
                      tc2_mma_bf16_acc(acc, a_lo + 2u * k, a_hi, b_lo + 2u * k, b_hi, idesc);
                  }
                }
              }
              if (!ok) break;
              if (leader) tc2_commit_both(&b_empty[b_slot]);
              __syncwarp();
              if (++b_slot == (uint32_t)p.b_slots) { b_slot = 0; b_par ^= 1u; }
            }
            if (!ok) break;
            if (kd < 2) {
              if (leader) tc2_commit_both(&a_empty[pl_slot[kd]]);
            } else {
#pragma unroll
              for (int j = 2; j < planes; ++j)
                if (leader) tc2_commit_both(&a_empty[pl_slot[j]]);
            }
          }
          a_slot += planes;
          while (a_slot >= (uint32_t)p.a_slots) { a_slot -= p.a_slots; a_par ^= 1u; }
        }
        if (ok && leader) tc2_commit_both(&tfull[buf]);
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int rh = row & 7, rw = row >> 3;
    uint32_t jcount = 0;
    bool ok = true;
    for (int pj = pair; pj < p.num_pair_jobs && ok; pj += npairs, ++jcount) {
      const uint32_t buf = jcount % p.n_bufs;
      const uint32_t use = jcount / p.n_bufs;
      if (!mbar_wait_cl(&tfull[buf], use & 1u, abort_flag, p.status, 76)) { ok = false; break; }
      tc_fence_after();
      const Job2 jc = decode_job2(p, pj, (int)rank);
      const int h = jc.h0 + rh, w = jc.w0 + rw;
      float gcnt = 0.f;  // valid voxels of this warp's 32 rows over the job's planes (lane 0 keeps the total)
      if (STATS) {
        if (lane < 16) { gn_acc[q][lane][0] = 0.f; gn_acc[q][lane][1] = 0.f; }
        __syncwarp();
      }
      for (int t = 0; t < TD; ++t) {
        const int d = jc.d0 + t;
        const bool valid = h < p.H && w < p.W && d < p.D && jc.n < p.N;
        long long vox = (((long long)jc.n * p.D + d) * p.H + h) * p.W + w;
        __nv_bfloat16* slab = nullptr;
        if (p.slab_mode) {
          if (d == 0) slab = p.slab_out[0];
          else if (d == p.D - 1) slab = p.slab_out[1];
          if (slab) vox = ((long long)jc.n * p.H + h) * p.W + w;
          else vox = (((long long)jc.n * (p.D - 2) + (d - 1)) * p.H + h) * p.W + w;
        }
        const uint32_t acc_i = buf * TD + t;
        const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + acc_i * p.BN;
        const int nchunk = p.BN / 32;
        if (STATS) gcnt += (float)__popc(__ballot_sync(0xffffffffu, valid));
        for (int ch = 0; ch < nchunk; ++ch) {
          uint32_t v[32];
          tmem_ld_32x32(tbase + ch * 32, v);
          tmem_ld_wait();
          float st[2][2] = {{0.f, 0.f}, {0.f, 0.f}};  // [half of the chunk][sum, sum of squares], as stored
          if (valid) {
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              const int col = jc.co0 + ch * 32 + g * 16;
              float f[16];
#pragma unroll
              for (int e = 0; e < 16; ++e) f[e] = __uint_as_float(v[g * 16 + e]);
              __nv_bfloat16* dst = nullptr;
              if (slab) {
                if (col < p.width0 + p.width1) dst = slab + vox * p.slab_ld + col;
              } else if (col < p.width0) {
                dst = p.out0 + vox * p.ld0 + col;
                if (p.bias) {
#pragma unroll
                  for (int e = 0; e < 16; ++e) f[e] += p.bias[col + e];
                }
              } else if (col - p.width0 < p.width1) {
                dst = p.out1 + vox * p.ld1 + (col - p.width0);
              }
              if (dst) {
                uint4 lo, hi;
                lo.x = pack_bf16x2(f[0], f[1]);
                lo.y = pack_bf16x2(f[2], f[3]);
                lo.z = pack_bf16x2(f[4], f[5]);
                lo.w = pack_bf16x2(f[6], f[7]);
                hi.x = pack_bf16x2(f[8], f[9]);
                hi.y = pack_bf16x2(f[10], f[11]);
                hi.z = pack_bf16x2(f[12], f[13]);
                hi.w = pack_bf16x2(f[14], f[15]);
                st_global_v8(dst, lo, hi);
                if (STATS) {
                  // the values as stored (bf16-rounded): the statistics describe the tensor the next pass reads
                  const uint32_t w8[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const float a0 = __uint_as_float(w8[e] << 16), a1 = __uint_as_float(w8[e] & 0xffff0000u);
                    st[g][0] += a0 + a1;
                    st[g][1] += a0 * a0 + a1 * a1;
                  }
                }
              }
            }
          }
          if (STATS) {
            // warp sums of the two 16-channel halves; lane 0 adds them to the job's group accumulators (fixed order)
#pragma unroll
            for (int o2 = 16; o2 > 0; o2 >>= 1) {
#pragma unroll
              for (int g = 0; g < 2; ++g) {
                st[g][0] += __shfl_xor_sync(0xffffffffu, st[g][0], o2);
                st[g][1] += __shfl_xor_sync(0xffffffffu, st[g][1], o2);
              }
            }
            if (lane == 0) {
#pragma unroll
              for (int g = 0; g < 2; ++g) {
                const int gl = (ch * 32 + g * 16) / p.gn_cg;  // group of this half inside the job's channel tile
                gn_acc[q][gl][0] += st[g][0];
                gn_acc[q][gl][1] += st[g][1];
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(map_to_rank(smem_u32(&tempty[acc_i]), 0));
      }
      if (STATS) {
        __syncwarp();
        const int groups_here = p.BN / p.gn_cg;
        const float n_vox = __shfl_sync(0xffffffffu, gcnt, 0);
        if (lane < groups_here && jc.n < p.N) {
          const float s1 = gn_acc[q][lane][0], s2 = gn_acc[q][lane][1];
          const float n_el = n_vox * (float)p.gn_cg;
          const float mean = n_el > 0.f ? s1 / n_el : 0.f;
          const float m2 = n_el > 0.f ? fmaxf(s2 - s1 * mean, 0.f) : 0.f;
          const int sj = ((jc.d0 / TD * p.tiles_h + jc.h0 / 8) * p.tiles_w + jc.w0 / 16) * 4 + q;
          const int g_glob = jc.co0 / p.gn_cg + lane;
          float* dst = p.gn_part + (((long long)jc.n * p.gn_splits + sj) * p.gn_groups + g_glob) * 3;
          dst[0] = n_el; dst[1] = mean; dst[2] = m2;
        }
        __syncwarp();  // gn_acc[q] is cleared by this warp at its next job
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let copies in flight land before the shared memory goes away
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000ll) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();  // the leader's MMAs read the peer's shared memory; arrives target the other CTA
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem2_dealloc(tmem_base, 512);
  }
}

static int g_p2_smem = 0, g_p2_sms = 0, g_p2_clusters = 0;
static int p2_setup() {
  if (g_p2_smem) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SB_ERR_DRIVER;
  int lim = 0, sms = 0;
  cudaDeviceGetAttribute(&lim, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const void* fns[6] = {(const void*)conv_plane2_kernel<1, false>, (const void*)conv_plane2_kernel<2, false>,
                        (const void*)conv_plane2_kernel<4, false>, (const void*)conv_plane2_kernel<1, true>,
                        (const void*)conv_plane2_kernel<2, true>, (const void*)conv_plane2_kernel<4, true>};
  for (int i = 0; i < 6; ++i)
    if (cudaFuncSetAttribute(fns[i], cudaFuncAttributeMaxDynamicSharedMemorySize, lim - 2048) != cudaSuccess)
      return SB_ERR_DRIVER;
  g_p2_smem = lim - 2048;
  g_p2_sms = sms;
  // SM pairs that can hold a cluster at the same time (a GPC with an odd SM count leaves one SM out)
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * (sms / 2));
  cfg.blockDim = dim3(224);
  cfg.dynamicSmemBytes = (size_t)g_p2_smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, conv_plane2_kernel<2, true>, &cfg) == cudaSuccess && n > 0 && n < sms / 2)
    g_p2_clusters = n;
  else
    g_p2_clusters = sms / 2;
  cudaGetLastError();
  return 0;
}

static int cdiv_p2(int a, int b) { return (a + b - 1) / b; }

// Shape rule of the pair kernel. Returns the widest tile (128 or 256) the call admits, 0 when it is not eligible.
int conv_plane2_bn(const SbConvArgs* a) {
  if (a->ksize != 3 || a->W < 16 || a->H < 8 || a->wpack == nullptr) return 0;
  if (a->cout_pad < 128 || a->cout_pad % 128 != 0) return 0;
  const int cin_tot = a->src_c[0] + a->src_c[1];
  if (a->src_c[0] % P2_BK != 0 || cin_tot % P2_BK != 0) return 0;
  const long long tiles = (long long)a->N * a->D * cdiv_p2(a->H, 8) * cdiv_p2(a->W, 16);
  if (tiles < 2) return 0;
  return a->cout_pad % 256 == 0 ? 256 : 128;
}

// Tile width BN and job depth TD (output planes that share one set of weight taps) by a cost model fitted to
// measurements on B200:  time ~ waves x (MMA cycles of a job x penalty + exposed epilogue), where
//   waves   = ceil(pair-jobs / SM pairs)               (small volumes: more, smaller jobs fill the machine)
//   penalty = 1.4 for (BN 128, TD 1): an 8 KB weight tap then feeds only four MMAs and the loop starves on
//             weight-tile traffic; 1.05 for (128, 2); 1.0 otherwise
//   exposed epilogue = TD x BN x 5 cycles when the accumulators cannot double-buffer (TD x BN = 512 columns).
// Ties go to the wider tile, then to the deeper job. Returns false when nothing fits.
static bool p2_choose(const SbConvArgs* a, int bn_max, int cblks, int clusters, int a_slot_bytes, int smem_budget,
                      int* bn_out, int* td_out) {
  const int tiles_h = cdiv_p2(a->H, 8), tiles_w = cdiv_p2(a->W, 16);
  double best = 0.0;
  bool found = false;
  for (int bn = bn_max; bn >= 128; bn /= 2) {
    const int b_slot_bytes = (bn / 2) * P2_ROWB;
    for (int td = 512 / bn; td >= 1; td /= 2) {
      if (td > a->D && td > 1) continue;
      if ((td + 2) * a_slot_bytes + 3 * b_slot_bytes > smem_budget) continue;
      const long long tl = (long long)a->N * cdiv_p2(a->D, td) * tiles_h * tiles_w;
      const long long jobs = ((tl + 1) / 2) * (a->cout_pad / bn);
      const long long waves = (jobs + clusters - 1) / clusters;
      const double penalty = bn == 128 ? (td == 1 ? 1.4 : td == 2 ? 1.05 : 1.0) : 1.0;
      const double mma = (double)cblks * 27.0 * td * P2_KSTEPS * (bn / 2) * penalty;
      const double epi = (td * bn == 512) ? td * bn * 5.0 : 0.0;
      const double cost = (double)waves * (mma + epi);
      if (!found || cost < best * 0.999) {
        best = cost;
        *bn_out = bn;
        *td_out = td;
        found = true;
      }
    }
  }
  return found;
}

// GroupNorm statistics from the epilogue: one destination, no slab outputs, groups of whole 16-channel halves of a
// TMEM chunk that do not straddle channel tiles, at most 16 groups per tile.
static bool p2_gn_ok(const SbConvArgs* a, int bn) {
  if (a->gn_groups < 1 || a->dst[1] != nullptr || a->slab_out[0] != nullptr) return false;
  if (a->dst_c[0] != a->cout_pad || a->cout_pad % a->gn_groups != 0) return false;
  const int cg = a->cout_pad / a->gn_groups;
  return cg % 16 == 0 && cg <= bn && bn % cg == 0 && bn / cg <= 16;
}

// Partials per sample the pair kernel would write for this call (0: it will not produce statistics).
int conv_plane2_gn_splits(const SbConvArgs* a) {
  const int bn_max = conv_plane2_bn(a);
  if (bn_max == 0 || p2_setup() != 0) return 0;
  const int cblks = (a->src_c[0] + a->src_c[1]) / P2_BK;
  const int a_tx = P2_RH * P2_RW * P2_ROWB;
  const int a_slot_bytes = ((a_tx + 1023) / 1024) * 1024;
  int bn = 0, td = 1;
  if (!p2_choose(a, bn_max, cblks, g_p2_clusters, a_slot_bytes, g_p2_smem - 1024, &bn, &td)) return 0;
  if (!p2_gn_ok(a, bn)) return 0;
  // the launcher's own refusals (it then falls back to the single-CTA kernels, which get no partial buffer)
  if (a->dst_c[0] % 16 || a->dst_ld[0] % 16 || (reinterpret_cast<uintptr_t>(a->dst[0]) & 31)) return 0;
  return cdiv_p2(a->D, td) * cdiv_p2(a->H, 8) * cdiv_p2(a->W, 16) * 4;
}

// Returns -1 when the shape is not eligible (the caller then uses the single-CTA kernels).
int conv_plane2_launch(const SbConvArgs* a, cudaStream_t stream) {
  const int bn_max = conv_plane2_bn(a);
  if (bn_max == 0) return -1;
  int rc = p2_setup();
  if (rc) return rc;
  Plane2Params p;
  memset(&p, 0, sizeof(p));
  const int cin_tot = a->src_c[0] + a->src_c[1];
  const int nsrc = a->src_c[1] > 0 ? 2 : 1;
  const int rowb = P2_ROWB;
  const int clusters = g_p2_clusters;
  const int cblks = cin_tot / P2_BK;
  p.a_tx = P2_RH * P2_RW * rowb;
  p.a_slot_bytes = ((p.a_tx + 1023) / 1024) * 1024;
  int td = 1;
  if (!p2_choose(a, bn_max, cblks, clusters, p.a_slot_bytes, g_p2_smem - 1024, &p.BN, &td)) return -1;
  p.N = a->N; p.D = a->D; p.H = a->H; p.W = a->W;
  p.tiles_h = cdiv_p2(a->H, 8);
  p.tiles_w = cdiv_p2(a->W, 16);
  p.tiles_co = a->cout_pad / p.BN;
  p.b_tx = (p.BN / 2) * rowb;
  p.b_slot_bytes = ((p.b_tx + 1023) / 1024) * 1024;
  const int max_acc = 512 / p.BN;
  p.TD = td;
  p.n_bufs = max_acc / td >= 2 ? 2 : 1;
  p.groups_d = cdiv_p2(a->D, td);
  const long long tiles = (long long)a->N * p.groups_d * p.tiles_h * p.tiles_w;
  p.num_pair_jobs = (int)(((tiles + 1) / 2) * p.tiles_co);
  const int budget = g_p2_smem - 1024;
  int a_slots = td + 3;
  while (a_slots > td + 2 && a_slots * p.a_slot_bytes + 3 * p.b_slot_bytes > budget) --a_slots;
  if (a_slots > P2_MAX_A) a_slots = P2_MAX_A;
  if (a_slots * p.a_slot_bytes + 3 * p.b_slot_bytes > budget) return -1;
  int b_slots = (budget - a_slots * p.a_slot_bytes) / p.b_slot_bytes;
  if (b_slots > P2_MAX_B) b_slots = P2_MAX_B;
  if (b_slots < 3) return -1;
  p.a_slots = a_slots;
  p.b_slots = b_slots;
  p.cblks0 = a->src_c[0] / P2_BK;
  p.cblks = cblks;
  for (int s = 0; s < nsrc; ++s) {
    const long long C = a->src_ld[s];
    const long long iD = a->in_d ? a->in_d : a->D, iH = a->in_h ? a->in_h : a->H, iW = a->in_w ? a->in_w : a->W;
    long long dims[5] = {a->src_c[s], iH, iW, iD, a->N};
    long long str[5] = {1, iW * C, C, iH * iW * C, iD * iH * iW * C};
    int box[5] = {P2_BK, P2_RH, P2_RW, 1, 1};
    rc = make_map_bf16(&p.mapA[s], a->src[s], 5, dims, str, box, rowb);
    if (rc) return rc;
  }
  if (nsrc == 1) p.mapA[1] = p.mapA[0];
  {
    long long dims[3] = {cin_tot, a->cout_pad, 27};
    long long str[3] = {1, cin_tot, (long long)a->cout_pad * cin_tot};
    int box[3] = {P2_BK, p.BN / 2, 1};
    rc = make_map_bf16(&p.mapB, a->wpack, 3, dims, str, box, rowb);
    if (rc) return rc;
  }
  p.out0 = (__nv_bfloat16*)a->dst[0];
  p.out1 = (__nv_bfloat16*)a->dst[1];
  p.width0 = a->dst_c[0];
  p.width1 = a->dst[1] ? a->dst_c[1] : 0;
  p.ld0 = a->dst_ld[0];
  p.ld1 = a->dst_ld[1];
  // the epilogue stores 16 channels (32 bytes) at a time
  if (p.width0 % 16 || p.width1 % 16 || p.ld0 % 16 || p.ld1 % 16) return -1;
  if ((reinterpret_cast<uintptr_t>(a->dst[0]) & 31) || (a->dst[1] && (reinterpret_cast<uintptr_t>(a->dst[1]) & 31)))
    return -1;
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
        int box[5] = {P2_BK, P2_RH, P2_RW, 1, 1};
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
  if (p.slab_mode && (p.slab_ld % 16 != 0 || a->D < 3)) return -1;
  if (p.slab_mode && ((reinterpret_cast<uintptr_t>(a->slab_out[0]) & 31) || (reinterpret_cast<uintptr_t>(a->slab_out[1]) & 31)))
    return -1;
  const int use = p.num_pair_jobs < clusters ? p.num_pair_jobs : clusters;
  const int grid = 2 * use;
  const size_t smem = (size_t)p.a_slots * p.a_slot_bytes + (size_t)p.b_slots * p.b_slot_bytes + 1024;
  if (a->gn_part != nullptr) {
    if (!p2_gn_ok(a, p.BN)) return SB_ERR_SHAPE;
    p.gn_part = a->gn_part;
    p.gn_groups = a->gn_groups;
    p.gn_cg = a->cout_pad / a->gn_groups;
    p.gn_splits = p.groups_d * p.tiles_h * p.tiles_w * 4;
    if (td == 4) conv_plane2_kernel<4, true><<<grid, 224, smem, stream>>>(p);
    else if (td == 2) conv_plane2_kernel<2, true><<<grid, 224, smem, stream>>>(p);
    else conv_plane2_kernel<1, true><<<grid, 224, smem, stream>>>(p);
  } else {
    if (td == 4) conv_plane2_kernel<4, false><<<grid, 224, smem, stream>>>(p);
    else if (td == 2) conv_plane2_kernel<2, false><<<grid, 224, smem, stream>>>(p);
    else conv_plane2_kernel<1, false><<<grid, 224, smem, stream>>>(p);
  }
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

}  // namespace sb

// Tile width and job depth the pair kernel would use for this call on a device with `clusters` SM pairs
// (no device needed: the host-side tests pin the selection). Returns 0 and fills bn / td, or -1 when the
// call is not eligible.
extern "C" int sb_conv_pair_plan(const SbConvArgs* a, int clusters, int* bn, int* td) {
  const int bn_max = sb::conv_plane2_bn(a);
  if (bn_max == 0 || clusters < 1) return -1;
  const int cblks = (a->src_c[0] + a->src_c[1]) / sb::P2_BK;
  const int a_tx = sb::P2_RH * sb::P2_RW * sb::P2_ROWB;
  const int a_slot_bytes = ((a_tx + 1023) / 1024) * 1024;
  const int budget = 232448 - 2048 - 1024;  // opt-in shared memory of an sm_100 CTA less the launcher's reserve
  return sb::p2_choose(a, bn_max, cblks, clusters, a_slot_bytes, budget, bn, td) ? 0 : -1;
}
