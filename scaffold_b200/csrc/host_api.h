// C ABI of libscaffold_b200.so. Every entry point takes raw device pointers and
// a CUDA stream, allocates nothing and returns 0 or an SB_ERR_* code; the
// Python layer (scaffold_b200/ops/_lib.py) mirrors these structs with ctypes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  SB_OK = 0,
  SB_ERR_DRIVER = 1,     // could not resolve / call the driver entry point
  SB_ERR_ALIGN = 2,      // pointer or stride violates a TMA alignment rule
  SB_ERR_TENSORMAP = 3,  // cuTensorMapEncodeTiled refused the description
  SB_ERR_SHAPE = 4,      // shape outside what the kernel supports
  SB_ERR_LAUNCH = 5,     // launch error
  SB_ERR_TOO_LARGE = 6,  // request exceeds a fixed capacity
};

// stride-1 "same" convolution (k = 1 or 3) over up to two channel-concatenated
// NDHWC bf16 sources into up to two channel-split NDHWC bf16 destinations
typedef struct {
  const void* src[2];
  int src_c[2];   // channels read from each source (src_c[1] = 0: one source)
  int src_ld[2];  // channel stride (elements per voxel) of each source
  int N, D, H, W;
  int ksize;
  const void* wpack;  // bf16 [taps][cout_pad][cin_total], taps ordered (kd,kh,kw)
  int cout_pad;       // rows per tap in wpack (multiple of 16)
  void* dst[2];
  int dst_c[2];   // channels stored into each destination (multiples of 8)
  int dst_ld[2];  // channel stride of each destination
  const float* bias;  // optional, added to destination 0 columns
  uint32_t* status;   // optional 4-word status block
  int force_plain;    // 0 automatic, 1..3 select a variant of the generic kernel, 4 automatic without the pair kernel
  // Spatially sharded volumes: the sources may carry a halo. in_* are the sources' spatial
  // extents (0 = same as D/H/W) and off_* the position of output voxel 0 inside them, so
  // input coordinate = output coordinate + tap - k/2 + off (negative offsets read zeros).
  int in_d, in_h, in_w;
  int off_d, off_h, off_w;
  // Depth-sharded volume with the halo fused into the kernel (plane-walk kernel only): the
  // sources hold this rank's planes only; plane -1 / plane in_d are read from landing slabs
  // [N,1,H,W,src_c] that the neighbours fill over NVLink, after the flag word reached the epoch.
  const void* halo_land[2][2];   // [source][0 = low face, 1 = high face], null = volume boundary
  const unsigned* halo_flag[2];  // per face; null = data already in place (no wait)
  unsigned halo_epoch;
  double halo_wait_s;
  // Backward-data of such a convolution: the output grid has D+2 planes; plane 0 and plane D+1
  // (gradient of the halo) go to slab_out[0] / slab_out[1] ([N,1,H,W,slab_ld]), the rest to dst.
  void* slab_out[2];
  int slab_ld;
  // Optional second packing of the same 3x3x3 weights, taps ordered (kh, kw, 2-kd): lets the
  // kd-fused kernel (conv_plane3.cu) fetch the three kd taps of a (kh, kw) pair as one box.
  const void* wpack_kd;
  // fp32 scratch for kernels that split the reduction (conv_small.cu); sb_conv_fwd_workspace() says how much
  float* workspace;
  long long workspace_elems;
  // GroupNorm statistics of the OUTPUT from the epilogue (kd-fused kernel, one destination): when gn_part is set,
  // every job also writes (count, mean, M2) of the bf16-rounded values it stored, per group of C / gn_groups
  // channels, into gn_part[N][splits][gn_groups][3] (splits = sb_conv_gn_splits(); the layout sb_gn_stats writes),
  // so the normalisation that follows skips its own pass over the tensor.
  float* gn_part;
  int gn_groups;
} SbConvArgs;

// One pass over fp32 3x3x3 weights [cout][cin][27] -> bf16 operand layouts (null = not wanted):
// fwd / fwd_kd [27][cout_pad][cin_pad], dgrad / dgrad_kd [27][cin_pad][cout_pad] (pack.cu).
// Input channel c goes to column c (c < real0) or c - real0 + pad0 (second concatenated source).
typedef struct {
  const float* w;
  int cout, cin, real0, pad0, cin_pad, cout_pad;
  void* fwd;
  void* fwd_kd;
  void* dgrad;
  void* dgrad_kd;
  // Volume processed with two spatial axes exchanged (a split along H or W runs as a split along depth): the
  // kernels then need the weight with the same two tap axes exchanged. 0 none, 1 kd <-> kh, 2 kd <-> kw.
  int tap_swap;
} SbPackArgs;

// One entry of the whole-model packing table (sb_pack_conv3_batch): tile0 / tiles_x are filled by sb_pack_conv3_plan.
typedef struct {
  SbPackArgs a;
  int tile0, tiles_x;
} SbPackJob;

// k=2,s=2 transposed convolution. Forward: src [N,D,H,W,cin] -> dst
// [N,2D,2H,2W,cout], wpack bf16 [8*cout][cin] (row = tap*cout + co).
// Backward-data (sb_convT_dgrad): src = gy [N,2D,2H,2W,cout] -> dst = gx
// [N,D,H,W,cin], wpack bf16 [4][wrows][2*cout] (outer = kd*2+kh, col = kw*cout+co).
typedef struct {
  const void* src;
  int src_ld;
  int N, D, H, W;  // the COARSE grid (input of forward / output of dgrad)
  int cin, cout;
  const void* wpack;
  int wrows;  // dgrad: rows per outer tap in wpack (cin padded to a multiple of 16)
  void* dst;
  int dst_ld;
  const float* bias;
  uint32_t* status;
} SbConvTArgs;

// Weight gradient: out[g][m][j] (fp32) = sum_voxels A[voxel, m] * B_g,j[voxel', n(j)]
// with deterministic split-K partials in `workspace` reduced by sb_wgrad_reduce.
typedef struct {
  const void* gy;  // NDHWC bf16 gradient w.r.t. conv output, [N,D,H,W,gy_ld]
  int gy_c, gy_ld;
  const void* x[2];  // NDHWC bf16 conv inputs (two when the input was a fused concat)
  int x_c[2], x_ld[2];
  int N, D, H, W;
  int ksize;          // 1 or 3 (same conv) ; 2 = k2s2 transposed (gy is the fine grid)
  float* workspace;   // fp32 [splits][taps][gy_c or M][cin_total]
  long long workspace_elems;
  float* dw;          // fp32 gradient in the parameter's own layout
  int dw_cout, dw_cin;  // real (unpadded) channel counts of the parameter
  int accumulate;     // add into dw instead of overwriting
  uint32_t* status;
  int splits;         // 0: choose
  // halo'd x (see SbConvArgs): extents of x (0 = same as the gy grid) and offset of voxel 0 in it
  int xin_d, xin_h, xin_w;
  int xoff_d, xoff_h, xoff_w;
  // depth halo of x kept as separate slabs [N,1,H,W,x_c[s]] (see SbConvArgs.halo_land); null = zeros
  const void* xhalo[2][2];
  // same exchange as SbPackArgs.tap_swap (3x3x3 only): the gradient is computed in the kernels' tap order and
  // stored into dw in the parameter's own order
  int tap_swap;
} SbWgradArgs;

// GroupNorm (+ReLU), channels-last bf16. `parts` lists the partial-statistics
// buffers to merge: this rank's own first, then the spatial peers' (device
// pointers valid on this GPU). S is the local voxel count per sample, S_total
// the voxel count per sample over all shards.
typedef struct {
  const void* x;
  const void* dy;
  void* y;
  const float* w;
  const float* b;
  float* mean;
  float* rstd;
  float* part;
  const float* parts[8];
  int n_parts;
  float* dw;
  float* db;
  int N, C, G;
  long long S, S_total;
  int nsplit;
  float eps;
  int relu;
  // cross-shard statistics over peer memory: when set, the merging kernels first wait (bounded)
  // until wait_flags[i] >= wait_epoch for every i < n_parts (flags and parts are local memory the
  // peers pushed into, see sb_gn_share)
  const unsigned* wait_flags;
  unsigned wait_epoch;
  double wait_s;
  unsigned* status;
  // sb_gn_stats / sb_gn_bwd_partial: when set, the last block of the launch also collapses the partials into
  // fin ([N*G*3] resp. [N*C*2], the output of sb_gn_stats_finalize / sb_gn_bwd_finalize): one launch instead of two
  float* fin;
} SbGnArgs;

// Stores `count` floats of `fin` into dst[r] for every r < world (peer pointers valid on this GPU),
// then publishes `epoch` into flags[r].
int sb_gn_share(const float* fin, long long count, void* const* dst, void* const* flags, int world,
                unsigned epoch, cudaStream_t stream);

// number of kernels this library launched so far in the process
long long sb_launch_count(void);
void sb_count_launch(int n);

int sb_gn_nsplit(int N, long long S, int C);
int sb_gn_stats(const SbGnArgs* a, cudaStream_t stream);
int sb_gn_apply(const SbGnArgs* a, cudaStream_t stream);
int sb_gn_bwd_partial(const SbGnArgs* a, cudaStream_t stream);
int sb_gn_bwd_dx(const SbGnArgs* a, cudaStream_t stream);

int sb_conv_fwd(const SbConvArgs* a, cudaStream_t stream);
long long sb_conv_fwd_workspace(const SbConvArgs* a);
// splits per sample of the statistics the call would write into gn_part; 0 = this call cannot produce them
int sb_conv_gn_splits(const SbConvArgs* a);
// tile width / job depth of the two-SM pair kernel for this call (-1: not eligible); needs no device
int sb_conv_pair_plan(const SbConvArgs* a, int clusters, int* bn, int* td);
int sb_convT_fwd(const SbConvTArgs* a, cudaStream_t stream);
int sb_convT_dgrad(const SbConvTArgs* a, cudaStream_t stream);
int sb_conv_wgrad(const SbWgradArgs* a, cudaStream_t stream);
long long sb_conv_wgrad_workspace(const SbWgradArgs* a);

#ifdef __cplusplus
}
#endif
