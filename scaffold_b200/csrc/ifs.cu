// GPU data generation: batched IFS chaos game and point-cloud rasterisation.
//
//   ifs_search_kernel   one thread per candidate: runs the float64 orbit and
//                       keeps only running statistics (min/max/mean/M2 per
//                       axis, runaway / non-finite flags) -> the acceptance
//                       test of the category search needs no point storage
//   ifs_points_kernel   one thread per instance: writes the float32 cloud
//   voxel_bbox / voxel_paint   per-cloud bounding box (block reduction), then
//                       isotropic normalise + centre + floor + clip and paint
//                       the class colour / label straight into the shard-local
//                       (3,d,h,w) fp32 volume and uint16 mask
//
// Role of the reference: ScaFFold/datagen/generate_fractal_points.py:23-126,
// ScaFFold/datagen/category_search.py:114-201, ScaFFold/datagen/volumegen.py:103-160,259-294.
#include "common.cuh"
#include "host_api.h"
#include "ifs_common.h"

namespace sb {
using namespace sbifs;

__global__ void ifs_search_kernel(const double* __restrict__ params, const unsigned long long* __restrict__ seeds,
                                  int batch, long long n, double* __restrict__ out) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  double P[26];
  for (int i = 0; i < 26; ++i) P[i] = params[(size_t)b * 26 + i];
  Rng rng{seeds[b]};
  Stats st;
  stats_init(st);
  double x = 0, y = 0, z = 0;
  const double p0 = P[12];
  for (long long i = 0; i < n; ++i) {
    if (i > 0) step(P, p0, rng, x, y, z);
    stats_add(st, x, y, z);
  }
  double* o = out + (size_t)b * 16;
  for (int a = 0; a < 3; ++a) {
    o[a] = st.mn[a];
    o[3 + a] = st.mx[a];
    o[6 + a] = st.mean[a];
    o[9 + a] = st.count > 0 ? st.m2[a] / (double)st.count : 0.0;
  }
  o[12] = (double)st.count;
  o[13] = st.runaway;
  o[14] = st.nonfinite;
  o[15] = 0;
}

__global__ void ifs_points_kernel(const double* __restrict__ params, const unsigned long long* __restrict__ seeds,
                                  int batch, long long n, float* __restrict__ pts, int* __restrict__ flags) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  double P[26];
  for (int i = 0; i < 26; ++i) P[i] = params[(size_t)b * 26 + i];
  Rng rng{seeds[b]};
  double x = 0, y = 0, z = 0;
  const double p0 = P[12];
  int bad = 0;
  float* o = pts + (size_t)b * n * 3;
  for (long long i = 0; i < n; ++i) {
    if (i > 0) step(P, p0, rng, x, y, z);
    if (!(x == x) || !(y == y) || !(z == z)) bad |= 2;
    if (fabs(x) > 1e10 || fabs(y) > 1e10 || fabs(z) > 1e10) bad |= 1;
    o[3 * i] = (float)x;
    o[3 * i + 1] = (float)y;
    o[3 * i + 2] = (float)z;
  }
  flags[b] = bad;
}

// bbox[cloud][6] = min xyz, max xyz ; one block per cloud
__global__ void __launch_bounds__(256) voxel_bbox_kernel(const float* __restrict__ pts, long long n,
                                                         float* __restrict__ bbox) {
  __shared__ float smin[3][256], smax[3][256];
  const float* p = pts + (size_t)blockIdx.x * n * 3;
  float mn[3] = {INFINITY, INFINITY, INFINITY}, mx[3] = {-INFINITY, -INFINITY, -INFINITY};
  for (long long i = threadIdx.x; i < n; i += 256)
    for (int a = 0; a < 3; ++a) {
      const float c = p[3 * i + a];
      mn[a] = fminf(mn[a], c);
      mx[a] = fmaxf(mx[a], c);
    }
  for (int a = 0; a < 3; ++a) { smin[a][threadIdx.x] = mn[a]; smax[a][threadIdx.x] = mx[a]; }
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s)
      for (int a = 0; a < 3; ++a) {
        smin[a][threadIdx.x] = fminf(smin[a][threadIdx.x], smin[a][threadIdx.x + s]);
        smax[a][threadIdx.x] = fmaxf(smax[a][threadIdx.x], smax[a][threadIdx.x + s]);
      }
    __syncthreads();
  }
  if (threadIdx.x < 3) {
    bbox[blockIdx.x * 6 + threadIdx.x] = smin[threadIdx.x][0];
    bbox[blockIdx.x * 6 + 3 + threadIdx.x] = smax[threadIdx.x][0];
  }
}

// Paints cloud `blockIdx.y` into the shard [lo, hi) of a G^3 grid. Later clouds overwrite earlier
// ones where they overlap only if launched later: callers paint the clouds of a volume one launch each.
__global__ void __launch_bounds__(256) voxel_paint_kernel(const float* __restrict__ pts, long long n,
                                                          const float* __restrict__ bbox, int G, int lo_d, int lo_h,
                                                          int lo_w, int sd, int sh, int sw, float r, float g,
                                                          float b, unsigned short label, float* __restrict__ vol,
                                                          unsigned short* __restrict__ mask) {
  const double mn[3] = {bbox[0], bbox[1], bbox[2]};
  const double ex[3] = {(double)bbox[3] - bbox[0], (double)bbox[4] - bbox[1], (double)bbox[5] - bbox[2]};
  const double ext = fmax(ex[0], fmax(ex[1], ex[2]));
  const double voxel = (ext + 1e-6) / G;
  const size_t plane = (size_t)sd * sh * sw;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    int idx[3];
    for (int a = 0; a < 3; ++a) {
      const double off = (G - ex[a] / voxel) / 2.0;
      long long v = (long long)floor(((double)pts[3 * i + a] - mn[a]) / voxel + off);
      idx[a] = (int)(v < 0 ? 0 : (v > G - 1 ? G - 1 : v));
    }
    const int d = idx[0] - lo_d, h = idx[1] - lo_h, w = idx[2] - lo_w;
    if (d < 0 || d >= sd || h < 0 || h >= sh || w < 0 || w >= sw) continue;
    const size_t o = ((size_t)d * sh + h) * sw + w;
    vol[o] = r;
    vol[plane + o] = g;
    vol[2 * plane + o] = b;
    mask[o] = label;
  }
}

}  // namespace sb

using namespace sb;

extern "C" int sb_ifs_search(const double* params, const unsigned long long* seeds, int batch, long long n,
                             double* out, cudaStream_t stream) {
  ifs_search_kernel<<<(batch + 63) / 64, 64, 0, stream>>>(params, seeds, batch, n, out);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_ifs_points(const double* params, const unsigned long long* seeds, int batch, long long n,
                             float* pts, int* flags, cudaStream_t stream) {
  ifs_points_kernel<<<(batch + 63) / 64, 64, 0, stream>>>(params, seeds, batch, n, pts, flags);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_voxel_bbox(const float* pts, int clouds, long long n, float* bbox, cudaStream_t stream) {
  voxel_bbox_kernel<<<clouds, 256, 0, stream>>>(pts, n, bbox);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}

extern "C" int sb_voxel_paint(const float* pts, long long n, const float* bbox, int G, const int* lo,
                              const int* shape, const float* rgb, int label, float* vol, unsigned short* mask,
                              cudaStream_t stream) {
  long long blocks = (n + 255) / 256;
  if (blocks > 1024) blocks = 1024;
  voxel_paint_kernel<<<(unsigned)blocks, 256, 0, stream>>>(pts, n, bbox, G, lo[0], lo[1], lo[2], shape[0], shape[1],
                                                          shape[2], rgb[0], rgb[1], rgb[2], (unsigned short)label,
                                                          vol, mask);
  sb_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? 0 : SB_ERR_LAUNCH;
}
