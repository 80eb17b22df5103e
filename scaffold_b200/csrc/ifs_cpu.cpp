// CPU side of the data generator: chaos-game orbits and point-cloud voxelisation.
// These are the oracles (and the CPU/gloo path) of the CUDA kernels in ifs.cu.
#include <cmath>
#include <cstring>

#include "host_api.h"
#include "ifs_common.h"

using namespace sbifs;

// out_stats[16]: min3, max3, mean3, var3 (population), count, runaway, nonfinite, unused
extern "C" int sb_ifs_orbit_cpu(const double* params, unsigned long long seed, long long n, float* out_points,
                                double* out_stats) {
  Rng rng{seed};
  Stats st;
  stats_init(st);
  double x = 0, y = 0, z = 0;
  const double p0 = params[12];
  for (long long i = 0; i < n; ++i) {
    if (i > 0) step(params, p0, rng, x, y, z);
    stats_add(st, x, y, z);
    if (out_points) {
      out_points[3 * i] = (float)x;
      out_points[3 * i + 1] = (float)y;
      out_points[3 * i + 2] = (float)z;
    }
  }
  if (out_stats) {
    for (int a = 0; a < 3; ++a) {
      out_stats[a] = st.mn[a];
      out_stats[3 + a] = st.mx[a];
      out_stats[6 + a] = st.mean[a];
      out_stats[9 + a] = st.count > 0 ? st.m2[a] / (double)st.count : 0.0;
    }
    out_stats[12] = (double)st.count;
    out_stats[13] = st.runaway;
    out_stats[14] = st.nonfinite;
    out_stats[15] = 0;
  }
  return 0;
}

// Isotropic normalisation + centring + floor + clip of a float32 point cloud into a G^3 grid;
// marks occupancy[d][h][w] = 1 (uint8, caller zeroes it). Returns SB_ERR_SHAPE on non-finite input.
// Role of the reference: ScaFFold/datagen/volumegen.py:103-160.
extern "C" int sb_voxelize_cpu(const float* pts, long long n, int G, unsigned char* occupancy) {
  double mn[3] = {1e300, 1e300, 1e300}, mx[3] = {-1e300, -1e300, -1e300};
  for (long long i = 0; i < n; ++i)
    for (int a = 0; a < 3; ++a) {
      const double c = pts[3 * i + a];
      if (!std::isfinite(c)) return SB_ERR_SHAPE;
      if (c < mn[a]) mn[a] = c;
      if (c > mx[a]) mx[a] = c;
    }
  double ext = 0;
  for (int a = 0; a < 3; ++a) ext = std::fmax(ext, mx[a] - mn[a]);
  const double voxel = (ext + 1e-6) / G;
  double off[3];
  for (int a = 0; a < 3; ++a) off[a] = (G - (mx[a] - mn[a]) / voxel) / 2.0;
  for (long long i = 0; i < n; ++i) {
    int idx[3];
    for (int a = 0; a < 3; ++a) {
      long long v = (long long)std::floor((pts[3 * i + a] - mn[a]) / voxel + off[a]);
      idx[a] = (int)(v < 0 ? 0 : (v > G - 1 ? G - 1 : v));
    }
    occupancy[((size_t)idx[0] * G + idx[1]) * G + idx[2]] = 1;
  }
  return 0;
}
