// IFS chaos game shared by the CPU library and the CUDA kernels: one orbit of
// a two-map affine iterated function system in float64.
//
//   params[2][13]: cols 0-8 row-major 3x3 matrix, 9-11 translation, 12 the
//   probability of map 0. x0 = 0; each step draws r in [0,1): map 0 if r < p0.
//   A coordinate beyond 1e10 in magnitude marks the orbit as runaway.
//
// The random stream is SplitMix64 seeded per orbit, identical on host and
// device, so the GPU generator is checked bit for bit against the CPU one.
// Role of the reference: ScaFFold/datagen/generate_fractal_points.py:23-126.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define SB_HD __host__ __device__ __forceinline__
#else
#define SB_HD inline
#endif

namespace sbifs {

struct Rng {
  uint64_t s;
};
SB_HD uint64_t next_u64(Rng& r) {
  uint64_t z = (r.s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
SB_HD double next_unit(Rng& r) { return (double)(next_u64(r) >> 11) * (1.0 / 9007199254740992.0); }

SB_HD void step(const double* P, double p0, Rng& rng, double& x, double& y, double& z) {
  const double r = next_unit(rng);
  const double* m = r < p0 ? P : P + 13;
  const double nx = x * m[0] + y * m[1] + z * m[2] + m[9];
  const double ny = x * m[3] + y * m[4] + z * m[5] + m[10];
  const double nz = x * m[6] + y * m[7] + z * m[8] + m[11];
  x = nx; y = ny; z = nz;
}

// Running statistics of an orbit (Welford per axis), enough for the acceptance test:
// finite, per-axis range > 0, variance of the normalised cloud above the threshold.
struct Stats {
  double mn[3], mx[3], mean[3], m2[3];
  long long count;
  int runaway, nonfinite;
};
SB_HD void stats_init(Stats& s) {
  for (int a = 0; a < 3; ++a) { s.mn[a] = 1e300; s.mx[a] = -1e300; s.mean[a] = 0.0; s.m2[a] = 0.0; }
  s.count = 0; s.runaway = 0; s.nonfinite = 0;
}
SB_HD void stats_add(Stats& s, double x, double y, double z) {
  const double v[3] = {x, y, z};
  s.count += 1;
  for (int a = 0; a < 3; ++a) {
    const double c = v[a];
    if (!(c == c) || c > 1e300 || c < -1e300) s.nonfinite = 1;
    if (c > 1e10 || c < -1e10) s.runaway = 1;
    if (c < s.mn[a]) s.mn[a] = c;
    if (c > s.mx[a]) s.mx[a] = c;
    const double d = c - s.mean[a];
    s.mean[a] += d / (double)s.count;
    s.m2[a] += d * (c - s.mean[a]);
  }
}

}  // namespace sbifs
