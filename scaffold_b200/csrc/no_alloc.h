// GroupNorm(+ReLU) forward for callers that must not allocate.
//
// This entry point has no counterpart in the reference; it exists for hosts of
// this library that cannot call cudaMalloc (or any allocating routine) at the
// point where they need a normalisation: code running between the begin and end
// of a stream capture, plugins that were handed a fixed memory budget at
// start-up, and runtimes that forbid allocation after initialisation because an
// allocation may synchronise the device.
//
// The two-pass kernel needs scratch memory for its per-split partial statistics.
// The ordinary entry points (sb_gn_stats / sb_gn_apply) take that scratch from
// the caller; this one keeps it in a fixed array inside the library:
//
//   * capacity: SB_GN_NOALLOC_SCRATCH_FLOATS floats (1 MiB) per GPU that loads
//     the library, held until the process exits;
//   * a call needs N * (nsplit + 1) * G * 3 floats, nsplit = sb_gn_nsplit(N, S, C);
//     larger requests are refused with SB_ERR_TOO_LARGE, nothing is launched;
//   * every call on a device shares the array. Nothing in it has to start at
//     zero (each call overwrites what it reads), but two calls that overlap on
//     the GPU (different streams, no ordering) race on it: serialise them;
//   * the first call on each device resolves the array's device address. Make
//     that first call outside any stream capture.
//
// x, y: bf16 [N, S, C] voxel-major; w, b: fp32 [C]; mean, rstd: fp32 [N, G]
// outputs (may be null). Returns 0 or an SB_ERR_* code.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SB_GN_NOALLOC_SCRATCH_FLOATS (1 << 18)

int sb_gn_forward_noalloc(const void* x, void* y, const float* w, const float* b, float* mean, float* rstd, int N,
                          long long S, int C, int G, float eps, int relu, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
