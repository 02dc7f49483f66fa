// Index checks of the debug build (-DNMTG_DEBUG_BOUNDS).  An index that comes from the caller's data (token ids, labels,
// sequence lengths, cache positions, gather indices) is always brought into range before it is used; the debug build
// also counts every such correction, so that a test run can assert that no kernel ever saw a bad index.  Nothing traps.
// Every translation unit that includes this header has its own counter and exports a reader for it with
// NMTG_BOUNDS_READER(name); nmtg_bounds_violations() in elementwise.cu sums the readers (-1: checks compiled out).
#pragma once
#include <cuda_runtime.h>

#ifdef NMTG_DEBUG_BOUNDS
namespace b200 {
namespace {
__device__ unsigned int tu_bounds_violations = 0;
}
}  // namespace b200
#define NMTG_BOUNDS_HIT() atomicAdd(&b200::tu_bounds_violations, 1u)
#define NMTG_BOUNDS_READER(name)                                                                                  \
  extern "C" long name() {                                                                                        \
    unsigned int v = 0;                                                                                           \
    if (cudaMemcpyFromSymbol(&v, b200::tu_bounds_violations, sizeof(v)) != cudaSuccess) return -2;                 \
    return static_cast<long>(v);                                                                                  \
  }
#else
#define NMTG_BOUNDS_HIT() ((void)0)
#define NMTG_BOUNDS_READER(name) \
  extern "C" long name() { return -1; }
#endif

namespace b200 {
// v clamped into [lo, hi]; a correction is counted in the debug build
__device__ __forceinline__ int checked_range(int v, int lo, int hi) {
  if (v < lo) { NMTG_BOUNDS_HIT(); return lo; }
  if (v > hi) { NMTG_BOUNDS_HIT(); return hi; }
  return v;
}
__device__ __forceinline__ long checked_range(long v, long lo, long hi) {
  if (v < lo) { NMTG_BOUNDS_HIT(); return lo; }
  if (v > hi) { NMTG_BOUNDS_HIT(); return hi; }
  return v;
}
}  // namespace b200
