// Cross-GPU flag primitives shared by the peer-memory kernels: release / acquire accesses at system scope and a
// bounded all-to-all barrier over per-rank flag rows (monotonically increasing epochs, never reset).
#pragma once
#include <cuda_runtime.h>
#include "ops_api.h"

namespace b200 {

constexpr int kMaxRanks = 16;
constexpr unsigned kFlagPolls = 1u << 22;

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Thread i < n publishes `epoch` in slot `rank` of peer i's flag row, then waits until slot i of the local
// row reaches `epoch`.  Returns false for the whole CTA when any wait ran out of polls (status = 5).
__device__ __forceinline__ bool peer_barrier(const NmtgPeerTable& t, int row, int epoch, int* status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < t.world) {
    __threadfence_system();
    st_release_sys(t.flags[threadIdx.x] + row * kMaxRanks + t.rank, epoch);
    const int* mine = t.flags[t.rank] + row * kMaxRanks + threadIdx.x;
    bool ok = false;
    for (unsigned i = 0; i < kFlagPolls; ++i) {
      if (ld_acquire_sys(mine) >= epoch) { ok = true; break; }
      if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
    }
    if (!ok) {
      s_fail = 1;
      if (status) atomicCAS(status, 0, 5 /* kTimeoutPeerFlag */);
    }
  }
  __syncthreads();
  return s_fail == 0;
}

}  // namespace b200
