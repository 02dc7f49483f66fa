// Cross-GPU flag primitives shared by the peer-memory kernels: release / acquire accesses at system scope and a
// bounded all-to-all barrier over per-rank flag rows (monotonically increasing epochs, never reset).
#pragma once
#include <cuda_runtime.h>
#include "ops_api.h"

namespace b200 {

constexpr int kMaxRanks = 16;
// Secondary bound of every flag wait (the primary one is NmtgPeerTable::timeout_ns of wall time): with the back-off
// below a poll takes a fraction of a microsecond at least, so this many polls is minutes.
constexpr unsigned kFlagPollCap = 1u << 30;

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
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Waits until *flag >= epoch.  Gives up after t.timeout_ns nanoseconds (or kFlagPollCap polls) and returns false.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, long long timeout_ns) {
  const unsigned long long t0 = global_timer_ns();
  for (unsigned i = 0; i < kFlagPollCap; ++i) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    if (i > 64) {
      __nanosleep(i > 4096 ? 256 : 32);
      if ((i & 63) == 0 && static_cast<long long>(global_timer_ns() - t0) > timeout_ns) return false;
    }
  }
  return false;
}

// Thread i < world publishes `epoch` in slot `rank` of peer i's flag row (when `publish` is set), then waits until
// slot i of the local row reaches `epoch`.  Returns false for the whole CTA when any wait ran out of time (status 5).
// Uses no shared memory (the verdict travels through the barrier's own OR), so kernels built on it can share an SM
// with a CTA that owns nearly all of the SM's shared memory.
__device__ __forceinline__ bool peer_barrier(const NmtgPeerTable& t, int row, int epoch, int* status, bool publish = true) {
  int fail = 0;
  if (threadIdx.x < t.world) {
    if (publish) {
      __threadfence_system();
      st_release_sys(t.flags[threadIdx.x] + row * kMaxRanks + t.rank, epoch);
    }
    if (!wait_flag(t.flags[t.rank] + row * kMaxRanks + threadIdx.x, epoch, t.timeout_ns)) {
      fail = 1;
      if (status) atomicCAS(status, 0, 5 /* kTimeoutPeerFlag */);
    }
  }
  return __syncthreads_or(fail) == 0;
}

// Publish only (no wait): slot `rank` of every peer's row.
__device__ __forceinline__ void peer_publish(const NmtgPeerTable& t, int row, int epoch) {
  if (threadIdx.x < t.world) {
    __threadfence_system();
    st_release_sys(t.flags[threadIdx.x] + row * kMaxRanks + t.rank, epoch);
  }
}

}  // namespace b200
