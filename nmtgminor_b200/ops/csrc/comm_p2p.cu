// Data-parallel gradient reduction fused with the optimiser, over peer-mapped (NVLink / NVSwitch) memory.
//
// Every rank keeps its flat fp32 gradient buffer and its flat bf16 parameter copy in memory that all other
// ranks of the node have mapped (CUDA IPC).  Rank r OWNS slice r of the flat parameter space: fp32 master
// weights and Adam moments exist only for that slice (optimiser state is sharded N ways).  One step is three
// launches per rank, each ordered after the previous one by the stream:
//
//   reduce_slice   waits (bounded) until every peer has published "gradients ready", then sums slice r of all
//                  N gradient buffers with direct 16-byte peer loads (each CTA fetches its own elements; no
//                  broadcast loads of any kind), writes the fp32 sum to a local buffer, accumulates the
//                  sum of squares of the slice and flags non-finite values.
//   update_slice   publishes the slice's sum of squares to every peer, waits (bounded) for all N partials,
//                  forms the global gradient norm / clip coefficient, applies Adam(W) to the owned slice,
//                  stores the refreshed bf16 parameters of the slice into EVERY rank's parameter copy with
//                  peer stores (the all-gather), and clears this rank's whole gradient buffer.
//   finish_step    publishes "parameters written" and waits (bounded) for all peers, so the next forward
//                  pass reads a complete parameter copy.
//
// Cross-GPU flags are monotonically increasing epochs written with st.release.sys and polled with
// ld.acquire.sys; a waiter that runs out of polls records kTimeoutPeerFlag in the status word and the
// kernel returns (the host raises), so a missing peer can never hang a GPU.  Bytes over NVLink per rank and
// step: (N-1)/N * P * 4 in (gradients) and (N-1)/N * P * 2 out (parameters), against 2 * (N-1)/N * P * 4 for
// a ring all-reduce followed by a replicated optimiser.
//
// Replaces DistributedDataParallel's bucketed NCCL all-reduce + GradScaler.unscale_ + clip_grad_norm +
// optimizer.step of the reference (onmt/train_utils/mp_trainer.py:381-387, 895-1016).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops_api.h"
#include "peer_sync.cuh"

namespace b200 {

int num_sms();

__global__ void __launch_bounds__(512)
reduce_slice_kernel(const NmtgPeerTable t, float* __restrict__ reduced, float* __restrict__ sq_out, int* __restrict__ nonfinite,
                    long slice_begin, long slice_len, const int* __restrict__ epoch_ptr, int* status) {
  const int epoch = *epoch_ptr;
  if (!peer_barrier(t, 0, epoch, status)) return;
  __shared__ float red[16];
  float acc = 0.f;
  const long n4 = slice_len >> 2;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int r = 0; r < t.world; ++r) {
      // start with my own buffer, then walk the ring so the peers' links are loaded evenly
      const int src = (t.rank + r) % t.world;
      const float4 v = reinterpret_cast<const float4*>(t.grads[src] + slice_begin)[i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    reinterpret_cast<float4*>(reduced)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  const bool bad = !isfinite(acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  if (bad) atomicOr(nonfinite, 1);
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) {
      if (isfinite(v)) atomicAdd(sq_out, v);
      else atomicOr(nonfinite, 1);
    }
  }
}

__global__ void __launch_bounds__(512)
update_slice_kernel(const NmtgPeerTable t, const float* __restrict__ reduced, float* __restrict__ master, float* __restrict__ m,
                    float* __restrict__ v, const NmtgAdamHyper* __restrict__ hp, const float* __restrict__ sq_local,
                    const int* __restrict__ nonfinite_local, long slice_begin, long slice_len, long total_len,
                    const int* __restrict__ epoch_ptr, int* status) {
  const int epoch = *epoch_ptr;
  // publish my partial (sum of squares, non-finite flag as a negative value) to every rank, then gather all
  if (threadIdx.x < t.world) {
    const float mine = (*nonfinite_local) ? -1.f : *sq_local;
    t.partials[threadIdx.x][(epoch & 1) * kMaxRanks + t.rank] = mine;
  }
  if (!peer_barrier(t, 1, epoch, status)) return;
  __shared__ float s_coef;
  __shared__ int s_skip;
  const NmtgAdamHyper h = *hp;
  if (threadIdx.x == 0) {
    float total = 0.f;
    int skip = 0;
    for (int r = 0; r < t.world; ++r) {
      const float p = ld_relaxed_sys_f32(&t.partials[t.rank][(epoch & 1) * kMaxRanks + r]);
      if (p < 0.f) skip = 1;
      total += p;
    }
    float coef = h.grad_scale;
    if (h.max_grad_norm > 0.f) {
      const float norm = sqrtf(total) * h.grad_scale;
      if (norm > h.max_grad_norm) coef *= h.max_grad_norm / (norm + 1e-6f);
    }
    s_coef = coef;
    s_skip = skip;
    if (blockIdx.x == 0 && t.norm_out) *t.norm_out = skip ? -1.f : sqrtf(total) * h.grad_scale;
  }
  __syncthreads();
  const float coef = s_coef;
  const bool skip = s_skip != 0;
  const long n4 = slice_len >> 2;
  if (!skip) {
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
      const float4 g4 = reinterpret_cast<const float4*>(reduced)[i];
      float4 p4 = reinterpret_cast<float4*>(master)[i];
      float4 m4 = reinterpret_cast<float4*>(m)[i];
      float4 v4 = reinterpret_cast<float4*>(v)[i];
      float gg[4] = {g4.x, g4.y, g4.z, g4.w}, pp[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w},
            vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float g = gg[j] * coef;
        if (!h.decoupled_wd && h.weight_decay != 0.f) g += h.weight_decay * pp[j];
        mm[j] = h.beta1 * mm[j] + (1.f - h.beta1) * g;
        vv[j] = h.beta2 * vv[j] + (1.f - h.beta2) * g * g;
        float upd = (mm[j] / h.bias_correction1) / (sqrtf(vv[j] / h.bias_correction2) + h.eps);
        if (h.decoupled_wd) upd += h.weight_decay * pp[j];
        pp[j] -= h.lr * upd;
      }
      reinterpret_cast<float4*>(master)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
      reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]), hi = __floats2bfloat162_rn(pp[2], pp[3]);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
#pragma unroll 4
      for (int r = 0; r < t.world; ++r) {
        const int dst = (t.rank + r) % t.world;
        reinterpret_cast<uint2*>(t.works[dst] + slice_begin)[i] = o;   // all-gather by peer stores
      }
    }
  }
  // every peer has finished reading my gradients (they passed the barrier above): clear the whole buffer
  if (h.zero_grad) {
    float4* g = reinterpret_cast<float4*>(t.grads[t.rank]);
    const long t4 = total_len >> 2;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < t4; i += static_cast<long>(gridDim.x) * blockDim.x) g[i] = z;
  }
  __threadfence_system();
}

// The epoch lives in device memory and is advanced here, so a captured CUDA graph can be replayed.
__global__ void finish_step_kernel(const NmtgPeerTable t, int* epoch_ptr, int* status) {
  const int epoch = *epoch_ptr;
  const bool ok = peer_barrier(t, 2, epoch, status);
  if (ok && threadIdx.x == 0) *epoch_ptr = epoch + 1;
}

// Stand-alone barrier used by the tests of the timeout path: waits on a row nobody else signals.
__global__ void wait_row_kernel(const NmtgPeerTable t, int row, int epoch, int* status) { peer_barrier(t, row, epoch, status); }

}  // namespace b200

using namespace b200;

static const char* err_str() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* nmtg_allreduce_adamw(const NmtgPeerTable* t, float* reduced, float* sq, int* nonfinite, float* master, float* m,
                                 float* v, const NmtgAdamHyper* hyper_dev, long slice_begin, long slice_len, long total_len,
                                 int* epoch_dev, int* status, cudaStream_t stream) {
  if (t->world < 1 || t->world > kMaxRanks) return "allreduce_adamw: world size out of range";
  if ((slice_begin % 4) || (slice_len % 4) || (total_len % 4)) return "allreduce_adamw: slices must be multiples of 4 elements";
  cudaMemsetAsync(sq, 0, sizeof(float), stream);
  cudaMemsetAsync(nonfinite, 0, sizeof(int), stream);
  long blocks = (slice_len / 4 + 511) / 512;
  const long cap = static_cast<long>(num_sms()) * 2;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  reduce_slice_kernel<<<static_cast<int>(blocks), 512, 0, stream>>>(*t, reduced, sq, nonfinite, slice_begin, slice_len, epoch_dev, status);
  const char* e = err_str();
  if (e) return e;
  update_slice_kernel<<<num_sms() * 2, 512, 0, stream>>>(*t, reduced, master, m, v, hyper_dev, sq, nonfinite, slice_begin, slice_len,
                                                         total_len, epoch_dev, status);
  if ((e = err_str())) return e;
  finish_step_kernel<<<1, 32, 0, stream>>>(*t, epoch_dev, status);
  return err_str();
}

const char* nmtg_peer_finish_step(const NmtgPeerTable* t, int* epoch_dev, int* status, cudaStream_t stream) {
  finish_step_kernel<<<1, 32, 0, stream>>>(*t, epoch_dev, status);
  return err_str();
}

const char* nmtg_peer_wait_row(const NmtgPeerTable* t, int row, int epoch, int* status, cudaStream_t stream) {
  wait_row_kernel<<<1, 32, 0, stream>>>(*t, row, epoch, status);
  return err_str();
}
