// Fully sharded data parallelism over peer-mapped memory (one node, NVLink / NVSwitch).
//
// The flat parameter space is cut into UNITS (one per Transformer layer, one for everything else).  Every unit is
// split into `world` equal pieces; rank r keeps, for every unit, piece r of the bf16 parameters, of the fp32 master
// weights and of the Adam moments, concatenated in "shard order".  Three kernels:
//
//   fsdp_gather   unit u -> local staging buffer: piece p of the unit is pulled from rank p's shard with 16-byte
//                 peer loads (every rank reads 1/world of the unit from every peer, so all links carry the same
//                 load).  It runs on a side stream one unit ahead of the GEMMs that consume the staging buffer.
//                 No flags are needed: shards only change inside fsdp_update, which every rank enters after the
//                 step barrier, and the previous step ended with a barrier too.
//   fsdp_reduce   after backward: waits (bounded) for "gradients ready" of all ranks, then for every unit sums this
//                 rank's piece over the N full gradient buffers (peer loads) into shard order, accumulates the
//                 squared norm and flags non-finite values: a reduce-scatter without a staging copy.
//   fsdp_update   exchanges the norm partials (bounded wait), applies Adam(W) to the shard, writes the refreshed
//                 bf16 parameters into the local shard that the next step's gathers read, clears the local
//                 gradient buffer.  The step ends with the shared finish barrier (peer_finish_step).
//
// Counterpart of FSDP's all-gather / reduce-scatter + optimizer.step in the reference (onmt/train_utils/
// mp_trainer.py:330-350 wrap, :895-1016 step).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops_api.h"
#include "peer_sync.cuh"

namespace b200 {

int num_sms();

__global__ void __launch_bounds__(256)
fsdp_gather_kernel(const NmtgPeerTable t, __nv_bfloat16* __restrict__ dst, long shard_off, long piece_len, long unit_len) {
  // element e of the unit lives in rank (e / piece_len)'s shard at shard_off + e % piece_len
  const long n8 = unit_len >> 3, p8 = piece_len >> 3;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long>(gridDim.x) * blockDim.x) {
    // walk the owners starting from this rank so that at any moment the peers serve different readers
    const long j = (i + static_cast<long>(t.rank) * p8) % n8;
    const int owner = static_cast<int>(j / p8);
    const long within = j - owner * p8;
    const uint4 v = reinterpret_cast<const uint4*>(t.works[owner] + shard_off)[within];
    reinterpret_cast<uint4*>(dst)[j] = v;
  }
}

__global__ void __launch_bounds__(512)
fsdp_reduce_kernel(const NmtgPeerTable t, const NmtgFsdpPieces pc, float* __restrict__ reduced, float* __restrict__ sq_out,
                   int* __restrict__ nonfinite, const int* __restrict__ epoch_ptr, int* status) {
  const int epoch = *epoch_ptr;
  if (!peer_barrier(t, 0, epoch, status)) return;
  __shared__ float red[16];
  float acc = 0.f;
  for (int u = 0; u < pc.n; ++u) {
    const long n4 = pc.len[u] >> 2;
    const long g0 = pc.global_begin[u];
    float4* out = reinterpret_cast<float4*>(reduced + pc.shard_off[u]);
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<long>(gridDim.x) * blockDim.x) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int r = 0; r < t.world; ++r) {
        const int src = (t.rank + r) % t.world;
        const float4 v = reinterpret_cast<const float4*>(t.grads[src] + g0)[i];
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      out[i] = s;
      acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
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
fsdp_update_kernel(const NmtgPeerTable t, const float* __restrict__ reduced, float* __restrict__ master, float* __restrict__ m,
                   float* __restrict__ v, const NmtgAdamHyper* __restrict__ hp, const float* __restrict__ sq_local,
                   const int* __restrict__ nonfinite_local, long shard_len, long total_len, const int* __restrict__ epoch_ptr,
                   int* status) {
  const int epoch = *epoch_ptr;
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
  if (!s_skip) {
    __nv_bfloat16* shard = reinterpret_cast<__nv_bfloat16*>(t.works[t.rank]);
    const long n4 = shard_len >> 2;
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
      reinterpret_cast<uint2*>(shard)[i] = o;
    }
  }
  if (h.zero_grad) {   // every peer has passed the barrier above, i.e. finished reading my gradients
    float4* g = reinterpret_cast<float4*>(t.grads[t.rank]);
    const long t4 = total_len >> 2;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < t4; i += static_cast<long>(gridDim.x) * blockDim.x) g[i] = z;
  }
  __threadfence_system();
}

}  // namespace b200

using namespace b200;

static const char* err_str() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* nmtg_fsdp_gather(const NmtgPeerTable* t, void* dst, long shard_off, long piece_len, long unit_len, int ctas,
                             cudaStream_t stream) {
  if (t->world < 1 || t->world > kMaxRanks) return "fsdp_gather: world size out of range";
  if ((shard_off % 8) || (piece_len % 8) || (unit_len % 8) || piece_len <= 0) return "fsdp_gather: sizes must be multiples of 8 elements";
  if (piece_len * t->world < unit_len) return "fsdp_gather: pieces do not cover the unit";
  if (reinterpret_cast<uintptr_t>(dst) & 15) return "fsdp_gather: unaligned staging buffer";
  if (ctas < 1) ctas = 32;
  fsdp_gather_kernel<<<ctas, 256, 0, stream>>>(*t, static_cast<__nv_bfloat16*>(dst), shard_off, piece_len, unit_len);
  return err_str();
}

const char* nmtg_fsdp_step(const NmtgPeerTable* t, const NmtgFsdpPieces* pieces, float* reduced, float* sq, int* nonfinite,
                           float* master, float* m, float* v, const NmtgAdamHyper* hyper_dev, long shard_len, long total_len,
                           int* epoch_dev, int* status, cudaStream_t stream) {
  if (t->world < 1 || t->world > kMaxRanks) return "fsdp_step: world size out of range";
  if (pieces->n < 1 || pieces->n > kFsdpMaxUnits) return "fsdp_step: too many units";
  for (int u = 0; u < pieces->n; ++u)
    if ((pieces->len[u] % 4) || (pieces->global_begin[u] % 4) || (pieces->shard_off[u] % 4)) return "fsdp_step: pieces must be multiples of 4 elements";
  if ((shard_len % 4) || (total_len % 4)) return "fsdp_step: lengths must be multiples of 4 elements";
  cudaMemsetAsync(sq, 0, sizeof(float), stream);
  cudaMemsetAsync(nonfinite, 0, sizeof(int), stream);
  fsdp_reduce_kernel<<<num_sms() * 2, 512, 0, stream>>>(*t, *pieces, reduced, sq, nonfinite, epoch_dev, status);
  const char* e = err_str();
  if (e) return e;
  fsdp_update_kernel<<<num_sms() * 2, 512, 0, stream>>>(*t, reduced, master, m, v, hyper_dev, sq, nonfinite, shard_len, total_len,
                                                        epoch_dev, status);
  if ((e = err_str())) return e;
  return nmtg_peer_finish_step(t, epoch_dev, status, stream);
}
