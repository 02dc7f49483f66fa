// Gradient reduction fused with the optimiser over peer-mapped (NVLink / NVSwitch) memory, for data parallelism
// and for fully sharded parameters.
//
// Every rank keeps its fp32 gradients (and, data parallel, its bf16 parameter copy) in memory that all other
// ranks of the node have mapped (CUDA IPC).  The flat parameter space is cut into UNITS - one per Transformer
// layer, everything else merged - and every unit into `world` pieces; rank r OWNS piece r of every unit: Adam
// moments (and, fully sharded, fp32 master weights and bf16 parameters) exist only for owned pieces.
//
//   reduce_unit    one launch per unit, enqueued on a communication stream as soon as the backward pass has
//                  produced the unit's last weight gradient, so the transfer overlaps the backward pass of the
//                  layers below.  Waits (bounded) until every peer has published "this unit is complete",
//                  then sums its piece over all N gradient buffers with 16-byte peer loads (each CTA fetches
//                  its own elements; no broadcast loads of any kind) into the shard-ordered `reduced` buffer.
//                  With rotating per-layer gradient buffers it also tells the peers when it has finished
//                  reading and clears its own copy once they all have.
//   update_pieces  after the last unit: exchanges the squared-norm partials, forms the global gradient norm
//                  and the clipping coefficient, applies Adam(W) to every owned piece and publishes the
//                  refreshed bf16 parameters - data parallel: stored into EVERY rank's parameter copy with peer
//                  stores (the all-gather); fully sharded: into the local shard that the gathers read.
//   finish_step    closing barrier, so the next forward pass reads complete parameters.
//
// Cross-GPU flags are monotonically increasing epochs written with st.release.sys and polled with
// ld.acquire.sys; a waiter that runs out of time records kTimeoutPeerFlag in the status word and the kernel
// returns (the host raises), so a missing peer can never hang a GPU.  Bytes over NVLink per rank and step, data
// parallel: (N-1)/N * P * 4 in (gradients) and (N-1)/N * P * 2 out (parameters), against 2 * (N-1)/N * P * 4
// for a ring all-reduce followed by a replicated optimiser.
//
// Replaces DistributedDataParallel's bucketed NCCL all-reduce + GradScaler.unscale_ + clip_grad_norm +
// optimizer.step (onmt/train_utils/mp_trainer.py:381-387, 895-1016) and FSDP's reduce-scatter + sharded
// optimizer step (onmt/train_utils/mp_trainer.py:314-341) of the reference.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops_api.h"
#include "peer_sync.cuh"

namespace b200 {

int num_sms();

// Sum of element groups i, i + stride, ... of all ranks' buffers; U groups per thread are in flight together.
template <int U>
__device__ __forceinline__ void reduce_elements(const NmtgPeerTable& t, float* __restrict__ reduced, long g0, long n4, long first,
                                                long stride, int accumulate) {
  for (long i = first; i < n4; i += U * stride) {
    float4 s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long j = i + u * stride;
      s[u] = (accumulate && j < n4) ? reinterpret_cast<const float4*>(reduced)[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll 4
    for (int r = 0; r < t.world; ++r) {
      // start with my own buffer, then walk the ring so the peers' links are loaded evenly
      const float* src = t.grads[(t.rank + r) % t.world] + g0;
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long j = i + u * stride;
        v[u] = j < n4 ? reinterpret_cast<const float4*>(src)[j] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) { s[u].x += v[u].x; s[u].y += v[u].y; s[u].z += v[u].z; s[u].w += v[u].w; }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long j = i + u * stride;
      if (j < n4) reinterpret_cast<float4*>(reduced)[j] = s[u];
    }
  }
}

// 128-thread CTAs at about 40 registers (5 K of the SM's 64 K): small enough to share an SM with a resident GEMM CTA
// (320 threads at up to 168 registers = 54 K, ~200 KB of shared memory), so the reduction runs beside the backward
// pass instead of waiting for an SM to drain.
// The wide form (512 threads, launched with a shared-memory request that no SM holding a GEMM or attention CTA can
// satisfy) is for SMs set aside for communication (nmtg_set_sm_reserve): a few such CTAs keep enough peer loads in flight
// to finish a layer's reduction long before the backward pass ends, without sharing an SM with the statically
// scheduled persistent kernels, which any co-resident work slows down as a whole.
constexpr int kReduceThreads = 128;
constexpr int kReduceWideThreads = 512;
constexpr int kReduceWideSmem = 96 * 1024;
template <int kThreads>
__global__ void __launch_bounds__(kThreads)
reduce_unit_kernel(const NmtgPeerTable t, int row, float* __restrict__ reduced, long g0, long len, int accumulate,
                   long zero_begin, long zero_len, int* __restrict__ counter, const int* __restrict__ epoch_ptr, int* status) {
  const int epoch = *epoch_ptr;
  if (!peer_barrier(t, row, epoch, status)) return;
  const long n4 = len >> 2;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  const long first = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  // Peer loads are latency bound: what counts is the number of 16-byte loads a thread has in flight.  Eight ranks give
  // eight per element; smaller worlds make up for it by working on several elements at once.
  if (t.world <= 2) reduce_elements<4>(t, reduced, g0, n4, first, stride, accumulate);
  else if (t.world <= 4) reduce_elements<2>(t, reduced, g0, n4, first, stride, accumulate);
  else reduce_elements<1>(t, reduced, g0, n4, first, stride, accumulate);
  if (zero_len <= 0) return;
  // Rotating gradient buffers: the LAST CTA of this launch to finish its loads tells every peer "rank `rank` has
  // read the unit"; everybody then waits for all peers' notices before clearing the local copy.
  __syncthreads();
  int last = 0;
  if (threadIdx.x == 0) {
    __threadfence();
    last = (atomicAdd(counter, 1) == static_cast<int>(gridDim.x) - 1);
  }
  if (__syncthreads_or(last)) {
    peer_publish(t, row + 1, epoch);
    if (threadIdx.x == 0) *counter = 0;      // ready for the next launch from this site
  }
  if (!peer_barrier(t, row + 1, epoch, status, /*publish=*/false)) return;
  float4* z = reinterpret_cast<float4*>(t.grads[t.rank] + zero_begin);
  const long z4 = zero_len >> 2;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < z4; i += stride) z[i] = zero;
}

__global__ void __launch_bounds__(512)
update_pieces_kernel(const NmtgPeerTable t, const NmtgPieces pc, const float* __restrict__ reduced, float* __restrict__ master,
                     float* __restrict__ m, float* __restrict__ v, const NmtgAdamHyper* __restrict__ hp,
                     const float* __restrict__ sq_local, const int* __restrict__ nonfinite_local, int mode, long zero_len,
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
      if (p < 0.f || !isfinite(p)) skip = 1;
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
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  if (!s_skip) {
    for (int u = 0; u < pc.n; ++u) {
      const long n4 = pc.len[u] >> 2;
      const long so = pc.shard_off[u], g0 = pc.global_begin[u];
      float* mp = master + (mode == 0 ? g0 : so);
      for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4; i += stride) {
        const float4 g4 = reinterpret_cast<const float4*>(reduced + so)[i];
        float4 p4 = reinterpret_cast<float4*>(mp)[i];
        float4 m4 = reinterpret_cast<float4*>(m + so)[i];
        float4 v4 = reinterpret_cast<float4*>(v + so)[i];
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
        reinterpret_cast<float4*>(mp)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
        reinterpret_cast<float4*>(m + so)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
        reinterpret_cast<float4*>(v + so)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
        __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]), hi = __floats2bfloat162_rn(pp[2], pp[3]);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        if (mode == 0) {
#pragma unroll 4
          for (int r = 0; r < t.world; ++r) {
            const int dst = (t.rank + r) % t.world;
            reinterpret_cast<uint2*>(t.works[dst] + g0)[i] = o;   // all-gather by peer stores
          }
        } else {
          reinterpret_cast<uint2*>(t.works[t.rank] + so)[i] = o;  // the shard that the next step's gathers read
        }
      }
    }
  }
  // every peer has finished reading my gradients (they passed the barrier above): clear the local space
  if (h.zero_grad && zero_len > 0) {
    float4* g = reinterpret_cast<float4*>(t.grads[t.rank]);
    const long t4 = zero_len >> 2;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < t4; i += stride) g[i] = z;
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

const char* nmtg_reduce_unit(const NmtgPeerTable* t, int row, float* reduced, long global_begin, long len, int accumulate,
                             long zero_begin, long zero_len, int* counter, const int* epoch_dev, int* status, int ctas,
                             cudaStream_t stream) {
  if (t->world < 1 || t->world > kMaxRanks) return "reduce_unit: world size out of range";
  if (row < 3 || row + 1 >= kNmtgFlagRows) return "reduce_unit: flag row out of range";
  if ((global_begin % 4) || (len % 4) || (zero_begin % 4) || (zero_len % 4) || len < 0)
    return "reduce_unit: ranges must be multiples of 4 elements";
  if (reinterpret_cast<uintptr_t>(reduced) & 15) return "reduce_unit: unaligned output";
  if (zero_len > 0 && !counter) return "reduce_unit: clearing the unit needs the launch counter";
  if (ctas < 0) {   // -ctas wide CTAs for the SMs that the compute kernels leave free
    static bool configured = false;
    if (!configured) {
      cudaError_t ce = cudaFuncSetAttribute(reduce_unit_kernel<kReduceWideThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            kReduceWideSmem);
      if (ce != cudaSuccess) return cudaGetErrorString(ce);
      configured = true;
    }
    long blocks = (len / 4 + kReduceWideThreads - 1) / kReduceWideThreads;
    if (blocks > -ctas) blocks = -ctas;
    if (blocks < 1) blocks = 1;
    reduce_unit_kernel<kReduceWideThreads><<<static_cast<int>(blocks), kReduceWideThreads, kReduceWideSmem, stream>>>(
        *t, row, reduced, global_begin, len, accumulate, zero_begin, zero_len, counter, epoch_dev, status);
    return err_str();
  }
  long blocks = (len / 4 + kReduceThreads - 1) / kReduceThreads;
  if (ctas < 1) ctas = 64;
  if (blocks > ctas) blocks = ctas;
  if (blocks < 1) blocks = 1;
  reduce_unit_kernel<kReduceThreads><<<static_cast<int>(blocks), kReduceThreads, 0, stream>>>(
      *t, row, reduced, global_begin, len, accumulate, zero_begin, zero_len, counter, epoch_dev, status);
  return err_str();
}

const char* nmtg_update_pieces(const NmtgPeerTable* t, const NmtgPieces* pieces, const float* reduced, float* master, float* m,
                               float* v, const NmtgAdamHyper* hyper_dev, const float* sq, const int* nonfinite, int mode,
                               long zero_len, const int* epoch_dev, int* status, cudaStream_t stream) {
  if (t->world < 1 || t->world > kMaxRanks) return "update_pieces: world size out of range";
  if (pieces->n < 1 || pieces->n > kNmtgMaxUnits) return "update_pieces: too many units";
  if (mode != 0 && mode != 1) return "update_pieces: unknown mode";
  for (int u = 0; u < pieces->n; ++u)
    if ((pieces->len[u] % 4) || (pieces->global_begin[u] % 4) || (pieces->shard_off[u] % 4))
      return "update_pieces: pieces must be multiples of 4 elements";
  if (zero_len % 4) return "update_pieces: lengths must be multiples of 4 elements";
  update_pieces_kernel<<<num_sms() * 2, 512, 0, stream>>>(*t, *pieces, reduced, master, m, v, hyper_dev, sq, nonfinite, mode,
                                                         zero_len, epoch_dev, status);
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
