// Flat-buffer optimiser kernels for sm_100a.  Parameters live in ONE contiguous fp32 master buffer with a
// bf16 working copy, gradients in one contiguous fp32 buffer, so "multi-tensor apply" is a single
// grid-stride launch with 16-byte accesses:
//   * sq_norm:   sum of squares of the gradients + non-finite detection -> device scalars
//   * adamw:     unscale, clip by global norm (coefficient computed on the device from the scalars, no host
//                round trip), Adam / AdamW update of the fp32 master, refresh of the bf16 working copy and
//                zeroing of the gradient buffer for the next step.  The step is skipped when a non-finite
//                gradient was seen (dynamic loss-scaling semantics).
// Hyper-parameters that change every step (lr, bias corrections) are read from a small device struct so a
// captured CUDA graph can be replayed with new values.
//
// Counterpart of the reference's fused_optim extension (onmt/modules/extensions/fused_optim/
// multi_tensor_adam.cu:24-170, multi_tensor_l2norm_kernel.cu:29-436, multi_tensor_scale_kernel.cu) and of
// GradScaler.unscale_ + clip_grad_norm + optimizer.step in onmt/train_utils/mp_trainer.py:965-1016.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops_api.h"

namespace b200 {

int num_sms();

__global__ void sq_norm_kernel(const float* __restrict__ g, long n, float* __restrict__ out_sq,
                               int* __restrict__ out_nonfinite) {
  __shared__ float red[32];
  float acc = 0.f;
  bool bad = false;
  const long n4 = n >> 2;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 v = reinterpret_cast<const float4*>(g)[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long i = (n4 << 2) + blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    acc += g[i] * g[i];
  bad = !isfinite(acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  if (bad) atomicOr(out_nonfinite, 1);
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) {
      if (isfinite(v)) atomicAdd(out_sq, v);
      else atomicOr(out_nonfinite, 1);
    }
  }
}

__global__ void adamw_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ work, float* __restrict__ grad,
                             float* __restrict__ m, float* __restrict__ v, long n, const NmtgAdamHyper* __restrict__ hp,
                             const float* __restrict__ grad_sq, const int* __restrict__ nonfinite) {
  const NmtgAdamHyper h = *hp;
  const bool skip = nonfinite && *nonfinite;
  float coef = h.grad_scale;  // multiplies raw gradients (1 / (loss_scale * normaliser))
  if (grad_sq && h.max_grad_norm > 0.f) {
    float norm = sqrtf(*grad_sq) * h.grad_scale;
    if (norm > h.max_grad_norm) coef *= h.max_grad_norm / (norm + 1e-6f);
  }
  const long n4 = n >> 2;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 g4 = reinterpret_cast<float4*>(grad)[i];
    if (skip) {
      if (h.zero_grad) __stcs(reinterpret_cast<float4*>(grad) + i, make_float4(0.f, 0.f, 0.f, 0.f));
      continue;
    }
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
      float mhat = mm[j] / h.bias_correction1;
      float denom = sqrtf(vv[j] / h.bias_correction2) + h.eps;
      float upd = mhat / denom;
      if (h.decoupled_wd) upd += h.weight_decay * pp[j];
      pp[j] -= h.lr * upd;
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (work) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]), hi = __floats2bfloat162_rn(pp[2], pp[3]);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(work)[i] = o;
    }
    // Clearing the gradient comes last and bypasses the usual write policy: a store to the line that was just
    // loaded, issued before the other loads of the iteration, made the whole kernel four times slower.
    if (h.zero_grad) __stcs(reinterpret_cast<float4*>(grad) + i, make_float4(0.f, 0.f, 0.f, 0.f));
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long n) {
  const long n4 = n >> 2;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 p = reinterpret_cast<const float4*>(src)[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
}

// ---------------------------------------------------------------------------------------------------------
// Dynamic loss scale kept on the device, so that a captured step never asks the host.
// state = { scale, clean steps since the last change, 1 / scale, skipped steps so far }
// ---------------------------------------------------------------------------------------------------------
// Before the update kernels: the gradients carry the loss scale, so the optimiser's gradient factor is divided by it.
__global__ void loss_scale_prepare_kernel(NmtgAdamHyper* hyper, const float* state) {
  if (threadIdx.x == 0 && blockIdx.x == 0) hyper->grad_scale = hyper->grad_scale / state[0];
}
// After the update kernels: a skipped step (non-finite gradient somewhere: local flag, or the global norm reported as
// negative by the sharded update) multiplies the scale by `backoff`; `interval` clean steps in a row multiply it by
// `growth`.  The scale stays within [min_scale, max_scale].
__global__ void loss_scale_update_kernel(float* state, const int* nonfinite, const float* norm, int interval, float growth,
                                         float backoff, float min_scale, float max_scale) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const bool skipped = (nonfinite && *nonfinite != 0) || (norm && !(*norm >= 0.f));
  float scale = state[0], clean = state[1];
  if (skipped) {
    scale = fmaxf(scale * backoff, min_scale);
    clean = 0.f;
    state[3] += 1.f;
  } else {
    clean += 1.f;
    if (clean >= static_cast<float>(interval)) {
      scale = fminf(scale * growth, max_scale);
      clean = 0.f;
    }
  }
  state[0] = scale;
  state[1] = clean;
  state[2] = 1.f / scale;
}

}  // namespace b200

using namespace b200;

static const char* last_err2() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* nmtg_sq_norm(const float* g, long n, float* out_sq, int* out_nonfinite, cudaStream_t stream) {
  if (n <= 0) return nullptr;
  long blocks = (n / 4 + 511) / 512;
  const long cap = static_cast<long>(num_sms()) * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  sq_norm_kernel<<<static_cast<int>(blocks), 512, 0, stream>>>(g, n, out_sq, out_nonfinite);
  return last_err2();
}

const char* nmtg_adamw_flat(float* master, void* work_bf16, float* grad, float* m, float* v, long n,
                            const NmtgAdamHyper* hyper_dev, const float* grad_sq, const int* nonfinite,
                            cudaStream_t stream) {
  if (n <= 0) return nullptr;
  if (n % 4) return "adamw: flat buffer length must be a multiple of 4";
  long blocks = (n / 4 + 255) / 256;
  const long cap = static_cast<long>(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  adamw_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(master, reinterpret_cast<__nv_bfloat16*>(work_bf16), grad, m,
                                                             v, n, hyper_dev, grad_sq, nonfinite);
  return last_err2();
}

const char* nmtg_cast_f32_bf16(const float* src, void* dst, long n, cudaStream_t stream) {
  if (n <= 0) return nullptr;
  if (n % 4) return "cast: length must be a multiple of 4";
  long blocks = (n / 4 + 255) / 256;
  const long cap = static_cast<long>(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  cast_f32_bf16_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), n);
  return last_err2();
}

const char* nmtg_loss_scale_prepare(NmtgAdamHyper* hyper_dev, const float* state, cudaStream_t stream) {
  loss_scale_prepare_kernel<<<1, 32, 0, stream>>>(hyper_dev, state);
  return last_err2();
}

const char* nmtg_loss_scale_update(float* state, const int* nonfinite, const float* norm, int interval, float growth,
                                   float backoff, float min_scale, float max_scale, cudaStream_t stream) {
  if (interval < 1) return "loss scale: the growth interval must be at least 1";
  loss_scale_update_kernel<<<1, 32, 0, stream>>>(state, nonfinite, norm, interval, growth, backoff, min_scale, max_scale);
  return last_err2();
}
