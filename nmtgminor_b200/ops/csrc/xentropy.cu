// Fused label-smoothed softmax cross-entropy for large vocabularies, forward and backward in ONE pass
// over HBM: a CTA owns one row of bf16 logits, stages it in shared memory while it computes the online
// max / sum-exp / sum, and then overwrites the row in place with the gradient
//     dlogit = grad_scale * (softmax - (1-eps) * onehot(y) - eps / V)
// (zero for rows whose label is the padding id).  The row loss
//     loss = (1-eps) * (lse - x[y]) + eps * (lse - mean(x))
// is written per row and summed into a scalar with one atomic per CTA.  Rows longer than the staging
// buffer are re-read from global memory (L2) in the second pass.
//
// Same mathematics as the reference's xentropy_cuda (onmt/modules/extensions/xentropy/
// xentropy_kernel.cu:382-432 forward, :545-569 backward), which runs two separate kernels.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <float.h>
#include "ops_api.h"
#include "bounds_check.cuh"

namespace b200 {

constexpr int kXentThreads = 512;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  float nm = fmaxf(m, m2);
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

template <bool STAGE>
__global__ void __launch_bounds__(kXentThreads)
xent_fused_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ row_loss,
                  float* __restrict__ row_lse, float* __restrict__ loss_sum, float* __restrict__ correct_sum, int rows,
                  int vocab, long ld, float smoothing, int pad_idx, const float* __restrict__ grad_scale_ptr,
                  float grad_scale_val, int write_grad) {
  extern __shared__ __align__(16) uint8_t xsm[];
  __shared__ float red_m[kXentThreads / 32], red_s[kXentThreads / 32], red_x[kXentThreads / 32];
  __shared__ int red_arg[kXentThreads / 32];
  __shared__ float red_best[kXentThreads / 32];
  __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(xsm);
  const int row = blockIdx.x;
  if (row >= rows) return;
  __nv_bfloat16* x = logits + static_cast<size_t>(row) * ld;
  const long label = labels[row];
  if (label != pad_idx && (label < 0 || label >= vocab)) NMTG_BOUNDS_HIT();   // treated as padding below
  const bool is_pad = (label == pad_idx) || label < 0 || label >= vocab;
  const int nvec = vocab >> 3;  // full 16-byte vectors (row start is 16-byte aligned when ld % 8 == 0)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  if (is_pad) {
    if (write_grad) {
      uint4 z = make_uint4(0, 0, 0, 0);
      for (int i = threadIdx.x; i < nvec; i += kXentThreads) reinterpret_cast<uint4*>(x)[i] = z;
      for (int i = nvec * 8 + threadIdx.x; i < vocab; i += kXentThreads) x[i] = __float2bfloat16(0.f);
    }
    if (threadIdx.x == 0) {
      if (row_loss) row_loss[row] = 0.f;
      if (row_lse) row_lse[row] = 0.f;
    }
    return;
  }

  float m = -FLT_MAX, s = 0.f, sx = 0.f, best = -FLT_MAX;
  int arg = 0;
  for (int i = threadIdx.x; i < nvec; i += kXentThreads) {
    uint4 u = reinterpret_cast<const uint4*>(x)[i];
    if (STAGE) reinterpret_cast<uint4*>(stage)[i] = u;
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(h[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > best) {
#pragma unroll
      for (int j = 7; j >= 0; --j)
        if (f[j] == lm) arg = i * 8 + j;
      best = lm;
    }
    float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc += __expf(f[j] - nm);
      sx += f[j];
    }
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = nvec * 8 + threadIdx.x; i < vocab; i += kXentThreads) {
    float f = __bfloat162float(x[i]);
    if (STAGE) stage[i] = x[i];
    if (f > best) { best = f; arg = i; }
    online_merge(m, s, f, 1.f);
    sx += f;
  }
  // warp then CTA reduction
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
    sx += __shfl_xor_sync(0xffffffffu, sx, o);
    float b2 = __shfl_xor_sync(0xffffffffu, best, o);
    int a2 = __shfl_xor_sync(0xffffffffu, arg, o);
    if (b2 > best || (b2 == best && a2 < arg)) { best = b2; arg = a2; }
  }
  if (lane == 0) { red_m[warp] = m; red_s[warp] = s; red_x[warp] = sx; red_best[warp] = best; red_arg[warp] = arg; }
  __syncthreads();
  m = red_m[0]; s = red_s[0]; sx = red_x[0]; best = red_best[0]; arg = red_arg[0];
#pragma unroll
  for (int w = 1; w < kXentThreads / 32; ++w) {
    online_merge(m, s, red_m[w], red_s[w]);
    sx += red_x[w];
    if (red_best[w] > best || (red_best[w] == best && red_arg[w] < arg)) { best = red_best[w]; arg = red_arg[w]; }
  }
  const float lse = m + __logf(s);
  const float xy = __bfloat162float(STAGE ? stage[label] : x[label]);
  if (threadIdx.x == 0) {
    float loss = (1.f - smoothing) * (lse - xy) + smoothing * (lse - sx / vocab);
    if (row_loss) row_loss[row] = loss;
    if (row_lse) row_lse[row] = lse;
    if (loss_sum) atomicAdd(loss_sum, loss);
    if (correct_sum && arg == label) atomicAdd(correct_sum, 1.f);
  }
  if (!write_grad) return;
  const float gs = grad_scale_ptr ? *grad_scale_ptr * grad_scale_val : grad_scale_val;
  const float uni = smoothing / vocab;
  const __nv_bfloat16* src = STAGE ? stage : x;
  for (int i = threadIdx.x; i < nvec; i += kXentThreads) {
    uint4 u = reinterpret_cast<const uint4*>(src)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(h[j]);
      float g0 = __expf(t.x - lse) - uni, g1 = __expf(t.y - lse) - uni;
      if (i * 8 + 2 * j == label) g0 -= (1.f - smoothing);
      if (i * 8 + 2 * j + 1 == label) g1 -= (1.f - smoothing);
      o2[j] = __floats2bfloat162_rn(g0 * gs, g1 * gs);
    }
    reinterpret_cast<uint4*>(x)[i] = o;
  }
  for (int i = nvec * 8 + threadIdx.x; i < vocab; i += kXentThreads) {
    float g = __expf(__bfloat162float(src[i]) - lse) - uni;
    if (i == label) g -= (1.f - smoothing);
    x[i] = __float2bfloat16(g * gs);
  }
}

}  // namespace b200

using namespace b200;

const char* nmtg_xent_fused(void* logits, const int64_t* labels, float* row_loss, float* row_lse, float* loss_sum,
                            float* correct_sum, int rows, int vocab, long ld, float smoothing, int pad_idx,
                            const float* grad_scale_ptr, float grad_scale_val, int write_grad, cudaStream_t stream) {
  if (rows <= 0) return nullptr;
  if (ld % 8) return "xent: leading dimension must be a multiple of 8 elements";
  const size_t need = static_cast<size_t>(vocab) * 2 + 16;
  cudaError_t e;
  if (need <= 200 * 1024) {
    static bool configured = false;
    if (!configured) {
      e = cudaFuncSetAttribute(xent_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return cudaGetErrorString(e);
      configured = true;
    }
    xent_fused_kernel<true><<<rows, kXentThreads, need, stream>>>(
        reinterpret_cast<__nv_bfloat16*>(logits), labels, row_loss, row_lse, loss_sum, correct_sum, rows, vocab, ld,
        smoothing, pad_idx, grad_scale_ptr, grad_scale_val, write_grad);
  } else {
    xent_fused_kernel<false><<<rows, kXentThreads, 0, stream>>>(
        reinterpret_cast<__nv_bfloat16*>(logits), labels, row_loss, row_lse, loss_sum, correct_sum, rows, vocab, ld,
        smoothing, pad_idx, grad_scale_ptr, grad_scale_val, write_grad);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

NMTG_BOUNDS_READER(nmtg_bounds_xentropy)
