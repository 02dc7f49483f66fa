// LayerNorm forward / backward for sm_100a.  One warp per row, 16-byte vector loads, the row is held in
// registers between the statistics pass and the normalisation pass, fp32 statistics saved for backward.
// Backward writes dx (optionally adding an incoming residual gradient) and accumulates the affine
// gradients of all rows of a CTA in shared memory before one fp32 atomic add per column into the
// (fp32, accumulating) gradient buffers.  Hidden size: any multiple of 8 up to 16384 (a warp per row up to 2048, a CTA per row above).
//
// Covers what the reference's fast_layer_norm_cuda does (onmt/modules/extensions/layer_norm/
// ln_fwd_kernels.cuh:7-108, ln_bwd_kernels.cuh:6-323) without the per-hidden-size kernel table.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <type_traits>
#include <cstdlib>
#include "ops_api.h"

namespace b200 {

constexpr int kLnWarps = 4;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// VPL = 16-byte vectors per lane (row length <= VPL * 256 elements)
template <int VPL>
__global__ void __launch_bounds__(kLnWarps * 32)
ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
              const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
              float* __restrict__ rstd, int rows, int hidden, float eps) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = hidden >> 3;
  for (int row = blockIdx.x * kLnWarps + warp; row < rows; row += gridDim.x * kLnWarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * hidden);
    float v[VPL][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        uint4 u = xr[vi];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(h[j]);
          v[i][2 * j] = f.x;
          v[i][2 * j + 1] = f.y;
          s += f.x + f.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
      }
    }
    const float mu = warp_sum(s) / hidden;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (lane + i * 32 < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float d = v[i][j] - mu;
          sq += d * d;
        }
      }
    }
    const float rs = rsqrtf(warp_sum(sq) / hidden + eps);
    if (lane == 0) {
      if (mean) mean[row] = mu;
      if (rstd) rstd[row] = rs;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * hidden);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
        uint4 b = __ldg(reinterpret_cast<const uint4*>(beta) + vi);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 gf = __bfloat1622float2(g2[j]), bf = __bfloat1622float2(b2[j]);
          o2[j] = __floats2bfloat162_rn((v[i][2 * j] - mu) * rs * gf.x + bf.x,
                                        (v[i][2 * j + 1] - mu) * rs * gf.y + bf.y);
        }
        yr[vi] = o;
      }
    }
  }
}

template <int VPL, int kWarps>
__global__ void __launch_bounds__(kWarps * 32, VPL <= 4 ? 16 / kWarps : 1)
ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
              const float* __restrict__ mean, const float* __restrict__ rstd,
              const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ dres,
              __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma, float* __restrict__ dbeta, int rows,
              int hidden) {
  extern __shared__ float s_acc[];  // [warps][2][hidden] : dgamma, dbeta partials, one slice per warp
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nvec = hidden >> 3;
  for (int i = threadIdx.x; i < kWarps * 2 * hidden; i += blockDim.x) s_acc[i] = 0.f;
  __syncthreads();
  float* wg = s_acc + warp * 2 * hidden;  // lanes own disjoint columns: plain read-modify-write
  float* wb = wg + hidden;
  // narrow rows keep the affine-gradient partial sums in registers; wide rows use the shared-memory slice
  constexpr bool kRegAcc = VPL <= 4;
  float ag[kRegAcc ? VPL : 1][8], ab[kRegAcc ? VPL : 1][8];
#pragma unroll
  for (int i = 0; i < (kRegAcc ? VPL : 1); ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) ag[i][j] = ab[i][j] = 0.f;

  for (int row = blockIdx.x * kWarps + warp; row < rows; row += gridDim.x * kWarps) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * hidden);
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * hidden);
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * hidden) : nullptr;
    // every global load of the row (dy, x and the residual-path gradient) is issued before anything waits on one;
    // the operands stay packed in registers and are unpacked again in the second pass
    uint4 av[VPL], bv[VPL], rv[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      av[i] = bv[i] = rv[i] = make_uint4(0u, 0u, 0u, 0u);
      if (vi < nvec) {
        av[i] = dyr[vi];
        bv[i] = xr[vi];
        if (rr) rv[i] = rr[vi];
      }
    }
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av[i]);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv[i]);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 d = __bfloat1622float2(a2[j]), xv = __bfloat1622float2(b2[j]), gf = __bfloat1622float2(g2[j]);
          float xh0 = (xv.x - mu) * rs, xh1 = (xv.y - mu) * rs;
          if constexpr (kRegAcc) {
            ag[i][2 * j] += d.x * xh0;
            ag[i][2 * j + 1] += d.y * xh1;
            ab[i][2 * j] += d.x;
            ab[i][2 * j + 1] += d.y;
          } else {
            const int c = vi * 8 + 2 * j;
            wg[c] += d.x * xh0;
            wg[c + 1] += d.y * xh1;
            wb[c] += d.x;
            wb[c + 1] += d.y;
          }
          float t0 = d.x * gf.x, t1 = d.y * gf.y;
          s1 += t0 + t1;
          s2 += t0 * xh0 + t1 * xh1;
        }
      }
    }
    s1 = warp_sum(s1) / hidden;
    s2 = warp_sum(s2) / hidden;
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * hidden);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av[i]);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv[i]);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv[i]);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 d = __bfloat1622float2(a2[j]), xv = __bfloat1622float2(b2[j]), gf = __bfloat1622float2(g2[j]);
          float2 add = __bfloat1622float2(r2[j]);       // zero when there is no residual-path gradient
          float xh0 = (xv.x - mu) * rs, xh1 = (xv.y - mu) * rs;
          float d0 = rs * (d.x * gf.x - s1 - xh0 * s2) + add.x;
          float d1 = rs * (d.y * gf.y - s1 - xh1 * s2) + add.y;
          o2[j] = __floats2bfloat162_rn(d0, d1);
        }
        dxr[vi] = o;
      }
    }
  }
  if constexpr (kRegAcc) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          wg[vi * 8 + j] = ag[i][j];
          wb[vi * 8 + j] = ab[i][j];
        }
      }
    }
  }
  // CTA-level reduction of the per-warp slices, then one atomic per column
  __syncthreads();
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      g += s_acc[w * 2 * hidden + i];
      b += s_acc[w * 2 * hidden + hidden + i];
    }
    if (dgamma) atomicAdd(dgamma + i, g);
    if (dbeta) atomicAdd(dbeta + i, b);
  }
}

// ---------------------------------------------------------------------------------------------------
// Rows longer than 2048 elements (up to 16384): one CTA of 256 threads per row, rows dealt round-robin over the grid.
// Thread t owns the 16-byte vectors t, t + 256, ... of every row, so its slice of the affine gradients stays in
// registers over all the rows of the CTA and costs one atomic per column and CTA at the end.
// ---------------------------------------------------------------------------------------------------
constexpr int kWideThreads = 256;
constexpr int kWideVec = 8;   // 8 vectors x 8 elements x 256 threads = 16384 elements

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kWideThreads / 32; ++w) t += red[w];
  __syncthreads();       // red may be written again right away
  return t;
}

__global__ void __launch_bounds__(kWideThreads)
ln_fwd_wide_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                   const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                   float* __restrict__ rstd, int rows, int hidden, float eps) {
  __shared__ float red[kWideThreads / 32];
  const int nvec = hidden >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * hidden);
    float v[kWideVec][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kWideVec; ++i) {
      const int vi = threadIdx.x + i * kWideThreads;
      if (vi < nvec) {
        const uint4 u = xr[vi];
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(u2[j]);
          v[i][2 * j] = f.x;
          v[i][2 * j + 1] = f.y;
          s += f.x + f.y;
        }
      }
    }
    const float mu = block_sum(s, red) / hidden;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kWideVec; ++i)
      if (threadIdx.x + i * kWideThreads < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) sq += (v[i][j] - mu) * (v[i][j] - mu);
      }
    const float rs = rsqrtf(block_sum(sq, red) / hidden + eps);
    if (threadIdx.x == 0) {
      if (mean) mean[row] = mu;
      if (rstd) rstd[row] = rs;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * hidden);
#pragma unroll
    for (int i = 0; i < kWideVec; ++i) {
      const int vi = threadIdx.x + i * kWideThreads;
      if (vi < nvec) {
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + vi), b = __ldg(reinterpret_cast<const uint4*>(beta) + vi);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 gf = __bfloat1622float2(g2[j]), bf = __bfloat1622float2(b2[j]);
          o2[j] = __floats2bfloat162_rn((v[i][2 * j] - mu) * rs * gf.x + bf.x, (v[i][2 * j + 1] - mu) * rs * gf.y + bf.y);
        }
        yr[vi] = o;
      }
    }
  }
}

__global__ void __launch_bounds__(kWideThreads)
ln_bwd_wide_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const float* __restrict__ mean,
                   const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ gamma,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma,
                   float* __restrict__ dbeta, int rows, int hidden) {
  __shared__ float red[kWideThreads / 32];
  const int nvec = hidden >> 3;
  float ag[kWideVec][8], ab[kWideVec][8];
#pragma unroll
  for (int i = 0; i < kWideVec; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) ag[i][j] = ab[i][j] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * hidden);
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * hidden);
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * hidden) : nullptr;
    const float mu = mean[row], rs = rstd[row];
    uint4 av[kWideVec], bv[kWideVec];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < kWideVec; ++i) {
      const int vi = threadIdx.x + i * kWideThreads;
      av[i] = bv[i] = make_uint4(0u, 0u, 0u, 0u);
      if (vi < nvec) {
        av[i] = dyr[vi];
        bv[i] = xr[vi];
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av[i]);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv[i]);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 d = __bfloat1622float2(a2[j]), xv = __bfloat1622float2(b2[j]), gf = __bfloat1622float2(g2[j]);
          const float xh0 = (xv.x - mu) * rs, xh1 = (xv.y - mu) * rs;
          ag[i][2 * j] += d.x * xh0;
          ag[i][2 * j + 1] += d.y * xh1;
          ab[i][2 * j] += d.x;
          ab[i][2 * j + 1] += d.y;
          const float t0 = d.x * gf.x, t1 = d.y * gf.y;
          s1 += t0 + t1;
          s2 += t0 * xh0 + t1 * xh1;
        }
      }
    }
    s1 = block_sum(s1, red) / hidden;
    s2 = block_sum(s2, red) / hidden;
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * hidden);
#pragma unroll
    for (int i = 0; i < kWideVec; ++i) {
      const int vi = threadIdx.x + i * kWideThreads;
      if (vi < nvec) {
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gamma) + vi);
        const uint4 r = rr ? rr[vi] : make_uint4(0u, 0u, 0u, 0u);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av[i]);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv[i]);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&r);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 d = __bfloat1622float2(a2[j]), xv = __bfloat1622float2(b2[j]), gf = __bfloat1622float2(g2[j]);
          const float2 add = __bfloat1622float2(r2[j]);
          const float xh0 = (xv.x - mu) * rs, xh1 = (xv.y - mu) * rs;
          o2[j] = __floats2bfloat162_rn(rs * (d.x * gf.x - s1 - xh0 * s2) + add.x, rs * (d.y * gf.y - s1 - xh1 * s2) + add.y);
        }
        dxr[vi] = o;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kWideVec; ++i) {
    const int vi = threadIdx.x + i * kWideThreads;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (dgamma) atomicAdd(dgamma + vi * 8 + j, ag[i][j]);
        if (dbeta) atomicAdd(dbeta + vi * 8 + j, ab[i][j]);
      }
    }
  }
}

template <typename F>
static const char* dispatch_vpl(int hidden, F&& f) {
  const int need = (hidden / 8 + 31) / 32;
  if (need <= 1) return f(std::integral_constant<int, 1>());
  if (need <= 2) return f(std::integral_constant<int, 2>());
  if (need <= 4) return f(std::integral_constant<int, 4>());
  if (need <= 5) return f(std::integral_constant<int, 5>());
  if (need <= 8) return f(std::integral_constant<int, 8>());
  return "layernorm: hidden size above 2048 belongs to the one-CTA-per-row kernels";
}

int num_sms();

}  // namespace b200

using namespace b200;

const char* nmtg_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                               int rows, int hidden, float eps, cudaStream_t stream) {
  if (rows <= 0) return nullptr;
  if (hidden % 8) return "layernorm: hidden size must be a multiple of 8";
  if (hidden > kWideVec * 8 * kWideThreads) return "layernorm: hidden size above 16384 is not supported";
  if (hidden > 2048) {
    const int g = rows < num_sms() * 4 ? rows : num_sms() * 4;
    ln_fwd_wide_kernel<<<g, kWideThreads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(gamma),
                                                       reinterpret_cast<const __nv_bfloat16*>(beta), reinterpret_cast<__nv_bfloat16*>(y),
                                                       mean, rstd, rows, hidden, eps);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
  }
  int grid = (rows + kLnWarps - 1) / kLnWarps;
  const int cap = num_sms() * 16;
  if (grid > cap) grid = cap;
  return dispatch_vpl(hidden, [&](auto vpl) -> const char* {
    ln_fwd_kernel<decltype(vpl)::value><<<grid, kLnWarps * 32, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(gamma),
        reinterpret_cast<const __nv_bfloat16*>(beta), reinterpret_cast<__nv_bfloat16*>(y), mean, rstd, rows, hidden,
        eps);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
  });
}

template <int kWarps>
static const char* launch_ln_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma,
                                 const void* dres, void* dx, float* dgamma, float* dbeta, int rows, int hidden,
                                 cudaStream_t stream) {
  int grid = (rows + kWarps - 1) / kWarps;
  const size_t smem = kWarps * 2 * static_cast<size_t>(hidden) * sizeof(float);
  return dispatch_vpl(hidden, [&](auto vpl) -> const char* {
    auto kern = ln_bwd_kernel<decltype(vpl)::value, kWarps>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    // exactly one wave of resident CTAs: a partial second wave would leave most SMs idle while it runs
    static int resident[16] = {0};
    int& occ = resident[decltype(vpl)::value];
    if (occ == 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kWarps * 32, smem) != cudaSuccess || n < 1) n = 1;
      occ = n;
    }
    const int cap = num_sms() * occ;
    if (grid > cap) grid = cap;
    kern<<<grid, kWarps * 32, smem, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x), mean, rstd,
        reinterpret_cast<const __nv_bfloat16*>(gamma), reinterpret_cast<const __nv_bfloat16*>(dres),
        reinterpret_cast<__nv_bfloat16*>(dx), dgamma, dbeta, rows, hidden);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
  });
}

const char* nmtg_layernorm_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma,
                               const void* dres, void* dx, float* dgamma, float* dbeta, int rows, int hidden,
                               cudaStream_t stream) {
  if (rows <= 0) return nullptr;
  if (hidden % 8) return "layernorm: hidden size must be a multiple of 8";
  if (hidden > kWideVec * 8 * kWideThreads) return "layernorm: hidden size above 16384 is not supported";
  if (hidden > 2048) {
    const int g = rows < num_sms() * 2 ? rows : num_sms() * 2;
    ln_bwd_wide_kernel<<<g, kWideThreads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),
                                                       mean, rstd, reinterpret_cast<const __nv_bfloat16*>(gamma),
                                                       reinterpret_cast<const __nv_bfloat16*>(dres), reinterpret_cast<__nv_bfloat16*>(dx),
                                                       dgamma, dbeta, rows, hidden);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
  }
  // Eight warps per CTA once there are enough rows: half as many CTAs end with their 2 * hidden atomics on the affine
  // gradients, the same number of warps per SM is resident (NMTG_LN_BWD_WARPS=4 restores the narrow CTAs for comparison)
  static const int forced = [] { const char* e = getenv("NMTG_LN_BWD_WARPS"); return e ? atoi(e) : 0; }();
  const bool wide = forced ? forced == 8 : rows >= 2048;
  return wide ? launch_ln_bwd<8>(dy, x, mean, rstd, gamma, dres, dx, dgamma, dbeta, rows, hidden, stream)
              : launch_ln_bwd<4>(dy, x, mean, rstd, gamma, dres, dx, dgamma, dbeta, rows, hidden, stream);
}
