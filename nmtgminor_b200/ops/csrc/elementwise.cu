// Memory-bound element-wise kernels for sm_100a (16-byte vector accesses, grid sized to the SM count):
//   * dropout_add:      y = residual + dropout(x)           (mask regenerated from counters, never stored)
//   * masked_scale:     dx = dy * keep / (1-p)              (same counters as the forward op)
//   * embed_fwd / bwd:  gather * scale + position row, dropout; backward scatter-adds into fp32 grads
//   * colsum:           column sums of a bf16 matrix (bias gradients) accumulated into fp32
// The dropout convention is shared with the GEMM epilogue: element e of the op with stream id s keeps
// its value iff byte (e & 3) of DropRng(seed, s).word(e >> 2) is >= round(256 p); the keep scale is
// 256 / (256 - round(256 p)).
//
// Counterpart of the reference's fused_dropout_add_cuda (onmt/modules/extensions/dropout_add/
// dropout.h:21-160) and of the PyTorch embedding/position code in onmt/models/transformers.py:163-207.
#include "b200_ptx.cuh"
#include "ops_api.h"
#include "bounds_check.cuh"

namespace b200 {

int num_sms();

// Debug build (-DNMTG_DEBUG_BOUNDS): out-of-range indices are counted (and still clamped, never trapped) so that a
// test run can assert that no kernel ever saw one; the release build only clamps.

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return o;
}

// One thread handles 16 consecutive elements (two 16-byte vectors, four hash words).
__global__ void dropout_add_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                   __nv_bfloat16* __restrict__ y, long n16, float p, unsigned long long seed,
                                   unsigned long long stream_id, const unsigned long long* seed_dev) {
  const DropRng rng(seed + (seed_dev ? *seed_dev : 0ull), stream_id, p);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n16;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float f[8], r[8];
      unpack8(reinterpret_cast<const uint4*>(x)[2 * i + h], f);
      if (res) unpack8(reinterpret_cast<const uint4*>(res)[2 * i + h], r);
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint32_t w = rng.word(static_cast<unsigned long long>(i) * 4 + h * 2 + g);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v = rng.keep(w, j) ? f[g * 4 + j] * rng.scale : 0.f;
          f[g * 4 + j] = res ? v + r[g * 4 + j] : v;
        }
      }
      reinterpret_cast<uint4*>(y)[2 * i + h] = pack8(f);
    }
  }
}

// dz = dropout-mask(dy) * act'(z): backward of ``dropout(act(z))`` for a stand-alone Linear with an activation, one pass
// (the mask is the one dropout_add / the GEMM epilogue drew for the same seed and stream).  One thread handles 8
// consecutive elements (one 16-byte vector, two hash words).  act: 1 ReLU, 2 GELU (erf), 3 SiLU.
__global__ void act_backward_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ z,
                                    __nv_bfloat16* __restrict__ dz, long n8, int act, float p, unsigned long long seed,
                                    unsigned long long stream_id, const unsigned long long* seed_dev) {
  const bool drop = p > 0.f;
  const DropRng rng(seed + ((drop && seed_dev) ? *seed_dev : 0ull), stream_id, p);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float g[8], a[8];
    unpack8(reinterpret_cast<const uint4*>(dy)[i], g);
    unpack8(reinterpret_cast<const uint4*>(z)[i], a);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t w = drop ? rng.word(static_cast<unsigned long long>(i) * 2 + h) : 0u;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = h * 4 + j;
        const float x = a[e];
        float d;
        if (act == 1) {
          d = x > 0.f ? 1.f : 0.f;
        } else if (act == 2) {
          d = 0.5f * (1.f + erff(x * 0.7071067811865476f)) + x * __expf(-0.5f * x * x) * 0.3989422804014327f;
        } else {
          const float sg = 1.f / (1.f + __expf(-x));
          d = sg * (1.f + x * (1.f - sg));
        }
        const float v = drop ? (rng.keep(w, j) ? g[e] * rng.scale : 0.f) : g[e];
        g[e] = v * d;
      }
    }
    reinterpret_cast<uint4*>(dz)[i] = pack8(g);
  }
}

// y = dropout-mask(x) (the mask of dropout_add with the same seed / stream) and colsum += column sums of y, in one
// pass: backward of ``dropout(linear(x) + bias)`` needs both the masked gradient and the bias gradient.  A thread keeps
// one group of 16 columns for all the rows it visits, so the partial sums stay in registers; the CTA's row slices are
// combined in shared memory and every CTA ends with one atomic per column.
template <int kGroups>     // 16-column groups per row; 256 % kGroups == 0
__global__ void __launch_bounds__(256)
dropout_colsum_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, float* __restrict__ colsum, int rows,
                      float p, unsigned long long seed, unsigned long long stream_id, const unsigned long long* seed_dev) {
  constexpr int kRowsPerIter = 256 / kGroups;
  __shared__ float part[kRowsPerIter][kGroups * 16 + 1];
  const DropRng rng(seed + (seed_dev ? *seed_dev : 0ull), stream_id, p);
  const int c = threadIdx.x % kGroups, rsub = threadIdx.x / kGroups;
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  for (long row = static_cast<long>(blockIdx.x) * kRowsPerIter + rsub; row < rows; row += static_cast<long>(gridDim.x) * kRowsPerIter) {
    const long i = row * kGroups + c;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(x)[2 * i + h], f);
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint32_t w = rng.word(static_cast<unsigned long long>(i) * 4 + h * 2 + g);
#pragma unroll
        for (int j = 0; j < 4; ++j) f[g * 4 + j] = rng.keep(w, j) ? f[g * 4 + j] * rng.scale : 0.f;
      }
      const uint4 packed = pack8(f);
      reinterpret_cast<uint4*>(y)[2 * i + h] = packed;
      float back[8];
      unpack8(packed, back);          // sum what was stored (bf16-rounded), as a separate pass over y would
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[h * 8 + j] += back[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) part[rsub][c * 16 + j] = acc[j];
  __syncthreads();
  for (int col = threadIdx.x; col < kGroups * 16; col += 256) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < kRowsPerIter; ++r) s += part[r][col];
    atomicAdd(colsum + col, s);
  }
}

__global__ void embed_fwd_kernel(const int64_t* __restrict__ tokens, const int64_t* __restrict__ positions,
                                 const __nv_bfloat16* __restrict__ table, const __nv_bfloat16* __restrict__ pos_table,
                                 __nv_bfloat16* __restrict__ out, int rows, int hidden, int vocab, int max_pos,
                                 float scale, float p, unsigned long long seed, unsigned long long stream_id,
                                 const unsigned long long* seed_dev) {
  const DropRng rng(seed + (seed_dev ? *seed_dev : 0ull), stream_id, p);
  const int n16 = hidden >> 4;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    long tok = tokens[row];
    if (tok < 0 || tok >= vocab) { NMTG_BOUNDS_HIT(); tok = 0; }
    long pos = positions ? positions[row] : 0;
    if (pos < 0) pos = 0;
    if (pos >= max_pos) { NMTG_BOUNDS_HIT(); pos = max_pos - 1; }
    const uint4* tr = reinterpret_cast<const uint4*>(table + static_cast<size_t>(tok) * hidden);
    const uint4* pr = pos_table ? reinterpret_cast<const uint4*>(pos_table + static_cast<size_t>(pos) * hidden) : nullptr;
    uint4* orow = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * hidden);
    for (int c = threadIdx.x; c < n16; c += blockDim.x) {
      const unsigned long long w0 = (static_cast<unsigned long long>(row) * n16 + c) * 4;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float f[8], q[8];
        unpack8(__ldg(tr + 2 * c + h), f);
        if (pr) unpack8(__ldg(pr + 2 * c + h), q);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const uint32_t w = p > 0.f ? rng.word(w0 + h * 2 + g) : 0xFFFFFFFFu;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float v = f[g * 4 + j] * scale + (pr ? q[g * 4 + j] : 0.f);
            if (p > 0.f) v = rng.keep(w, j) ? v * rng.scale : 0.f;
            f[g * 4 + j] = v;
          }
        }
        orow[2 * c + h] = pack8(f);
      }
    }
  }
}

// dTable[tok] += scale * keep * dy[row]   (fp32, vector red.add); optional dPos[pos] += keep * dy[row]
__global__ void embed_bwd_kernel(const int64_t* __restrict__ tokens, const int64_t* __restrict__ positions,
                                 const __nv_bfloat16* __restrict__ dy, float* __restrict__ dtable,
                                 float* __restrict__ dpos, int rows, int hidden, int vocab, int max_pos, float scale,
                                 float p, unsigned long long seed, unsigned long long stream_id,
                                 const unsigned long long* seed_dev, int pad_idx) {
  const DropRng rng(seed + (seed_dev ? *seed_dev : 0ull), stream_id, p);
  const int n16 = hidden >> 4;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    long tok = tokens[row];
    if (tok < 0 || tok >= vocab || tok == pad_idx) continue;
    long pos = positions ? positions[row] : 0;
    if (pos < 0) pos = 0;
    if (pos >= max_pos) pos = max_pos - 1;
    const uint4* dr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * hidden);
    float* trow = dtable + static_cast<size_t>(tok) * hidden;
    float* prow = dpos ? dpos + static_cast<size_t>(pos) * hidden : nullptr;
    for (int c = threadIdx.x; c < n16; c += blockDim.x) {
      const unsigned long long w0 = (static_cast<unsigned long long>(row) * n16 + c) * 4;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float f[8];
        unpack8(dr[2 * c + h], f);
        if (p > 0.f) {
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            const uint32_t w = rng.word(w0 + h * 2 + g);
#pragma unroll
            for (int j = 0; j < 4; ++j) f[g * 4 + j] = rng.keep(w, j) ? f[g * 4 + j] * rng.scale : 0.f;
          }
        }
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          float* t = trow + c * 16 + h * 8 + g * 4;
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(t), "f"(f[g * 4] * scale),
                       "f"(f[g * 4 + 1] * scale), "f"(f[g * 4 + 2] * scale), "f"(f[g * 4 + 3] * scale)
                       : "memory");
          if (prow) {
            float* q = prow + c * 16 + h * 8 + g * 4;
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(q), "f"(f[g * 4]), "f"(f[g * 4 + 1]),
                         "f"(f[g * 4 + 2]), "f"(f[g * 4 + 3])
                         : "memory");
          }
        }
      }
    }
  }
}

// out[c] += sum_r x[r, c]; CTA tile: 32 rows-lanes x 64 columns, rows strided over the grid's y dimension
__global__ void colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int rows, int cols,
                              long ld) {
  __shared__ float part[8][64];
  const int c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 8 warps
  float a0 = 0.f, a1 = 0.f;
  const int c = c0 + tx * 2;
  if (c < cols) {
    for (int r = blockIdx.y * 8 + ty; r < rows; r += gridDim.y * 8) {
      __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + static_cast<size_t>(r) * ld + c);
      float2 f = __bfloat1622float2(v);
      a0 += f.x;
      a1 += f.y;
    }
  }
  part[ty][tx * 2] = a0;
  part[ty][tx * 2 + 1] = a1;
  __syncthreads();
  if (threadIdx.x < 64 && c0 + threadIdx.x < cols) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += part[w][threadIdx.x];
    atomicAdd(out + c0 + threadIdx.x, s);
  }
}

// Wide variant: a warp covers 256 consecutive columns with 16-byte loads (cols % 8 == 0, ld % 8 == 0)
__global__ void colsum_wide_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int rows, int cols,
                                   long ld) {
  __shared__ float part[8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + lane * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < cols) {
    for (int r = blockIdx.y * 8 + warp; r < rows; r += gridDim.y * 8) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * ld + c0), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < cols) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += part[w][threadIdx.x];
    atomicAdd(out + c, s);
  }
}

}  // namespace b200

using namespace b200;

static const char* last_err() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* nmtg_dropout_add(const void* x, const void* residual, void* y, long n, float p, unsigned long long seed,
                             unsigned long long stream_id, const unsigned long long* seed_dev, cudaStream_t stream) {
  if (n <= 0) return nullptr;
  if (n % 16) return "dropout_add: element count must be a multiple of 16";
  const long n16 = n / 16;
  long blocks = (n16 + 255) / 256;
  const long cap = static_cast<long>(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  dropout_add_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(residual),
      reinterpret_cast<__nv_bfloat16*>(y), n16, p, seed, stream_id, seed_dev);
  return last_err();
}

const char* nmtg_act_backward(const void* dy, const void* z, void* dz, long n, int act, float p, unsigned long long seed,
                              unsigned long long stream_id, const unsigned long long* seed_dev, cudaStream_t stream) {
  if (n <= 0) return nullptr;
  if (n % 8) return "act_backward: element count must be a multiple of 8";
  if (act < 1 || act > 3) return "act_backward: activation must be ReLU (1), GELU (2) or SiLU (3)";
  const long n8 = n / 8;
  long blocks = (n8 + 255) / 256;
  const long cap = static_cast<long>(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  act_backward_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(z),
      reinterpret_cast<__nv_bfloat16*>(dz), n8, act, p, seed, stream_id, seed_dev);
  return last_err();
}

const char* nmtg_dropout_colsum(const void* x, void* y, float* colsum, int rows, int cols, float p, unsigned long long seed,
                                unsigned long long stream_id, const unsigned long long* seed_dev, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return nullptr;
  const int groups = cols / 16;
  if (cols % 16 || groups > 256 || (256 % groups) != 0) return "dropout_colsum: columns must be 16 * a divisor of 256";
  const int rows_per_iter = 256 / groups;
  long blocks = (static_cast<long>(rows) + rows_per_iter - 1) / rows_per_iter;
  const long cap = static_cast<long>(num_sms()) * 4;
  if (blocks > cap) blocks = cap;
  auto go = [&](auto tag) {
    dropout_colsum_kernel<decltype(tag)::value><<<static_cast<int>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(y), colsum, rows, p, seed, stream_id, seed_dev);
  };
  switch (groups) {
    case 256: go(std::integral_constant<int, 256>()); break;
    case 128: go(std::integral_constant<int, 128>()); break;
    case 64: go(std::integral_constant<int, 64>()); break;
    case 32: go(std::integral_constant<int, 32>()); break;
    case 16: go(std::integral_constant<int, 16>()); break;
    case 8: go(std::integral_constant<int, 8>()); break;
    default: return "dropout_colsum: unsupported column count";
  }
  return last_err();
}

const char* nmtg_embed_fwd(const int64_t* tokens, const int64_t* positions, const void* table, const void* pos_table,
                           void* out, int rows, int hidden, int vocab, int max_pos, float scale, float p,
                           unsigned long long seed, unsigned long long stream_id, const unsigned long long* seed_dev,
                           cudaStream_t stream) {
  if (rows <= 0) return nullptr;
  if (hidden % 16) return "embed: hidden size must be a multiple of 16";
  int grid = rows < num_sms() * 8 ? rows : num_sms() * 8;
  embed_fwd_kernel<<<grid, 64, 0, stream>>>(tokens, positions, reinterpret_cast<const __nv_bfloat16*>(table),
                                            reinterpret_cast<const __nv_bfloat16*>(pos_table),
                                            reinterpret_cast<__nv_bfloat16*>(out), rows, hidden, vocab, max_pos, scale,
                                            p, seed, stream_id, seed_dev);
  return last_err();
}

const char* nmtg_embed_bwd(const int64_t* tokens, const int64_t* positions, const void* dy, float* dtable, float* dpos,
                           int rows, int hidden, int vocab, int max_pos, float scale, float p, unsigned long long seed,
                           unsigned long long stream_id, const unsigned long long* seed_dev, int pad_idx,
                           cudaStream_t stream) {
  if (rows <= 0) return nullptr;
  if (hidden % 16) return "embed: hidden size must be a multiple of 16";
  int grid = rows < num_sms() * 8 ? rows : num_sms() * 8;
  embed_bwd_kernel<<<grid, 64, 0, stream>>>(tokens, positions, reinterpret_cast<const __nv_bfloat16*>(dy), dtable, dpos,
                                            rows, hidden, vocab, max_pos, scale, p, seed, stream_id, seed_dev, pad_idx);
  return last_err();
}

const char* nmtg_colsum(const void* x, float* out, int rows, int cols, long ld, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return nullptr;
  if (cols % 2 || ld % 2) return "colsum: column count and leading dimension must be even";
  if (cols % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    dim3 g((cols + 255) / 256, 1);
    int gy = (num_sms() * 4) / g.x;
    if (gy < 1) gy = 1;
    if (gy > (rows + 7) / 8) gy = (rows + 7) / 8;
    g.y = gy;
    colsum_wide_kernel<<<g, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), out, rows, cols, ld);
    return last_err();
  }
  dim3 grid((cols + 63) / 64, 1);
  int gy = (num_sms() * 4) / grid.x;
  if (gy < 1) gy = 1;
  if (gy > (rows + 7) / 8) gy = (rows + 7) / 8;
  grid.y = gy;
  colsum_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), out, rows, cols, ld);
  return last_err();
}

NMTG_BOUNDS_READER(nmtg_bounds_elementwise)
extern "C" long nmtg_bounds_xentropy();
extern "C" long nmtg_bounds_decode();
extern "C" long nmtg_bounds_sequence();
extern "C" long nmtg_bounds_attention_short();

// Number of out-of-range indices corrected by the kernels of this library since load; -1 when the checks are compiled out.
extern "C" long nmtg_bounds_violations() {
  long total = 0;
  const long parts[] = {nmtg_bounds_elementwise(), nmtg_bounds_xentropy(), nmtg_bounds_decode(), nmtg_bounds_sequence(),
                        nmtg_bounds_attention_short()};
  for (long v : parts) {
    if (v < 0) return v;
    total += v;
  }
  return total;
}
