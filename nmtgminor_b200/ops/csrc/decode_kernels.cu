// Inference-side kernels for sm_100a: one beam-search step (log-softmax + masks + per-sentence top-2K without ever
// writing [rows, V] log-probabilities), row gather for hypothesis reordering, append into preallocated key/value
// caches and single-query attention over them (self-attention over the growing cache, encoder-decoder attention
// over a per-sentence cache shared by the hypotheses of that sentence).
//
// They replace, in the reference, F.log_softmax + topk + index_select of onmt/inference/fast_translator.py:420-900 /
// onmt/inference/search.py:60-140 and the torch.cat caches of onmt/modules/optimized/self_attention_func.py:162-174.
#include "b200_ptx.cuh"
#include "seq_api.h"
#include "bounds_check.cuh"

namespace b200 {
namespace {

const char* launch_err() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

template <typename T> __device__ __forceinline__ float ldv(const T* p);
template <> __device__ __forceinline__ float ldv<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldv<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

struct Best {
  float v;
  int i;
};
// order: larger value first, ties by smaller index
__device__ __forceinline__ bool better(const Best& a, const Best& b) { return a.v > b.v || (a.v == b.v && a.i < b.i); }
// strictly after `p` in that order
__device__ __forceinline__ bool after(float v, int i, const Best& p) { return v < p.v || (v == p.v && i > p.i); }

__device__ __forceinline__ Best block_best(Best x, Best* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    if (better(y, x)) x = y;
  }
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = x;
  __syncthreads();
  Best r = red[0];
  for (int k = 1; k < nw; ++k)
    if (better(red[k], r)) r = red[k];
  return r;
}

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float y = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, y) : v + y;
  }
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float r = red[0];
  for (int k = 1; k < nw; ++k) r = is_max ? fmaxf(r, red[k]) : r + red[k];
  return r;
}

// Stage 1: one block per hypothesis row.  cand[r, 0:2K] = best 2K of scores[r] + masked log-softmax(logits[r]).
// kStage: the row is first copied into shared memory, so the 2K + 2 passes over it never leave the SM.
template <typename T, bool kStage>
__global__ void beam_row_topk_kernel(const T* __restrict__ logits, long ld, const float* __restrict__ scores,
                                     const uint8_t* __restrict__ force_eos, float* __restrict__ row_lse,
                                     float* __restrict__ cand_val, int* __restrict__ cand_idx, int K2, int V, int pad, int eos,
                                     int ban_eos) {
  extern __shared__ __align__(16) uint8_t stage_raw[];
  __shared__ float redf[32];
  __shared__ Best redb[32];
  const int r = blockIdx.x;
  const T* x = logits + static_cast<long>(r) * ld;
  if (kStage) {
    T* st = reinterpret_cast<T*>(stage_raw);
    constexpr int kPer = 16 / sizeof(T);
    if ((ld % kPer) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
      const int nvec = V / kPer;
      for (int i = threadIdx.x; i < nvec; i += blockDim.x)
        reinterpret_cast<uint4*>(st)[i] = reinterpret_cast<const uint4*>(x)[i];
      for (int v = nvec * kPer + threadIdx.x; v < V; v += blockDim.x) st[v] = x[v];
    } else {
      for (int v = threadIdx.x; v < V; v += blockDim.x) st[v] = x[v];
    }
    __syncthreads();
    x = st;
  }
  float mx = -INFINITY;
  for (int v = threadIdx.x; v < V; v += blockDim.x) mx = fmaxf(mx, ldv(x + v));
  mx = block_reduce(mx, redf, true);
  float s = 0.f;
  for (int v = threadIdx.x; v < V; v += blockDim.x) s += __expf(ldv(x + v) - mx);
  s = block_reduce(s, redf, false);
  const float lse = mx + __logf(s);
  if (threadIdx.x == 0) row_lse[r] = lse;
  const float base = scores[r] - lse;
  // per-row control byte: 1 = only EOS may follow, 2 = EOS is banned (same as ban_eos, but readable by a replayed graph)
  const uint8_t fe = force_eos ? force_eos[r] : 0;
  const bool only_eos = fe == 1;
  if (fe == 2) ban_eos = 1;
  float* cv = cand_val + static_cast<long>(r) * K2;
  int* ci = cand_idx + static_cast<long>(r) * K2;
  if (only_eos || base == -INFINITY) {
    // one live candidate (or none): no search needed
    for (int j = threadIdx.x; j < K2; j += blockDim.x) {
      const bool live = only_eos && j == 0 && base != -INFINITY;
      cv[j] = live ? ldv(x + eos) + base : -INFINITY;
      ci[j] = live ? eos : (j == eos ? (eos + K2) % V : j);
    }
    return;
  }
  if constexpr (kStage) {
    // The masks are written into the staged copy, so the selection passes compare raw values only.
    T* st = reinterpret_cast<T*>(stage_raw);
    __syncthreads();
    if (threadIdx.x == 0) {
      if (pad >= 0 && pad < V) st[pad] = static_cast<T>(-INFINITY);
      if (ban_eos && eos >= 0 && eos < V) st[eos] = static_cast<T>(-INFINITY);
    }
    __syncthreads();
    constexpr int kPer = 16 / sizeof(T);
    const int nvec = V / kPer;
    Best prev{INFINITY, -1};
    for (int j = 0; j < K2; ++j) {
      Best mine{-INFINITY, 0x7fffffff};
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        const uint4 u = reinterpret_cast<const uint4*>(st)[i];
        const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
          const float f = static_cast<float>(e[k]);
          if (f > mine.v || (f == mine.v && mine.i == 0x7fffffff)) {
            const int v = i * kPer + k;
            if (after(f, v, prev)) { mine.v = f; mine.i = v; }
          }
        }
      }
      for (int v = nvec * kPer + threadIdx.x; v < V; v += blockDim.x) {
        const float f = static_cast<float>(st[v]);
        if ((f > mine.v || (f == mine.v && v < mine.i)) && after(f, v, prev)) { mine.v = f; mine.i = v; }
      }
      const Best b = block_best(mine, redb);
      if (threadIdx.x == 0) {
        cv[j] = b.v + base;
        ci[j] = b.i == 0x7fffffff ? 0 : b.i;
      }
      prev = b;
    }
  } else {
    Best prev{INFINITY, -1};
    for (int j = 0; j < K2; ++j) {
      Best mine{-INFINITY, 0x7fffffff};
      for (int v = threadIdx.x; v < V; v += blockDim.x) {
        float val = ldv(x + v);
        if (v == pad || (ban_eos && v == eos)) val = -INFINITY;
        if (val != val) val = -INFINITY;
        if (after(val, v, prev)) {
          Best c{val, v};
          if (better(c, mine)) mine = c;
        }
      }
      const Best b = block_best(mine, redb);
      if (threadIdx.x == 0) {
        cv[j] = b.v + base;
        ci[j] = b.i == 0x7fffffff ? 0 : b.i;
      }
      prev = b;
    }
  }
}

template <typename T>
const char* launch_row_topk(const T* logits, long ld, const float* scores, const uint8_t* force_eos, float* row_lse,
                            float* cand_val, int* cand_idx, int R, int K2, int V, int pad, int eos, int ban_eos,
                            cudaStream_t stream) {
  const int threads = V >= 8192 ? 512 : (V >= 1024 ? 256 : 64);
  const size_t need = static_cast<size_t>(V) * sizeof(T) + 16;
  if (need <= 200 * 1024) {
    if (need > 48 * 1024) {
      static bool configured = false;
      if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(beam_row_topk_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        configured = true;
      }
    }
    beam_row_topk_kernel<T, true><<<R, threads, need, stream>>>(logits, ld, scores, force_eos, row_lse, cand_val, cand_idx, K2, V,
                                                                 pad, eos, ban_eos);
  } else {
    beam_row_topk_kernel<T, false><<<R, threads, 0, stream>>>(logits, ld, scores, force_eos, row_lse, cand_val, cand_idx, K2, V,
                                                              pad, eos, ban_eos);
  }
  return nullptr;
}

// Stage 2: one block per sentence; merge K rows of 2K candidates into the best 2K (sorted, best first).
__global__ void beam_merge_kernel(const float* __restrict__ cand_val, const int* __restrict__ cand_idx,
                                  float* __restrict__ out_scores, long* __restrict__ out_index, int K, int K2, int V) {
  __shared__ Best redb[32];
  const int b = blockIdx.x;
  const int n = K * K2;
  const float* cv = cand_val + static_cast<long>(b) * n;
  const int* ci = cand_idx + static_cast<long>(b) * n;
  Best prev{INFINITY, -1};
  for (int j = 0; j < K2; ++j) {
    Best mine{-INFINITY, 0x7fffffff};
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      const float val = cv[c];
      if (after(val, c, prev)) {
        Best t{val, c};
        if (better(t, mine)) mine = t;
      }
    }
    const Best w = block_best(mine, redb);
    if (threadIdx.x == 0) {
      const int c = w.i == 0x7fffffff ? 0 : w.i;
      out_scores[static_cast<long>(b) * K2 + j] = w.v;
      out_index[static_cast<long>(b) * K2 + j] = static_cast<long>(c / K2) * V + ci[c];
    }
    prev = w;
  }
}

__global__ void gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const long* __restrict__ index,
                                   int rows, int src_rows, long stride16, long copy16, const int* __restrict__ filled_dev,
                                   long unit16) {
  // filled_dev (optional): number of `unit16`-sized units at the start of every row that hold data, read on the
  // device so that a captured graph copies the right amount at every replay
  if (filled_dev) {
    const long want = static_cast<long>(*filled_dev) * unit16;
    copy16 = want < stride16 ? want : stride16;
  }
  if (copy16 <= 0) return;
  const long total = static_cast<long>(rows) * copy16;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / copy16, c = i % copy16;
    const long from = checked_range(static_cast<long>(index[r]), 0L, static_cast<long>(src_rows) - 1);
    dst[r * stride16 + c] = src[from * stride16 + c];
  }
}

__global__ void cache_append_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new, long ld,
                                    __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int R, int hid,
                                    int cap, int pos, const int* __restrict__ pos_dev) {
  if (pos_dev) pos = *pos_dev;
  if (pos < 0 || pos >= cap) {
    if (blockIdx.x == 0 && threadIdx.x == 0) NMTG_BOUNDS_HIT();
    return;
  }
  const int n16 = hid >> 3;
  const long total = static_cast<long>(R) * n16;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / n16, c = i % n16;
    const long d = ((r * cap + pos) * hid) / 8 + c;
    reinterpret_cast<uint4*>(k_cache)[d] = reinterpret_cast<const uint4*>(k_new + r * ld)[c];
    reinterpret_cast<uint4*>(v_cache)[d] = reinterpret_cast<const uint4*>(v_new + r * ld)[c];
  }
}

// One warp per (row, head).  Scores: one key per lane (the 128-byte key row is read with eight 16-byte loads);
// values: see the second half of the kernel (four positions per load instruction, probabilities from shared memory).
__global__ void decode_attn_kernel(const __nv_bfloat16* __restrict__ q, long q_ld, const __nv_bfloat16* __restrict__ k_cache,
                                   const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ lengths,
                                   __nv_bfloat16* __restrict__ out, int R, int heads, int cap, int len_all, int kv_div,
                                   float scale, const int* __restrict__ len_dev, int len_add) {
  extern __shared__ float probs[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long item = blockIdx.x * static_cast<long>(blockDim.x >> 5) + wib;
  if (item >= static_cast<long>(R) * heads) return;
  const int r = static_cast<int>(item / heads), h = static_cast<int>(item % heads);
  const int kr = r / kv_div;
  int len = lengths ? lengths[kr] : (len_dev ? *len_dev + len_add : len_all);
  len = len < 0 ? 0 : (len > cap ? cap : len);
  float* p = probs + static_cast<long>(wib) * cap;
  const int hid = heads * 64;
  const __nv_bfloat16* kb = k_cache + (static_cast<long>(kr) * cap) * hid + h * 64;
  const __nv_bfloat16* vb = v_cache + (static_cast<long>(kr) * cap) * hid + h * 64;
  float qf[64];
  {
    const uint4* qp = reinterpret_cast<const uint4*>(q + static_cast<long>(r) * q_ld + h * 64);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 u = qp[c];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = __bfloat1622float2(h2[j]);
        qf[c * 8 + 2 * j] = t.x * scale;
        qf[c * 8 + 2 * j + 1] = t.y * scale;
      }
    }
  }
  float mx = -INFINITY;
  for (int j = lane; j < len; j += 32) {
    const uint4* kp = reinterpret_cast<const uint4*>(kb + static_cast<long>(j) * hid);
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 u = kp[c];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float2 t = __bfloat1622float2(h2[jj]);
        s = fmaf(t.x, qf[c * 8 + 2 * jj], s);
        s = fmaf(t.y, qf[c * 8 + 2 * jj + 1], s);
      }
    }
    p[j] = s;
    mx = fmaxf(mx, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int j = lane; j < len; j += 32) {
    const float e = __expf(p[j] - mx);
    p[j] = e;
    sum += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  // values: a 128-byte value row is read by eight lanes with one 16-byte load each, so one load instruction of the
  // warp covers four cache positions; eight such loads (32 positions) are in flight before any is used.  Lane
  // (sub, part) accumulates dimensions part*8 .. part*8+7 over positions sub, sub+4, ...; the four partial sums of a
  // dimension are combined with two shuffles.
  const int sub = lane >> 3, part = lane & 7;
  float acc[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) acc[d] = 0.f;
  for (int j0 = 0; j0 < len; j0 += 32) {
    uint4 v[8];
    float pj[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = j0 + u * 4 + sub;
      const bool in = j < len;
      v[u] = in ? *reinterpret_cast<const uint4*>(vb + static_cast<long>(j) * hid + part * 8) : make_uint4(0u, 0u, 0u, 0u);
      pj[u] = in ? p[j] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        const float2 t = __bfloat1622float2(h2[d]);
        acc[2 * d] = fmaf(pj[u], t.x, acc[2 * d]);
        acc[2 * d + 1] = fmaf(pj[u], t.y, acc[2 * d + 1]);
      }
    }
  }
#pragma unroll
  for (int d = 0; d < 8; ++d) {
    acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], 8);
    acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], 16);
  }
  if (sub == 0) {
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int d = 0; d < 4; ++d) o2[d] = __floats2bfloat162_rn(acc[2 * d] * inv, acc[2 * d + 1] * inv);
    *reinterpret_cast<uint4*>(out + (static_cast<long>(r) * heads + h) * 64 + part * 8) = o;
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

const char* nmtg_beam_topk(const void* logits, long ld, int dtype, const float* scores, const uint8_t* force_eos,
                           float* row_lse, float* cand_val, int* cand_idx, float* out_scores, long* out_index, int B, int K,
                           int V, int pad, int eos, int ban_eos, cudaStream_t stream) {
  if (B <= 0 || K <= 0 || V <= 0) return nullptr;
  const int K2 = 2 * K;
  if (K2 > V) return "beam_topk: vocabulary smaller than twice the beam";
  if (ld < V) return "beam_topk: row stride smaller than the vocabulary";
  const int R = B * K;
  const char* err;
  if (dtype == 0)
    err = launch_row_topk<float>(static_cast<const float*>(logits), ld, scores, force_eos, row_lse, cand_val, cand_idx, R, K2, V,
                                 pad, eos, ban_eos, stream);
  else
    err = launch_row_topk<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(logits), ld, scores, force_eos, row_lse, cand_val,
                                         cand_idx, R, K2, V, pad, eos, ban_eos, stream);
  if (err) return err;
  beam_merge_kernel<<<B, K * K2 >= 256 ? 256 : 64, 0, stream>>>(cand_val, cand_idx, out_scores, out_index, K, K2, V);
  return launch_err();
}

const char* nmtg_gather_rows(const void* src, void* dst, const long* index, int rows, int src_rows, long row_stride_bytes,
                             long copy_bytes, const int* filled_dev, long unit_bytes, cudaStream_t stream) {
  if (filled_dev) {
    if (unit_bytes <= 0 || (unit_bytes % 16)) return "gather_rows: unit size must be a positive multiple of 16 bytes";
    copy_bytes = row_stride_bytes;       // grid sized for the worst case; the kernel reads the real amount
  }
  if (rows <= 0 || copy_bytes <= 0) return nullptr;
  if (src_rows <= 0) return "gather_rows: the source has no rows";
  if ((row_stride_bytes % 16) || (copy_bytes % 16) || copy_bytes > row_stride_bytes)
    return "gather_rows: sizes must be multiples of 16 bytes with copy <= stride";
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) return "gather_rows: unaligned pointer";
  const long total = rows * (copy_bytes / 16);
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  gather_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst),
                                                                        index, rows, src_rows, row_stride_bytes / 16, copy_bytes / 16,
                                                                        filled_dev, unit_bytes / 16);
  return launch_err();
}

const char* nmtg_decode_attn(const void* q, long q_ld, const void* k_cache, const void* v_cache, const int* lengths,
                             void* out, int R, int heads, int cap, int len, int kv_div, float scale, const int* len_dev,
                             int len_add, cudaStream_t stream) {
  if (R <= 0 || heads <= 0) return nullptr;
  if (kv_div <= 0 || cap <= 0 || len > cap) return "decode_attn: bad cache geometry";
  if (q_ld % 8) return "decode_attn: query row stride must be a multiple of 8 elements";
  const int warps = 4;
  const size_t smem = static_cast<size_t>(warps) * cap * sizeof(float);
  if (smem > 200 * 1024) return "decode_attn: cache capacity too large for one warp's probabilities";
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decode_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return cudaGetErrorString(e);
  }
  const long items = static_cast<long>(R) * heads;
  decode_attn_kernel<<<static_cast<unsigned>((items + warps - 1) / warps), warps * 32, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(q), q_ld, static_cast<const __nv_bfloat16*>(k_cache),
      static_cast<const __nv_bfloat16*>(v_cache), lengths, static_cast<__nv_bfloat16*>(out), R, heads, cap, len, kv_div, scale,
      len_dev, len_add);
  return launch_err();
}

const char* nmtg_cache_append(const void* k_new, const void* v_new, long ld, void* k_cache, void* v_cache, int R, int heads,
                              int cap, int pos, const int* pos_dev, cudaStream_t stream) {
  if (R <= 0) return nullptr;
  if (!pos_dev && (pos < 0 || pos >= cap)) return "cache_append: position outside the cache";
  if (ld % 8) return "cache_append: row stride must be a multiple of 8 elements";
  const int hid = heads * 64;
  const long total = static_cast<long>(R) * (hid / 8);
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  cache_append_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(k_new), static_cast<const __nv_bfloat16*>(v_new), ld,
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), R, hid, cap, pos, pos_dev);
  return launch_err();
}

}  // extern "C"

NMTG_BOUNDS_READER(nmtg_bounds_decode)
