// Sequence-model kernels for sm_100a that are bandwidth- or latency-bound rather than GEMM-shaped:
//   * transducer joint (broadcast add of acoustic and label states, ReLU, dropout; packed or dense) and its backward
//   * transducer (RNN-T) loss: alpha/beta lattices by anti-diagonal wavefronts, gradient with optional fused
//     log-softmax backward
//   * diagonal complex linear recurrence (LRU) as a warp-level scan along time, both directions, with backward
//   * Cauchy kernel coefficients of S4 (sum_n a_n / (b_l - c_n)) with backward
//   * warp-per-row softmax with key mask and dropout, and its backward
//
// Behavioural counterparts in the reference: onmt/modules/extensions/transducer/transducer_joint_kernel.cu:171-633,
// transducer_loss_kernel.cu:32-380, blru/blru_kernel.cu:41-165,
// onmt/models/speech_recognizer/mssm/ssm_kernel/ssm_kernel_coefficient_binding_cuda.cu:31-276,
// multihead_attn/softmax_apex.h (softmax / dropout / masked variants).
#include "b200_ptx.cuh"
#include "seq_api.h"
#include "bounds_check.cuh"

namespace b200 {
namespace {

const char* launch_err() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

// ------------------------------------------------------------------------------------------------------------
// 4-element vectors of fp32 / bf16
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.x));
    float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    uint2 t;
    *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = t;
  }
};

// row of (b, t, u) in the joint / loss lattice
struct Lattice {
  int T, U, packed;
  const long* off;
  __device__ __forceinline__ long row(int b, int t, int u, int ub) const {
    if (packed) return (b ? off[b - 1] : 0) + static_cast<long>(t) * ub + u;
    return (static_cast<long>(b) * T + t) * U + u;
  }
};

// ---- transducer joint ---------------------------------------------------------------------------------------
template <typename T>
__global__ void joint_fwd_kernel(const T* __restrict__ f, const T* __restrict__ g, const int* __restrict__ f_len,
                                 const int* __restrict__ g_len, Lattice lat, T* __restrict__ out, int H, int relu, float p,
                                 unsigned long long seed, unsigned long long stream_id) {
  const int t = blockIdx.x, b = blockIdx.y;
  const int tb = f_len[b], ub = g_len[b];
  const DropRng rng(seed, stream_id, p);
  const bool t_ok = t < tb;
  if (lat.packed && !t_ok) return;
  const T* frow = f + (static_cast<long>(b) * lat.T + t) * H;
  const int u_end = lat.packed ? ub : lat.U;
  for (int h = threadIdx.x * 4; h < H; h += blockDim.x * 4) {
    float fv[4] = {0.f, 0.f, 0.f, 0.f};
    if (t_ok) Vec4<T>::load(frow + h, fv);
    for (int u = 0; u < u_end; ++u) {
      const long r = lat.row(b, t, u, ub);
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (t_ok && u < ub) {
        Vec4<T>::load(g + (static_cast<long>(b) * lat.U + u) * H + h, v);
        const unsigned long long e = static_cast<unsigned long long>(r) * H + h;   // multiple of 4
        const uint32_t w = p > 0.f ? rng.word(e >> 2) : 0xFFFFFFFFu;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float s = v[j] + fv[j];
          if (relu) s = fmaxf(s, 0.f);
          if (p > 0.f) s = rng.keep(w, j) ? s * rng.scale : 0.f;
          v[j] = s;
        }
      }
      Vec4<T>::store(out + r * H + h, v);
    }
  }
}

// mode 0: df (block per (t, b), sum over u); mode 1: dg (block per (u, b), sum over t)
template <typename T>
__global__ void joint_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ out, const int* __restrict__ f_len,
                                 const int* __restrict__ g_len, Lattice lat, T* __restrict__ dst, int H, int relu, float p,
                                 unsigned long long seed, unsigned long long stream_id, float scale, int mode) {
  const int x = blockIdx.x, b = blockIdx.y;
  const int tb = f_len[b], ub = g_len[b];
  const DropRng rng(seed, stream_id, p);
  const int own_len = mode == 0 ? tb : ub, other_len = mode == 0 ? ub : tb;
  const int own_max = mode == 0 ? lat.T : lat.U;
  T* drow = dst + (static_cast<long>(b) * own_max + x) * H;
  for (int h = threadIdx.x * 4; h < H; h += blockDim.x * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (x < own_len) {
      for (int y = 0; y < other_len; ++y) {
        const int t = mode == 0 ? x : y, u = mode == 0 ? y : x;
        const long r = lat.row(b, t, u, ub);
        float d[4], o[4];
        Vec4<T>::load(dout + r * H + h, d);
        if (relu) Vec4<T>::load(out + r * H + h, o);
        const unsigned long long e = static_cast<unsigned long long>(r) * H + h;
        const uint32_t w = (p > 0.f && !relu) ? rng.word(e >> 2) : 0xFFFFFFFFu;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float m = 1.f;
          if (relu) m = o[j] > 0.f ? rng.scale : 0.f;             // kept and positive (scale is 1 without dropout)
          else if (p > 0.f) m = rng.keep(w, j) ? rng.scale : 0.f;
          acc[j] += d[j] * m;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] *= scale;
    Vec4<T>::store(drow + h, acc);
  }
}

// ---- transducer loss ----------------------------------------------------------------------------------------
__device__ __forceinline__ float log_add(float a, float b) {
  if (a == -INFINITY) return b;
  if (b == -INFINITY) return a;
  const float m = fmaxf(a, b);
  return m + log1pf(expf(-fabsf(a - b)));
}

// blockIdx.y == 0: alpha, == 1: beta.  Anti-diagonal d = t + u; the previous diagonal lives in shared memory.
__global__ void rnnt_lattice_kernel(const float* __restrict__ x, const int* __restrict__ label,
                                    const int* __restrict__ f_len, const int* __restrict__ y_len, Lattice lat,
                                    float* __restrict__ alpha, float* __restrict__ beta, float* __restrict__ loss, int V,
                                    int blank) {
  extern __shared__ float sm[];
  const int b = blockIdx.x;
  // lengths beyond the lattice and labels outside the vocabulary are brought into range (and counted in the debug build)
  const int tb = checked_range(f_len[b], 0, lat.T), ub = checked_range(y_len[b] + 1, 0, lat.U);
  float* prev = sm;
  float* cur = sm + lat.U + 1;
  const int* lab = label + static_cast<long>(b) * (lat.U - 1);
  const bool is_beta = blockIdx.y == 1;
  float* dst = (is_beta ? beta : alpha) + static_cast<long>(b) * lat.T * lat.U;
  if (tb <= 0 || ub <= 0) {
    if (is_beta && threadIdx.x == 0) loss[b] = 0.f;
    return;
  }
  const int nd = tb + ub - 1;
  for (int step = 0; step < nd; ++step) {
    const int d = is_beta ? nd - 1 - step : step;
    for (int u = threadIdx.x; u < ub; u += blockDim.x) {
      const int t = d - u;
      if (t < 0 || t >= tb) continue;
      float v;
      if (!is_beta) {
        if (t == 0 && u == 0) v = 0.f;
        else {
          float a = -INFINITY, c = -INFINITY;
          if (t > 0) a = prev[u] + x[lat.row(b, t - 1, u, ub) * V + blank];
          if (u > 0) c = prev[u - 1] + x[lat.row(b, t, u - 1, ub) * V + checked_range(lab[u - 1], 0, V - 1)];
          v = log_add(a, c);
        }
      } else {
        const long r = lat.row(b, t, u, ub) * V;
        if (t == tb - 1 && u == ub - 1) v = x[r + blank];
        else {
          float a = -INFINITY, c = -INFINITY;
          if (t < tb - 1) a = prev[u] + x[r + blank];
          if (u < ub - 1) c = prev[u + 1] + x[r + checked_range(lab[u], 0, V - 1)];
          v = log_add(a, c);
        }
        if (t == 0 && u == 0) loss[b] = -v;
      }
      cur[u] = v;
      dst[static_cast<long>(t) * lat.U + u] = v;
    }
    __syncthreads();
    float* tmp = prev; prev = cur; cur = tmp;
  }
}

__global__ void rnnt_grad_kernel(const float* __restrict__ x, const float* __restrict__ loss_grad,
                                 const float* __restrict__ alpha, const float* __restrict__ beta,
                                 const int* __restrict__ label, const int* __restrict__ f_len,
                                 const int* __restrict__ y_len, Lattice lat, float* __restrict__ dx, int V, int blank,
                                 int fuse_softmax) {
  const int b = blockIdx.y;
  const int t = blockIdx.x / lat.U, u = blockIdx.x % lat.U;
  const int tb = min(max(f_len[b], 0), lat.T), ub = min(max(y_len[b] + 1, 0), lat.U);   // counted once, in the lattice kernel
  const bool valid = t < tb && u < ub;
  if (!valid && lat.packed) return;
  const long r = lat.row(b, t, u, ub) * V;
  if (!valid) {
    for (int v = threadIdx.x; v < V; v += blockDim.x) dx[r + v] = 0.f;
    return;
  }
  const float* al = alpha + static_cast<long>(b) * lat.T * lat.U;
  const float* be = beta + static_cast<long>(b) * lat.T * lat.U;
  const float ll = be[0], a = al[static_cast<long>(t) * lat.U + u], g = loss_grad[b];
  const int lab = u < ub - 1 ? min(max(label[static_cast<long>(b) * (lat.U - 1) + u], 0), V - 1) : -1;
  float db = 0.f, dl = 0.f;
  if (t < tb - 1) db = -g * expf(a + be[static_cast<long>(t + 1) * lat.U + u] + x[r + blank] - ll);
  else if (u == ub - 1) db = -g * expf(a + x[r + blank] - ll);
  if (lab >= 0) dl = -g * expf(a + be[static_cast<long>(t) * lat.U + u + 1] + x[r + lab] - ll);
  const float tot = db + dl;
  for (int v = threadIdx.x; v < V; v += blockDim.x) {
    float d = (v == blank ? db : 0.f) + (v == lab ? dl : 0.f);
    if (fuse_softmax) d -= expf(x[r + v]) * tot;
    dx[r + v] = d;
  }
}

// ---- complex helpers ---------------------------------------------------------------------------------------
__device__ __forceinline__ float2 cmul(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }
__device__ __forceinline__ float2 cconj(float2 a) { return make_float2(a.x, -a.y); }
__device__ __forceinline__ float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 cinv(float2 d) {
  const float s = 1.f / (d.x * d.x + d.y * d.y);
  return make_float2(d.x * s, -d.y * s);
}

// ---- LRU scan: one warp per (b, n) row, 32 time steps per iteration ----------------------------------------------
// grad == false: h = scan(x).  grad == true: x holds dL/dh, the scan runs against the recurrence direction with
// conj(lambda), the result is dL/dx, and dlambda[n] += sum_t conj(h_prev(t)) * dx_t.
template <bool kGrad>
__global__ void lru_scan_kernel(const float2* __restrict__ lambda, const float2* __restrict__ x, const float2* __restrict__ hfwd,
                                const int* __restrict__ lengths, float2* __restrict__ y, float2* __restrict__ dlambda, int B,
                                int N, int L, int direction) {
  const int lane = threadIdx.x & 31;
  const long row = blockIdx.x * static_cast<long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= static_cast<long>(B) * N) return;
  const int b = static_cast<int>(row / N), n = static_cast<int>(row % N);
  int len = lengths[b];
  len = len < 0 ? 0 : (len > L ? L : len);
  int dir = direction == 2 ? (n < N / 2 ? 0 : 1) : direction;   // direction of the recurrence
  float2 lam = lambda[n];
  if (kGrad) { lam = cconj(lam); dir ^= 1; }
  float2 pw[5];                                                   // lambda^(2^k)
  pw[0] = lam;
#pragma unroll
  for (int k = 1; k < 5; ++k) pw[k] = cmul(pw[k - 1], pw[k - 1]);
  float2 lane_pow = make_float2(1.f, 0.f);                        // lambda^(lane + 1)
#pragma unroll
  for (int k = 0; k < 5; ++k)
    if ((lane + 1) & (1 << k)) lane_pow = cmul(lane_pow, pw[k]);
  if (lane == 31) lane_pow = cmul(pw[4], pw[4]);                 // 32 = 2^5 is not covered by the loop above
  const float2* xr = x + row * L;
  const float2* hr = kGrad ? hfwd + row * L : nullptr;
  float2* yr = y + row * L;
  float2 carry = make_float2(0.f, 0.f), dl = make_float2(0.f, 0.f);
  for (int base = 0; base < len; base += 32) {
    const int i = base + lane;
    const bool ok = i < len;
    const int pos = dir == 0 ? i : len - 1 - i;
    float2 v = ok ? xr[pos] : make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 5; ++k) {
      const int o = 1 << k;
      float2 up;
      up.x = __shfl_up_sync(0xffffffffu, v.x, o);
      up.y = __shfl_up_sync(0xffffffffu, v.y, o);
      if (lane >= o) v = cadd(v, cmul(pw[k], up));
    }
    v = cadd(v, cmul(lane_pow, carry));
    if (ok) {
      yr[pos] = v;
      if (kGrad) {
        // the forward recurrence ran opposite to this scan: its predecessor of `pos` is the next element here
        const int prev = dir == 0 ? pos + 1 : pos - 1;              // dir is already flipped
        if (prev >= 0 && prev < len) dl = cadd(dl, cmul(cconj(hr[prev]), v));
      }
    }
    carry.x = __shfl_sync(0xffffffffu, v.x, 31);
    carry.y = __shfl_sync(0xffffffffu, v.y, 31);
  }
  for (int i = len + lane; i < L; i += 32) yr[i] = make_float2(0.f, 0.f);
  if (kGrad) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      dl.x += __shfl_xor_sync(0xffffffffu, dl.x, o);
      dl.y += __shfl_xor_sync(0xffffffffu, dl.y, o);
    }
    if (lane == 0) {
      atomicAdd(&dlambda[n].x, dl.x);
      atomicAdd(&dlambda[n].y, dl.y);
    }
  }
}

// ---- Cauchy kernel coefficients ----------------------------------------------------------------------------
__global__ void cauchy_fwd_kernel(const float2* __restrict__ a, const float2* __restrict__ b, const float2* __restrict__ c,
                                  float2* __restrict__ out, int I, int Q, int L, int H, int N) {
  const long total = static_cast<long>(I) * Q * L * H;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const int h = static_cast<int>(idx % H);
    const int l = static_cast<int>((idx / H) % L);
    const int q = static_cast<int>((idx / (static_cast<long>(H) * L)) % Q);
    const int i = static_cast<int>(idx / (static_cast<long>(H) * L * Q));
    const float2 bl = b[(static_cast<long>(q) * L + l) * H + h];
    const float2* ar = a + ((static_cast<long>(i) * Q + q) * H + h) * N;
    const float2* cr = c + static_cast<long>(q) * N;
    float2 acc = make_float2(0.f, 0.f);
    for (int n = 0; n < N; ++n) {
      const float2 cn = cr[n];
      acc = cadd(acc, cmul(ar[n], cinv(make_float2(bl.x - cn.x, bl.y - cn.y))));
    }
    out[idx] = acc;
  }
}

__device__ __forceinline__ float2 block_sum2(float2 v, float2* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
  }
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float2 s = make_float2(0.f, 0.f);
  for (int k = 0; k < nw; ++k) s = cadd(s, red[k]);
  return s;
}

// block per (h, q); threads stride over l.  db[q, l, h] is owned by one thread of one block.
__global__ void cauchy_bwd_kernel(const float2* __restrict__ a, const float2* __restrict__ b, const float2* __restrict__ c,
                                  const float2* __restrict__ dout, float2* __restrict__ da, float2* __restrict__ db,
                                  float2* __restrict__ dc, int I, int Q, int L, int H, int N) {
  __shared__ float2 red[32];
  const int h = blockIdx.x, q = blockIdx.y;
  for (int i = 0; i < I; ++i) {
    for (int n = 0; n < N; ++n) {
      const float2 cn = c[static_cast<long>(q) * N + n];
      const long ai = ((static_cast<long>(i) * Q + q) * H + h) * N + n;
      const float2 an = a[ai];
      float2 s_da = make_float2(0.f, 0.f), s_dc = make_float2(0.f, 0.f);
      for (int l = threadIdx.x; l < L; l += blockDim.x) {
        const long bi = (static_cast<long>(q) * L + l) * H + h;
        const float2 bl = b[bi];
        const float2 r = cinv(make_float2(bl.x - cn.x, bl.y - cn.y));
        const float2 g = dout[((static_cast<long>(i) * Q + q) * L + l) * H + h];
        s_da = cadd(s_da, cmul(cconj(r), g));
        const float2 t2 = cmul(cconj(cmul(an, cmul(r, r))), g);
        s_dc = cadd(s_dc, t2);
        float2 cur = db[bi];
        db[bi] = make_float2(cur.x - t2.x, cur.y - t2.y);
      }
      const float2 tda = block_sum2(s_da, red);
      const float2 tdc = block_sum2(s_dc, red);
      if (threadIdx.x == 0) {
        da[ai] = tda;
        atomicAdd(&dc[static_cast<long>(q) * N + n].x, tdc.x);
        atomicAdd(&dc[static_cast<long>(q) * N + n].y, tdc.y);
      }
    }
  }
}

// ---- softmax (+mask, +dropout): one warp per row ------------------------------------------------------------
template <typename T> __device__ __forceinline__ float ld1(const T* p);
template <> __device__ __forceinline__ float ld1<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st1(T* p, float v);
template <> __device__ __forceinline__ void st1<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st1<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, const uint8_t* __restrict__ mask, T* __restrict__ y,
                                   T* __restrict__ yd, int rows, int cols, int rows_per_mask, float scale, float p,
                                   unsigned long long seed, unsigned long long stream_id) {
  const int lane = threadIdx.x & 31;
  const long row = blockIdx.x * static_cast<long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const DropRng rng(seed, stream_id, p);
  const T* xr = x + row * cols;
  const uint8_t* mr = mask ? mask + (row / rows_per_mask) * cols : nullptr;
  float mx = -INFINITY;
  for (int c = lane; c < cols; c += 32)
    if (!mr || !mr[c]) mx = fmaxf(mx, ld1(xr + c) * scale);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int c = lane; c < cols; c += 32)
    if (!mr || !mr[c]) sum += __expf(ld1(xr + c) * scale - mx);
  sum = warp_sum(sum);
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  for (int c = lane; c < cols; c += 32) {
    float v = (!mr || !mr[c]) ? __expf(ld1(xr + c) * scale - mx) * inv : 0.f;
    st1(y + row * cols + c, v);
    if (yd) {
      const unsigned long long e = static_cast<unsigned long long>(row) * cols + c;
      if (p > 0.f) v = rng.keep(rng.word(e >> 2), static_cast<int>(e & 3)) ? v * rng.scale : 0.f;
      st1(yd + row * cols + c, v);
    }
  }
}

template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ dyd, const T* __restrict__ y, T* __restrict__ dx, int rows, int cols,
                                   float scale, float p, unsigned long long seed, unsigned long long stream_id) {
  const int lane = threadIdx.x & 31;
  const long row = blockIdx.x * static_cast<long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const DropRng rng(seed, stream_id, p);
  float dot = 0.f;
  for (int c = lane; c < cols; c += 32) {
    const unsigned long long e = static_cast<unsigned long long>(row) * cols + c;
    float g = ld1(dyd + row * cols + c);
    if (p > 0.f) g = rng.keep(rng.word(e >> 2), static_cast<int>(e & 3)) ? g * rng.scale : 0.f;
    dot += g * ld1(y + row * cols + c);
  }
  dot = warp_sum(dot);
  for (int c = lane; c < cols; c += 32) {
    const unsigned long long e = static_cast<unsigned long long>(row) * cols + c;
    float g = ld1(dyd + row * cols + c);
    if (p > 0.f) g = rng.keep(rng.word(e >> 2), static_cast<int>(e & 3)) ? g * rng.scale : 0.f;
    st1(dx + row * cols + c, scale * ld1(y + row * cols + c) * (g - dot));
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

const char* nmtg_transducer_joint_fwd(const void* f, const void* g, const int* f_len, const int* g_len,
                                      const long* batch_offset, void* out, int B, int T, int U, int H, int dtype,
                                      int packed, int relu, float p, unsigned long long seed,
                                      unsigned long long stream_id, cudaStream_t stream) {
  if (H % 4) return "transducer joint: hidden size must be a multiple of 4";
  if (packed && !batch_offset) return "transducer joint: packed output needs batch_offset";
  if (B <= 0 || T <= 0 || U <= 0) return nullptr;
  Lattice lat{T, U, packed, batch_offset};
  dim3 grid(T, B);
  const int threads = H >= 512 ? 128 : 64;
  if (dtype == 0)
    joint_fwd_kernel<float><<<grid, threads, 0, stream>>>(static_cast<const float*>(f), static_cast<const float*>(g), f_len,
                                                           g_len, lat, static_cast<float*>(out), H, relu, p, seed, stream_id);
  else
    joint_fwd_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(f), static_cast<const __nv_bfloat16*>(g), f_len, g_len, lat,
        static_cast<__nv_bfloat16*>(out), H, relu, p, seed, stream_id);
  return launch_err();
}

const char* nmtg_transducer_joint_bwd(const void* dout, const void* out, const int* f_len, const int* g_len,
                                      const long* batch_offset, void* df, void* dg, int B, int T, int U, int H,
                                      int dtype, int packed, int relu, float p, unsigned long long seed,
                                      unsigned long long stream_id, float scale, cudaStream_t stream) {
  if (H % 4) return "transducer joint: hidden size must be a multiple of 4";
  if (relu && !out) return "transducer joint backward: the forward output is needed with relu";
  if (B <= 0 || T <= 0 || U <= 0) return nullptr;
  Lattice lat{T, U, packed, batch_offset};
  const int threads = H >= 512 ? 128 : 64;
  for (int mode = 0; mode < 2; ++mode) {
    dim3 grid(mode == 0 ? T : U, B);
    void* dst = mode == 0 ? df : dg;
    if (dtype == 0)
      joint_bwd_kernel<float><<<grid, threads, 0, stream>>>(static_cast<const float*>(dout), static_cast<const float*>(out),
                                                             f_len, g_len, lat, static_cast<float*>(dst), H, relu, p, seed,
                                                             stream_id, scale, mode);
    else
      joint_bwd_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(out), f_len, g_len, lat,
          static_cast<__nv_bfloat16*>(dst), H, relu, p, seed, stream_id, scale, mode);
  }
  return launch_err();
}

const char* nmtg_transducer_loss_fwd(const float* x, const int* label, const int* f_len, const int* y_len,
                                     const long* batch_offset, float* alpha, float* beta, float* loss, int B, int T,
                                     int U, int V, int blank, int packed, cudaStream_t stream) {
  if (packed && !batch_offset) return "transducer loss: packed input needs batch_offset";
  if (blank < 0 || blank >= V) return "transducer loss: blank index out of range";
  if (B <= 0) return nullptr;
  Lattice lat{T, U, packed, batch_offset};
  const size_t smem = 2 * static_cast<size_t>(U + 1) * sizeof(float);
  if (smem > 48 * 1024) return "transducer loss: label dimension too large (U + 1 > 6144)";
  const int threads = U >= 256 ? 256 : (U >= 64 ? 128 : 32);
  rnnt_lattice_kernel<<<dim3(B, 2), threads, smem, stream>>>(x, label, f_len, y_len, lat, alpha, beta, loss, V, blank);
  return launch_err();
}

const char* nmtg_transducer_loss_bwd(const float* x, const float* loss_grad, const float* alpha, const float* beta,
                                     const int* label, const int* f_len, const int* y_len, const long* batch_offset,
                                     float* dx, int B, int T, int U, int V, int blank, int packed, int fuse_softmax,
                                     cudaStream_t stream) {
  if (packed && !batch_offset) return "transducer loss: packed input needs batch_offset";
  if (B <= 0 || T <= 0 || U <= 0) return nullptr;
  if (B > 65535) return "transducer loss: batch too large";
  Lattice lat{T, U, packed, batch_offset};
  const int threads = V >= 1024 ? 256 : 128;
  rnnt_grad_kernel<<<dim3(T * U, B), threads, 0, stream>>>(x, loss_grad, alpha, beta, label, f_len, y_len, lat, dx, V, blank,
                                                           fuse_softmax);
  return launch_err();
}

const char* nmtg_lru_scan_fwd(const float2* lambda, const float2* x, const int* lengths, float2* h, int B, int N, int L,
                              int direction, cudaStream_t stream) {
  if (direction < 0 || direction > 2) return "lru scan: direction must be 0, 1 or 2";
  if (B <= 0 || N <= 0 || L <= 0) return nullptr;
  const long rows = static_cast<long>(B) * N;
  lru_scan_kernel<false><<<static_cast<unsigned>((rows + 3) / 4), 128, 0, stream>>>(lambda, x, nullptr, lengths, h, nullptr, B,
                                                                                    N, L, direction);
  return launch_err();
}

const char* nmtg_lru_scan_bwd(const float2* lambda, const float2* grad_h, const float2* h, const int* lengths,
                              float2* dx, float2* dlambda, int B, int N, int L, int direction, cudaStream_t stream) {
  if (direction < 0 || direction > 2) return "lru scan: direction must be 0, 1 or 2";
  if (B <= 0 || N <= 0 || L <= 0) return nullptr;
  const long rows = static_cast<long>(B) * N;
  lru_scan_kernel<true><<<static_cast<unsigned>((rows + 3) / 4), 128, 0, stream>>>(lambda, grad_h, h, lengths, dx, dlambda, B,
                                                                                   N, L, direction);
  return launch_err();
}

const char* nmtg_cauchy_fwd(const float2* a, const float2* b, const float2* c, float2* out, int I, int Q, int L, int H,
                            int N, cudaStream_t stream) {
  const long total = static_cast<long>(I) * Q * L * H;
  if (total <= 0) return nullptr;
  const long blocks = (total + 255) / 256;
  cauchy_fwd_kernel<<<static_cast<unsigned>(blocks > 148 * 16 ? 148 * 16 : blocks), 256, 0, stream>>>(a, b, c, out, I, Q, L, H, N);
  return launch_err();
}

const char* nmtg_cauchy_bwd(const float2* a, const float2* b, const float2* c, const float2* dout, float2* da, float2* db,
                            float2* dc, int I, int Q, int L, int H, int N, cudaStream_t stream) {
  if (I <= 0 || Q <= 0 || L <= 0 || H <= 0 || N <= 0) return nullptr;
  if (Q > 65535) return "cauchy backward: too many heads";
  cauchy_bwd_kernel<<<dim3(H, Q), 128, 0, stream>>>(a, b, c, dout, da, db, dc, I, Q, L, H, N);
  return launch_err();
}

const char* nmtg_softmax_dropout_fwd(const void* x, const uint8_t* pad_mask, void* y, void* yd, int rows, int cols,
                                     int rows_per_mask, int dtype, float scale, float p, unsigned long long seed,
                                     unsigned long long stream_id, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return nullptr;
  if (pad_mask && rows_per_mask <= 0) return "softmax: rows_per_mask must be positive";
  const unsigned blocks = static_cast<unsigned>((rows + 3) / 4);
  if (dtype == 0)
    softmax_fwd_kernel<float><<<blocks, 128, 0, stream>>>(static_cast<const float*>(x), pad_mask, static_cast<float*>(y),
                                                          static_cast<float*>(yd), rows, cols, rows_per_mask, scale, p, seed,
                                                          stream_id);
  else
    softmax_fwd_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), pad_mask, static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(yd), rows,
        cols, rows_per_mask, scale, p, seed, stream_id);
  return launch_err();
}

const char* nmtg_softmax_dropout_bwd(const void* dyd, const void* y, void* dx, int rows, int cols, int dtype, float scale,
                                     float p, unsigned long long seed, unsigned long long stream_id,
                                     cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return nullptr;
  const unsigned blocks = static_cast<unsigned>((rows + 3) / 4);
  if (dtype == 0)
    softmax_bwd_kernel<float><<<blocks, 128, 0, stream>>>(static_cast<const float*>(dyd), static_cast<const float*>(y),
                                                          static_cast<float*>(dx), rows, cols, scale, p, seed, stream_id);
  else
    softmax_bwd_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(dyd),
                                                                  static_cast<const __nv_bfloat16*>(y),
                                                                  static_cast<__nv_bfloat16*>(dx), rows, cols, scale, p, seed,
                                                                  stream_id);
  return launch_err();
}

}  // extern "C"

NMTG_BOUNDS_READER(nmtg_bounds_sequence)
