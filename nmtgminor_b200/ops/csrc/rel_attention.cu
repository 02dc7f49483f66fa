// Transformer-XL style relative-position self-attention for packed short sequences (T <= 128, head size 64):
//
//   s_ij = ((q_i + u) . k_j + (q_i + w) . r_(i-j)) * scale,   p = dropout(softmax_j(s)),   ctx_i = sum_j p_ij v_j
//
// One CTA per (sequence, head).  Keys, values and the window of 2T-1 relative-position rows that this sequence can
// address are staged in shared memory (rows padded to 33 words so that lanes walking over keys hit distinct banks);
// the relative shift of the reference (pad + reshape of the [T, 2T-1] score matrix) is index arithmetic here:
// distance i - j lives in window row T-1-i+j.  A warp owns a query: lanes run over keys for the scores and the
// softmax, then over the 64 feature columns for the value product.  The backward kernel recomputes the
// probabilities from the saved log-sum-exp, owns dq per query, and accumulates dk / dv / dr in shared memory
// (fp32) before one write-out per CTA; du / dw are reduced per warp.
//
// Counterpart of the reference's relative_self_attn kernels (onmt/modules/extensions/multihead_attn_blaslt/
// relative_self_attn_cuda.cu:28-371: batched GEMMs + shift + softmax-dropout kernels).
#include "b200_ptx.cuh"
#include "seq_api.h"

namespace b200 {
namespace {

constexpr int kMaxT = 128;
constexpr int kRowWords = 33;    // 64 bf16 = 32 words + 1 word of padding
constexpr int kWarps = 8;

struct RelArgs {
  const __nv_bfloat16* qkv;   // [N, 3H]: q | k | v
  const __nv_bfloat16* r;     // [L, H]: row r_center - d holds distance d
  const float* u;             // [heads, 64]  (r_w_bias)
  const float* w;             // [heads, 64]  (r_r_bias)
  const int* cu;              // [B + 1]
  float* lse;                 // [heads, N]
  int heads, H, r_center, L, N, causal;
  float scale, p;
  unsigned long long seed, stream_id;
};

__device__ __forceinline__ float2 ldw(const uint32_t* row, int word) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + word));
}

// stage rows [row0, row0 + n) x 64 columns at column offset col of a bf16 matrix with leading dimension ld
__device__ __forceinline__ void stage_rows(uint32_t* dst, const __nv_bfloat16* src, long ld, long row0, int n, int col) {
  for (int i = threadIdx.x; i < n * 32; i += blockDim.x) {
    const int rr = i >> 5, wd = i & 31;
    dst[rr * kRowWords + wd] = *reinterpret_cast<const uint32_t*>(src + (row0 + rr) * ld + col + 2 * wd);
  }
}

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

// scores of query i against keys lane, lane + 32, ... (at most 4 per lane); masked entries are -inf
__device__ __forceinline__ void scores_for_query(const uint32_t* Ks, const uint32_t* Rs, const float* qu, const float* qw, int i,
                                                 int T, int causal, float scale, int lane, float (&s)[4]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int j = lane + 32 * c;
    float acc = -INFINITY;
    if (j < T && !(causal && j > i)) {
      const uint32_t* kr = Ks + j * kRowWords;
      const uint32_t* rr = Rs + (T - 1 - i + j) * kRowWords;
      float a = 0.f;
#pragma unroll 8
      for (int wd = 0; wd < 32; ++wd) {
        const float2 kk = ldw(kr, wd), r2 = ldw(rr, wd);
        a = fmaf(qu[2 * wd], kk.x, a);
        a = fmaf(qu[2 * wd + 1], kk.y, a);
        a = fmaf(qw[2 * wd], r2.x, a);
        a = fmaf(qw[2 * wd + 1], r2.y, a);
      }
      acc = a * scale;
    }
    s[c] = acc;
  }
}

__global__ void __launch_bounds__(kWarps * 32)
rel_attn_fwd_kernel(const RelArgs p, __nv_bfloat16* __restrict__ out) {
  extern __shared__ uint32_t sm[];
  const int b = blockIdx.x, h = blockIdx.y;
  const int t0 = p.cu[b], T = p.cu[b + 1] - t0;
  if (T <= 0 || T > kMaxT) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t* Ks = sm;
  uint32_t* Vs = Ks + T * kRowWords;
  uint32_t* Rs = Vs + T * kRowWords;
  float* scratch = reinterpret_cast<float*>(Rs + (2 * T - 1) * kRowWords);
  float* qu = scratch + warp * (128 + kMaxT);
  float* qw = qu + 64;
  float* pw = qw + 64;
  const long ld = 3L * p.H;
  stage_rows(Ks, p.qkv, ld, t0, T, p.H + h * 64);
  stage_rows(Vs, p.qkv, ld, t0, T, 2 * p.H + h * 64);
  stage_rows(Rs, p.r, p.H, p.r_center - (T - 1), 2 * T - 1, h * 64);
  __syncthreads();
  const DropRng rng(p.seed, p.stream_id, p.p);
  for (int i = warp; i < T; i += kWarps) {
    {
      const float2 q2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p.qkv + (t0 + i) * ld + h * 64 + 2 * lane));
      qu[2 * lane] = q2.x + p.u[h * 64 + 2 * lane];
      qu[2 * lane + 1] = q2.y + p.u[h * 64 + 2 * lane + 1];
      qw[2 * lane] = q2.x + p.w[h * 64 + 2 * lane];
      qw[2 * lane + 1] = q2.y + p.w[h * 64 + 2 * lane + 1];
    }
    __syncwarp();
    float s[4];
    scores_for_query(Ks, Rs, qu, qw, i, T, p.causal, p.scale, lane, s);
    const float mx = warp_max(fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3])));
    float e[4], sum = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      e[c] = s[c] == -INFINITY ? 0.f : __expf(s[c] - mx);
      sum += e[c];
    }
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    if (lane == 0) p.lse[static_cast<long>(h) * p.N + t0 + i] = sum > 0.f ? mx + __logf(sum) : 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = lane + 32 * c;
      float pv = e[c] * inv;
      if (p.p > 0.f) {
        const unsigned long long el = (static_cast<unsigned long long>(t0 + i) * p.heads + h) * kMaxT + j;
        pv = rng.keep(rng.word(el >> 2), static_cast<int>(el & 3)) ? pv * rng.scale : 0.f;
      }
      if (j < kMaxT) pw[j] = pv;
    }
    __syncwarp();
    float2 acc = make_float2(0.f, 0.f);
    const int jend = p.causal ? i + 1 : T;
    for (int j = 0; j < jend; ++j) {
      const float2 v2 = ldw(Vs + j * kRowWords, lane);
      acc.x = fmaf(pw[j], v2.x, acc.x);
      acc.y = fmaf(pw[j], v2.y, acc.y);
    }
    *reinterpret_cast<__nv_bfloat162*>(out + static_cast<long>(t0 + i) * p.H + h * 64 + 2 * lane) = __floats2bfloat162_rn(acc.x, acc.y);
    __syncwarp();
  }
}

__global__ void __launch_bounds__(kWarps * 32)
rel_attn_bwd_kernel(const RelArgs p, const __nv_bfloat16* __restrict__ dctx, __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dr,
                    float* __restrict__ du, float* __restrict__ dw) {
  extern __shared__ uint32_t sm[];
  const int b = blockIdx.x, h = blockIdx.y;
  const int t0 = p.cu[b], T = p.cu[b + 1] - t0;
  if (T <= 0 || T > kMaxT) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nr = 2 * T - 1;
  uint32_t* Ks = sm;
  uint32_t* Vs = Ks + T * kRowWords;
  uint32_t* Rs = Vs + T * kRowWords;
  float* dK = reinterpret_cast<float*>(Rs + nr * kRowWords);
  float* dV = dK + T * 64;
  float* dR = dV + T * 64;
  float* scratch = dR + nr * 64;
  float* qu = scratch + warp * (192 + 2 * kMaxT);
  float* qw = qu + 64;
  float* dO = qw + 64;
  float* dSw = dO + 64;
  float* pdw = dSw + kMaxT;
  const long ld = 3L * p.H;
  stage_rows(Ks, p.qkv, ld, t0, T, p.H + h * 64);
  stage_rows(Vs, p.qkv, ld, t0, T, 2 * p.H + h * 64);
  stage_rows(Rs, p.r, p.H, p.r_center - (T - 1), nr, h * 64);
  for (int i = threadIdx.x; i < (2 * T + nr) * 64; i += blockDim.x) dK[i] = 0.f;     // dK, dV, dR are contiguous
  __syncthreads();
  const DropRng rng(p.seed, p.stream_id, p.p);
  float2 du_acc = make_float2(0.f, 0.f), dw_acc = make_float2(0.f, 0.f);
  const int d0 = 2 * lane;
  for (int i = warp; i < T; i += kWarps) {
    {
      const float2 q2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p.qkv + (t0 + i) * ld + h * 64 + d0));
      const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dctx + static_cast<long>(t0 + i) * p.H + h * 64 + d0));
      qu[d0] = q2.x + p.u[h * 64 + d0];
      qu[d0 + 1] = q2.y + p.u[h * 64 + d0 + 1];
      qw[d0] = q2.x + p.w[h * 64 + d0];
      qw[d0 + 1] = q2.y + p.w[h * 64 + d0 + 1];
      dO[d0] = g2.x;
      dO[d0 + 1] = g2.y;
    }
    __syncwarp();
    float s[4];
    scores_for_query(Ks, Rs, qu, qw, i, T, p.causal, p.scale, lane, s);
    const float lse = p.lse[static_cast<long>(h) * p.N + t0 + i];
    float pr[4], dp[4], dsum = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = lane + 32 * c;
      pr[c] = 0.f;
      dp[c] = 0.f;
      if (s[c] != -INFINITY) {
        float pv = __expf(s[c] - lse), keep = 1.f;
        if (p.p > 0.f) {
          const unsigned long long el = (static_cast<unsigned long long>(t0 + i) * p.heads + h) * kMaxT + j;
          keep = rng.keep(rng.word(el >> 2), static_cast<int>(el & 3)) ? rng.scale : 0.f;
        }
        const uint32_t* vr = Vs + j * kRowWords;
        float a = 0.f;
#pragma unroll 8
        for (int wd = 0; wd < 32; ++wd) {
          const float2 v2 = ldw(vr, wd);
          a = fmaf(dO[2 * wd], v2.x, a);
          a = fmaf(dO[2 * wd + 1], v2.y, a);
        }
        pr[c] = pv;
        dp[c] = a * keep;                 // gradient reaching the un-dropped probability
        dsum += pv * dp[c];
        if (j < kMaxT) pdw[j] = pv * keep;
      } else if (j < kMaxT) {
        pdw[j] = 0.f;
      }
    }
    dsum = warp_sum(dsum);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int j = lane + 32 * c;
      if (j < kMaxT) dSw[j] = pr[c] * (dp[c] - dsum) * p.scale;
    }
    __syncwarp();
    float2 ac = make_float2(0.f, 0.f), bd = make_float2(0.f, 0.f);
    const int jend = p.causal ? i + 1 : T;
    for (int j = 0; j < jend; ++j) {
      const float ds = dSw[j], pd = pdw[j];
      const int x = T - 1 - i + j;
      const float2 kk = ldw(Ks + j * kRowWords, lane), rr = ldw(Rs + x * kRowWords, lane);
      ac.x = fmaf(ds, kk.x, ac.x);
      ac.y = fmaf(ds, kk.y, ac.y);
      bd.x = fmaf(ds, rr.x, bd.x);
      bd.y = fmaf(ds, rr.y, bd.y);
      atomicAdd(&dK[j * 64 + d0], ds * qu[d0]);
      atomicAdd(&dK[j * 64 + d0 + 1], ds * qu[d0 + 1]);
      atomicAdd(&dR[x * 64 + d0], ds * qw[d0]);
      atomicAdd(&dR[x * 64 + d0 + 1], ds * qw[d0 + 1]);
      atomicAdd(&dV[j * 64 + d0], pd * dO[d0]);
      atomicAdd(&dV[j * 64 + d0 + 1], pd * dO[d0 + 1]);
    }
    *reinterpret_cast<__nv_bfloat162*>(dqkv + (t0 + i) * ld + h * 64 + d0) = __floats2bfloat162_rn(ac.x + bd.x, ac.y + bd.y);
    du_acc.x += ac.x; du_acc.y += ac.y;
    dw_acc.x += bd.x; dw_acc.y += bd.y;
    __syncwarp();
  }
  atomicAdd(&du[h * 64 + d0], du_acc.x);
  atomicAdd(&du[h * 64 + d0 + 1], du_acc.y);
  atomicAdd(&dw[h * 64 + d0], dw_acc.x);
  atomicAdd(&dw[h * 64 + d0 + 1], dw_acc.y);
  __syncthreads();
  for (int i = threadIdx.x; i < T * 32; i += blockDim.x) {
    const int j = i >> 5, wd = i & 31;
    *reinterpret_cast<__nv_bfloat162*>(dqkv + (t0 + j) * ld + p.H + h * 64 + 2 * wd) = __floats2bfloat162_rn(dK[j * 64 + 2 * wd], dK[j * 64 + 2 * wd + 1]);
    *reinterpret_cast<__nv_bfloat162*>(dqkv + (t0 + j) * ld + 2 * p.H + h * 64 + 2 * wd) = __floats2bfloat162_rn(dV[j * 64 + 2 * wd], dV[j * 64 + 2 * wd + 1]);
  }
  for (int i = threadIdx.x; i < nr * 64; i += blockDim.x) {
    const int x = i >> 6, d = i & 63;
    atomicAdd(&dr[static_cast<long>(p.r_center - (T - 1) + x) * p.H + h * 64 + d], dR[i]);
  }
}

size_t fwd_smem(int T) { return static_cast<size_t>(4 * T - 1) * kRowWords * 4 + kWarps * (128 + kMaxT) * 4; }
size_t bwd_smem(int T) {
  return static_cast<size_t>(4 * T - 1) * kRowWords * 4 + static_cast<size_t>(4 * T - 1) * 64 * 4 + kWarps * (192 + 2 * kMaxT) * 4;
}

const char* check(const RelArgs& a, int max_len) {
  if (a.H != a.heads * 64) return "rel_attn: head size must be 64";
  if (max_len < 1 || max_len > kMaxT) return "rel_attn: sequences longer than 128 are not supported by this kernel";
  if (a.r_center - (max_len - 1) < 0 || a.r_center + (max_len - 1) >= a.L) return "rel_attn: position table does not cover the distances";
  return nullptr;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

const char* nmtg_rel_attn_fwd(const void* qkv, const void* r, const float* u, const float* w, const int* cu, void* out, float* lse,
                              int B, int N, int heads, int max_len, int r_center, int L, int causal, float scale, float p,
                              unsigned long long seed, unsigned long long stream_id, cudaStream_t stream) {
  if (B <= 0) return nullptr;
  RelArgs a{static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(r), u, w, cu, lse, heads, heads * 64, r_center, L, N,
            causal, scale, p, seed, stream_id};
  if (const char* e = check(a, max_len)) return e;
  const size_t smem = fwd_smem(max_len);
  cudaError_t err = cudaFuncSetAttribute(rel_attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(fwd_smem(kMaxT)));
  if (err != cudaSuccess) return cudaGetErrorString(err);
  rel_attn_fwd_kernel<<<dim3(B, heads), kWarps * 32, smem, stream>>>(a, static_cast<__nv_bfloat16*>(out));
  err = cudaGetLastError();
  return err == cudaSuccess ? nullptr : cudaGetErrorString(err);
}

const char* nmtg_rel_attn_bwd(const void* qkv, const void* r, const float* u, const float* w, const int* cu, const float* lse,
                              const void* dctx, void* dqkv, float* dr, float* du, float* dw, int B, int N, int heads, int max_len,
                              int r_center, int L, int causal, float scale, float p, unsigned long long seed,
                              unsigned long long stream_id, cudaStream_t stream) {
  if (B <= 0) return nullptr;
  RelArgs a{static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(r), u, w, cu, const_cast<float*>(lse), heads,
            heads * 64, r_center, L, N, causal, scale, p, seed, stream_id};
  if (const char* e = check(a, max_len)) return e;
  const size_t smem = bwd_smem(max_len);
  if (smem > 227 * 1024) return "rel_attn backward: shared memory budget exceeded";
  cudaError_t err = cudaFuncSetAttribute(rel_attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bwd_smem(kMaxT)));
  if (err != cudaSuccess) return cudaGetErrorString(err);
  rel_attn_bwd_kernel<<<dim3(B, heads), kWarps * 32, smem, stream>>>(a, static_cast<const __nv_bfloat16*>(dctx),
                                                                     static_cast<__nv_bfloat16*>(dqkv), dr, du, dw);
  err = cudaGetLastError();
  return err == cudaSuccess ? nullptr : cudaGetErrorString(err);
}

}  // extern "C"
