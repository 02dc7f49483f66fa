// Shared declarations of the attention kernels (general multi-tile kernels and the persistent pipelined
// kernels for sequences that fit one 128-row tile).
#pragma once
#include "b200_ptx.cuh"
#include "ops_api.h"

namespace b200 {

bool cached_tmap(CUtensorMap* out, const void* base, long rows, long cols, long ld, int br, int bc);
bool cached_tmap_f32(CUtensorMap* out, const void* base, long rows, long cols, long ld, int br, int bc);

constexpr int kHd = 64;          // head dimension
constexpr int kTile = 128;       // query / key tile
constexpr int kTileBytes = kTile * kHd * 2;   // 16 KB : one [128 x 64] bf16 tile
constexpr int kPBytes = kTile * kTile * 2;    // 32 KB : P or dS as two [128 x 64] slabs
constexpr float kNegBig = -1.0e30f;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnArgs {
  const int* cu_q;
  const int* cu_k;
  int num_heads;
  int causal;
  float scale;
  float dropout_p;
  unsigned long long seed, stream_id;
  const unsigned long long* seed_dev;
  int kstride;            // multiple of 16, >= longest key sequence: dropout counter stride per query row
  __nv_bfloat16* out; int ld_out;       // fwd: O ; bwd: unused
  float* lse; long lse_stride;          // [heads, lse_stride]
  __nv_bfloat16* p_debug; long p_stride_row;  // optional [heads, total_q, kstride] dropped probabilities
  // backward
  const __nv_bfloat16* o; int ld_o;
  const __nv_bfloat16* d_o; int ld_do;
  __nv_bfloat16* dq; int ld_dq;
  __nv_bfloat16* dk; int ld_dk;
  __nv_bfloat16* dv; int ld_dv;
  float* dq_acc; int ld_dqacc;          // fp32 accumulation buffer for multi-key-tile sequences
  const float* delta;                   // rowsum(dO * O), laid out like lse; null: computed in the kernel per tile
  int dq_tma;                           // 1: dQ tiles are added to dq_acc by TMA reductions (tensor map given to the kernel)
  int total_q;
  int total_k;            // allocated rows of q / k (>= cu[batch]): rows past the last sequence are cleared by the kernels
  int batch;
  int* status;
  // optional additive score bias [batch, heads, q, k] in natural-log units (k contiguous; element strides below), added
  // to S * scale before the softmax; dbias (same layout, zero-initialised by the caller) receives its gradient
  const float* bias; long bias_sb, bias_sh, bias_sq;
  float* dbias;
};

// scores of 32 key columns of one query row -> base-2 domain with the bias added: r = r * scale_log2 + bias * log2 e.
// `brow` points at the bias of the first of the 32 columns (null: the row is outside the sequence), `ncols` of them exist.
__device__ __forceinline__ void add_bias32(uint32_t (&r)[32], const float* brow, int ncols, float scale_log2) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float bv = (brow != nullptr && j < ncols) ? __ldg(brow + j) * 1.4426950408889634f : 0.f;
    r[j] = __float_as_uint(fmaf(__uint_as_float(r[j]), scale_log2, bv));
  }
}

// Clears rows [first_row, end_row) of a bf16 matrix (width a multiple of 8 columns, 16-byte aligned rows) with the
// whole grid.  Those rows belong to no sequence, so nothing else in the kernel touches them and no ordering is
// needed; callers can therefore hand the kernels uninitialised output buffers.
__device__ __forceinline__ void zero_tail_rows(__nv_bfloat16* base, int ld, int width, int first_row, int end_row) {
  if (base == nullptr || first_row >= end_row) return;
  const long bid = blockIdx.x + static_cast<long>(gridDim.x) * (blockIdx.y + static_cast<long>(gridDim.y) * blockIdx.z);
  const long nb = static_cast<long>(gridDim.x) * gridDim.y * gridDim.z;
  const int vec = width >> 3;
  const long total = static_cast<long>(end_row - first_row) * vec;
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (long i = bid * blockDim.x + threadIdx.x; i < total; i += nb * blockDim.x) {
    const long r = first_row + i / vec;
    const int c = static_cast<int>(i % vec) << 3;
    *reinterpret_cast<uint4*>(base + r * ld + c) = z;
  }
}
__device__ __forceinline__ void zero_tail_fwd(const AttnArgs& p) {
  zero_tail_rows(p.out, p.ld_out, p.num_heads * 64, p.cu_q[p.batch], p.total_q);
}
__device__ __forceinline__ void zero_tail_bwd(const AttnArgs& p) {
  const int w = p.num_heads * 64;
  zero_tail_rows(p.dq, p.ld_dq, w, p.cu_q[p.batch], p.total_q);
  const int k_end = p.cu_k[p.batch];
  zero_tail_rows(p.dk, p.ld_dk, w, k_end, p.total_k);
  zero_tail_rows(p.dv, p.ld_dv, w, k_end, p.total_k);
}

// nk UMMA k-steps reading A from a_addr (+ k * a_step bytes) and B from b_addr (+ k * b_step bytes)
__device__ __forceinline__ void umma_steps(uint32_t d_tmem, uint32_t a_addr, uint32_t a_lbo, uint32_t a_step,
                                           uint32_t b_addr, uint32_t b_lbo, uint32_t b_step, uint32_t idesc, int nk,
                                           bool accumulate_first) {
  const uint64_t adesc = make_smem_desc_sw128(a_addr, a_lbo, 1024);
  const uint64_t bdesc = make_smem_desc_sw128(b_addr, b_lbo, 1024);
  for (int k = 0; k < nk; ++k)
    umma_bf16(d_tmem, adesc + static_cast<uint64_t>((k * a_step) >> 4), bdesc + static_cast<uint64_t>((k * b_step) >> 4),
              idesc, (accumulate_first || k > 0) ? 1u : 0u);
}

// Dropout factors (0 or keep scale) for 32 consecutive probabilities starting at element index `base`
// (a multiple of 4): multiplies pv[] in place.
__device__ __forceinline__ void apply_dropout32(const DropRng& rng, unsigned long long base, float (&pv)[32]) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const uint32_t w = rng.word((base >> 2) + g);
#pragma unroll
    for (int j = 0; j < 4; ++j) pv[g * 4 + j] = rng.keep(w, j) ? pv[g * 4 + j] * rng.scale : 0.f;
  }
}

// ---------------------------------------------------------------------------------------------------
// Backward arithmetic on 16 key columns of one query row (shared by the single-tile and the multi-tile kernels).  Working
// on 16 columns at a time keeps few values live per thread, which is what lets the compiler interleave independent
// elements: holding whole 32- or 64-column chunks of S, dP, P and dS at once made these loops latency-bound.
// ---------------------------------------------------------------------------------------------------
// bit j = element (base + j) is kept; base a multiple of 4
__device__ __forceinline__ uint32_t drop_mask16(const DropRng& rng, unsigned long long base) {
  uint32_t m = 0;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint32_t w = rng.word((base >> 2) + g);
#pragma unroll
    for (int j = 0; j < 4; ++j) m |= (rng.keep(w, j) ? 1u : 0u) << (g * 4 + j);
  }
  return m;
}

// Probabilities from the raw scores (P = 2^(sc * sl2 - lse2); sl2 = 1 when the scores were converted already) and
// dS = P * (dP_dropped - D), packed to bf16 (two 16-byte vectors each).  c0: first column inside the key tile (columns
// >= k_lim do not exist); causal: key position kpos0 + j must not exceed q_pos.  A row past the sequence has lse2 = +inf,
// so its probabilities are 0 without a per-element test.  dS is kept without the softmax scale (applied when dQ and dK
// leave TMEM).  ds_out (optional): the 16 fp32 dS values of the existing pairs, for the gradient of an additive bias.
// kMasked / kDrop are compile-time so that the common case (a tile inside both sequences, below the diagonal, no dropout)
// carries no per-element predicate: with run-time flags the compiler evaluated the validity test and both dropout variants
// for every element, which doubled the instruction count of the loop.
template <bool kMasked, bool kDrop>
__device__ __forceinline__ void bwd_compute16_t(const uint32_t (&sc)[16], const uint32_t (&dp)[16], uint32_t keep,
                                                float keep_scale, float Drow, float sl2, float lse2, int c0, int k_lim,
                                                bool causal, int kpos0, int q_pos, uint4 (&vp)[2], uint4 (&vds)[2],
                                                float* ds_out) {
#pragma unroll
  for (int g2 = 0; g2 < 2; ++g2) {
    __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&vp[g2]);
    __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&vds[g2]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float pd[2], ds[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int idx = g2 * 8 + 2 * j + e;
        float prob = ex2_approx(fmaf(__uint_as_float(sc[idx]), sl2, -lse2));
        bool valid = true;
        if (kMasked) {
          valid = c0 + idx < k_lim && (!causal || kpos0 + idx <= q_pos);
          prob = valid ? prob : 0.f;
        }
        const float d = __uint_as_float(dp[idx]);
        if (kDrop) {
          const float kf = ((keep >> idx) & 1u) ? keep_scale : 0.f;
          pd[e] = prob * kf;
          ds[e] = prob * fmaf(d, kf, -Drow);
        } else {
          pd[e] = prob;
          ds[e] = prob * (d - Drow);
        }
        if (ds_out != nullptr && valid) ds_out[idx] = ds[e];
      }
      a2[j] = __floats2bfloat162_rn(pd[0], pd[1]);
      b2[j] = __floats2bfloat162_rn(ds[0], ds[1]);
    }
  }
}
__device__ __forceinline__ void bwd_compute16(const uint32_t (&sc)[16], const uint32_t (&dp)[16], uint32_t keep, bool do_drop,
                                              float keep_scale, float Drow, float sl2, float lse2, int c0, int k_lim,
                                              bool causal, int kpos0, int q_pos, uint4 (&vp)[2], uint4 (&vds)[2],
                                              float* ds_out = nullptr) {
  const bool full = !causal && c0 + 16 <= k_lim;
  if (!do_drop) {
    if (full) bwd_compute16_t<false, false>(sc, dp, keep, keep_scale, Drow, sl2, lse2, c0, k_lim, causal, kpos0, q_pos, vp, vds, ds_out);
    else bwd_compute16_t<true, false>(sc, dp, keep, keep_scale, Drow, sl2, lse2, c0, k_lim, causal, kpos0, q_pos, vp, vds, ds_out);
  } else {
    if (full) bwd_compute16_t<false, true>(sc, dp, keep, keep_scale, Drow, sl2, lse2, c0, k_lim, causal, kpos0, q_pos, vp, vds, ds_out);
    else bwd_compute16_t<true, true>(sc, dp, keep, keep_scale, Drow, sl2, lse2, c0, k_lim, causal, kpos0, q_pos, vp, vds, ds_out);
  }
}
// the two vectors of bwd_compute16 into the 128-byte-swizzled staging tiles (row t, columns c0 .. c0 + 15 of the tile)
__device__ __forceinline__ void bwd_store16(const uint4 (&vp)[2], const uint4 (&vds)[2], int c0, int t, uint8_t* sP, uint8_t* sDS) {
#pragma unroll
  for (int g2 = 0; g2 < 2; ++g2) {
    const int chunk = (c0 >> 3) + g2;     // 16-byte chunk of the row: 8 per 64-key slab
    const uint32_t off = (chunk >> 3) * kTileBytes + sw128_offset(t, chunk & 7);
    *reinterpret_cast<uint4*>(sP + off) = vp[g2];
    *reinterpret_cast<uint4*>(sDS + off) = vds[g2];
  }
}

// scores of 16 key columns -> base-2 domain with an additive bias: r = r * scale_log2 + bias * log2 e
__device__ __forceinline__ void add_bias16(uint32_t (&r)[16], const float* brow, int ncols, float scale_log2) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float bv = (brow != nullptr && j < ncols) ? __ldg(brow + j) * 1.4426950408889634f : 0.f;
    r[j] = __float_as_uint(fmaf(__uint_as_float(r[j]), scale_log2, bv));
  }
}

}  // namespace b200
