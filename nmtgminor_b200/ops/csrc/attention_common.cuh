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

}  // namespace b200
