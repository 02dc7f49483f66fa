// Shared pieces of the tcgen05 GEMM kernels (single-CTA and CTA-pair variants): argument block and the
// fused epilogue applied to one 32-column chunk of an accumulator row.
#pragma once
#include "b200_ptx.cuh"
#include "ops_api.h"

namespace b200 {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kEpilogueWarps = 8;   // two warps per TMEM lane quarter, interleaved over 32-column chunks

struct GemmArgs {
  int M, N, K;
  int a_mn_major, b_mn_major;
  int split_k;             // >= 1; > 1 requires out_fp32 and atomic accumulation
  int stream_k;            // CTA-pair kernel, fp32 accumulating output: equal runs of (tile, k-block) pairs per cluster
  float alpha;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ld_res] or null, added last
  int ld_res;
  const __nv_bfloat16* aux;       // [M, ld_aux] activation-backward operand or null
  int ld_aux;
  void* out;
  int ld_out;
  int out_fp32;
  int accumulate;          // fp32 output only: out += result
  __nv_bfloat16* preact;   // optional [M, ld_out]: value after bias, before activation
  uint32_t* mask;          // optional [M, ld_mask] sign bits of the output (written, or read by kActMaskBwd)
  int ld_mask;
  float* colsum;           // optional fp32 [N]: += column sums of the stored bf16 output (TMA-store epilogue)
  int act;
  float dropout_p;
  unsigned long long seed, stream_id;
  const unsigned long long* seed_dev;
  int* status;
  int tma_store;           // bf16 output leaves through shared memory and TMA stores (CTA-pair kernel)
  int ablate;              // profiling aid: 1 = read the accumulator but skip arithmetic and stores, 2 = skip the epilogue body,
                           // 3 (traced kernel only) = also skip the MMAs: operand streaming alone
  long long* trace;        // profiling aid: when set, the CTA-pair kernel writes up to 16 cycle counters per cluster (see gemm2cta_tcgen05.cu)
};

// In-kernel gather of the B operand (fully sharded parameters), CTA-pair kernel.  The matrix is `units` blocks of
// 4 KB, claimed four at a time through the cursor counters[1]; block u belongs to segment u / seg_units, and the TMA
// producer loads tiles of a segment only after counters[2 + segment] has reached the segment's block count.
// n_seg == 0: no gather.
constexpr int kGatherBlockBytes = 4096;
constexpr int kGatherMaxSegs = 128;
struct GatherArgs {
  int n_seg;
  int rank, world;
  const unsigned short* shards[16];
  long shard_off, piece_len, unit_off;
  unsigned short* dst;      // local staging address of the matrix
  long units;               // 4 KB blocks in the matrix
  int seg_units;            // blocks per segment (the last segment may have fewer)
  int* counters;            // [0]: CTAs that have left the kernel, [1]: next unclaimed block, [2 + s]: finished blocks of segment s
};

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad(float x) {
  float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
  float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + __expf(-x)); }

// One thread = one accumulator row; processes columns [col0, col0 + 32) read from TMEM address `taddr`:
// alpha, bias, optional pre-activation store, activation or activation gradient, dropout, residual, store
// (bf16, fp32, fp32 accumulate, or fp32 red.add for split-K).  Warp-collective (contains a tcgen05.ld).
// `stage_row` (optional): instead of writing bf16 results to global memory, place the 64-byte row fragment in a
// shared-memory staging row laid out for a 128-byte-swizzled TMA store (logical 16-byte chunk j of row r sits at
// chunk j ^ (r & 7)); `stage_half` selects the left / right 32 columns of the 64-column staging tile.
// Feature bits of the epilogue.  A kernel instantiated with a mask contains only the code of those features (the
// run-time checks inside still apply), which keeps the epilogue a short straight-line sequence: with everything
// compiled in, each 32-column chunk jumps over a dozen large unused blocks and the warps wait on instruction fetch
// rather than on arithmetic.  kEpiAll is the general kernel.
constexpr uint32_t kEpiBias = 1u, kEpiPreact = 2u, kEpiActFwd = 4u, kEpiActBwd = 8u, kEpiMaskBwd = 16u, kEpiDrop = 32u,
                   kEpiMaskOut = 64u, kEpiRes = 128u, kEpiF32 = 256u, kEpiBf16 = 512u,
                   kEpiRagged = 1024u /* N not a multiple of 64: partial column chunks */,
                   kEpiColsum = 2048u /* column sums of the output, pair kernel only */, kEpiAll = 4095u;

// Features a problem needs (host side).
inline uint32_t gemm_epilogue_features(const GemmArgs& a) {
  uint32_t f = 0;
  if (a.bias) f |= kEpiBias;
  if (a.preact) f |= kEpiPreact;
  if (a.act == kActMaskBwd) f |= kEpiMaskBwd;
  else if (a.act >= kActReluBwd) f |= kEpiActBwd;
  else if (a.act != 0) f |= kEpiActFwd;
  if (a.dropout_p > 0.f) f |= kEpiDrop;
  if (a.mask && a.act != kActMaskBwd) f |= kEpiMaskOut;
  if (a.residual) f |= kEpiRes;
  f |= a.out_fp32 ? kEpiF32 : kEpiBf16;
  if (a.N % 64) f |= kEpiRagged;
  if (a.colsum) f |= kEpiColsum;
  return f;
}

template <uint32_t kFeat = kEpiAll>
__device__ __forceinline__ void gemm_epilogue_chunk(const GemmArgs& p, const DropRng& rng, const bool do_drop, const int row,
                                                    const bool row_ok, const int col0, const uint32_t taddr,
                                                    uint8_t* stage_row = nullptr, const int stage_half = 0,
                                                    const int stage_r = 0) {
    const bool full_cols = !(kFeat & kEpiRagged) || (col0 + 32 <= p.N);
    // global operands of the epilogue are requested BEFORE the TMEM load so their latency overlaps it
    uint4 aux_v[4], res_v[4];
    const bool aux_vec = (kFeat & kEpiActBwd) && row_ok && full_cols && p.act >= kActReluBwd && p.act != kActMaskBwd && (p.ld_aux & 7) == 0;
    uint32_t mask_word = 0;
    if ((kFeat & kEpiMaskBwd) && p.act == kActMaskBwd && row_ok) mask_word = p.mask[static_cast<size_t>(row) * p.ld_mask + (col0 >> 5)];
    const bool res_vec = (kFeat & kEpiRes) && row_ok && full_cols && p.residual != nullptr && (p.ld_res & 7) == 0;
    if (aux_vec) {
      const uint4* ap4 = reinterpret_cast<const uint4*>(p.aux + static_cast<size_t>(row) * p.ld_aux + col0);
#pragma unroll
      for (int g = 0; g < 4; ++g) aux_v[g] = ap4[g];
    }
    if (res_vec) {
      const uint4* rp4 = reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(row) * p.ld_res + col0);
#pragma unroll
      for (int g = 0; g < 4; ++g) res_v[g] = rp4[g];
    }
    uint32_t r[32];
    tmem_ld32(taddr, r);
    tmem_ld_wait();
    if (!row_ok || p.ablate == 1) return;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
    if ((kFeat & kEpiBias) && p.bias) {
      if (full_cols) {
        const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 b = __ldg(bp + g);
          const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(b2[j]);
            v[g * 8 + 2 * j] += f.x;
            v[g * 8 + 2 * j + 1] += f.y;
          }
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
      }
    }
    if ((kFeat & kEpiPreact) && p.preact) {
      __nv_bfloat16* pp = p.preact + static_cast<size_t>(row) * p.ld_out + col0;
      if (full_cols) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[g * 8 + 2 * j], v[g * 8 + 2 * j + 1]);
          reinterpret_cast<uint4*>(pp)[g] = o;
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) pp[j] = __float2bfloat16(v[j]);
      }
    }
    // activation (forward) or activation-gradient (backward; aux holds h or z)
    if ((kFeat & kEpiMaskBwd) && p.act == kActMaskBwd) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = ((mask_word >> j) & 1u) ? v[j] : 0.f;
    } else if ((kFeat & kEpiActBwd) && p.act >= kActReluBwd) {
      const __nv_bfloat16* ap = p.aux + static_cast<size_t>(row) * p.ld_aux + col0;
      float av[32];
      if (aux_vec) {
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {
          uint4 u = aux_v[g4];
          const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(u2[j]);
            av[g4 * 8 + 2 * j] = f.x;
            av[g4 * 8 + 2 * j + 1] = f.y;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) av[j] = (col0 + j < p.N) ? __bfloat162float(ap[j]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float a = av[j];
        float g;
        if (p.act == kActReluBwd) g = a > 0.f ? 1.f : 0.f;  // aux = relu output (after dropout)
        else if (p.act == kActGeluBwd) g = gelu_grad(a);
        else { float s = sigmoid_f(a); g = s * (1.f + a * (1.f - s)); }
        v[j] *= g;
      }
    } else if ((kFeat & kEpiActFwd) && p.act == kActRelu) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
    } else if ((kFeat & kEpiActFwd) && p.act == kActGelu) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = gelu_f(v[j]);
    } else if ((kFeat & kEpiActFwd) && p.act == kActSilu) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = v[j] * sigmoid_f(v[j]);
    }
    if ((kFeat & kEpiDrop) && do_drop) {
      // element index = row * N + col; 4 consecutive elements share one hash word (one byte each)
      const unsigned long long w0 = (static_cast<unsigned long long>(row) * p.N + col0) >> 2;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const uint32_t w = rng.word(w0 + g);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[g * 4 + j] = rng.keep(w, j) ? v[g * 4 + j] * rng.scale : 0.f;
      }
    }
    if ((kFeat & kEpiMaskOut) && p.mask && p.act != kActMaskBwd) {
      uint32_t bits = 0;
#pragma unroll
      for (int j = 0; j < 32; ++j) bits |= (v[j] > 0.f ? 1u : 0u) << j;
      p.mask[static_cast<size_t>(row) * p.ld_mask + (col0 >> 5)] = bits;
    }
    if ((kFeat & kEpiRes) && p.residual) {
      const __nv_bfloat16* rp = p.residual + static_cast<size_t>(row) * p.ld_res + col0;
      if (res_vec) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 b = res_v[g];
          const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(b2[j]);
            v[g * 8 + 2 * j] += f.x;
            v[g * 8 + 2 * j + 1] += f.y;
          }
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) v[j] += __bfloat162float(rp[j]);
      }
    }
    if ((kFeat & kEpiF32) && (p.out_fp32 || !(kFeat & kEpiBf16))) {
      float* op = reinterpret_cast<float*>(p.out) + static_cast<size_t>(row) * p.ld_out + col0;
      // accumulation into an existing fp32 buffer goes through the L2 reduction unit as well: no read round trip
      if (p.split_k > 1 || p.accumulate || p.stream_k) {
        if (full_cols) {
#pragma unroll
          for (int g = 0; g < 8; ++g)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(op + g * 4), "f"(v[g * 4]),
                         "f"(v[g * 4 + 1]), "f"(v[g * 4 + 2]), "f"(v[g * 4 + 3])
                         : "memory");
        } else {
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) atomicAdd(op + j, v[j]);
        }
      } else if (full_cols) {
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          float4 o = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
          if (p.accumulate) {
            float4 old = reinterpret_cast<float4*>(op)[g];
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          reinterpret_cast<float4*>(op)[g] = o;
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) op[j] = p.accumulate ? op[j] + v[j] : v[j];
      }
    } else if (!(kFeat & kEpiBf16)) {
      // fp32-only kernel asked for bf16 output: the host never selects this combination
    } else if (stage_row != nullptr) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[g * 8 + 2 * j], v[g * 8 + 2 * j + 1]);
        *reinterpret_cast<uint4*>(stage_row + (((stage_half * 4 + g) ^ (stage_r & 7)) << 4)) = o;
      }
    } else {
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ld_out + col0;
      if (full_cols) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[g * 8 + 2 * j], v[g * 8 + 2 * j + 1]);
          reinterpret_cast<uint4*>(op)[g] = o;
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) op[j] = __float2bfloat16(v[j]);
      }
    }
}

}  // namespace b200
