// Warp-specialised forward pass of the multi-tile (general) attention kernels for sm_100a, head_dim 64.
//
// One CTA owns TWO neighbouring 128-query tiles of one (sequence, head) and walks over the key tiles once for both, so K
// and V tiles are fetched once per 256 queries and the softmax of one query tile runs under the MMAs of the other:
//
//   warps 0-3   softmax of query tile 0: thread = query row (TMEM lane), all 128 key columns of the tile
//   warps 4-7   softmax of query tile 1
//   warp 10     TMA producer: Q tiles once, K and V tiles through rings of three stages each
//   warps 8, 9  MMA issuers, one per query tile: S_g = Q_g K^T as soon as the softmax warps have read the previous S_g,
//               and O_g += P_g V as soon as P_g is stored
//
// TMEM (512 columns): S of tile 0 | S of tile 1 | O of tile 0 | O of tile 1 | P of tile 0 | P of tile 1 (64 columns each:
// 128 bf16 probabilities per row, two per column).  P never touches shared memory: the softmax threads store it into
// tensor memory and the P V product reads its A operand from there, so that product costs only V's shared-memory
// bandwidth - an M = 128, N <= 128 MMA with both operands in shared memory saturates the 128 B/clock of the SM on its
// own, and every other shared-memory access slows it down.  O accumulates in TMEM over the key tiles.  A softmax thread reads its whole row of S (128 values) into registers in one go, so S is read once and the MMA
// of the next key tile may overwrite it right away.  The row maximum that the exponentials refer to is only moved when
// the new tile exceeds it by more than 2^8 (probabilities then stay below 256, harmless in fp32 / bf16); only then are
// the 64 accumulator columns of the row rescaled in TMEM, which after the first tiles of a sequence is rare.  The final
// division uses the row sum taken against the same reference, so the result is the exact softmax.  Arithmetic and masks
// are those of attn_fwd_kernel (attention_tcgen05.cu), which stays for calls with attention dropout (hashing the mask
// words in the one softmax warp per scheduler cost more than the pipelining gained: 0.21 against 0.15 ms on 8 x 1000 x 16
// heads), with an additive bias and for short sequences.  Every wait is bounded (status word).
//
// Counterpart in the reference: fmha_fprop_kernel_1xN.h of its bundled FlashAttention and the cuBLAS + warp-softmax
// forward of onmt/modules/extensions/multihead_attn/self_multihead_attn_cuda.cu:23-231.
#include "attention_common.cuh"

namespace b200 {

constexpr int kFwsThreads = 352;
constexpr int kFwsStages = 3;
constexpr int kFwsSmem = 2 * kTileBytes + 2 * kFwsStages * kTileBytes + 512 + 1024;

// Time stamps (SM clock) of CTA (0, 0, 0) when ablation bit 128 is set: [key tile][16] = softmax warp 0: S ready, row
// loaded, maximum, exponentials, packed, previous product done, staged | MMA warp: S of tile 0 issued, P V of tile 0
// issued, S of tile 1 issued, P V of tile 1 issued.  A timing aid, read back with nmtg_attn_fws_trace.
constexpr int kFwsTraceTiles = 32;
__device__ long long g_fws_trace[kFwsTraceTiles * 16];
#define FWS_STAMP(tile, slot)                                                                             \
  do {                                                                                                    \
    if (trace && (tile) < kFwsTraceTiles) g_fws_trace[(tile) * 16 + (slot)] = clock64();                  \
  } while (0)

__global__ void __launch_bounds__(kFwsThreads, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const AttnArgs p, const int ablate) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                  // [2] query tiles
  uint8_t* sK = sQ + 2 * kTileBytes;                   // [3] key tiles
  uint8_t* sV = sK + kFwsStages * kTileBytes;          // [3] value tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kFwsStages * kTileBytes);
  uint64_t* q_full = bars;           // TMA -> MMA
  uint64_t* k_full = bars + 1;       // [3] TMA -> MMA
  uint64_t* k_free = bars + 4;       // [3] S of both query tiles done -> TMA
  uint64_t* v_full = bars + 7;       // [3]
  uint64_t* v_free = bars + 10;      // [3] P V of both query tiles done -> TMA
  uint64_t* s_full = bars + 13;      // [2] S_g ready -> softmax warps g
  uint64_t* s_free = bars + 15;      // [2] S_g read -> MMA
  uint64_t* p_full = bars + 17;      // [2] P_g stored in tensor memory -> MMA
  uint64_t* pv_done = bars + 19;     // [2] P_g V of a key tile done: P_g may be overwritten, O_g may be touched
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  zero_tail_fwd(p);
  const int b = blockIdx.z, h = blockIdx.y;
  const int q_begin = p.cu_q[b], q_end = p.cu_q[b + 1];
  const int k_begin = p.cu_k[b], k_len = p.cu_k[b + 1] - k_begin;
  const int qt0 = 2 * blockIdx.x;
  if (q_begin + qt0 * kTile >= q_end) return;   // uniform for the CTA, before any barrier or TMEM use
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kt = (k_len + kTile - 1) / kTile;
  // per query tile g: first row, rows inside the sequence (0: the tile does not exist), key tiles it attends to
  int q0[2], q_rows[2], nkt[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    q0[g] = q_begin + (qt0 + g) * kTile;
    q_rows[g] = max(0, min(kTile, q_end - q0[g]));
    nkt[g] = q_rows[g] > 0 ? (p.causal ? min(total_kt, ((qt0 + g) * kTile + q_rows[g] + kTile - 1) / kTile) : total_kt) : 0;
  }
  const int nkt_max = max(nkt[0], nkt[1]);
  const bool trace = (ablate & 128) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (warp == 0 || warp == 8 || warp == 9);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kFwsStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_free[i], 2);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_free[i], 2);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 128);
      mbar_init(&p_full[i], 128);
      mbar_init(&pv_done[i], 1);
    }
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 9) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 10) {
    // ---- TMA producer --------------------------------------------------------------------------------------------
    if (lane == 0 && nkt_max > 0) {
      mbar_expect_tx(q_full, (q_rows[1] > 0 ? 2 : 1) * kTileBytes);
      tma_load_2d(sQ, &tmap_q, q_full, h * kHd, q0[0]);
      if (q_rows[1] > 0) tma_load_2d(sQ + kTileBytes, &tmap_q, q_full, h * kHd, q0[1]);
      for (int kt = 0; kt < nkt_max; ++kt) {
        const int st = kt % kFwsStages;
        const uint32_t par = ((kt / kFwsStages) & 1) ^ 1;
        if (kt >= kFwsStages && !mbar_wait(&k_free[st], par, abort_word, p.status, kTimeoutSmemEmpty)) break;
        mbar_expect_tx(&k_full[st], kTileBytes);
        tma_load_2d(sK + st * kTileBytes, &tmap_k, &k_full[st], h * kHd, k_begin + kt * kTile);
        if (kt >= kFwsStages && !mbar_wait(&v_free[st], par, abort_word, p.status, kTimeoutSmemEmpty)) break;
        mbar_expect_tx(&v_full[st], kTileBytes);
        tma_load_2d(sV + st * kTileBytes, &tmap_v, &v_full[st], h * kHd, k_begin + kt * kTile);
      }
    }
  } else if (warp == 8 || warp == 9) {
    // ---- MMA issuers: one warp per query tile ------------------------------------------------------------------------
    // An MMA of these shapes is 32 to 64 clocks of tensor-core work, less than it costs a single thread that shares its
    // scheduler with two softmax warps to issue it; with one issuer per query tile the two chains S_g -> P_g V are issued
    // side by side.  K and V stages are released by both issuers (two arrivals each).
    const int g = warp - 8;
    const int n = g ? nkt[1] : nkt[0], n_other = g ? nkt[0] : nkt[1];
    if (lane == 0 && n > 0 && mbar_wait(q_full, 0, abort_word, p.status, kTimeoutTmaFull)) {
      const uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(kTile, kHd, 0, 1);
      const uint32_t tS = tmem_base + g * kTile, tO = tmem_base + 256 + g * 64, tP = tmem_base + 384 + g * 64;
      const uint32_t qa = smem_u32(sQ + g * kTileBytes);
      // The events of one query tile come in a fixed order - S of key tile k read (s_free) before P of key tile k stored
      // (p_full) - so the issuer blocks on them one after the other.  A blocked mbarrier wait costs no issue slots; an
      // issuer that polls its barriers in a loop shares a scheduler with two softmax warps and slowed them down enough
      // for them to finish thousands of clocks after the rest of their warpgroup.
      bool ok = true;
      auto issue_s = [&](int kt) -> bool {
        const int st = kt % kFwsStages;
        if (!mbar_wait(&k_full[st], (kt / kFwsStages) & 1, abort_word, p.status, kTimeoutTmaFull)) return false;
        if (kt > 0 && !mbar_wait(&s_free[g], (kt - 1) & 1, abort_word, p.status, kTimeoutTmemEmpty)) return false;
        tc_fence_after_sync();
        if (g == 0) FWS_STAMP(kt, 14);
        umma_steps(tS, qa, 16, 32, smem_u32(sK + st * kTileBytes), 16, 32, idesc_s, kHd / 16, false);
        if (g == 0) FWS_STAMP(kt, 15);
        umma_commit(&s_full[g]);
        umma_commit(&k_free[st]);
        if (kt >= n_other) umma_commit(&k_free[st]);     // the other query tile never reads this key tile
        FWS_STAMP(kt, 8 + 2 * g);
        return true;
      };
      ok = issue_s(0);
      for (int kt = 0; kt < n && ok; ++kt) {
        if (kt + 1 < n) ok = issue_s(kt + 1);
        if (!ok) break;
        const int st = kt % kFwsStages;
        // O_g += P_g V of key tile kt
        ok = mbar_wait(&p_full[g], kt & 1, abort_word, p.status, kTimeoutTmemEmpty) &&
             mbar_wait(&v_full[st], (kt / kFwsStages) & 1, abort_word, p.status, kTimeoutTmaFull);
        if (!ok) break;
        if (g == 0) FWS_STAMP(kt, 7);
        tc_fence_after_sync();
        // A = P from tensor memory (8 columns per 16 keys), B = V (MN-major, 16 keys = 2048 bytes per k-step)
        const uint64_t vdesc = make_smem_desc_sw128(smem_u32(sV + st * kTileBytes), 8192, 1024);
        if (g == 0) FWS_STAMP(kt, 12);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ts(tO, tP + k * 8, vdesc + static_cast<uint64_t>((k * 2048) >> 4), idesc_o, (kt > 0 || k > 0) ? 1u : 0u);
        if (g == 0) FWS_STAMP(kt, 13);
        umma_commit(&pv_done[g]);
        umma_commit(&v_free[st]);
        if (kt >= n_other) umma_commit(&v_free[st]);
        FWS_STAMP(kt, 9 + 2 * g);
      }
    }
  } else {
    // ---- softmax warps -------------------------------------------------------------------------------------------
    const int g = warp >> 2;
    const int t = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + g * kTile + lane_sel;
    const uint32_t tO = tmem_base + 256 + g * 64 + lane_sel;
    const uint32_t tP = tmem_base + 384 + g * 64 + lane_sel;
    const int n = g ? nkt[1] : nkt[0];
    const int my_q0 = g ? q0[1] : q0[0], my_rows = g ? q_rows[1] : q_rows[0];
    const int qt = qt0 + g;
    const int q_pos = qt * kTile + t;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    float m_run = kNegBig, l_run = 0.f;     // reference maximum (base-2 domain) and the row sum taken against it
    bool ok = true;

    for (int kt = 0; kt < n && ok; ++kt) {
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[g], kt & 1, abort_word, p.status, kTimeoutTmemFull));
      if (!ok) break;
      tc_fence_after_sync();
      FWS_STAMP(kt, 0);
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld32(tS, r0);
      tmem_ld32(tS + 32, r1);
      tmem_ld32(tS + 64, r2);
      tmem_ld32(tS + 96, r3);
      tmem_ld_wait();
      FWS_STAMP(kt, 1);
      tc_fence_before_sync();
      mbar_arrive(&s_free[g]);            // the whole row is in registers: S of the next key tile may overwrite this one
      const int kcols = min(kTile, k_len - kt * kTile);
      const bool full = kcols == kTile && (!p.causal || kt < qt);
      if (!full) {
        // scores of pairs that do not exist become a large negative number once, so the loops below need no tests
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int kp = kt * kTile + j;
          if (!(j < kcols && (!p.causal || kp <= q_pos))) r0[j] = __float_as_uint(kNegBig);
          if (!(j + 32 < kcols && (!p.causal || kp + 32 <= q_pos))) r1[j] = __float_as_uint(kNegBig);
          if (!(j + 64 < kcols && (!p.causal || kp + 64 <= q_pos))) r2[j] = __float_as_uint(kNegBig);
          if (!(j + 96 < kcols && (!p.causal || kp + 96 <= q_pos))) r3[j] = __float_as_uint(kNegBig);
        }
      }
      // row maximum of the raw scores (scale > 0: the maximum commutes with the scaling)
      float m0 = kNegBig, m1 = kNegBig, m2 = kNegBig, m3 = kNegBig;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        m0 = fmaxf(m0, __uint_as_float(r0[j]));
        m1 = fmaxf(m1, __uint_as_float(r1[j]));
        m2 = fmaxf(m2, __uint_as_float(r2[j]));
        m3 = fmaxf(m3, __uint_as_float(r3[j]));
      }
      const float m_tile = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * scale_log2;
      float alpha = 1.f;
      if (m_tile > m_run + 8.f) {          // also true for the first tile (m_run = -1e30)
        alpha = ex2_approx(m_run - m_tile);
        m_run = m_tile;
      }
      const bool rescale = kt > 0 && __any_sync(0xffffffffu, alpha != 1.f);
      FWS_STAMP(kt, 2);
      // probabilities against the reference maximum, in place; masked scores (-1e30 * scale) give exactly 0
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float e0 = ex2_approx(fmaf(__uint_as_float(r0[j]), scale_log2, -m_run));
        const float e1 = ex2_approx(fmaf(__uint_as_float(r1[j]), scale_log2, -m_run));
        const float e2 = ex2_approx(fmaf(__uint_as_float(r2[j]), scale_log2, -m_run));
        const float e3 = ex2_approx(fmaf(__uint_as_float(r3[j]), scale_log2, -m_run));
        s0 += e0;
        s1 += e1;
        s2 += e2;
        s3 += e3;
        r0[j] = __float_as_uint(e0);
        r1[j] = __float_as_uint(e1);
        r2[j] = __float_as_uint(e2);
        r3[j] = __float_as_uint(e3);
      }
      l_run = l_run * alpha + ((s0 + s1) + (s2 + s3));
      FWS_STAMP(kt, 3);
      // bf16 packing first (the 128 fp32 values die here), then the wait for the previous product
      uint32_t pk0[32], pk1[32];     // keys 0..63 and 64..127 of the row, two bf16 per word
      {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t(&r)[32] = c == 0 ? r0 : (c == 1 ? r1 : (c == 2 ? r2 : r3));
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            (c < 2 ? pk0 : pk1)[(c & 1) * 16 + j] = *reinterpret_cast<const uint32_t*>(&v);
          }
        }
      }
      FWS_STAMP(kt, 4);
      if (kt > 0) {
        // P V of the previous key tile has had this whole softmax to complete: the staging tile and O are free
        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[g], (kt - 1) & 1, abort_word, p.status, kTimeoutTmemFull));
        if (!ok) break;
        tc_fence_after_sync();
        FWS_STAMP(kt, 5);
        if (rescale) {                      // some row of this warp moved its reference: O *= alpha (1 for the others)
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t o[32];
            tmem_ld32(tO + hh * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st32(tO + hh * 32, o);
          }
        }
      }
      tmem_st32(tP, pk0);
      tmem_st32(tP + 32, pk1);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&p_full[g]);
      FWS_STAMP(kt, 6);
    }
    if (ok && n > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[g], (n - 1) & 1, abort_word, p.status, kTimeoutTmemFull));
      if (ok) {
        tc_fence_after_sync();
        uint32_t o0[32], o1[32];
        tmem_ld32(tO, o0);
        tmem_ld32(tO + 32, o1);
        tmem_ld_wait();
        if (t < my_rows) {
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
          __nv_bfloat16* orow = p.out + static_cast<size_t>(my_q0 + t) * p.ld_out + h * kHd;
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int e = (g4 & 3) * 8 + 2 * j;
              o2[j] = __floats2bfloat162_rn(__uint_as_float(g4 < 4 ? o0[e] : o1[e]) * inv, __uint_as_float(g4 < 4 ? o0[e + 1] : o1[e + 1]) * inv);
            }
            reinterpret_cast<uint4*>(orow)[g4] = o;
          }
          if (p.lse)
            p.lse[static_cast<size_t>(h) * p.lse_stride + my_q0 + t] = l_run > 0.f ? (m_run + __log2f(l_run)) * 0.6931471805599453f : 0.f;
        }
      }
    } else if (ok && n == 0 && t < my_rows) {
      // a query row without keys (empty key sequence): zero output
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      __nv_bfloat16* orow = p.out + static_cast<size_t>(my_q0 + t) * p.ld_out + h * kHd;
      for (int g4 = 0; g4 < 8; ++g4) reinterpret_cast<uint4*>(orow)[g4] = z;
      if (p.lse) p.lse[static_cast<size_t>(h) * p.lse_stride + my_q0 + t] = 0.f;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_word) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

int get_attn_bwd_ablation();

const char* launch_attn_fwd_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a, int max_q,
                               cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(attn_fwd_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwsSmem);
    if (ce != cudaSuccess) return cudaGetErrorString(ce);
    configured = true;
  }
  dim3 grid((max_q + 2 * kTile - 1) / (2 * kTile), a.num_heads, a.batch);
  if (a.dropout_p > 0.f) return "attention: the warp-specialised forward kernel has no dropout";
  attn_fwd_ws_kernel<<<grid, kFwsThreads, kFwsSmem, stream>>>(tq, tk, tv, a, get_attn_bwd_ablation());
  cudaError_t ce = cudaGetLastError();
  return ce == cudaSuccess ? nullptr : cudaGetErrorString(ce);
}

}  // namespace b200

// copies the time stamps of the last traced launch (ablation bit 128) to host memory; returns the number of values
int nmtg_attn_fws_trace(long long* out, int capacity) {
  const int n = b200::kFwsTraceTiles * 16 < capacity ? b200::kFwsTraceTiles * 16 : capacity;
  if (cudaMemcpyFromSymbol(out, b200::g_fws_trace, n * sizeof(long long)) != cudaSuccess) return -1;
  return n;
}
