// Persistent, warp-specialised, software-pipelined attention for sequences that fit ONE 128-row tile
// (query and key length <= 128: every sentence-level translation batch).  A work item is one
// (sequence, head) pair; each CTA (one per SM) walks a strided list of items and overlaps, across items,
//   TMA loads of Q / K / V (/ dO)        - producer warp, multi-slot shared-memory ring
//   tcgen05 MMAs into TMEM               - MMA warp, issues S(i+1) before the second-stage MMAs of item i
//   softmax / dS math and the epilogues  - 128-thread groups, thread t = tile row t = TMEM lane t
// so that per-item latencies (global loads, MMA completion, TMEM reads) are hidden instead of summed, which
// is what dominates when a sentence has only 20..100 tokens.
//
// forward : two softmax groups alternate items (TMEM: S0 S1 | O0 O1), three Q/K/V slots.
// backward: 256 math threads (query row x half of the key columns) on one item, a warpgroup that prepares D / log-sum-exp
//           of the next item and writes dQ, dK, dV of the previous one; TMEM holds two sets (S dP, reused for dV dQ dK),
//           two Q/K/V/dO slots; P and dS are staged once in shared memory and consumed K-major (dQ = dS K) and MN-major
//           (dV = P^T dO, dK = dS^T Q).
// MMA reduction lengths are trimmed to the real sequence lengths (multiples of 16).
// Same numerics, dropout counters and interfaces as the general kernels in attention_tcgen05.cu.
#include "attention_common.cuh"
#include "bounds_check.cuh"

namespace b200 {

int num_sms();

struct Item {
  int q0 = 0, q_len = 0, k0 = 0, k_len = 0, h = 0;
  bool valid = false;
};

__device__ __forceinline__ Item get_item(const AttnArgs& p, int item) {
  Item it;
  const int b = item / p.num_heads;
  it.h = item - b * p.num_heads;
  it.q0 = p.cu_q[b];
  it.q_len = p.cu_q[b + 1] - it.q0;
  it.k0 = p.cu_k[b];
  it.k_len = p.cu_k[b + 1] - it.k0;
  it.valid = it.q_len > 0 && it.k_len > 0 && it.q_len <= kTile && it.k_len <= kTile;
  // a sequence that does not fit one tile (or offsets that run backwards) is skipped by every role of the kernel; the host
  // dispatch sends such batches to the general kernels, so meeting one here means the offsets are wrong
  if (!it.valid && (it.q_len < 0 || it.k_len < 0 || it.q_len > kTile || it.k_len > kTile) && threadIdx.x == 0) NMTG_BOUNDS_HIT();
  return it;
}

// ---------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------
constexpr int kFwdSlots = 3;
constexpr int kFwdSlotBytes = 3 * kTileBytes;
constexpr int kFwdShortThreads = 320;   // warps 0-3 / 4-7: softmax groups, warp 8: TMA producer, warp 9: MMA issuer
constexpr int kFwdShortSmem = kFwdSlots * kFwdSlotBytes + 2 * kPBytes + 256 + 1024;

__global__ void __launch_bounds__(kFwdShortThreads, 1)
attn_fwd_short_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const AttnArgs p, const int num_items) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sSlots = smem;
  uint8_t* sP = smem + kFwdSlots * kFwdSlotBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kPBytes);
  uint64_t* slot_full = bars;
  uint64_t* slot_empty = bars + 3;
  uint64_t* s_full = bars + 6;
  uint64_t* s_empty = bars + 8;
  uint64_t* p_full = bars + 10;
  uint64_t* o_full = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  zero_tail_fwd(p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 3; ++i) { mbar_init(&slot_full[i], 1); mbar_init(&slot_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 128);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_full[i], 1);
    }
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 9) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    if (lane == 0) {
      int it = 0;
      for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
        const Item w = get_item(p, item);
        if (!w.valid) continue;
        const int slot = it % kFwdSlots;
        if (!mbar_wait(&slot_empty[slot], ((it / kFwdSlots) & 1) ^ 1, abort_word, p.status, kTimeoutSmemEmpty)) break;
        uint8_t* s = sSlots + slot * kFwdSlotBytes;
        mbar_expect_tx(&slot_full[slot], kFwdSlotBytes);
        tma_load_2d(s, &tmap_q, &slot_full[slot], w.h * kHd, w.q0);
        tma_load_2d(s + kTileBytes, &tmap_k, &slot_full[slot], w.h * kHd, w.k0);
        tma_load_2d(s + 2 * kTileBytes, &tmap_v, &slot_full[slot], w.h * kHd, w.k0);
        ++it;
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(kTile, kHd, 0, 1);
      int it = 0;
      bool have_prev = false, ok = true;
      int prev_it = 0, prev_klen = 0;
      auto issue_pv = [&](int j, int k_len) -> bool {
        const int g = j & 1, slot = j % kFwdSlots;
        if (!mbar_wait(&p_full[g], (j >> 1) & 1, abort_word, p.status, kTimeoutTmemEmpty)) return false;
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(sP + g * kPBytes);
        const uint32_t va = smem_u32(sSlots + slot * kFwdSlotBytes + 2 * kTileBytes);
        const uint32_t tO = tmem_base + 256 + g * kHd;
        const int nk = (k_len + 15) >> 4;
        for (int k = 0; k < nk; ++k) {
          const uint64_t ad = make_smem_desc_sw128(pa + (k >> 2) * kTileBytes + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(va + k * 2048, 8192, 1024);
          umma_bf16(tO, ad, bd, idesc_o, k > 0 ? 1u : 0u);
        }
        umma_commit(&o_full[g]);
        umma_commit(&slot_empty[slot]);
        return true;
      };
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const Item w = get_item(p, item);
        if (!w.valid) continue;
        const int slot = it % kFwdSlots, g = it & 1;
        if (!mbar_wait(&slot_full[slot], (it / kFwdSlots) & 1, abort_word, p.status, kTimeoutTmaFull)) { ok = false; break; }
        if (!mbar_wait(&s_empty[g], ((it >> 1) & 1) ^ 1, abort_word, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(sSlots + slot * kFwdSlotBytes);
        umma_steps(tmem_base + g * kTile, qa, 16, 32, qa + kTileBytes, 16, 32, idesc_s, kHd / 16, false);
        umma_commit(&s_full[g]);
        if (have_prev) ok = issue_pv(prev_it, prev_klen);
        have_prev = true;
        prev_it = it;
        prev_klen = w.k_len;
        ++it;
      }
      if (ok && have_prev) issue_pv(prev_it, prev_klen);
    }
  } else if (warp < 8) {
    const int g = warp >> 2;
    const int t = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + g * kTile, tO = tmem_base + 256 + g * kHd;
    uint8_t* myP = sP + g * kPBytes;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const bool do_drop = p.dropout_p > 0.f;
    const unsigned long long seed = p.seed + ((do_drop && p.seed_dev) ? *p.seed_dev : 0ull);
    int it = 0;
    int item = blockIdx.x;
    Item nxt = item < num_items ? get_item(p, item) : Item{};
    while (item < num_items) {
      const Item w = nxt;
      item += gridDim.x;
      if (item < num_items) nxt = get_item(p, item);   // loads for the next item overlap this item's work
      if (!w.valid) continue;
      const int my = ((it & 1) == g);
      const uint32_t ph = (it >> 1) & 1;
      ++it;
      if (!my) continue;
      if (!mbar_wait(&s_full[g], ph, abort_word, p.status, kTimeoutTmemFull)) break;
      tc_fence_after_sync();
      const bool warp_active = (warp & 3) * 32 < w.q_len;
      const int nchunks = (w.k_len + 31) >> 5;
      float row_sum = 0.f, row_max = kNegBig;
      if (warp_active) {
        const DropRng rng(seed, (p.stream_id << 16) | static_cast<unsigned long long>(w.h), p.dropout_p);
        // two column chunks (64 scores) per round: both TMEM loads are in flight before the single wait
#pragma unroll 1
        for (int c0 = 0; c0 < nchunks; c0 += 2) {
          uint32_t r0[32], r1[32];
          tmem_ld32(tS + lane_sel + c0 * 32, r0);
          if (c0 + 1 < nchunks) tmem_ld32(tS + lane_sel + (c0 + 1) * 32, r1);
          tmem_ld_wait();
          // raw-score maximum (scale > 0: scaling commutes with the maximum); a chunk whose 32 key columns all exist
          // (and no causal mask) needs no per-element test
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int c = c0 + half;
            if (c >= nchunks) break;
            if (!p.causal && (c + 1) * 32 <= w.k_len) {
              float m0 = kNegBig, m1 = kNegBig, m2 = kNegBig, m3 = kNegBig;
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                m0 = fmaxf(m0, __uint_as_float(half == 0 ? r0[j] : r1[j]));
                m1 = fmaxf(m1, __uint_as_float(half == 0 ? r0[j + 1] : r1[j + 1]));
                m2 = fmaxf(m2, __uint_as_float(half == 0 ? r0[j + 2] : r1[j + 2]));
                m3 = fmaxf(m3, __uint_as_float(half == 0 ? r0[j + 3] : r1[j + 3]));
              }
              row_max = fmaxf(row_max, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = c * 32 + j;
                const bool valid = col < w.k_len && (!p.causal || col <= t);
                row_max = fmaxf(row_max, valid ? __uint_as_float(half == 0 ? r0[j] : r1[j]) : kNegBig);
              }
            }
          }
        }
        row_max *= scale_log2;         // from here on in the base-2 domain: P = 2^(S * scale * log2 e - row_max)
#pragma unroll 1
        for (int c0 = 0; c0 < nchunks; c0 += 2) {
          uint32_t r0[32], r1[32];
          tmem_ld32(tS + lane_sel + c0 * 32, r0);
          if (c0 + 1 < nchunks) tmem_ld32(tS + lane_sel + (c0 + 1) * 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int c = c0 + half;
            if (c >= nchunks) break;
            float pv[32];
            if (!p.causal && (c + 1) * 32 <= w.k_len) {
              float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                pv[j] = ex2_approx(fmaf(__uint_as_float(half == 0 ? r0[j] : r1[j]), scale_log2, -row_max));
                pv[j + 1] = ex2_approx(fmaf(__uint_as_float(half == 0 ? r0[j + 1] : r1[j + 1]), scale_log2, -row_max));
                pv[j + 2] = ex2_approx(fmaf(__uint_as_float(half == 0 ? r0[j + 2] : r1[j + 2]), scale_log2, -row_max));
                pv[j + 3] = ex2_approx(fmaf(__uint_as_float(half == 0 ? r0[j + 3] : r1[j + 3]), scale_log2, -row_max));
                s0 += pv[j];
                s1 += pv[j + 1];
                s2 += pv[j + 2];
                s3 += pv[j + 3];
              }
              row_sum += (s0 + s1) + (s2 + s3);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = c * 32 + j;
                const bool valid = col < w.k_len && (!p.causal || col <= t);
                const float sv = __uint_as_float(half == 0 ? r0[j] : r1[j]);
                const float e = valid ? ex2_approx(fmaf(sv, scale_log2, -row_max)) : 0.f;
                row_sum += e;
                pv[j] = e;
              }
            }
            if (do_drop) apply_dropout32(rng, static_cast<unsigned long long>(w.q0 + t) * p.kstride + c * 32, pv);
#pragma unroll
            for (int g4 = 0; g4 < 4; ++g4) {
              uint4 o;
              __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(pv[g4 * 8 + 2 * j], pv[g4 * 8 + 2 * j + 1]);
              const int chunk = c * 4 + g4;
              *reinterpret_cast<uint4*>(myP + (chunk >> 3) * kTileBytes + sw128_offset(t, chunk & 7)) = o;
            }
          }
        }
      }
      tc_fence_before_sync();
      fence_async_smem();
      mbar_arrive(&p_full[g]);
      mbar_arrive(&s_empty[g]);
      if (!mbar_wait(&o_full[g], ph, abort_word, p.status, kTimeoutTmemFull)) break;
      tc_fence_after_sync();
      if (warp_active) {
        const float inv = row_sum > 0.f ? 1.f / row_sum : 0.f;
        __nv_bfloat16* orow = p.out + static_cast<size_t>(w.q0 + t) * p.ld_out + w.h * kHd;
        uint32_t r0[32], r1[32];
        tmem_ld32(tO + lane_sel, r0);
        tmem_ld32(tO + lane_sel + 32, r1);
        tmem_ld_wait();
        if (t < w.q_len) {
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int e = (g4 & 3) * 8 + 2 * j;
              const float a = __uint_as_float(g4 < 4 ? r0[e] : r1[e]), b = __uint_as_float(g4 < 4 ? r0[e + 1] : r1[e + 1]);
              o2[j] = __floats2bfloat162_rn(a * inv, b * inv);
            }
            reinterpret_cast<uint4*>(orow)[g4] = o;
          }
          if (p.lse) p.lse[static_cast<size_t>(w.h) * p.lse_stride + w.q0 + t] = row_sum > 0.f ? (row_max + __log2f(row_sum)) * 0.6931471805599453f : 0.f;
        }
      }
      tc_fence_before_sync();
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

// ---------------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------------
// Roles (448 threads):
//   warps 0-3 / 4-7   math: thread = (query row, half); half h owns key columns [32 c + 16 h, 32 c + 16 h + 16) of every
//                     32-column chunk c, so all 256 threads work on the SAME item and each holds few values at a time
//                     (the math is issue-bound: with one warp per scheduler and most registers tied up in TMEM chunks the
//                     compiler could not interleave independent elements, which is what made the one-group version slow)
//   warps 8-11        D = rowsum(dO * O) and the log-sum-exp of item i+1 into shared memory, then dQ / dK / dV of item i-1
//   warp 12           TMA producer          warp 13   MMA issuer
// TMEM holds two sets of 256 columns, set = item & 1:
//   columns   0..127  S  = Q K^T          later  dV (0..63) and dQ (64..127)
//   columns 128..255  dP = dO V^T         later  dK (128..191)
// so the S / dP MMAs of item i+1 run while the gradients of item i-1 are still being read out of the other set.
// P and dS are staged in ONE pair of shared-memory tiles; the math threads wait for the gradient MMAs of the previous
// item (pds_free) only right before their first store, after the exponentials of the new item are done.
constexpr int kBwdSlots = 2;
constexpr int kBwdSlotBytes = 4 * kTileBytes;   // Q, K, V, dO
constexpr int kBwdShortThreads = 448;
constexpr int kBwdRowBytes = 2 * 2 * kTile * 4; // D and log-sum-exp of two items in flight
constexpr int kBwdShortSmem = kBwdSlots * kBwdSlotBytes + 2 * kPBytes + kBwdRowBytes + 256 + 1024;
constexpr uint32_t kBwdIssuePolls = 1u << 22;   // polls of the MMA warp without progress before it gives up

// One gradient row (64 fp32 accumulator columns of this thread's TMEM lane) scaled, packed to bf16 and stored.
__device__ __forceinline__ void bwd_store_row(uint32_t taddr, __nv_bfloat16* drow, float osc, bool store) {
  uint32_t r0[32], r1[32];
  tmem_ld32(taddr, r0);
  tmem_ld32(taddr + 32, r1);
  tmem_ld_wait();
  if (store) {
#pragma unroll
    for (int g4 = 0; g4 < 8; ++g4) {
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = (g4 & 3) * 8 + 2 * j;
        o2[j] = __floats2bfloat162_rn(__uint_as_float(g4 < 4 ? r0[e] : r1[e]) * osc, __uint_as_float(g4 < 4 ? r0[e + 1] : r1[e + 1]) * osc);
      }
      reinterpret_cast<uint4*>(drow)[g4] = o;
    }
  }
}

__global__ void __launch_bounds__(kBwdShortThreads, 1)
attn_bwd_short_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                      const AttnArgs p, const int num_items, const int ablate) {
  // `ablate` (0 in production) switches parts of the work off while keeping every barrier hand-shake, so that a timing run
  // can tell which role bounds the item rate (results are then meaningless):
  //   1 no P / dS math   2 no gradient read-out   4 no gradient MMAs   8 no S / dP MMAs   16 no TMA loads
  //   32 no D / log-sum-exp loads   64 no dropout masks
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sSlots = smem;
  uint8_t* sP = smem + kBwdSlots * kBwdSlotBytes;
  uint8_t* sDS = sP + kPBytes;
  float* sD = reinterpret_cast<float*>(sDS + kPBytes);   // [2][128] rowsum(dO * O) of the items in flight
  float* sL = sD + 2 * kTile;                            // [2][128] log-sum-exp * log2 e (+inf for rows past the sequence)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + kPBytes + kBwdRowBytes);
  uint64_t* slot_full = bars;        // [2] TMA -> MMA
  uint64_t* slot_empty = bars + 2;   // [2] gradient MMAs done -> TMA
  uint64_t* sdp_full = bars + 4;     // [2] S / dP ready -> math group
  uint64_t* set_free = bars + 6;     // [2] gradients read out -> MMA may overwrite the set
  uint64_t* grads_full = bars + 8;   // [2] gradient MMAs done -> epilogue group
  uint64_t* pds_full = bars + 10;    // P / dS staged -> MMA
  uint64_t* pds_free = bars + 11;    // gradient MMAs done -> math threads may overwrite P / dS
  uint64_t* d_full = bars + 12;      // [2] D / log-sum-exp rows written -> math threads
  uint64_t* d_free = bars + 14;      // [2] rows read -> may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  zero_tail_bwd(p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&slot_full[i], 1);
      mbar_init(&slot_empty[i], 1);
      mbar_init(&sdp_full[i], 1);
      mbar_init(&set_free[i], 128);
      mbar_init(&grads_full[i], 1);
      mbar_init(&d_full[i], 128);
      mbar_init(&d_free[i], 256);
    }
    mbar_init(pds_full, 256);
    mbar_init(pds_free, 1);
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 13) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 12) {
    if (lane == 0) {
      int it = 0;
      for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
        const Item w = get_item(p, item);
        if (!w.valid) continue;
        const int slot = it & 1;
        if (!mbar_wait(&slot_empty[slot], ((it >> 1) & 1) ^ 1, abort_word, p.status, kTimeoutSmemEmpty)) break;
        uint8_t* s = sSlots + slot * kBwdSlotBytes;
        if (ablate & 16) {
          mbar_arrive(&slot_full[slot]);
          ++it;
          continue;
        }
        mbar_expect_tx(&slot_full[slot], kBwdSlotBytes);
        tma_load_2d(s, &tmap_q, &slot_full[slot], w.h * kHd, w.q0);
        tma_load_2d(s + kTileBytes, &tmap_k, &slot_full[slot], w.h * kHd, w.k0);
        tma_load_2d(s + 3 * kTileBytes, &tmap_do, &slot_full[slot], w.h * kHd, w.q0);
        tma_load_2d(s + 2 * kTileBytes, &tmap_v, &slot_full[slot], w.h * kHd, w.k0);
        ++it;
      }
    }
  } else if (warp == 13) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_dq = make_idesc_bf16(kTile, kHd, 0, 1);
      const uint32_t idesc_dkv = make_idesc_bf16(kTile, kHd, 1, 1);
      // Two queues served in whichever order their inputs arrive: S / dP of item s_it (needs its tiles and a free TMEM
      // set) and the gradients of item g_it (needs P / dS).  Blocking on one would hold back the other: the tiles of item
      // i + 1 land about a TMA round trip after the gradients of item i - 1 completed.
      int s_it = 0, g_it = 0;
      unsigned long long lens = 0;   // (q_len, k_len) bytes of items g_it .. s_it (at most three alive), 16 bits per item
      int item = blockIdx.x;
      auto next_valid = [&]() {
        while (item < num_items) {
          const Item w = get_item(p, item);
          if (w.valid) {
            const int sh = (s_it & 3) * 16;
            lens = (lens & ~(0xFFFFull << sh)) | (static_cast<unsigned long long>((w.q_len << 8) | w.k_len) << sh);
            return true;
          }
          item += gridDim.x;
        }
        return false;
      };
      bool more = next_valid();
      uint32_t idle = 0;
      while (more || g_it < s_it) {
        bool progressed = false;
        if (g_it < s_it && mbar_test_wait(pds_full, g_it & 1)) {
          tc_fence_after_sync();
          const int s = g_it & 1;
          const uint32_t set = tmem_base + s * 256;
          const uint32_t base = smem_u32(sSlots + s * kBwdSlotBytes);
          const uint32_t qa = base, ka = base + kTileBytes, doa = base + 3 * kTileBytes;
          const uint32_t pa = smem_u32(sP), dsa = smem_u32(sDS);
          const uint32_t lw = static_cast<uint32_t>(lens >> ((g_it & 3) * 16)) & 0xFFFFu;
          const int nkq = ((lw >> 8) + 15) >> 4, nkk = ((lw & 0xFFu) + 15) >> 4;
          // dV = P^T dO, dK = dS^T Q : A read MN-major (keys = M, two 64-key slabs), reduction over query rows
          if (!(ablate & 4)) {
            umma_steps(set, pa, kTileBytes, 2048, doa, 8192, 2048, idesc_dkv, nkq, false);
            umma_steps(set + 128, dsa, kTileBytes, 2048, qa, 8192, 2048, idesc_dkv, nkq, false);
          }
          // dQ = dS K : A K-major (slab per 64 keys), B = K tile MN-major, reduction over keys
          for (int k = 0; k < ((ablate & 4) ? 0 : nkk); ++k) {
            const uint64_t ad = make_smem_desc_sw128(dsa + (k >> 2) * kTileBytes + (k & 3) * 32, 16, 1024);
            const uint64_t bd = make_smem_desc_sw128(ka + k * 2048, 8192, 1024);
            umma_bf16(set + 64, ad, bd, idesc_dq, k > 0 ? 1u : 0u);
          }
          umma_commit(pds_free);
          umma_commit(&grads_full[s]);
          umma_commit(&slot_empty[s]);
          ++g_it;
          progressed = true;
        }
        if (more && s_it - g_it < 2 && mbar_test_wait(&slot_full[s_it & 1], (s_it >> 1) & 1) &&
            mbar_test_wait(&set_free[s_it & 1], ((s_it >> 1) & 1) ^ 1)) {
          tc_fence_after_sync();
          const int s = s_it & 1;
          const uint32_t set = tmem_base + s * 256;
          const uint32_t base = smem_u32(sSlots + s * kBwdSlotBytes);
          if (!(ablate & 8)) {
            umma_steps(set, base, 16, 32, base + kTileBytes, 16, 32, idesc_s, kHd / 16, false);                              // Q K^T
            umma_steps(set + 128, base + 3 * kTileBytes, 16, 32, base + 2 * kTileBytes, 16, 32, idesc_s, kHd / 16, false);   // dO V^T
          }
          umma_commit(&sdp_full[s]);
          ++s_it;
          item += gridDim.x;
          more = next_valid();
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else {
          if (++idle > 4096) {        // a few microseconds of plain polling first: a sleep here delays every waiter
            if (*abort_word) break;
            if (idle > kBwdIssuePolls) {
              *abort_word = 1;
              if (p.status) atomicCAS(p.status, 0, static_cast<int>(kTimeoutTmemEmpty));
              break;
            }
            __nanosleep(idle > 65536 ? 256 : 32);
          }
        }
      }
    }
  } else if (warp < 8) {
    // ---- math threads: P and dS of every item, 16 of every 32 key columns each ---------------------------------------
    const int half = warp >> 2;
    const int t = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const bool do_drop = p.dropout_p > 0.f && !(ablate & 64);
    const unsigned long long seed = p.seed + ((do_drop && p.seed_dev) ? *p.seed_dev : 0ull);
    int it = 0;
    int item = blockIdx.x;
    Item nxt = item < num_items ? get_item(p, item) : Item{};
    while (item < num_items) {
      const Item w = nxt;
      item += gridDim.x;
      if (item < num_items) nxt = get_item(p, item);   // the next item's descriptor is fetched under this item's work
      if (!w.valid) continue;
      const int s = it & 1;
      const uint32_t set = tmem_base + s * 256 + lane_sel + half * 16;
      if (!__all_sync(0xffffffffu, mbar_wait(&d_full[s], (it >> 1) & 1, abort_word, p.status, kTimeoutTmemFull))) break;
      const float Drow = sD[s * kTile + t], lse2 = sL[s * kTile + t];
      mbar_arrive(&d_free[s]);
      if (!__all_sync(0xffffffffu, mbar_wait(&sdp_full[s], (it >> 1) & 1, abort_word, p.status, kTimeoutTmemFull))) break;
      tc_fence_after_sync();
      const int nchunks = (w.k_len + 31) >> 5;
      const int q_rows16 = ((w.q_len + 15) >> 4) << 4;   // rows the MN-major MMAs will read
      const bool warp_writes = (warp & 3) * 32 < q_rows16 && !(ablate & 1);
      bool may_store = it == 0, ok = true;
      if (warp_writes) {
        const DropRng rng(seed, (p.stream_id << 16) | static_cast<unsigned long long>(w.h), p.dropout_p);
        const unsigned long long row_base = static_cast<unsigned long long>(w.q0 + t) * p.kstride + half * 16;
        // two chunks (2 x 16 columns of this thread) per round: four TMEM loads in flight before the single wait
#pragma unroll 1
        for (int c = 0; c < nchunks; c += 2) {
          const bool two = c + 1 < nchunks;
          uint32_t s0[16], d0[16], s1[16], d1[16];
          tmem_ld16(set + c * 32, s0);
          tmem_ld16(set + 128 + c * 32, d0);
          if (two) {
            tmem_ld16(set + (c + 1) * 32, s1);
            tmem_ld16(set + 128 + (c + 1) * 32, d1);
          }
          uint32_t km0 = 0xffffu, km1 = 0xffffu;
          if (do_drop) {   // the mask words are hashed while the TMEM loads are in flight
            km0 = drop_mask16(rng, row_base + c * 32);
            if (two) km1 = drop_mask16(rng, row_base + (c + 1) * 32);
          }
          tmem_ld_wait();
          // all of the arithmetic comes before the wait for the staging tiles: it overlaps the previous item's gradient MMAs
          uint4 p0[2], e0[2], p1[2], e1[2];
          bwd_compute16(s0, d0, km0, do_drop, rng.scale, Drow, scale_log2, lse2, c * 32 + half * 16, w.k_len, p.causal != 0,
                        c * 32 + half * 16, t, p0, e0);
          if (two)
            bwd_compute16(s1, d1, km1, do_drop, rng.scale, Drow, scale_log2, lse2, (c + 1) * 32 + half * 16, w.k_len,
                          p.causal != 0, (c + 1) * 32 + half * 16, t, p1, e1);
          if (!may_store) {   // the gradient MMAs of the previous item still read the staging tiles
            ok = __all_sync(0xffffffffu, mbar_wait(pds_free, (it - 1) & 1, abort_word, p.status, kTimeoutSmemEmpty));
            if (!ok) break;
            may_store = true;
          }
          bwd_store16(p0, e0, c * 32 + half * 16, t, sP, sDS);
          if (two) bwd_store16(p1, e1, (c + 1) * 32 + half * 16, t, sP, sDS);
        }
      }
      if (ok && !may_store) {
        // No thread may run ahead: S / dP and the D rows are double-buffered, so without this wait a thread with nothing to
        // write could reach its arrival for the NEXT item while the others still write this one, and complete the phase
        // early.  pds_free(it - 1) implies that phase it - 1 of pds_full is complete.
        ok = __all_sync(0xffffffffu, mbar_wait(pds_free, (it - 1) & 1, abort_word, p.status, kTimeoutSmemEmpty));
      }
      if (!ok) break;
      tc_fence_before_sync();
      fence_async_smem();
      mbar_arrive(pds_full);
      ++it;
    }
  } else if (warp < 12) {
    // ---- D / log-sum-exp rows of item i, then dQ row t (queries) and dK / dV row t (keys) of item i - 1 --------------
    const int wq = warp - 8;
    const int t = wq * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(wq * 32) << 16;
    const float kInf = __int_as_float(0x7f800000);
    int it = 0;
    int item = blockIdx.x;
    Item nxt = item < num_items ? get_item(p, item) : Item{};
    Item prev{};
    bool ok = true;
    auto read_out = [&](const Item& w, int j) -> bool {
      const int s = j & 1;
      const uint32_t set = tmem_base + s * 256 + lane_sel;
      if (!__all_sync(0xffffffffu, mbar_wait(&grads_full[s], (j >> 1) & 1, abort_word, p.status, kTimeoutTmemFull))) return false;
      tc_fence_after_sync();
      if (!(ablate & 2)) {
        const size_t col = static_cast<size_t>(w.h) * kHd;
        if (wq * 32 < w.q_len)
          bwd_store_row(set + 64, p.dq + static_cast<size_t>(w.q0 + t) * p.ld_dq + col, p.scale, t < w.q_len);
        if (wq * 32 < w.k_len) {
          // dK carries the softmax scale that dS left out
          bwd_store_row(set + 128, p.dk + static_cast<size_t>(w.k0 + t) * p.ld_dk + col, p.scale, t < w.k_len);
          bwd_store_row(set, p.dv + static_cast<size_t>(w.k0 + t) * p.ld_dv + col, 1.f, t < w.k_len);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&set_free[s]);
      return true;
    };
    while (item < num_items && ok) {
      const Item w = nxt;
      item += gridDim.x;
      if (item < num_items) {
        nxt = get_item(p, item);
        if (nxt.valid && t < nxt.q_len) {   // the rows this thread reads in the next iteration, on their way to L2 now
          prefetch_l2(p.o + static_cast<size_t>(nxt.q0 + t) * p.ld_o + nxt.h * kHd);
          prefetch_l2(p.d_o + static_cast<size_t>(nxt.q0 + t) * p.ld_do + nxt.h * kHd);
        }
      }
      if (!w.valid) continue;
      const int s = it & 1;
      float Drow = 0.f, lse2 = kInf;
      if (t < w.q_len && !(ablate & 32)) {
        const uint4* orow = reinterpret_cast<const uint4*>(p.o + static_cast<size_t>(w.q0 + t) * p.ld_o + w.h * kHd);
        const uint4* drow = reinterpret_cast<const uint4*>(p.d_o + static_cast<size_t>(w.q0 + t) * p.ld_do + w.h * kHd);
        uint4 a[8], d[8];
#pragma unroll
        for (int g4 = 0; g4 < 8; ++g4) { a[g4] = orow[g4]; d[g4] = drow[g4]; }
        lse2 = p.lse[static_cast<size_t>(w.h) * p.lse_stride + w.q0 + t] * 1.4426950408889634f;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int g4 = 0; g4 < 8; ++g4) {
          const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a[g4]);
          const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d[g4]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 x = __bfloat1622float2(a2[j]), y = __bfloat1622float2(d2[j]);
            acc[j] = fmaf(x.x, y.x, fmaf(x.y, y.y, acc[j]));
          }
        }
        Drow = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      } else if (t < w.q_len) {
        lse2 = 0.f;
      }
      // the rows of item it - 2 have been read by every math thread
      if (!__all_sync(0xffffffffu, mbar_wait(&d_free[s], ((it >> 1) & 1) ^ 1, abort_word, p.status, kTimeoutSmemEmpty))) { ok = false; break; }
      sD[s * kTile + t] = Drow;
      sL[s * kTile + t] = lse2;
      mbar_arrive(&d_full[s]);
      if (it > 0) ok = read_out(prev, it - 1);
      prev = w;
      ++it;
    }
    if (ok && it > 0) read_out(prev, it - 1);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_word) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 13) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

static int g_attn_bwd_ablate = 0;
void set_attn_bwd_ablation(int bits) { g_attn_bwd_ablate = bits; }
int get_attn_bwd_ablation() { return g_attn_bwd_ablate; }

const char* launch_attn_fwd_short(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a,
                                  int num_items, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(attn_fwd_short_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdShortSmem);
    if (ce != cudaSuccess) return cudaGetErrorString(ce);
    configured = true;
  }
  const int grid = num_items < num_sms() ? num_items : num_sms();
  attn_fwd_short_kernel<<<grid, kFwdShortThreads, kFwdShortSmem, stream>>>(tq, tk, tv, a, num_items);
  cudaError_t ce = cudaGetLastError();
  return ce == cudaSuccess ? nullptr : cudaGetErrorString(ce);
}

const char* launch_attn_bwd_short(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                                  const AttnArgs& a, int num_items, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(attn_bwd_short_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdShortSmem);
    if (ce != cudaSuccess) return cudaGetErrorString(ce);
    configured = true;
  }
  const int grid = num_items < num_sms() ? num_items : num_sms();
  attn_bwd_short_kernel<<<grid, kBwdShortThreads, kBwdShortSmem, stream>>>(tq, tk, tv, tdo, a, num_items, g_attn_bwd_ablate);
  cudaError_t ce = cudaGetLastError();
  return ce == cudaSuccess ? nullptr : cudaGetErrorString(ce);
}

}  // namespace b200

NMTG_BOUNDS_READER(nmtg_bounds_attention_short)

void nmtg_set_attn_bwd_ablation(int bits) { b200::set_attn_bwd_ablation(bits); }
