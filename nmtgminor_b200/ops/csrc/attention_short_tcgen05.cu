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
// backward: one group (TMEM: S dP | dQ dK dV), two Q/K/V/dO slots; P and dS are staged once in shared
//           memory and consumed K-major (dQ = dS K) and MN-major (dV = P^T dO, dK = dS^T Q).
// MMA reduction lengths are trimmed to the real sequence lengths (multiples of 16).
// Same numerics, dropout counters and interfaces as the general kernels in attention_tcgen05.cu.
#include "attention_common.cuh"

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
constexpr int kBwdSlots = 2;
constexpr int kBwdSlotBytes = 4 * kTileBytes;   // Q, K, V, dO
constexpr int kBwdShortThreads = 192;   // warps 0-3: math group, warp 4: TMA producer, warp 5: MMA issuer
constexpr int kBwdShortSmem = kBwdSlots * kBwdSlotBytes + 2 * kPBytes + 256 + 1024;

__global__ void __launch_bounds__(kBwdShortThreads, 1)
attn_bwd_short_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                      const AttnArgs p, const int num_items) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sSlots = smem;
  uint8_t* sP = smem + kBwdSlots * kBwdSlotBytes;
  uint8_t* sDS = sP + kPBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + kPBytes);
  uint64_t* slot_full = bars;        // [2]
  uint64_t* slot_empty = bars + 2;   // [2]
  uint64_t* sdp_full = bars + 4;
  uint64_t* sdp_empty = bars + 5;
  uint64_t* pds_full = bars + 6;
  uint64_t* grads_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  zero_tail_bwd(p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&slot_full[i], 1); mbar_init(&slot_empty[i], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_empty, 128);
    mbar_init(pds_full, 128);
    mbar_init(grads_full, 1);
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 5) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDQ = tmem_base + 256, tDK = tmem_base + 320,
                 tDV = tmem_base + 384;

  if (warp == 4) {
    if (lane == 0) {
      int it = 0;
      for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
        const Item w = get_item(p, item);
        if (!w.valid) continue;
        const int slot = it & 1;
        if (!mbar_wait(&slot_empty[slot], ((it >> 1) & 1) ^ 1, abort_word, p.status, kTimeoutSmemEmpty)) break;
        uint8_t* s = sSlots + slot * kBwdSlotBytes;
        mbar_expect_tx(&slot_full[slot], kBwdSlotBytes);
        tma_load_2d(s, &tmap_q, &slot_full[slot], w.h * kHd, w.q0);
        tma_load_2d(s + kTileBytes, &tmap_k, &slot_full[slot], w.h * kHd, w.k0);
        tma_load_2d(s + 2 * kTileBytes, &tmap_v, &slot_full[slot], w.h * kHd, w.k0);
        tma_load_2d(s + 3 * kTileBytes, &tmap_do, &slot_full[slot], w.h * kHd, w.q0);
        ++it;
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_dq = make_idesc_bf16(kTile, kHd, 0, 1);
      const uint32_t idesc_dkv = make_idesc_bf16(kTile, kHd, 1, 1);
      int it = 0;
      bool have_prev = false, ok = true;
      int prev_it = 0, prev_q = 0, prev_k = 0;
      auto issue_grads = [&](int j, int q_len, int k_len) -> bool {
        const int slot = j & 1;
        if (!mbar_wait(pds_full, j & 1, abort_word, p.status, kTimeoutTmemEmpty)) return false;
        tc_fence_after_sync();
        const uint32_t base = smem_u32(sSlots + slot * kBwdSlotBytes);
        const uint32_t qa = base, ka = base + kTileBytes, doa = base + 3 * kTileBytes;
        const uint32_t pa = smem_u32(sP), dsa = smem_u32(sDS);
        const int nkq = (q_len + 15) >> 4, nkk = (k_len + 15) >> 4;
        // dV = P^T dO, dK = dS^T Q : A read MN-major (keys = M, two 64-key slabs), reduction over query rows
        umma_steps(tDV, pa, kTileBytes, 2048, doa, 8192, 2048, idesc_dkv, nkq, false);
        umma_steps(tDK, dsa, kTileBytes, 2048, qa, 8192, 2048, idesc_dkv, nkq, false);
        // dQ = dS K : A K-major (slab per 64 keys), B = K tile MN-major, reduction over keys
        for (int k = 0; k < nkk; ++k) {
          const uint64_t ad = make_smem_desc_sw128(dsa + (k >> 2) * kTileBytes + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(ka + k * 2048, 8192, 1024);
          umma_bf16(tDQ, ad, bd, idesc_dq, k > 0 ? 1u : 0u);
        }
        umma_commit(grads_full);
        umma_commit(&slot_empty[slot]);
        return true;
      };
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const Item w = get_item(p, item);
        if (!w.valid) continue;
        const int slot = it & 1;
        if (!mbar_wait(&slot_full[slot], (it >> 1) & 1, abort_word, p.status, kTimeoutTmaFull)) { ok = false; break; }
        if (!mbar_wait(sdp_empty, (it & 1) ^ 1, abort_word, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t base = smem_u32(sSlots + slot * kBwdSlotBytes);
        umma_steps(tS, base, 16, 32, base + kTileBytes, 16, 32, idesc_s, kHd / 16, false);                       // Q K^T
        umma_steps(tDP, base + 3 * kTileBytes, 16, 32, base + 2 * kTileBytes, 16, 32, idesc_s, kHd / 16, false);  // dO V^T
        umma_commit(sdp_full);
        if (have_prev) ok = issue_grads(prev_it, prev_q, prev_k);
        have_prev = true;
        prev_it = it;
        prev_q = w.q_len;
        prev_k = w.k_len;
        ++it;
      }
      if (ok && have_prev) issue_grads(prev_it, prev_q, prev_k);
    }
  } else if (warp < 4) {
    const int t = warp * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const bool do_drop = p.dropout_p > 0.f;
    const unsigned long long seed = p.seed + ((do_drop && p.seed_dev) ? *p.seed_dev : 0ull);
    int it = 0;
    int item = blockIdx.x;
    Item nxt = item < num_items ? get_item(p, item) : Item{};
    while (item < num_items) {
      const Item w = nxt;
      item += gridDim.x;
      if (item < num_items) nxt = get_item(p, item);
      if (!w.valid) continue;
      const uint32_t ph = it & 1;
      ++it;
      const bool row_ok = t < w.q_len;
      float Drow = 0.f, lse = 0.f;
      if (row_ok) {   // overlaps the S / dP MMAs
        const uint4* orow = reinterpret_cast<const uint4*>(p.o + static_cast<size_t>(w.q0 + t) * p.ld_o + w.h * kHd);
        const uint4* drow = reinterpret_cast<const uint4*>(p.d_o + static_cast<size_t>(w.q0 + t) * p.ld_do + w.h * kHd);
        uint4 a[8], d[8];
#pragma unroll
        for (int g4 = 0; g4 < 8; ++g4) { a[g4] = orow[g4]; d[g4] = drow[g4]; }
        lse = p.lse[static_cast<size_t>(w.h) * p.lse_stride + w.q0 + t];
#pragma unroll
        for (int g4 = 0; g4 < 8; ++g4) {
          const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a[g4]);
          const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d[g4]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 x = __bfloat1622float2(a2[j]), y = __bfloat1622float2(d2[j]);
            Drow += x.x * y.x + x.y * y.y;
          }
        }
      }
      const float lse2 = row_ok ? lse * 1.4426950408889634f : __int_as_float(0x7f800000);
      if (!mbar_wait(sdp_full, ph, abort_word, p.status, kTimeoutTmemFull)) break;
      tc_fence_after_sync();
      const int nchunks = (w.k_len + 31) >> 5;
      const int q_rows16 = ((w.q_len + 15) >> 4) << 4;   // rows the MN-major MMAs will read
      const bool warp_writes = warp * 32 < q_rows16;
      if (warp_writes) {
        const DropRng rng(seed, (p.stream_id << 16) | static_cast<unsigned long long>(w.h), p.dropout_p);
#pragma unroll 1
        for (int c0 = 0; c0 < nchunks; c0 += 2) {
          uint32_t rs0[32], rd0[32], rs1[32], rd1[32];
          tmem_ld32(tS + lane_sel + c0 * 32, rs0);
          tmem_ld32(tDP + lane_sel + c0 * 32, rd0);
          if (c0 + 1 < nchunks) {
            tmem_ld32(tS + lane_sel + (c0 + 1) * 32, rs1);
            tmem_ld32(tDP + lane_sel + (c0 + 1) * 32, rd1);
          }
          tmem_ld_wait();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int c = c0 + half;
            if (c >= nchunks) break;
            // P = 2^(S * scale * log2 e - lse * log2 e); a row past the sequence has lse2 = +inf, so its P is 0 without a
            // per-element test; dS is kept without the softmax scale (applied when dQ / dK leave TMEM).  A chunk whose 32
            // key columns all exist (and no causal mask) takes the branch without per-element masks.
            float pd[32], ds[32];
            const bool chunk_full = !p.causal && (c + 1) * 32 <= w.k_len;
            if (chunk_full && !do_drop) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float sv = __uint_as_float(half == 0 ? rs0[j] : rs1[j]);
                const float dv = __uint_as_float(half == 0 ? rd0[j] : rd1[j]);
                pd[j] = ex2_approx(fmaf(sv, scale_log2, -lse2));
                ds[j] = pd[j] * (dv - Drow);
              }
            } else {
              float kf[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) kf[j] = 1.f;
              if (do_drop) apply_dropout32(rng, static_cast<unsigned long long>(w.q0 + t) * p.kstride + c * 32, kf);
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int col = c * 32 + j;
                const bool valid = chunk_full || (col < w.k_len && (!p.causal || col <= t));
                const float sv = __uint_as_float(half == 0 ? rs0[j] : rs1[j]);
                const float dv = __uint_as_float(half == 0 ? rd0[j] : rd1[j]);
                const float pr = valid ? ex2_approx(fmaf(sv, scale_log2, -lse2)) : 0.f;
                pd[j] = pr * kf[j];
                ds[j] = pr * (dv * kf[j] - Drow);
              }
            }
#pragma unroll
            for (int g4 = 0; g4 < 4; ++g4) {
              uint4 o1, o2v;
              __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&o1);
              __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&o2v);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                a2[j] = __floats2bfloat162_rn(pd[g4 * 8 + 2 * j], pd[g4 * 8 + 2 * j + 1]);
                b2[j] = __floats2bfloat162_rn(ds[g4 * 8 + 2 * j], ds[g4 * 8 + 2 * j + 1]);
              }
              const int chunk = c * 4 + g4;
              const uint32_t off = (chunk >> 3) * kTileBytes + sw128_offset(t, chunk & 7);
              *reinterpret_cast<uint4*>(sP + off) = o1;
              *reinterpret_cast<uint4*>(sDS + off) = o2v;
            }
          }
        }
      }
      tc_fence_before_sync();
      fence_async_smem();
      mbar_arrive(pds_full);
      mbar_arrive(sdp_empty);
      if (!mbar_wait(grads_full, ph, abort_word, p.status, kTimeoutTmemFull)) break;
      tc_fence_after_sync();
      // dQ row t (queries), dK / dV row t (keys): all TMEM loads of a row are issued before one wait
      const bool q_warp = warp * 32 < w.q_len, k_warp = warp * 32 < w.k_len;
      if (q_warp) {
        uint32_t r0[32], r1[32];
        tmem_ld32(tDQ + lane_sel, r0);
        tmem_ld32(tDQ + lane_sel + 32, r1);
        tmem_ld_wait();
        if (row_ok) {
          __nv_bfloat16* drow = p.dq + static_cast<size_t>(w.q0 + t) * p.ld_dq + w.h * kHd;
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int e = (g4 & 3) * 8 + 2 * j;
              o2[j] = __floats2bfloat162_rn(__uint_as_float(g4 < 4 ? r0[e] : r1[e]) * p.scale, __uint_as_float(g4 < 4 ? r0[e + 1] : r1[e + 1]) * p.scale);
            }
            reinterpret_cast<uint4*>(drow)[g4] = o;
          }
        }
      }
      if (k_warp) {
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* dst = which == 0 ? p.dk : p.dv;
          const int ld = which == 0 ? p.ld_dk : p.ld_dv;
          const uint32_t tsrc = which == 0 ? tDK : tDV;
          const float osc = which == 0 ? p.scale : 1.f;      // dK carries the softmax scale that dS left out
          uint32_t r0[32], r1[32];
          tmem_ld32(tsrc + lane_sel, r0);
          tmem_ld32(tsrc + lane_sel + 32, r1);
          tmem_ld_wait();
          if (t < w.k_len) {
            __nv_bfloat16* drow = dst + static_cast<size_t>(w.k0 + t) * ld + w.h * kHd;
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
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

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
  attn_bwd_short_kernel<<<grid, kBwdShortThreads, kBwdShortSmem, stream>>>(tq, tk, tv, tdo, a, num_items);
  cudaError_t ce = cudaGetLastError();
  return ce == cudaSuccess ? nullptr : cudaGetErrorString(ce);
}

}  // namespace b200
