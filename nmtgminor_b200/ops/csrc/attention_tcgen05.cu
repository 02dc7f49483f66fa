// Variable-length (packed) multi-head attention for sm_100a, head_dim 64, forward and backward, on
// tcgen05 tensor cores with TMEM accumulators and TMA-fed 128-byte-swizzled shared-memory tiles.
//
// Sequences are packed along the token dimension and described by cumulative offsets (cu_seqlens), so
// key padding never exists; self-attention (optionally causal) and encoder-decoder attention (separate
// query / key offsets) use the same kernels.  One CTA = one (128-query tile, head, sequence) in forward
// and one (128-key tile, head, sequence) in backward.  Two warpgroups of 128 threads each: thread t of a
// warpgroup owns TMEM lane t = tile row t and half of that row's columns, so the softmax needs one
// shared-memory exchange of the row maximum per tile and no shuffles.
//
// forward:   S = Q K^T (UMMA, K-major x K-major) -> online softmax in registers -> P (bf16, swizzled
//            smem) -> O_tile = P V (UMMA, V consumed MN-major straight from its [keys, d] TMA tile).
// backward:  S, dP = dO V^T recomputed per query tile; dV += P^T dO, dK += dS^T Q accumulate in TMEM
//            over query tiles (A operands read MN-major from the same smem that holds P / dS);
//            dQ = dS K per tile (written directly when the sequence has a single key tile, else
//            accumulated in an fp32 buffer with vector red.add).
// Dropout on P is regenerated from its counters in backward; nothing but the row log-sum-exp is saved.
//
// Replaces the reference's cuBLAS-strided-batched + warp-softmax attention extensions
// (onmt/modules/extensions/multihead_attn/self_multihead_attn_cuda.cu:23-612, encdec_multihead_attn_
// bias_cuda.cu:22-612, softmax_apex.h) and its bundled FlashAttention-v1 mma.sync kernels
// (onmt/modules/extensions/flashattn/src/fmha_fprop_kernel_1xN.h, fmha_dgrad_kernel_1xN_loop.h).
#include "attention_common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------------
// 256 threads: two warpgroups own the same 128 query rows (TMEM lanes) and split the 128 score columns and the 64 output
// columns between them, so every scheduler has four warps (two CTAs per SM) to hide TMEM loads and exponentials behind.
template <bool kBias>
__global__ void __launch_bounds__(256, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTileBytes;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sP = sV + kTileBytes;
  float* sRed = reinterpret_cast<float*>(sP + kPBytes);        // [2][128]: row maxima / row sums of the two warpgroups
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRed + 2 * kTile);  // [0]=Q [1]=K [2]=MMA [3]=V
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  zero_tail_fwd(p);
  const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int q_begin = p.cu_q[b], q_end = p.cu_q[b + 1];
  const int k_begin = p.cu_k[b], k_len = p.cu_k[b + 1] - k_begin;
  const int q0 = q_begin + qt * kTile;
  if (q0 >= q_end) return;  // uniform for the CTA, before any barrier or TMEM use
  const int q_rows = min(kTile, q_end - q0);
  const int t = threadIdx.x & 127, warp = t >> 5, grp = threadIdx.x >> 7;
  const bool leader = threadIdx.x == 0;

  if (leader) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    mbar_init(&bars[3], 1);
    *abort_word = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 32) tmem_alloc(tmem_slot, 256);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;         // 128 columns
  const uint32_t tO = tmem_base + 128;   // 64 columns
  const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;

  if (leader) {
    mbar_expect_tx(&bars[0], kTileBytes);
    tma_load_2d(sQ, &tmap_q, &bars[0], h * kHd, q0);
  }
  const uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);
  const uint32_t idesc_o = make_idesc_bf16(kTile, kHd, 0, 1);

  float m_run = kNegBig, l_run = 0.f;          // running maximum in the base-2 domain, running sum of my 64 columns
  const float scale_log2 = p.scale * 1.4426950408889634f;
  // with an additive bias (kBias) the scores are brought into the base-2 domain, and the bias added, right after they are
  // read from TMEM, so the factor that the softmax below applies is 1
  const float sl2 = kBias ? 1.f : scale_log2;
  const float* bias_row = (kBias && t < q_rows)
      ? p.bias + static_cast<long>(b) * p.bias_sb + static_cast<long>(h) * p.bias_sh + static_cast<long>(qt * kTile + t) * p.bias_sq
      : nullptr;
  float o_acc[32];                             // my warpgroup's 32 of the 64 output columns
#pragma unroll
  for (int j = 0; j < 32; ++j) o_acc[j] = 0.f;

  const int q_pos = qt * kTile + t;  // position inside the sequence
  int num_kt = (k_len + kTile - 1) / kTile;
  if (p.causal) num_kt = min(num_kt, (qt * kTile + q_rows + kTile - 1) / kTile);
  const bool do_drop = p.dropout_p > 0.f;
  const DropRng rng(p.seed + ((do_drop && p.seed_dev) ? *p.seed_dev : 0ull),
                    (p.stream_id << 16) | static_cast<unsigned long long>(h), p.dropout_p);
  uint32_t ph_kv = 0, ph_mma = 0;
  bool ok = true;

  // The K tile of the next iteration is requested as soon as S = Q K^T of this one has been computed, the V tile as soon
  // as O = P V has: both loads run under the softmax of the tile in between.
  if (leader && num_kt > 0) {
    mbar_expect_tx(&bars[1], kTileBytes);
    tma_load_2d(sK, &tmap_k, &bars[1], h * kHd, k_begin);
    mbar_expect_tx(&bars[3], kTileBytes);
    tma_load_2d(sV, &tmap_v, &bars[3], h * kHd, k_begin);
  }
  for (int kt = 0; kt < num_kt && ok; ++kt) {
    if (leader) {
      if (kt == 0) ok = mbar_wait(&bars[0], 0, abort_word, p.status, kTimeoutTmaFull);
      if (ok) ok = mbar_wait(&bars[1], ph_kv, abort_word, p.status, kTimeoutTmaFull);
      if (ok) {
        tc_fence_after_sync();
        umma_steps(tS, smem_u32(sQ), 16, 32, smem_u32(sK), 16, 32, idesc_s, kHd / 16, false);
        umma_commit(&bars[2]);
      }
    }
    if (!mbar_wait(&bars[2], ph_mma, abort_word, p.status, kTimeoutTmemFull)) { ok = false; break; }
    ph_mma ^= 1;
    tc_fence_after_sync();
    if (leader && kt + 1 < num_kt) {       // the MMA that read sK has completed
      mbar_expect_tx(&bars[1], kTileBytes);
      tma_load_2d(sK, &tmap_k, &bars[1], h * kHd, k_begin + (kt + 1) * kTile);
    }

    // ---- softmax over this key tile: two passes over my 64 of the 128 score columns of my row ---------
    // Scores stay in the base-2 domain (score * scale * log2 e), so one FMA + one ex2 makes a probability.  A tile whose
    // 128 x 128 scores are all inside the sequence (and below the diagonal when causal) skips the per-element masks.
    const int kcols = min(kTile, k_len - kt * kTile);
    const bool full = kcols == kTile && (!p.causal || kt < qt);
    float tile_max = kNegBig;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int c = 2 * grp + cc;
      uint32_t r[32];
      tmem_ld32(tS + lane_sel + c * 32, r);
      tmem_ld_wait();
      if (kBias) add_bias32(r, bias_row ? bias_row + kt * kTile + c * 32 : nullptr, kcols - c * 32, scale_log2);
      if (full) {
        float m0 = __uint_as_float(r[0]), m1 = __uint_as_float(r[1]), m2 = __uint_as_float(r[2]), m3 = __uint_as_float(r[3]);
#pragma unroll
        for (int j = 4; j < 32; j += 4) {
          m0 = fmaxf(m0, __uint_as_float(r[j]));
          m1 = fmaxf(m1, __uint_as_float(r[j + 1]));
          m2 = fmaxf(m2, __uint_as_float(r[j + 2]));
          m3 = fmaxf(m3, __uint_as_float(r[j + 3]));
        }
        tile_max = fmaxf(tile_max, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = c * 32 + j;
          const bool valid = col < kcols && (!p.causal || kt * kTile + col <= q_pos);
          tile_max = fmaxf(tile_max, valid ? __uint_as_float(r[j]) : kNegBig);
        }
      }
    }
    sRed[grp * kTile + t] = tile_max;
    __syncthreads();                                            // the other warpgroup's half of the row maximum
    tile_max = fmaxf(tile_max, sRed[(grp ^ 1) * kTile + t]);
    const float m_new = fmaxf(m_run, tile_max * sl2);           // scale > 0: the maximum commutes with the scaling
    const float alpha = ex2_approx(m_run - m_new);
    float row_sum = 0.f;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int c = 2 * grp + cc;
      uint32_t r[32];
      tmem_ld32(tS + lane_sel + c * 32, r);
      tmem_ld_wait();
      if (kBias) add_bias32(r, bias_row ? bias_row + kt * kTile + c * 32 : nullptr, kcols - c * 32, scale_log2);
      float pv[32];
      if (full) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          pv[j] = ex2_approx(fmaf(__uint_as_float(r[j]), sl2, -m_new));
          pv[j + 1] = ex2_approx(fmaf(__uint_as_float(r[j + 1]), sl2, -m_new));
          pv[j + 2] = ex2_approx(fmaf(__uint_as_float(r[j + 2]), sl2, -m_new));
          pv[j + 3] = ex2_approx(fmaf(__uint_as_float(r[j + 3]), sl2, -m_new));
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
          const bool valid = col < kcols && (!p.causal || kt * kTile + col <= q_pos);
          const float e = valid ? ex2_approx(fmaf(__uint_as_float(r[j]), sl2, -m_new)) : 0.f;
          row_sum += e;
          pv[j] = e;
        }
      }
      if (do_drop) {
        const unsigned long long base = static_cast<unsigned long long>(q0 + t) * p.kstride + kt * kTile + c * 32;
        apply_dropout32(rng, base, pv);
      }
      // bf16, swizzled K-major slabs of 64 keys
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(pv[g * 8 + 2 * j], pv[g * 8 + 2 * j + 1]);
        const int chunk = c * 4 + g;  // 16-byte chunk index along the 128 keys
        *reinterpret_cast<uint4*>(sP + (chunk >> 3) * kTileBytes + sw128_offset(t, chunk & 7)) = o;
      }
    }
    l_run = l_run * alpha + row_sum;
    m_run = m_new;
    tc_fence_before_sync();
    fence_async_smem();
    __syncthreads();
    if (leader) {
      if (mbar_wait(&bars[3], ph_kv, abort_word, p.status, kTimeoutTmaFull)) {
        tc_fence_after_sync();
        // O_tile = P V : A = P (K-major, two slabs of 4 k-steps), B = V (MN-major, 16 keys per k-step)
        umma_steps(tO, smem_u32(sP), 16, 32, smem_u32(sV), 8192, 2048, idesc_o, 4, false);
        umma_steps(tO, smem_u32(sP) + kTileBytes, 16, 32, smem_u32(sV) + 4 * 2048, 8192, 2048, idesc_o, 4, true);
        umma_commit(&bars[2]);
      }
    }
    ph_kv ^= 1;
    if (!mbar_wait(&bars[2], ph_mma, abort_word, p.status, kTimeoutTmemFull)) { ok = false; break; }
    ph_mma ^= 1;
    tc_fence_after_sync();
    if (leader && kt + 1 < num_kt) {       // the MMA that read sV has completed
      mbar_expect_tx(&bars[3], kTileBytes);
      tma_load_2d(sV, &tmap_v, &bars[3], h * kHd, k_begin + (kt + 1) * kTile);
    }
    {
      uint32_t r[32];
      tmem_ld32(tO + lane_sel + grp * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) o_acc[j] = o_acc[j] * alpha + __uint_as_float(r[j]);
    }
    tc_fence_before_sync();
    __syncthreads();  // K, V, P shared-memory tiles and both TMEM regions are free again
  }

  // the row sum is the sum of the two warpgroups' halves (both used the same running maximum)
  sRed[grp * kTile + t] = l_run;
  __syncthreads();
  l_run += sRed[(grp ^ 1) * kTile + t];
  if (ok && t < q_rows) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* orow = p.out + static_cast<size_t>(q0 + t) * p.ld_out + h * kHd + grp * 32;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(o_acc[g * 8 + 2 * j] * inv, o_acc[g * 8 + 2 * j + 1] * inv);
      reinterpret_cast<uint4*>(orow)[g] = o;
    }
    if (p.lse && grp == 0)
      p.lse[static_cast<size_t>(h) * p.lse_stride + q0 + t] = l_run > 0.f ? (m_run + __log2f(l_run)) * 0.6931471805599453f : 0.f;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_word) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (threadIdx.x < 32) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

// ---------------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------------
// 256 threads: two warpgroups own the same 128 rows (TMEM lanes) and split the columns of every tile between them, so
// each scheduler has two warps to switch between while the other waits on TMEM loads and exponentials.
template <bool kBias>
__global__ void __launch_bounds__(256)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                const __grid_constant__ CUtensorMap tmap_dq, const AttnArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sQ0 = sV + kTileBytes;         // Q / dO tiles are double-buffered: the next query tile is fetched while
  uint8_t* sDO0 = sQ0 + kTileBytes;       // this one is being worked on
  uint8_t* sQ1 = sDO0 + kTileBytes;
  uint8_t* sDO1 = sQ1 + kTileBytes;
  uint8_t* sP = sDO1 + kTileBytes;
  uint8_t* sDS = sP + kPBytes;
  uint8_t* sDQ = sDS + kPBytes;           // fp32 dQ staging: one [128 x 32] 128-byte-swizzled slab per warpgroup
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDQ + 2 * kTileBytes);  // [0]=KV [1]=Q,dO buffer 0 [2]=dV,dK,dQ MMAs [3]=Q,dO buffer 1 [4]=S,dP MMAs
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  zero_tail_bwd(p);
  const int b = blockIdx.z, h = blockIdx.y, kt = blockIdx.x;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int k_begin = p.cu_k[b], k_len = p.cu_k[b + 1] - k_begin;
  const int k0 = k_begin + kt * kTile;
  if (kt * kTile >= k_len) return;
  const int k_rows = min(kTile, k_len - kt * kTile);
  const bool single_kt = k_len <= kTile;
  const int t = threadIdx.x & 127, warp = t >> 5, grp = threadIdx.x >> 7;
  const bool leader = threadIdx.x == 0;

  if (leader) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    mbar_init(&bars[3], 1);
    mbar_init(&bars[4], 1);
    *abort_word = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 32) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDQ = tmem_base + 256, tDK = tmem_base + 320,
                 tDV = tmem_base + 384;
  const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;

  if (leader) {
    mbar_expect_tx(&bars[0], 2 * kTileBytes);
    tma_load_2d(sK, &tmap_k, &bars[0], h * kHd, k0);
    tma_load_2d(sV, &tmap_v, &bars[0], h * kHd, k0);
  }
  const uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);    // S, dP : K-major x K-major, N = 128
  const uint32_t idesc_dq = make_idesc_bf16(kTile, kHd, 0, 1);     // dQ    : K-major A, MN-major B, N = 64
  const uint32_t idesc_dkv = make_idesc_bf16(kTile, kHd, 1, 1);    // dK,dV : MN-major A and B, N = 64

  const float scale_log2 = p.scale * 1.4426950408889634f;
  const float sl2 = kBias ? 1.f : scale_log2;      // with a bias the scores are converted when they are read (add_bias32)
  const bool do_drop = p.dropout_p > 0.f;
  const DropRng rng(p.seed + ((do_drop && p.seed_dev) ? *p.seed_dev : 0ull),
                    (p.stream_id << 16) | static_cast<unsigned long long>(h), p.dropout_p);

  const int num_qt = (q_len + kTile - 1) / kTile;
  const int qt_first = p.causal ? (kt * kTile) / kTile : 0;  // query tiles before the key tile see none of it
  uint32_t ph_mma = 0, ph_s = 0;
  bool ok = true;
  bool first = true;

  // S = Q K^T and dP = dO V^T of query tile i+1 are issued right behind the dV / dK / dQ products of tile i, so they run
  // while the threads move dQ of tile i out of TMEM; the first pair is issued here.
  if (leader && qt_first < num_qt) {
    mbar_expect_tx(&bars[1], 2 * kTileBytes);
    tma_load_2d(sQ0, &tmap_q, &bars[1], h * kHd, q_begin + qt_first * kTile);
    tma_load_2d(sDO0, &tmap_do, &bars[1], h * kHd, q_begin + qt_first * kTile);
    ok = mbar_wait(&bars[0], 0, abort_word, p.status, kTimeoutTmaFull);
    if (ok) ok = mbar_wait(&bars[1], 0, abort_word, p.status, kTimeoutTmaFull);
    if (ok) {
      tc_fence_after_sync();
      umma_steps(tS, smem_u32(sQ0), 16, 32, smem_u32(sK), 16, 32, idesc_s, kHd / 16, false);
      umma_steps(tDP, smem_u32(sDO0), 16, 32, smem_u32(sV), 16, 32, idesc_s, kHd / 16, false);
      umma_commit(&bars[4]);
    }
  }
  float nxt_D = 0.f, nxt_lse = 0.f;
  if (p.delta && qt_first < num_qt && qt_first * kTile + t < q_len) {
    nxt_D = p.delta[static_cast<size_t>(h) * p.lse_stride + q_begin + qt_first * kTile + t];
    nxt_lse = p.lse[static_cast<size_t>(h) * p.lse_stride + q_begin + qt_first * kTile + t];
  }
  for (int qt = qt_first; qt < num_qt && ok; ++qt) {
    const int q0 = q_begin + qt * kTile;
    const int q_rows = min(kTile, q_len - qt * kTile);
    const int it = qt - qt_first, buf = it & 1;
    uint8_t* sQ = buf ? sQ1 : sQ0;
    uint8_t* sDO = buf ? sDO1 : sDO0;
    if (leader && qt + 1 < num_qt) {
      // the other buffer was last read by the MMAs of the previous iteration, which have completed
      uint64_t* nb = buf ? &bars[1] : &bars[3];
      mbar_expect_tx(nb, 2 * kTileBytes);
      tma_load_2d(buf ? sQ0 : sQ1, &tmap_q, nb, h * kHd, q0 + kTile);
      tma_load_2d(buf ? sDO0 : sDO1, &tmap_do, nb, h * kHd, q0 + kTile);
    }
    // D = rowsum(dO * O) and the saved log-sum-exp of my query row.  With the precomputed D both are one float per row:
    // the values of the NEXT tile are requested here and used an iteration later, so their latency is never waited for.
    const bool row_ok = t < q_rows;
    float Drow = 0.f, lse = 0.f;
    if (p.delta) {
      Drow = nxt_D;
      lse = nxt_lse;
      const int nrow = q0 + kTile + t;
      if (qt + 1 < num_qt && nrow < q_begin + q_len) {
        nxt_D = p.delta[static_cast<size_t>(h) * p.lse_stride + nrow];
        nxt_lse = p.lse[static_cast<size_t>(h) * p.lse_stride + nrow];
      }
    } else if (row_ok) {
      const uint4* orow = reinterpret_cast<const uint4*>(p.o + static_cast<size_t>(q0 + t) * p.ld_o + h * kHd);
      const uint4* drow = reinterpret_cast<const uint4*>(p.d_o + static_cast<size_t>(q0 + t) * p.ld_do + h * kHd);
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        uint4 a = orow[g], d = drow[g];
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 x = __bfloat1622float2(a2[j]), y = __bfloat1622float2(d2[j]);
          Drow += x.x * y.x + x.y * y.y;
        }
      }
      lse = p.lse[static_cast<size_t>(h) * p.lse_stride + q0 + t];
    }
    if (!mbar_wait(&bars[4], ph_s, abort_word, p.status, kTimeoutTmemFull)) { ok = false; break; }
    ph_s ^= 1;
    tc_fence_after_sync();

    const int q_pos = qt * kTile + t;
    // P = 2^(S * scale * log2 e - lse * log2 e); dS is kept WITHOUT the softmax scale (dQ and dK are scaled when they
    // leave TMEM: 64 multiplies per row instead of 128 per row and tile).  A tile with all 128 x 128 scores inside both
    // sequences (and below the diagonal when causal) and no dropout takes the branch without per-element masks.
    const bool full = q_rows == kTile && k_rows == kTile && (!p.causal || kt < qt);
    const float lse2 = lse * 1.4426950408889634f;
#pragma unroll 1
    for (int c = 2 * grp; c < 2 * grp + 2; ++c) {      // this warpgroup's 64 of the 128 key columns
      uint32_t rs[32], rd[32];
      tmem_ld32(tS + lane_sel + c * 32, rs);
      tmem_ld32(tDP + lane_sel + c * 32, rd);
      tmem_ld_wait();
      const long bias_off = kBias ? static_cast<long>(b) * p.bias_sb + static_cast<long>(h) * p.bias_sh +
                                        static_cast<long>(q_pos) * p.bias_sq + kt * kTile + c * 32
                                  : 0;
      if (kBias) add_bias32(rs, row_ok ? p.bias + bias_off : nullptr, k_rows - c * 32, scale_log2);
      float pd[32], ds[32];
      if (full && !do_drop && !kBias) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          pd[j] = ex2_approx(fmaf(__uint_as_float(rs[j]), scale_log2, -lse2));
          ds[j] = pd[j] * (__uint_as_float(rd[j]) - Drow);
        }
      } else {
        float kf[32];
        const unsigned long long base = static_cast<unsigned long long>(q0 + t) * p.kstride + kt * kTile + c * 32;
#pragma unroll
        for (int j = 0; j < 32; ++j) kf[j] = 1.f;
        if (do_drop) apply_dropout32(rng, base, kf);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = c * 32 + j;
          const bool valid = row_ok && col < k_rows && (!p.causal || kt * kTile + col <= q_pos);
          const float pr = valid ? ex2_approx(fmaf(__uint_as_float(rs[j]), sl2, -lse2)) : 0.f;
          pd[j] = pr * kf[j];
          ds[j] = pr * (__uint_as_float(rd[j]) * kf[j] - Drow);
          // the gradient of the bias is dS before the softmax scale; every (query, key) pair is visited by one thread
          if (kBias && p.dbias && valid) p.dbias[bias_off + j] = ds[j];
        }
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o1, o2v;
        __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&o1);
        __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&o2v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          a2[j] = __floats2bfloat162_rn(pd[g * 8 + 2 * j], pd[g * 8 + 2 * j + 1]);
          b2[j] = __floats2bfloat162_rn(ds[g * 8 + 2 * j], ds[g * 8 + 2 * j + 1]);
        }
        const int chunk = c * 4 + g;
        const uint32_t off = (chunk >> 3) * kTileBytes + sw128_offset(t, chunk & 7);
        *reinterpret_cast<uint4*>(sP + off) = o1;
        *reinterpret_cast<uint4*>(sDS + off) = o2v;
      }
    }
    if (t == 0) tma_store_wait_read();                 // last tile's dQ slab has been read by its reduction
    tc_fence_before_sync();
    fence_async_smem();
    __syncthreads();
    if (leader) {
      tc_fence_after_sync();
      // dV += P^T dO : A = P read MN-major (M = keys: two 64-key slabs, LBO = slab size), K = 128 query rows
      umma_steps(tDV, smem_u32(sP), kTileBytes, 2048, smem_u32(sDO), 8192, 2048, idesc_dkv, 8, !first);
      // dK += dS^T Q
      umma_steps(tDK, smem_u32(sDS), kTileBytes, 2048, smem_u32(sQ), 8192, 2048, idesc_dkv, 8, !first);
      // dQ = dS K : A = dS K-major (two slabs of 4 k-steps), B = K tile MN-major
      umma_steps(tDQ, smem_u32(sDS), 16, 32, smem_u32(sK), 8192, 2048, idesc_dq, 4, false);
      umma_steps(tDQ, smem_u32(sDS) + kTileBytes, 16, 32, smem_u32(sK) + 4 * 2048, 8192, 2048, idesc_dq, 4, true);
      umma_commit(&bars[2]);
      if (qt + 1 < num_qt) {
        // every thread has read S and dP of this tile (barrier above): the next pair may overwrite them
        const int nit = it + 1;
        if (mbar_wait((nit & 1) ? &bars[3] : &bars[1], (nit >> 1) & 1, abort_word, p.status, kTimeoutTmaFull)) {
          tc_fence_after_sync();
          umma_steps(tS, smem_u32(buf ? sQ0 : sQ1), 16, 32, smem_u32(sK), 16, 32, idesc_s, kHd / 16, false);
          umma_steps(tDP, smem_u32(buf ? sDO0 : sDO1), 16, 32, smem_u32(sV), 16, 32, idesc_s, kHd / 16, false);
          umma_commit(&bars[4]);
        }
      }
    }
    first = false;
    if (!mbar_wait(&bars[2], ph_mma, abort_word, p.status, kTimeoutTmemFull)) { ok = false; break; }
    ph_mma ^= 1;
    tc_fence_after_sync();
#pragma unroll 1
    for (int c = grp; c < grp + 1; ++c) {               // 32 of the 64 dQ columns per warpgroup
      uint32_t r[32];
      tmem_ld32(tDQ + lane_sel + c * 32, r);
      tmem_ld_wait();
      if (row_ok || (!single_kt && p.dq_tma)) {      // rows past the sequence hold exact zeros: harmless in the tile sum
        if (single_kt) {
          __nv_bfloat16* drow = p.dq + static_cast<size_t>(q0 + t) * p.ld_dq + h * kHd + c * 32;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              o2[j] = __floats2bfloat162_rn(__uint_as_float(r[g * 8 + 2 * j]) * p.scale, __uint_as_float(r[g * 8 + 2 * j + 1]) * p.scale);
            reinterpret_cast<uint4*>(drow)[g] = o;
          }
        } else if (p.dq_tma) {
          // my 32 values go to the staging slab of my warpgroup (conflict-free thanks to the swizzle); one thread per
          // warpgroup hands the slab to the TMA unit after the barrier below: whole 128-byte lines reach the L2 reduction
          // units, where a row-per-thread red.add sends 16-byte fragments of 32 different lines per instruction
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float4 o = make_float4(__uint_as_float(r[g * 4]) * p.scale, __uint_as_float(r[g * 4 + 1]) * p.scale,
                                   __uint_as_float(r[g * 4 + 2]) * p.scale, __uint_as_float(r[g * 4 + 3]) * p.scale);
            *reinterpret_cast<float4*>(sDQ + grp * kTileBytes + sw128_offset(t, g)) = o;
          }
        } else {
          float* arow = p.dq_acc + static_cast<size_t>(q0 + t) * p.ld_dqacc + h * kHd + c * 32;
#pragma unroll
          for (int g = 0; g < 8; ++g)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(arow + g * 4),
                         "f"(__uint_as_float(r[g * 4]) * p.scale), "f"(__uint_as_float(r[g * 4 + 1]) * p.scale),
                         "f"(__uint_as_float(r[g * 4 + 2]) * p.scale), "f"(__uint_as_float(r[g * 4 + 3]) * p.scale)
                         : "memory");
        }
      }
    }
    tc_fence_before_sync();
    if (!single_kt && p.dq_tma) fence_async_smem();
    __syncthreads();
    if (!single_kt && p.dq_tma && t == 0) {          // one thread per warpgroup: dq_acc[q0 .. q0+127, my 32 columns] += slab
      tma_reduce_add_2d(&tmap_dq, sDQ + grp * kTileBytes, h * kHd + grp * 32, q0);
      tma_store_commit();
    }
  }
  if (t == 0) tma_store_wait_all();                  // the slabs must outlive the reductions that read them

  // dK, dV of my key row
  if (ok && !first) {
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* dst = which == 0 ? p.dk : p.dv;
      const int ld = which == 0 ? p.ld_dk : p.ld_dv;
      const uint32_t tsrc = which == 0 ? tDK : tDV;
#pragma unroll 1
      for (int c = grp; c < grp + 1; ++c) {
        uint32_t r[32];
        tmem_ld32(tsrc + lane_sel + c * 32, r);
        tmem_ld_wait();
        if (t < k_rows) {
          __nv_bfloat16* drow = dst + static_cast<size_t>(k0 + t) * ld + h * kHd + c * 32;
          const float osc = which == 0 ? p.scale : 1.f;     // dK carries the softmax scale that dS left out
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              o2[j] = __floats2bfloat162_rn(__uint_as_float(r[g * 8 + 2 * j]) * osc, __uint_as_float(r[g * 8 + 2 * j + 1]) * osc);
            reinterpret_cast<uint4*>(drow)[g] = o;
          }
        }
      }
    }
  } else if (ok && t < k_rows && grp == 0) {
    // no query tile attends to this key tile: zero gradients
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* dst = which == 0 ? p.dk : p.dv;
      const int ld = which == 0 ? p.ld_dk : p.ld_dv;
      uint4 z = make_uint4(0, 0, 0, 0);
      for (int g = 0; g < 8; ++g) reinterpret_cast<uint4*>(dst + static_cast<size_t>(k0 + t) * ld + h * kHd)[g] = z;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_word) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (threadIdx.x < 32) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[h, row] = sum_j dO[row, h*64 + j] * O[row, h*64 + j]; one thread per (row, head), neighbours read neighbouring
// 128-byte runs
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, int ld_o, const __nv_bfloat16* __restrict__ d_o, int ld_do,
                                  float* __restrict__ delta, long stride, int total_q, int heads) {
  const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long>(total_q) * heads) return;
  const int row = static_cast<int>(i / heads), h = static_cast<int>(i % heads);
  const uint4* orow = reinterpret_cast<const uint4*>(o + static_cast<size_t>(row) * ld_o + h * kHd);
  const uint4* drow = reinterpret_cast<const uint4*>(d_o + static_cast<size_t>(row) * ld_do + h * kHd);
  float acc = 0.f;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    uint4 a = orow[g], d = drow[g];
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = __bfloat1622float2(a2[j]), y = __bfloat1622float2(d2[j]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  delta[static_cast<size_t>(h) * stride + row] = acc;
}

// dq (bf16) = dq_acc (fp32) for rows of sequences with more than one key tile
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, int ld_acc, __nv_bfloat16* __restrict__ dq, int ld_dq,
                                       const int* __restrict__ cu_q, const int* __restrict__ cu_k, int width) {
  const int b = blockIdx.y;
  if (cu_k[b + 1] - cu_k[b] <= kTile) return;
  const int q_begin = cu_q[b], q_end = cu_q[b + 1];
  const int w4 = width >> 2;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < static_cast<long>(q_end - q_begin) * w4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int r = q_begin + static_cast<int>(i / w4), c = static_cast<int>(i % w4) * 4;
    float4 v = *reinterpret_cast<const float4*>(acc + static_cast<size_t>(r) * ld_acc + c);
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dq + static_cast<size_t>(r) * ld_dq + c) = o;
  }
}

constexpr int kFwdSmem = 3 * kTileBytes + kPBytes + 1024 + 64 + 1024;
constexpr int kBwdSmem = 8 * kTileBytes + 2 * kPBytes + 64 + 1024;

}  // namespace b200

namespace b200 {
const char* launch_attn_fwd_short(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a,
                                  int num_items, cudaStream_t stream);
const char* launch_attn_bwd_short(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                                  const AttnArgs& a, int num_items, cudaStream_t stream);
const char* launch_attn_fwd_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a, int max_q,
                               cudaStream_t stream);
const char* launch_attn_bwd_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                               const CUtensorMap& tdq, const AttnArgs& a, dim3 grid, cudaStream_t stream);
}  // namespace b200

using namespace b200;

// 0 = automatic, 1 = always the general multi-tile kernels, 2 = the general kernels without their warp-specialised variants
static int g_attn_variant = 0;
void nmtg_set_attention_variant(int v) { g_attn_variant = v; }

static const char* check_ptr(const void* p, int ld) {
  if ((reinterpret_cast<uintptr_t>(p) & 15) || (ld % 8)) return "attention: tensors must be 16-byte aligned with ld % 8 == 0";
  return nullptr;
}

const char* nmtg_attn_fwd(const AttnDesc* d, cudaStream_t stream) {
  if (d->batch <= 0 || d->num_heads <= 0) return nullptr;
  if (d->head_dim != kHd) return "attention: only head_dim 64 is implemented";
  const char* e;
  if ((e = check_ptr(d->q, d->ld_q)) || (e = check_ptr(d->k, d->ld_k)) || (e = check_ptr(d->v, d->ld_v)) ||
      (e = check_ptr(d->out, d->ld_out)))
    return e;
  const int width = d->num_heads * kHd;
  CUtensorMap tq, tk, tv;
  if (!cached_tmap(&tq, d->q, d->total_q, width, d->ld_q, kTile, kHd)) return "attention: tensor map (q) failed";
  if (!cached_tmap(&tk, d->k, d->total_k, width, d->ld_k, kTile, kHd)) return "attention: tensor map (k) failed";
  if (!cached_tmap(&tv, d->v, d->total_k, width, d->ld_v, kTile, kHd)) return "attention: tensor map (v) failed";
  AttnArgs a = {};
  a.cu_q = d->cu_q; a.cu_k = d->cu_k; a.num_heads = d->num_heads; a.causal = d->causal; a.scale = d->scale;
  a.dropout_p = d->dropout_p; a.seed = d->seed; a.stream_id = d->stream_id; a.seed_dev = d->seed_dev; a.kstride = d->kstride;
  a.out = reinterpret_cast<__nv_bfloat16*>(d->out); a.ld_out = d->ld_out;
  a.lse = d->lse; a.lse_stride = d->lse_stride;
  a.p_debug = nullptr; a.total_q = d->total_q; a.total_k = d->total_k; a.batch = d->batch; a.status = d->status;
  a.bias = d->bias; a.bias_sb = d->bias_sb; a.bias_sh = d->bias_sh; a.bias_sq = d->bias_sq; a.dbias = nullptr;
  if (g_attn_variant == 0 && d->max_q <= kTile && d->max_k <= kTile && !d->bias)
    return launch_attn_fwd_short(tq, tk, tv, a, d->batch * d->num_heads, stream);
  // Long sequences without attention dropout: the warp-specialised kernel (attention_fwd_ws_tcgen05.cu), two query tiles
  // per CTA.  Measured against the kernel below: 0.233 / 0.264 ms on 8 x 1500 x 20 heads, but 0.070 / 0.053 ms on
  // 8 x 448 causal (too few CTAs of 256 queries for 148 SMs), hence the length threshold; variant 1 ignores it (tests).
  if (!d->bias && d->dropout_p <= 0.f && g_attn_variant != 2 && d->max_q > (g_attn_variant == 1 ? kTile : 4 * kTile))
    return launch_attn_fwd_ws(tq, tk, tv, a, d->max_q, stream);
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem);
    if (ce == cudaSuccess) ce = cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem);
    if (ce != cudaSuccess) return cudaGetErrorString(ce);
    configured = true;
  }
  dim3 grid((d->max_q + kTile - 1) / kTile, d->num_heads, d->batch);
  if (d->bias) attn_fwd_kernel<true><<<grid, 256, kFwdSmem, stream>>>(tq, tk, tv, a);
  else attn_fwd_kernel<false><<<grid, 256, kFwdSmem, stream>>>(tq, tk, tv, a);
  cudaError_t ce = cudaGetLastError();
  return ce == cudaSuccess ? nullptr : cudaGetErrorString(ce);
}

const char* nmtg_attn_bwd(const AttnDesc* d, cudaStream_t stream) {
  if (d->batch <= 0 || d->num_heads <= 0) return nullptr;
  if (d->head_dim != kHd) return "attention: only head_dim 64 is implemented";
  const char* e;
  if ((e = check_ptr(d->q, d->ld_q)) || (e = check_ptr(d->k, d->ld_k)) || (e = check_ptr(d->v, d->ld_v)) ||
      (e = check_ptr(d->out, d->ld_out)) || (e = check_ptr(d->d_out, d->ld_dout)) || (e = check_ptr(d->dq, d->ld_dq)) ||
      (e = check_ptr(d->dk, d->ld_dk)) || (e = check_ptr(d->dv, d->ld_dv)))
    return e;
  if (d->max_k > kTile && !d->dq_acc) return "attention backward: sequences above 128 keys need the fp32 dq buffer";
  const int width = d->num_heads * kHd;
  CUtensorMap tq, tk, tv, tdo;
  if (!cached_tmap(&tq, d->q, d->total_q, width, d->ld_q, kTile, kHd)) return "attention: tensor map (q) failed";
  if (!cached_tmap(&tk, d->k, d->total_k, width, d->ld_k, kTile, kHd)) return "attention: tensor map (k) failed";
  if (!cached_tmap(&tv, d->v, d->total_k, width, d->ld_v, kTile, kHd)) return "attention: tensor map (v) failed";
  if (!cached_tmap(&tdo, d->d_out, d->total_q, width, d->ld_dout, kTile, kHd)) return "attention: tensor map (dO) failed";
  AttnArgs a = {};
  a.cu_q = d->cu_q; a.cu_k = d->cu_k; a.num_heads = d->num_heads; a.causal = d->causal; a.scale = d->scale;
  a.dropout_p = d->dropout_p; a.seed = d->seed; a.stream_id = d->stream_id; a.seed_dev = d->seed_dev; a.kstride = d->kstride;
  a.lse = d->lse; a.lse_stride = d->lse_stride;
  a.o = reinterpret_cast<const __nv_bfloat16*>(d->out); a.ld_o = d->ld_out;
  a.d_o = reinterpret_cast<const __nv_bfloat16*>(d->d_out); a.ld_do = d->ld_dout;
  a.dq = reinterpret_cast<__nv_bfloat16*>(d->dq); a.ld_dq = d->ld_dq;
  a.dk = reinterpret_cast<__nv_bfloat16*>(d->dk); a.ld_dk = d->ld_dk;
  a.dv = reinterpret_cast<__nv_bfloat16*>(d->dv); a.ld_dv = d->ld_dv;
  a.dq_acc = d->dq_acc; a.ld_dqacc = d->ld_dqacc;
  a.total_q = d->total_q; a.total_k = d->total_k; a.batch = d->batch; a.status = d->status;
  a.bias = d->bias; a.bias_sb = d->bias_sb; a.bias_sh = d->bias_sh; a.bias_sq = d->bias_sq; a.dbias = d->dbias;
  if (g_attn_variant == 0 && d->max_q <= kTile && d->max_k <= kTile && !d->bias)
    return launch_attn_bwd_short(tq, tk, tv, tdo, a, d->batch * d->num_heads, stream);
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
    if (ce == cudaSuccess) ce = cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
    if (ce != cudaSuccess) return cudaGetErrorString(ce);
    configured = true;
  }
  if (d->delta && d->max_k > kTile) {
    const long n = static_cast<long>(d->total_q) * d->num_heads;
    attn_delta_kernel<<<static_cast<int>((n + 255) / 256), 256, 0, stream>>>(a.o, a.ld_o, a.d_o, a.ld_do, d->delta, d->lse_stride,
                                                                            d->total_q, d->num_heads);
    a.delta = d->delta;
  }
  CUtensorMap tdq = tq;       // placeholder when the reductions go through red.add
  a.dq_tma = 0;
  if (d->dq_acc && d->max_k > kTile && (reinterpret_cast<uintptr_t>(d->dq_acc) & 15) == 0 && d->ld_dqacc % 4 == 0 &&
      cached_tmap_f32(&tdq, d->dq_acc, d->total_q, width, d->ld_dqacc, kTile, 32))
    a.dq_tma = 1;
  dim3 grid((d->max_k + kTile - 1) / kTile, d->num_heads, d->batch);
  cudaError_t ce = cudaSuccess;
  if (!d->bias && a.delta && a.dq_tma && g_attn_variant != 2 && (g_attn_variant == 1 || d->max_k > 4 * kTile)) {
    // long sequences: the warp-specialised, pipelined kernel (attention_bwd_ws_tcgen05.cu); 0.587 / 0.664 ms on 8 x 1500 x 20
    // heads and 0.313 / 0.336 ms on 8 x 1000 x 16 heads against the kernel below, level with it at 448 tokens
    if ((e = launch_attn_bwd_ws(tq, tk, tv, tdo, tdq, a, grid, stream))) return e;
  } else {
    if (d->bias) attn_bwd_kernel<true><<<grid, 256, kBwdSmem, stream>>>(tq, tk, tv, tdo, tdq, a);
    else attn_bwd_kernel<false><<<grid, 256, kBwdSmem, stream>>>(tq, tk, tv, tdo, tdq, a);
    ce = cudaGetLastError();
    if (ce != cudaSuccess) return cudaGetErrorString(ce);
  }
  if (d->max_k > kTile) {
    dim3 g2(64, d->batch);
    attn_dq_convert_kernel<<<g2, 256, 0, stream>>>(d->dq_acc, d->ld_dqacc, reinterpret_cast<__nv_bfloat16*>(d->dq), d->ld_dq,
                                                   d->cu_q, d->cu_k, width);
    ce = cudaGetLastError();
    if (ce != cudaSuccess) return cudaGetErrorString(ce);
  }
  return nullptr;
}

// ---------------------------------------------------------------------------------------------------
// Backward pass with a built-in accumulation buffer (see attention_noalloc.h for the contract).
// ---------------------------------------------------------------------------------------------------
#include "attention_noalloc.h"
#include <cstdio>

namespace b200 {
bool make_tmap_2d_nobind(CUtensorMap* out, const void* base, long rows, long cols, long ld, int box_rows, int box_cols, bool f32);
}

// The fp32 dQ accumulation buffer of the no-allocation entry point.  In host code this name is only a handle
// for cudaGetSymbolAddress, never a pointer that a kernel may receive.
static __device__ __align__(256) float g_attn_noalloc_scratch[NMTG_ATTN_NOALLOC_MAX_FLOATS];
static float* g_attn_noalloc_ptr[64] = {};   // device address of the array, per device ordinal
static bool g_attn_noalloc_smem_set[64] = {}; // the backward kernel's shared-memory limit was raised on this device

static int noalloc_fail(int code, const char* msg, char* err, int err_len) {
  if (err && err_len > 0) snprintf(err, static_cast<size_t>(err_len), "%s", msg);
  return code;
}

extern "C" int nmtg_attn_bwd_noalloc(const void* q, int ld_q, const void* k, int ld_k, const void* v, int ld_v, const void* out,
                                     int ld_out, const float* lse, long lse_stride, const void* d_out, int ld_dout, void* dq,
                                     int ld_dq, void* dk, int ld_dk, void* dv, int ld_dv, const int* cu_q, const int* cu_k,
                                     int batch, int num_heads, int max_q, int max_k, int total_q, int total_k, int causal,
                                     float scale, float dropout_p, unsigned long long seed, unsigned long long stream_id,
                                     int* status, cudaStream_t stream, char* err, int err_len) {
  if (batch <= 0 || num_heads <= 0 || total_q <= 0 || total_k <= 0) return 0;
  const void* ptrs[] = {q, k, v, out, d_out, dq, dk, dv};
  const int lds[] = {ld_q, ld_k, ld_v, ld_out, ld_dout, ld_dq, ld_dk, ld_dv};
  for (int i = 0; i < 8; ++i)
    if (!ptrs[i] || (reinterpret_cast<uintptr_t>(ptrs[i]) & 15) || (lds[i] % 8))
      return noalloc_fail(1, "attention: tensors must be non-null, 16-byte aligned, with leading dimensions % 8 == 0", err, err_len);
  if (!lse || !cu_q || !cu_k) return noalloc_fail(1, "attention: lse / cu_q / cu_k must not be null", err, err_len);
  const int width = num_heads * kHd;
  const bool needs_buffer = max_k > kTile;
  const long need = static_cast<long>(total_q) * width;
  if (needs_buffer && need > NMTG_ATTN_NOALLOC_MAX_FLOATS) {
    char msg[200];
    snprintf(msg, sizeof(msg), "attention backward without allocation: total_q * heads * 64 = %ld floats exceeds the built-in "
             "buffer of %ld floats", need, static_cast<long>(NMTG_ATTN_NOALLOC_MAX_FLOATS));
    return noalloc_fail(2, msg, err, err_len);
  }
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess || dev < 0 || dev >= 64) return noalloc_fail(3, "cudaGetDevice failed", err, err_len);
  // Binds the device's primary context to the calling thread (the descriptor encoder below is a driver entry point and
  // needs one); unlike the regular path's cudaFree(nullptr) this is legal while another thread captures a stream.
  ce = cudaSetDevice(dev);
  if (ce != cudaSuccess) return noalloc_fail(3, cudaGetErrorString(ce), err, err_len);
  if (!g_attn_noalloc_ptr[dev]) {   // first call on this device: resolve the array's device address
    float* p = nullptr;
    ce = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_noalloc_scratch);
    if (ce != cudaSuccess || !p) return noalloc_fail(3, cudaGetErrorString(ce), err, err_len);
    g_attn_noalloc_ptr[dev] = p;
  }
  float* scratch = g_attn_noalloc_ptr[dev];
  if (needs_buffer) {   // the array still holds the previous call's sums
    ce = cudaMemsetAsync(scratch, 0, static_cast<size_t>(need) * sizeof(float), stream);
    if (ce != cudaSuccess) return noalloc_fail(3, cudaGetErrorString(ce), err, err_len);
  }
  CUtensorMap tq, tk, tv, tdo;
  if (!make_tmap_2d_nobind(&tq, q, total_q, width, ld_q, kTile, kHd, false) ||
      !make_tmap_2d_nobind(&tk, k, total_k, width, ld_k, kTile, kHd, false) ||
      !make_tmap_2d_nobind(&tv, v, total_k, width, ld_v, kTile, kHd, false) ||
      !make_tmap_2d_nobind(&tdo, d_out, total_q, width, ld_dout, kTile, kHd, false))
    return noalloc_fail(3, "attention: cuTensorMapEncodeTiled failed", err, err_len);
  AttnArgs a = {};
  a.cu_q = cu_q; a.cu_k = cu_k; a.num_heads = num_heads; a.causal = causal; a.scale = scale;
  a.dropout_p = dropout_p; a.seed = seed; a.stream_id = stream_id; a.seed_dev = nullptr;
  a.kstride = (max_k + 15) / 16 * 16;
  a.lse = const_cast<float*>(lse); a.lse_stride = lse_stride;
  a.o = reinterpret_cast<const __nv_bfloat16*>(out); a.ld_o = ld_out;
  a.d_o = reinterpret_cast<const __nv_bfloat16*>(d_out); a.ld_do = ld_dout;
  a.dq = reinterpret_cast<__nv_bfloat16*>(dq); a.ld_dq = ld_dq;
  a.dk = reinterpret_cast<__nv_bfloat16*>(dk); a.ld_dk = ld_dk;
  a.dv = reinterpret_cast<__nv_bfloat16*>(dv); a.ld_dv = ld_dv;
  a.dq_acc = scratch; a.ld_dqacc = width;
  a.total_q = total_q; a.total_k = total_k; a.batch = batch; a.status = status;
  if (!g_attn_noalloc_smem_set[dev]) {   // once per device, like the address look-up above
    ce = cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
    if (ce != cudaSuccess) return noalloc_fail(3, cudaGetErrorString(ce), err, err_len);
    g_attn_noalloc_smem_set[dev] = true;
  }
  CUtensorMap tdq = tq;       // placeholder when no accumulation buffer is needed
  a.dq_tma = (needs_buffer && make_tmap_2d_nobind(&tdq, scratch, total_q, width, width, kTile, 32, true)) ? 1 : 0;
  dim3 grid((max_k + kTile - 1) / kTile, num_heads, batch);
  attn_bwd_kernel<false><<<grid, 256, kBwdSmem, stream>>>(tq, tk, tv, tdo, tdq, a);
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return noalloc_fail(3, cudaGetErrorString(ce), err, err_len);
  if (needs_buffer) {
    dim3 g2(64, batch);
    attn_dq_convert_kernel<<<g2, 256, 0, stream>>>(scratch, width, reinterpret_cast<__nv_bfloat16*>(dq), ld_dq, cu_q, cu_k, width);
    ce = cudaGetLastError();
    if (ce != cudaSuccess) return noalloc_fail(3, cudaGetErrorString(ce), err, err_len);
  }
  return 0;
}
