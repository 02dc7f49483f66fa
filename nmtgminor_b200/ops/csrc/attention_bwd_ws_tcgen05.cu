// Warp-specialised backward pass of the multi-tile (general) attention kernels for sm_100a, head_dim 64.
//
// One CTA owns one 128-key tile of one (sequence, head) and walks over the query tiles that attend to it, like
// attn_bwd_kernel (attention_tcgen05.cu), whose arithmetic, operand layouts and dropout counters it shares.  There every
// thread took part in every phase, so the tensor cores idled while P / dS were being computed and the threads idled while
// the five products of a tile ran.  Here the phases belong to different warps and are pipelined across query tiles:
//
//   warps 0-3 / 4-7   math: thread = (query row, half); half h owns key columns [32 c + 16 h, 32 c + 16 h + 16) of every
//                     32-column chunk c.  P = 2^(S - lse), dS = P (dP - D), packed to bf16 into swizzled staging tiles.
//   warps 8-11        dQ of tile i - 1: TMEM -> fp32 staging -> TMA reduce-add into the accumulation buffer; at the end
//                     dK and dV of the key tile.
//   warp 12           TMA producer (K, V once; Q and dO of every query tile, double-buffered)
//   warp 13           MMA issuer: S / dP of tile i + 1 in two 64-key halves as soon as the math threads have read the
//                     half of tile i out of TMEM, then dV, dK, dQ of tile i once its P / dS are staged.
//
// TMEM (512 columns): S 0..127 | dP 128..255 | dK 256..319 | dV 320..383 | dQ of even tiles 384..447 | odd tiles 448..511.
// S and dP are single-buffered, but produced and consumed in halves: while one math warpgroup works on its half of tile
// i, the tensor cores already compute the other warpgroup's half of tile i + 1.  Shared memory (224 KB): K, V | three Q / dO
// buffers (a tile's loads take about 1.5 us under load, so the tile after next must be on its way while this one is worked
// on) | one P staging tile (dV, its only reader, is the first product of a tile and done before the next tile's first
// store) | two dS staging tiles (read by dK and dQ; the tile's dS buffer then doubles as the fp32 staging of its dQ for the
// TMA reduction).  Every wait is bounded (status word) as in the other kernels.
//
// Counterpart in the reference: the dgrad loop of its bundled FlashAttention
// (onmt/modules/extensions/flashattn/src/fmha_dgrad_kernel_1xN_loop.h) and the strided-batched backward GEMMs of
// onmt/modules/extensions/multihead_attn/self_multihead_attn_cuda.cu:232-612.
#include "attention_common.cuh"

namespace b200 {

constexpr int kWsThreads = 448;
constexpr int kWsSmem = 2 * kTileBytes + 6 * kTileBytes + 3 * kPBytes + 256 + 1024;
constexpr uint32_t kWsIssuePolls = 1u << 22;   // polls of the MMA warp without progress before it gives up

// Time stamps (SM clock) of CTA (0, 0, 0) when ablation bit 128 is set: [tile][16] = math warp 0: S lo ready, loaded,
// computed, stored, S hi ready, loaded, computed, stored | MMA warp: S lo issued, S hi issued, products issued | dQ warps:
// products done, staged, handed over | TMA warp: loads issued.  A timing aid, read back with nmtg_attn_ws_trace.
constexpr int kWsTraceTiles = 32;
__device__ long long g_ws_trace[kWsTraceTiles * 16];
#define WS_STAMP(tile, slot)                                                                              \
  do {                                                                                                    \
    if (trace && (tile) < kWsTraceTiles) g_ws_trace[(tile) * 16 + (slot)] = clock64();                    \
  } while (0)

// 64 fp32 accumulator columns of this thread's TMEM lane, scaled, packed to bf16 and stored as one row
__device__ __forceinline__ void ws_store_row(uint32_t taddr, __nv_bfloat16* drow, float osc, bool store) {
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

__global__ void __launch_bounds__(kWsThreads, 1)
attn_bwd_ws_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                   const __grid_constant__ CUtensorMap tmap_dq, const AttnArgs p, const int ablate) {
  // `ablate` (0 in production) switches parts of the work off while keeping every barrier hand-shake, for timing runs that
  // tell which role bounds the tile rate (results are then meaningless): 1 no P / dS arithmetic and stores, 2 no dQ
  // read-out, 4 no gradient MMAs, 8 no S / dP MMAs, 32 dQ staged but not added to the accumulation buffer
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sQD = sV + kTileBytes;              // buffer b (tile % 3): Q at sQD + b * 2 tiles, dO one tile behind it
  uint8_t* sPst = sQD + 6 * kTileBytes;        // P staging (single)
  uint8_t* sDSst = sPst + kPBytes;             // dS staging, buffer tile & 1
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDSst + 2 * kPBytes);
  uint64_t* kv_full = bars;          // TMA -> MMA
  uint64_t* qdo_full = bars + 1;     // [3] TMA -> MMA
  uint64_t* qdo_free = bars + 4;     // [3] dV and dK of the tile done -> TMA
  uint64_t* s_full = bars + 7;       // [2] S / dP of keys 0..63 (0) and 64..127 (1) ready -> math
  uint64_t* s_free = bars + 9;       // [2] that half has been read out of TMEM -> MMA
  uint64_t* pds_full = bars + 11;    // [2] P / dS staged -> MMA
  uint64_t* ds_free = bars + 13;     // [2] dK, dQ done and the dQ staged in the dS buffer handed to the TMA unit -> math
  uint64_t* grads_full = bars + 15;  // [2] dV, dK, dQ of the tile done -> dQ warps
  uint64_t* dq_free = bars + 17;     // [2] dQ read out of TMEM -> MMA
  uint64_t* p_free = bars + 19;      // dV of the tile done -> math (next tile's P may be stored)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  zero_tail_bwd(p);
  const int b = blockIdx.z, h = blockIdx.y, kt = blockIdx.x;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int k_begin = p.cu_k[b], k_len = p.cu_k[b + 1] - k_begin;
  if (kt * kTile >= k_len) return;   // uniform for the CTA, before any barrier or TMEM use
  const int k0 = k_begin + kt * kTile;
  const int k_rows = min(kTile, k_len - kt * kTile);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qt = (q_len + kTile - 1) / kTile;
  const int qt_first = p.causal ? kt : 0;          // query tiles before the key tile see none of it
  const int n_tiles = max(0, num_qt - qt_first);
  const bool trace = (ablate & 128) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 &&
                     (warp == 0 || warp >= 8);

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(p_free, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 256);
      mbar_init(&pds_full[i], 256);
      mbar_init(&ds_free[i], 1);
      mbar_init(&grads_full[i], 1);
      mbar_init(&dq_free[i], 128);
    }
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 13) tmem_alloc(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDK = tmem_base + 256, tDV = tmem_base + 320, tDQ = tmem_base + 384;

  if (warp == 12) {
    // ---- TMA producer --------------------------------------------------------------------------------------------
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(kv_full, 2 * kTileBytes);
      tma_load_2d(sK, &tmap_k, kv_full, h * kHd, k0);
      tma_load_2d(sV, &tmap_v, kv_full, h * kHd, k0);
      for (int i = 0; i < n_tiles; ++i) {
        const int s = i % 3;
        if (i >= 3 && !mbar_wait(&qdo_free[s], ((i / 3) & 1) ^ 1, abort_word, p.status, kTimeoutSmemEmpty)) break;
        uint8_t* dst = sQD + s * 2 * kTileBytes;
        const int row = q_begin + (qt_first + i) * kTile;
        WS_STAMP(i, 14);
        mbar_expect_tx(&qdo_full[s], 2 * kTileBytes);
        tma_load_2d(dst, &tmap_q, &qdo_full[s], h * kHd, row);
        tma_load_2d(dst + kTileBytes, &tmap_do, &qdo_full[s], h * kHd, row);
      }
    }
  } else if (warp == 13) {
    // ---- MMA issuer ----------------------------------------------------------------------------------------------
    if (lane == 0 && n_tiles > 0 && mbar_wait(kv_full, 0, abort_word, p.status, kTimeoutTmaFull)) {
      const uint32_t idesc_s = make_idesc_bf16(kTile, 64, 0, 0);       // S, dP halves: K-major x K-major, N = 64 keys
      const uint32_t idesc_dq = make_idesc_bf16(kTile, kHd, 0, 1);     // dQ    : K-major A, MN-major B
      const uint32_t idesc_dkv = make_idesc_bf16(kTile, kHd, 1, 1);    // dK,dV : MN-major A and B
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      // Two queues served in whichever order their inputs arrive: the halves of S / dP of tile s_it, and the gradient
      // products of tile g_it.  The S queue is polled first: the math threads wait for nothing else.
      int s_it = 0, s_half = 0, g_it = 0;
      uint32_t idle = 0;
      while (g_it < n_tiles) {
        bool progressed = false;
        if (s_it < n_tiles) {
          const int s = s_it % 3;
          const bool ready = (s_half == 1 || mbar_test_wait(&qdo_full[s], (s_it / 3) & 1)) &&
                             (s_it == 0 || mbar_test_wait(&s_free[s_half], (s_it - 1) & 1));
          if (ready) {
            tc_fence_after_sync();
            const uint32_t qa = smem_u32(sQD + s * 2 * kTileBytes), doa = qa + kTileBytes;
            const uint32_t koff = s_half * 64 * 128;     // keys 64..127 start 64 rows (of 128 bytes) into the K / V tiles
            if (!(ablate & 8)) {
              umma_steps(tS + s_half * 64, qa, 16, 32, ka + koff, 16, 32, idesc_s, kHd / 16, false);      // Q K^T
              umma_steps(tDP + s_half * 64, doa, 16, 32, va + koff, 16, 32, idesc_s, kHd / 16, false);    // dO V^T
            }
            umma_commit(&s_full[s_half]);
            WS_STAMP(s_it, 8 + s_half);
            if (s_half == 1) ++s_it;
            s_half ^= 1;
            progressed = true;
          }
        }
        if (g_it < s_it) {
          const int s = g_it & 1;
          if (mbar_test_wait(&pds_full[s], (g_it >> 1) & 1) && (g_it < 2 || mbar_test_wait(&dq_free[s], ((g_it >> 1) & 1) ^ 1))) {
            tc_fence_after_sync();
            const int qb = g_it % 3;
            const uint32_t qa = smem_u32(sQD + qb * 2 * kTileBytes), doa = qa + kTileBytes;
            const uint32_t pa = smem_u32(sPst), dsa = smem_u32(sDSst + s * kPBytes);
            const uint32_t dq = tDQ + s * 64;
            // dV += P^T dO, dK += dS^T Q : A read MN-major (M = keys: two 64-key slabs), reduction over the 128 query rows
            if (!(ablate & 4)) {
              umma_steps(tDV, pa, kTileBytes, 2048, doa, 8192, 2048, idesc_dkv, 8, g_it > 0);
            }
            umma_commit(p_free);            // dV is the only reader of the P staging tile
            if (!(ablate & 4)) umma_steps(tDK, dsa, kTileBytes, 2048, qa, 8192, 2048, idesc_dkv, 8, g_it > 0);
            umma_commit(&qdo_free[qb]);    // dV and dK were the last readers of the Q / dO tiles: the tile after next can be fetched
            if (!(ablate & 4)) {
              // dQ = dS K : A = dS K-major (two slabs of 4 k-steps), B = K tile MN-major
              umma_steps(dq, dsa, 16, 32, ka, 8192, 2048, idesc_dq, 4, false);
              umma_steps(dq, dsa + kTileBytes, 16, 32, ka + 4 * 2048, 8192, 2048, idesc_dq, 4, true);
            }
            umma_commit(&grads_full[s]);
            WS_STAMP(g_it, 10);
            ++g_it;
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
        } else if (++idle > 4096) {      // a few microseconds of plain polling first: a sleep here delays every waiter
          if (*abort_word) break;
          if (idle > kWsIssuePolls) {
            *abort_word = 1;
            if (p.status) atomicCAS(p.status, 0, static_cast<int>(kTimeoutTmemEmpty));
            break;
          }
          __nanosleep(idle > 65536 ? 256 : 32);
        }
      }
    }
  } else if (warp < 8) {
    // ---- math threads --------------------------------------------------------------------------------------------
    // thread = (query row, half): half h owns key columns [32 c + 16 h, 32 c + 16 h + 16) of every 32-column chunk c, so all
    // 256 threads work through keys 0..63 (round 0) and then 64..127 (round 1) of the tile together
    const int half = warp >> 2;
    const int t = (warp & 3) * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const float kInf = __int_as_float(0x7f800000);
    const bool do_drop = p.dropout_p > 0.f;
    const DropRng rng(p.seed + ((do_drop && p.seed_dev) ? *p.seed_dev : 0ull),
                      (p.stream_id << 16) | static_cast<unsigned long long>(h), p.dropout_p);
    const float* drow_ptr = p.delta + static_cast<size_t>(h) * p.lse_stride + q_begin;
    const float* lrow_ptr = p.lse + static_cast<size_t>(h) * p.lse_stride + q_begin;
    float nxt_D = 0.f, nxt_lse2 = kInf;        // a row past the sequence: +inf makes every probability 0
    if (n_tiles > 0 && qt_first * kTile + t < q_len) {
      nxt_D = drow_ptr[qt_first * kTile + t];
      nxt_lse2 = lrow_ptr[qt_first * kTile + t] * 1.4426950408889634f;
    }
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int qt = qt_first + i, s = i & 1;
      const int q0 = q_begin + qt * kTile;
      const float Drow = nxt_D, lse2 = nxt_lse2;
      nxt_D = 0.f;
      nxt_lse2 = kInf;
      if (i + 1 < n_tiles && (qt + 1) * kTile + t < q_len) {     // requested a tile ahead: never waited for
        nxt_D = drow_ptr[(qt + 1) * kTile + t];
        nxt_lse2 = lrow_ptr[(qt + 1) * kTile + t] * 1.4426950408889634f;
      }
      uint8_t* sP = sPst;
      uint8_t* sDS = sDSst + s * kPBytes;
      const bool causal_here = p.causal != 0 && kt >= qt;    // tiles below the diagonal need no causal test
      const int q_pos = qt * kTile + t;
      const unsigned long long row_base = static_cast<unsigned long long>(q0 + t) * p.kstride + kt * kTile + half * 16;
      bool may_store = i < 1;
#pragma unroll 1
      for (int r = 0; r < 2 && ok; ++r) {
        ok = __all_sync(0xffffffffu, mbar_wait(&s_full[r], i & 1, abort_word, p.status, kTimeoutTmemFull));
        if (!ok) break;
        tc_fence_after_sync();
        WS_STAMP(i, r * 4);
        if (ablate & 1) {
          tc_fence_before_sync();
          mbar_arrive(&s_free[r]);
          if (!may_store) {
            ok = __all_sync(0xffffffffu, mbar_wait(p_free, (i - 1) & 1, abort_word, p.status, kTimeoutSmemEmpty)) &&
                 (i < 2 || __all_sync(0xffffffffu, mbar_wait(&ds_free[s], ((i >> 1) & 1) ^ 1, abort_word, p.status, kTimeoutSmemEmpty)));
            may_store = true;
          }
          continue;
        }
        const int c = 2 * r;
        const int c0a = c * 32 + half * 16, c0b = c0a + 32;
        uint32_t s0[16], d0[16], s1[16], d1[16];
        tmem_ld16(tS + lane_sel + c0a, s0);
        tmem_ld16(tDP + lane_sel + c0a, d0);
        tmem_ld16(tS + lane_sel + c0b, s1);
        tmem_ld16(tDP + lane_sel + c0b, d1);
        uint32_t km0 = 0xffffu, km1 = 0xffffu;
        if (do_drop) {   // the mask words are hashed while the TMEM loads are in flight
          km0 = drop_mask16(rng, row_base + c * 32);
          km1 = drop_mask16(rng, row_base + (c + 1) * 32);
        }
        tmem_ld_wait();
        WS_STAMP(i, r * 4 + 1);
        tc_fence_before_sync();
        mbar_arrive(&s_free[r]);       // this half of S / dP may be overwritten by the next query tile
        uint4 p0[2], e0[2], p1[2], e1[2];
        bwd_compute16(s0, d0, km0, do_drop, rng.scale, Drow, scale_log2, lse2, c0a, k_rows, causal_here, kt * kTile + c0a, q_pos,
                      p0, e0);
        bwd_compute16(s1, d1, km1, do_drop, rng.scale, Drow, scale_log2, lse2, c0b, k_rows, causal_here, kt * kTile + c0b, q_pos,
                      p1, e1);
        WS_STAMP(i, r * 4 + 2);
        if (!may_store) {
          // dV of the previous tile reads the P staging tile; dK / dQ of tile i - 2 read this dS staging tile, which then
          // held that tile's dQ until the TMA unit had read it
          ok = __all_sync(0xffffffffu, mbar_wait(p_free, (i - 1) & 1, abort_word, p.status, kTimeoutSmemEmpty)) &&
               (i < 2 || __all_sync(0xffffffffu, mbar_wait(&ds_free[s], ((i >> 1) & 1) ^ 1, abort_word, p.status, kTimeoutSmemEmpty)));
          if (!ok) break;
          may_store = true;
        }
        bwd_store16(p0, e0, c0a, t, sP, sDS);
        bwd_store16(p1, e1, c0b, t, sP, sDS);
        WS_STAMP(i, r * 4 + 3);
      }
      if (!ok) break;
      fence_async_smem();
      mbar_arrive(&pds_full[s]);
    }
  } else if (warp < 12) {
    // ---- dQ of every tile, then dK / dV ------------------------------------------------------------------------------
    const int wq = warp - 8;
    const int t = wq * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(wq * 32) << 16;
    const bool single_kt = k_len <= kTile;
    bool ok = true;
    for (int i = 0; i < n_tiles && ok; ++i) {
      const int s = i & 1;
      const int q0 = q_begin + (qt_first + i) * kTile;
      ok = __all_sync(0xffffffffu, mbar_wait(&grads_full[s], (i >> 1) & 1, abort_word, p.status, kTimeoutTmemFull));
      if (!ok) break;
      tc_fence_after_sync();
      WS_STAMP(i, 11);
      if (ablate & 2) {
        tc_fence_before_sync();
        mbar_arrive(&dq_free[s]);
        if (t == 0) mbar_arrive(&ds_free[s]);
        continue;
      }
      uint32_t r0[32], r1[32];
      tmem_ld32(tDQ + s * 64 + lane_sel, r0);
      tmem_ld32(tDQ + s * 64 + lane_sel + 32, r1);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&dq_free[s]);
      if (single_kt) {
        // the only key tile of its sequence: dQ is final, written as bf16 (the conversion pass skips such sequences)
        if (qt_first * kTile + i * kTile + t < q_len) {
          __nv_bfloat16* drow = p.dq + static_cast<size_t>(q0 + t) * p.ld_dq + static_cast<size_t>(h) * kHd;
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4) {
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int e = (g4 & 3) * 8 + 2 * j;
              o2[j] = __floats2bfloat162_rn(__uint_as_float(g4 < 4 ? r0[e] : r1[e]) * p.scale,
                                            __uint_as_float(g4 < 4 ? r0[e + 1] : r1[e + 1]) * p.scale);
            }
            reinterpret_cast<uint4*>(drow)[g4] = o;
          }
        }
        if (t == 0) mbar_arrive(&ds_free[s]);      // nothing was staged: the products' completion frees the tile
        continue;
      }
      // fp32 staging in the dS buffer of this tile (its products have completed): two [128 x 32] 128-byte-swizzled slabs.
      // Rows past the sequence hold exact zeros (their dS is zero), so the whole tile can be added.
      uint8_t* stage = sDSst + s * kPBytes;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        *reinterpret_cast<float4*>(stage + sw128_offset(t, g)) =
            make_float4(__uint_as_float(r0[g * 4]) * p.scale, __uint_as_float(r0[g * 4 + 1]) * p.scale,
                        __uint_as_float(r0[g * 4 + 2]) * p.scale, __uint_as_float(r0[g * 4 + 3]) * p.scale);
        *reinterpret_cast<float4*>(stage + kTileBytes + sw128_offset(t, g)) =
            make_float4(__uint_as_float(r1[g * 4]) * p.scale, __uint_as_float(r1[g * 4 + 1]) * p.scale,
                        __uint_as_float(r1[g * 4 + 2]) * p.scale, __uint_as_float(r1[g * 4 + 3]) * p.scale);
      }
      fence_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      WS_STAMP(i, 12);
      if (t == 0) {
        if (!(ablate & 32)) {
          tma_reduce_add_2d(&tmap_dq, stage, h * kHd, q0);
          tma_reduce_add_2d(&tmap_dq, stage + kTileBytes, h * kHd + 32, q0);
        }
        tma_store_commit();
        tma_store_wait_read();           // the staging tile has been read: the math threads may reuse it
        WS_STAMP(i, 13);
        mbar_arrive(&ds_free[s]);
      }
    }
    if (t == 0) tma_store_wait_all();
    const size_t col = static_cast<size_t>(h) * kHd;
    if (ok && n_tiles > 0) {
      // the last grads_full wait above covers every accumulation into dK and dV; dK carries the softmax scale that dS left out
      tc_fence_after_sync();
      ws_store_row(tDK + lane_sel, p.dk + static_cast<size_t>(k0 + t) * p.ld_dk + col, p.scale, t < k_rows);
      ws_store_row(tDV + lane_sel, p.dv + static_cast<size_t>(k0 + t) * p.ld_dv + col, 1.f, t < k_rows);
    } else if (n_tiles == 0 && t < k_rows) {
      // no query tile attends to this key tile: zero gradients
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      for (int g = 0; g < 8; ++g) {
        reinterpret_cast<uint4*>(p.dk + static_cast<size_t>(k0 + t) * p.ld_dk + col)[g] = z;
        reinterpret_cast<uint4*>(p.dv + static_cast<size_t>(k0 + t) * p.ld_dv + col)[g] = z;
      }
    }
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

int get_attn_bwd_ablation();

const char* launch_attn_bwd_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                               const CUtensorMap& tdq, const AttnArgs& a, dim3 grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(attn_bwd_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWsSmem);
    if (ce != cudaSuccess) return cudaGetErrorString(ce);
    configured = true;
  }
  attn_bwd_ws_kernel<<<grid, kWsThreads, kWsSmem, stream>>>(tq, tk, tv, tdo, tdq, a, get_attn_bwd_ablation());
  cudaError_t ce = cudaGetLastError();
  return ce == cudaSuccess ? nullptr : cudaGetErrorString(ce);
}

}  // namespace b200

// copies the time stamps of the last traced launch (ablation bit 128) to host memory; returns the number of values
int nmtg_attn_ws_trace(long long* out, int capacity) {
  const int n = b200::kWsTraceTiles * 16 < capacity ? b200::kWsTraceTiles * 16 : capacity;
  if (cudaMemcpyFromSymbol(out, b200::g_ws_trace, n * sizeof(long long)) != cudaSuccess) return -1;
  return n;
}
