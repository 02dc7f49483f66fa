// CTA-pair bf16 GEMM for sm_100a: two CTAs of a cluster (two SMs) cooperate on one 256 x BN output tile
// with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and its own HALF of the B tile, so
// per SM the shared-memory traffic (TMA writes + UMMA operand reads) per flop drops by a third compared
// with the single-CTA kernel, which is what keeps the tensor pipe fed at large tile sizes.
//
//   rank 0 (leader): TMA producer + UMMA issuer for the pair + epilogue of rows [m0, m0 + 128)
//   rank 1         : TMA producer for its operand halves       + epilogue of rows [m0 + 128, m0 + 256)
//
// Synchronisation (all mbarriers live in shared memory; remote ones are addressed through the cluster
// window, no broadcast forms are used anywhere):
//   full[s]       on the leader, count 1 + 2 x stage bytes: both CTAs' TMA loads complete_tx on it
//   empty[s]      on each CTA, signalled by two tcgen05.commit of the leader (local + peer address)
//   tmem_full[a]  on each CTA, same two-commit scheme after the last k-block of a tile
//   tmem_empty[a] on the leader, count 2 x 256: every epilogue thread of both CTAs arrives (peer: remote arrive)
// Every wait is bounded; all exits go through the final cluster barrier so a CTA never leaves while its peer
// may still touch its shared memory.
#include "gemm_common.cuh"

namespace b200 {

bool cached_tmap(CUtensorMap* out, const void* base, long rows, long cols, long ld, int br, int bc);
int num_sms();
int gemm_sms();

constexpr int kPairThreads = 32 * (2 + kEpilogueWarps);

template <int BN>
struct PairSmem {
  static constexpr int kABytes = BM * BK * 2;            // 16 KB : this CTA's 128 rows of A
  static constexpr int kBBytes = (BN / 2) * BK * 2;      // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 6 : 8;
  static constexpr int kStagingOffset = kStages * kStageBytes;          // 8 epilogue warps x [32 rows x 128 B]
  static constexpr int kStagingBytes = kEpilogueWarps * 32 * 128;
  static constexpr int kBarOffset = kStagingOffset + kStagingBytes;
  static constexpr int kTotal = kBarOffset + 512 + 1024;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into THIS CTA's shared memory that reports its bytes to an mbarrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <int BN, bool kTrace, uint32_t kFeat>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_out, const GemmArgs p, const GatherArgs g) {
  using S = PairSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + S::kStages;
  uint64_t* tmem_full = empty_bar + S::kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (p.N + BN - 1) / BN;
  const int num_kb_total = (p.K + BK - 1) / BK;
  const int kb_per_split = (num_kb_total + p.split_k - 1) / p.split_k;   // host guarantees no split is empty
  const int num_mn = num_m * num_n;
  const int num_tiles = num_mn * p.split_k;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  // Work distribution.  Default: whole (tile, split) units dealt round-robin.  p.stream_k (fp32 accumulating output
  // only): the (tile, k-block) pairs are laid end to end and every cluster takes one contiguous, equally long run of
  // them, which may end in the middle of a tile; partial tiles meet in the output through the red.add epilogue, so
  // no fix-up pass is needed and no cluster idles when the tile count is not a multiple of the cluster count.
  const long sk_total = static_cast<long>(num_mn) * num_kb_total;
  const long sk_per = sk_total / num_clusters, sk_rem = sk_total % num_clusters;
  const long sk_begin = cluster_id * sk_per + (cluster_id < sk_rem ? cluster_id : sk_rem);
  const long sk_end = sk_begin + sk_per + (cluster_id < sk_rem ? 1 : 0);
  const long first_work = p.stream_k ? sk_begin : cluster_id;
  auto next_work = [&](long& cursor, int& mn, int& kb_begin, int& kb_end) -> bool {
    if (!p.stream_k) {
      if (cursor >= num_tiles) return false;
      const int tile = static_cast<int>(cursor);
      mn = tile % num_mn;
      kb_begin = (tile / num_mn) * kb_per_split;
      kb_end = min(kb_begin + kb_per_split, num_kb_total);
      cursor += num_clusters;
      return true;
    }
    if (cursor >= sk_end) return false;
    mn = static_cast<int>(cursor / num_kb_total);
    kb_begin = static_cast<int>(cursor % num_kb_total);
    const long left = sk_end - cursor;
    kb_end = (kb_begin + left < num_kb_total) ? static_cast<int>(kb_begin + left) : num_kb_total;
    cursor += kb_end - kb_begin;
    return true;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < S::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 2 * 32 * kEpilogueWarps);
    }
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();      // barriers of both CTAs are initialised and TMEM is allocated before anyone proceeds
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) --------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long cursor = first_work;
      int mn, kb_begin, kb_end;
      // Sharded B operand: segments of the matrix that are known to have arrived in the local staging buffer
      // (K-major B: segment = BN / 2 rows, i.e. one CTA's half tile; MN-major B: segment = one 64-row k-block).
      uint32_t seg_seen[kGatherMaxSegs / 32] = {};
      auto seg_ready = [&](int sgm) -> bool {
        if (g.n_seg == 0 || sgm >= g.n_seg || ((seg_seen[sgm >> 5] >> (sgm & 31)) & 1u)) return true;
        const long left = g.units - static_cast<long>(sgm) * g.seg_units;
        const int need = left < g.seg_units ? static_cast<int>(left) : g.seg_units;
        const int* ctr = g.counters + 2 + sgm;
        for (uint32_t i = 0; i < B200_WAIT_POLLS; ++i) {
          if (ld_acquire_gpu(ctr) >= need) {
            fence_proxy_async_all();     // the copies were ordinary stores; the loads below go through the async proxy
            seg_seen[sgm >> 5] |= 1u << (sgm & 31);
            return true;
          }
          if (i > 16) {
            if (*abort_word) return false;
            __nanosleep(i > 4096 ? 256 : 32);
          }
        }
        *abort_word = 1;
        if (p.status) atomicCAS(p.status, 0, kTimeoutGather);
        return false;
      };
      while (ok && next_work(cursor, mn, kb_begin, kb_end)) {
        const int m0 = (mn % num_m) * (2 * BM) + static_cast<int>(rank) * BM;   // my 128 rows of the pair tile
        const int n0 = (mn / num_m) * BN + static_cast<int>(rank) * (BN / 2);   // my half of the B tile
        if (!p.b_mn_major && !seg_ready(n0 / (BN / 2))) { ok = false; break; }
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (p.b_mn_major && !seg_ready(kb)) { ok = false; break; }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word, p.status, kTimeoutSmemEmpty)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);   // the leader's barrier
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * S::kStageBytes);
          if (!p.a_mn_major) {
            tma_load_2d_pair(sa, &tmap_a, bar, kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmap_a, bar, m0 + j * 64, kb * BK);
          }
          if (!p.b_mn_major) {
            tma_load_2d_pair(sb, &tmap_b, bar, kb * BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(sb + j * (BK * 128), &tmap_b, bar, n0 + j * 64, kb * BK);
          }
          if (++stage == S::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- UMMA issuer (leader only) -------------------------------
    if (leader && lane == 0) {
      const uint32_t idesc = make_idesc_bf16(2 * BM, BN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, b_lbo = p.b_mn_major ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? (16 * 128) >> 4 : 32 >> 4;
      const uint32_t b_kstep = p.b_mn_major ? (16 * 128) >> 4 : 32 >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      // cycle counters for p.trace: [0] issuer loop, [1] waiting for a free accumulator, [2] waiting for operands,
      // [3] start of the loop until the first operands have landed
      const long long t_begin = kTrace ? clock64() : 0;
      long long t_wait_acc = 0, t_wait_ops = 0, t_first = 0;
      long cursor = first_work;
      int mn, kb_begin, kb_end;
      for (; ok && next_work(cursor, mn, kb_begin, kb_end); ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        long long t0 = kTrace ? clock64() : 0;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_word, p.status, kTimeoutTmemEmpty)) break;
        if (kTrace) t_wait_acc += clock64() - t0;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          t0 = kTrace ? clock64() : 0;
          if (!mbar_wait(&full_bar[stage], phase, abort_word, p.status, kTimeoutTmaFull)) { ok = false; break; }
          if (kTrace) {
            const long long t1 = clock64();
            t_wait_ops += t1 - t0;
            if (t_first == 0) t_first = t1 - t_begin;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
          const uint64_t adesc = make_smem_desc_sw128(sa, a_lbo, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sb, b_lbo, 1024);
          if (!kTrace || p.ablate != 3) {     // traced ablation 3: stream the operands only, no tensor-core work
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_bf16_pair(d_tmem, adesc + static_cast<uint64_t>(k * a_kstep), bdesc + static_cast<uint64_t>(k * b_kstep), idesc,
                             (kb > kb_begin || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 0));
          umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          if (++stage == S::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          umma_commit_pair(map_to_cta(smem_u32(&tmem_full[acc]), 0));
          umma_commit_pair(map_to_cta(smem_u32(&tmem_full[acc]), 1));
        }
      }
      if (kTrace && p.trace) {
        long long* tr = p.trace + cluster_id * 16;
        tr[0] = clock64() - t_begin;
        tr[1] = t_wait_acc;
        tr[2] = t_wait_ops;
        tr[3] = t_first;
      }
    }
  } else {
    // ------------------------------- epilogue (8 warps, both CTAs) ---------------------------
    const int q = warp & 3;
    const int chunk_par = (warp - 2) >> 2;
    const bool do_drop = p.dropout_p > 0.f;
    const DropRng rng(p.seed + ((do_drop && p.seed_dev) ? *p.seed_dev : 0ull), p.stream_id, p.dropout_p);
    int it = 0;
    // cycle counters for p.trace (first epilogue warp of the leader): [4] loop, [5] waiting for a finished accumulator,
    // [6] the last tile's epilogue (the part no later main loop can hide), [7] tiles
    const bool tracing = kTrace && p.trace != nullptr && leader && warp == 2 && lane == 0;
    const long long e_begin = tracing ? clock64() : 0;
    long long e_wait = 0, e_last = 0, e_drain = 0, e_chunks = 0, e_issue = 0;
    long cursor = first_work;
    int mn, kb_begin, kb_end;
    // ---- gather of a sharded B operand (fully sharded parameters), done by these warps WHILE they wait for
    // accumulators.  The matrix is a run of 4 KB blocks; the CTAs that are running claim four consecutive blocks at
    // a time from a shared cursor (a CTA that has not been scheduled yet holds nobody up, and the segments complete
    // in order), each thread moves 16 bytes of every claimed block (four peer loads in flight), then the blocks'
    // segment counters are raised.  Element e of the unit lives in rank e / piece_len's shard; a 16-byte group never
    // straddles two owners (pieces are multiples of 64 elements).  One round: thread 0 looks whether the awaited
    // accumulator is complete (then the epilogue goes first) and otherwise claims blocks; the verdict reaches the
    // other 255 threads through shared memory and a named barrier.
    __shared__ int s_claim[2];
    int claim_slot = 0;
    bool gather_left = g.n_seg > 0;
    const int gt = threadIdx.x - 64;
    auto gather_rounds = [&](uint64_t* wait_bar, uint32_t wait_phase) {
      while (gather_left) {
        if (gt == 0) {
          int c = -1;
          if (wait_bar == nullptr || !mbar_try_wait(wait_bar, wait_phase)) c = atomicAdd(g.counters + 1, 4);
          s_claim[claim_slot] = c;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpilogueWarps) : "memory");
        const long u0 = s_claim[claim_slot];
        claim_slot ^= 1;
        if (u0 < 0) return;                       // the accumulator is ready: epilogue first, gather again later
        if (u0 >= g.units || *abort_word) { gather_left = false; return; }
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (u0 + j < g.units) {
            const long e = g.unit_off + (u0 + j) * (kGatherBlockBytes / 2) + gt * 8;
            const int owner = static_cast<int>(e / g.piece_len);
            const long within = e - owner * g.piece_len;
            v[j] = *reinterpret_cast<const uint4*>(g.shards[owner] + g.shard_off + within);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (u0 + j < g.units) *reinterpret_cast<uint4*>(g.dst + (u0 + j) * (kGatherBlockBytes / 2) + gt * 8) = v[j];
        fence_proxy_async_all();
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpilogueWarps) : "memory");
        if (gt < 4 && u0 + gt < g.units) atomicAdd(g.counters + 2 + static_cast<int>((u0 + gt) / g.seg_units), 1);
      }
    };
    for (; next_work(cursor, mn, kb_begin, kb_end); ++it) {
      const int m0 = (mn % num_m) * (2 * BM) + static_cast<int>(rank) * BM;
      const int n0 = (mn / num_m) * BN;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const long long e0 = tracing ? clock64() : 0;
      gather_rounds(&tmem_full[acc], acc_phase);
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_word, p.status, kTimeoutTmemFull)) break;
      if (tracing) { e_last = clock64(); e_wait += e_last - e0; }
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      if ((kFeat & kEpiBf16) && p.tma_store) {
        // 64-column groups: both 32-column halves go to this warp's staging tile, one TMA store per group writes
        // full 128-byte lines (rows / columns outside the matrix are clipped by the copy engine)
        uint8_t* stage = smem + S::kStagingOffset + (warp - 2) * (32 * 128);
#pragma unroll 1
        for (int g = chunk_par; g < BN / 64; g += kEpilogueWarps / 4) {
          const int col0 = n0 + g * 64;
          if (col0 >= p.N || p.ablate >= 2) break;
          const long long c0 = tracing ? clock64() : 0;
          if (lane == 0) tma_store_wait_read();        // the previous store of this warp has drained its staging tile
          __syncwarp();
          const long long c1 = tracing ? clock64() : 0;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (col0 + half * 32 < p.N)
              gemm_epilogue_chunk<kFeat>(p, rng, do_drop, row, row_ok, col0 + half * 32,
                                  tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + g * 64 + half * 32,
                                  stage + lane * 128, half, lane);
          }
          const long long c2 = tracing ? clock64() : 0;
          fence_async_smem();
          __syncwarp();
          if ((kFeat & kEpiColsum) && p.colsum) {
            // column sums of the staged 32 x 64 tile: lane l owns columns 2l, 2l+1 (one 32-bit word per row; the
            // swizzle keeps the 32 lanes on 32 different banks), rows outside the matrix are skipped
            const int rows_here = min(32, p.M - (m0 + q * 32));
            float s0 = 0.f, s1 = 0.f;
            for (int r = 0; r < rows_here; ++r) {
              const uint32_t w = *reinterpret_cast<const uint32_t*>(stage + r * 128 + ((((lane >> 2) ^ (r & 7)) << 4) | ((lane & 3) << 2)));
              const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
              s0 += f.x;
              s1 += f.y;
            }
            const int c = col0 + 2 * lane;
            if (c < p.N) atomicAdd(p.colsum + c, s0);
            if (c + 1 < p.N) atomicAdd(p.colsum + c + 1, s1);
          }
          if (lane == 0) {
            tma_store_2d(&tmap_out, stage, col0, m0 + q * 32);
            tma_store_commit();
          }
          if (tracing) {
            e_drain += c1 - c0;
            e_chunks += c2 - c1;
            e_issue += clock64() - c2;
          }
        }
      } else {
#pragma unroll 1
        for (int c = chunk_par; c < BN / 32; c += kEpilogueWarps / 4) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N || p.ablate >= 2) break;
          gemm_epilogue_chunk<kFeat>(p, rng, do_drop, row, row_ok, col0, tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32);
        }
      }
      tc_fence_before_sync();
      mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
    }
    gather_rounds(nullptr, 0);      // blocks that nobody has claimed yet (none, unless this CTA ran out of tiles early)
    if (p.tma_store && lane == 0) tma_store_wait_all();   // staging must outlive the copies that read it
    if (tracing) {
      long long* tr = p.trace + cluster_id * 16;
      const long long e_end = clock64();
      tr[4] = e_end - e_begin;
      tr[5] = e_wait;
      tr[6] = e_end - e_last;
      tr[7] = it;
      tr[8] = e_drain;       // waiting for the previous TMA store to release the staging tile
      tr[9] = e_chunks;      // accumulator loads, arithmetic, staging writes
      tr[10] = e_issue;      // proxy fence + issuing the store
    }
  }

  // ------------------------------- teardown --------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_word) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();      // the peer may still signal barriers in my shared memory until it gets here
  if (warp == 1) {
    tc_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
  if (g.n_seg > 0 && threadIdx.x == 0) {
    // the last CTA to leave puts the counters back to zero for the next launch that uses them (every CTA has
    // finished its tiles by now, so nobody polls them any more)
    __threadfence();
    if (atomicAdd(g.counters, 1) == static_cast<int>(gridDim.x) - 1) {
      for (int i = 0; i < g.n_seg; ++i) g.counters[2 + i] = 0;
      g.counters[0] = 0;
      g.counters[1] = 0;
      __threadfence();
    }
  }
}

template <int BN, bool kTrace, uint32_t kFeat>
static const char* launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmArgs& args, int grid,
                               cudaStream_t stream, const GatherArgs& g) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<BN, kTrace, kFeat>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem<BN>::kTotal);
    if (e != cudaSuccess) return cudaGetErrorString(e);
    configured = true;
  }
  gemm_pair_kernel<BN, kTrace, kFeat><<<grid, kPairThreads, PairSmem<BN>::kTotal, stream>>>(ta, tb, tc, args, g);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

// CTA-pair path; BN = 256 or 128; a.split_k splits must all be non-empty.  Returns nullptr on success.
int g_pair_generic_epilogue = 0;   // gemm variant 31: always run the general epilogue (30 = specialised, default)
int g_pair_tma_store = 1;     // set to 0 (gemm variant 20) to force per-thread global stores, for A/B measurements

// True when the CTA-pair kernel can gather this B operand itself (see GatherArgs); fills `g`.
bool plan_pair_gather(const GemmDesc* d, int bn, GatherArgs* g) {
  *g = GatherArgs{};
  const NmtgGather* src = d->gather;
  if (!src) return false;
  const long row_len = d->b_mn_major ? d->N : d->K;          // contiguous matrix: ldb == row length
  const long rows = d->b_mn_major ? d->K : d->N;
  if (d->ldb != row_len) return false;
  const long bytes = rows * row_len * 2;
  const long seg_rows = d->b_mn_major ? BK : bn / 2;
  const long seg_bytes = seg_rows * row_len * 2;
  if (bytes % kGatherBlockBytes || seg_bytes % kGatherBlockBytes) return false;
  const long n_seg = (rows + seg_rows - 1) / seg_rows;
  if (n_seg > kGatherMaxSegs || src->world < 1 || src->world > 16 || (src->piece_len % 64) || (src->unit_off % 8) ||
      (src->shard_off % 8) || !src->counters)
    return false;
  g->n_seg = static_cast<int>(n_seg);
  g->rank = src->rank; g->world = src->world;
  for (int i = 0; i < src->world; ++i) g->shards[i] = src->shards[i];
  g->shard_off = src->shard_off; g->piece_len = src->piece_len; g->unit_off = src->unit_off;
  g->dst = reinterpret_cast<unsigned short*>(const_cast<void*>(d->b));
  g->units = bytes / kGatherBlockBytes;
  g->seg_units = static_cast<int>(seg_bytes / kGatherBlockBytes);
  g->counters = src->counters;
  return true;
}

// Stand-alone copy of a sharded B operand into its staging place, for the GEMM paths that cannot gather in-kernel.
__global__ void __launch_bounds__(256) gather_copy_kernel(const NmtgGather g, unsigned short* __restrict__ dst, long n8) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long e = g.unit_off + i * 8;
    const int owner = static_cast<int>(e / g.piece_len);
    const long within = e - owner * g.piece_len;
    reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(g.shards[owner] + g.shard_off + within);
  }
}

const char* launch_gather_copy(const GemmDesc* d, cudaStream_t stream) {
  const NmtgGather* g = d->gather;
  const long row_len = d->b_mn_major ? d->N : d->K, rows = d->b_mn_major ? d->K : d->N;
  if (d->ldb != row_len) return "gemm: a sharded operand must be contiguous";
  const long n = rows * row_len;
  if ((n % 8) || (g->unit_off % 8) || (g->piece_len % 8) || (g->shard_off % 8) || g->world < 1 || g->world > 16)
    return "gemm: sharded operand offsets must be multiples of 8 elements";
  long blocks = (n / 8 + 255) / 256;
  if (blocks > 2L * num_sms()) blocks = 2L * num_sms();
  gather_copy_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(*g, reinterpret_cast<unsigned short*>(const_cast<void*>(d->b)), n / 8);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* launch_gemm_pair(const GemmDesc* d, const GemmArgs& a, int bn, cudaStream_t stream) {
  GatherArgs g;
  if (d->gather && !plan_pair_gather(d, bn, &g)) return "gemm: this sharded operand cannot be gathered inside the kernel";
  if (!d->gather) g = GatherArgs{};
  CUtensorMap ta, tb;
  bool ok;
  if (!d->a_mn_major) ok = cached_tmap(&ta, d->a, d->M, d->K, d->lda, BM, BK);
  else ok = cached_tmap(&ta, d->a, d->K, d->M, d->lda, BK, 64);
  if (!ok) return "gemm: cuTensorMapEncodeTiled failed for A";
  if (!d->b_mn_major) ok = cached_tmap(&tb, d->b, d->N, d->K, d->ldb, bn / 2, BK);
  else ok = cached_tmap(&tb, d->b, d->K, d->N, d->ldb, BK, 64);
  if (!ok) return "gemm: cuTensorMapEncodeTiled failed for B";
  // bf16 results leave through shared memory + TMA stores when nothing else has to be written per element
  GemmArgs args = a;
  CUtensorMap tc = ta;
  args.tma_store = 0;
  if (!d->out_fp32 && a.split_k == 1 && d->preact == nullptr && (d->ld_out % 8) == 0 && (g_pair_tma_store || a.colsum)) {
    if (cached_tmap(&tc, d->out, d->M, d->N, d->ld_out, 32, 64)) args.tma_store = 1;
    else tc = ta;
  }
  if (a.colsum && !args.tma_store) return "gemm: the column-sum output needs the bf16 TMA-store epilogue (no split-K, no pre-activation)";
  const long tiles = static_cast<long>((d->M + 2 * BM - 1) / (2 * BM)) * ((d->N + bn - 1) / bn) * a.split_k;
  const int max_clusters = gemm_sms() / 2;
  const int clusters = a.stream_k ? max_clusters : static_cast<int>(tiles < max_clusters ? tiles : max_clusters);
  if (bn != 256) return launch_pair<128, false, kEpiAll>(ta, tb, tc, args, clusters * 2, stream, g);
  if (args.trace != nullptr) return launch_pair<256, true, kEpiAll>(ta, tb, tc, args, clusters * 2, stream, g);
  // the specialised epilogues of the shapes a training step is made of; anything else takes the general kernel
  constexpr uint32_t kPlain = kEpiBf16;
  constexpr uint32_t kFc1 = kEpiBf16 | kEpiBias | kEpiActFwd | kEpiDrop | kEpiMaskOut;
  constexpr uint32_t kOutRes = kEpiBf16 | kEpiBias | kEpiDrop | kEpiRes;
  constexpr uint32_t kDgradMask = kEpiBf16 | kEpiMaskBwd | kEpiColsum;
  constexpr uint32_t kAccum = kEpiF32;
  // GELU / SiLU feed-forward blocks (speech and pretrained-decoder models) keep the pre-activation instead of sign bits
  constexpr uint32_t kFc1Preact = kEpiBf16 | kEpiBias | kEpiActFwd | kEpiDrop | kEpiPreact;
  constexpr uint32_t kDgradAct = kEpiBf16 | kEpiActBwd | kEpiDrop;
  const uint32_t need = g_pair_generic_epilogue ? kEpiAll : gemm_epilogue_features(args);
  const int grid = clusters * 2;
  if ((need & ~kPlain) == 0) return launch_pair<256, false, kPlain>(ta, tb, tc, args, grid, stream, g);
  if ((need & ~kAccum) == 0) return launch_pair<256, false, kAccum>(ta, tb, tc, args, grid, stream, g);
  if ((need & ~kDgradMask) == 0) return launch_pair<256, false, kDgradMask>(ta, tb, tc, args, grid, stream, g);
  if ((need & ~kOutRes) == 0) return launch_pair<256, false, kOutRes>(ta, tb, tc, args, grid, stream, g);
  if ((need & ~kFc1) == 0) return launch_pair<256, false, kFc1>(ta, tb, tc, args, grid, stream, g);
  if ((need & ~kFc1Preact) == 0) return launch_pair<256, false, kFc1Preact>(ta, tb, tc, args, grid, stream, g);
  if ((need & ~kDgradAct) == 0) return launch_pair<256, false, kDgradAct>(ta, tb, tc, args, grid, stream, g);
  return launch_pair<256, false, kEpiAll>(ta, tb, tc, args, grid, stream, g);
}

}  // namespace b200
