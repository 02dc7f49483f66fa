// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128-byte swizzle) ->
// tcgen05.mma with fp32 accumulators in TMEM -> fused epilogue read back with tcgen05.ld.
//
//   C[M,N] = epilogue( alpha * sum_k A(m,k) * B(n,k) )
//
// A and B may each be stored "K-major" (row = M/N index, K contiguous; the layout of activations X[M,K]
// and of Linear weights W[N,K]) or "MN-major" (row = K index, M/N contiguous), so the same mainloop
// serves forward (X W^T), data-gradient (dY W) and weight-gradient (dY^T X) products without any
// transposed copy.  Roles: warp 0 = TMA producer, warp 1 = UMMA issuer (owns TMEM), warps 2..5 =
// epilogue.  Two accumulator buffers in TMEM let the epilogue of tile i overlap the mainloop of tile
// i+1.  Optional split-K (weight gradients of small matrices) accumulates with vector red.add into an
// fp32 output.
//
// Replaces the cuBLAS / cuBLASLt GEMM + separate element-wise kernels of the reference
// (onmt/modules/extensions/mlp/mlp_relu_cuda.cu:82-190,445-1292; mlp_blaslt/mlp_gelu_cuda.cu:212-471;
// multihead_attn/self_multihead_attn_cuda.cu:91,284; dropout_add/dropout.h:21-160).
#include "gemm_common.cuh"

#include <mutex>
#include <unordered_map>
#include <string>
#include <cstring>
#include <cstdio>

namespace b200 {

constexpr int kGemmThreads = 32 * (2 + kEpilogueWarps);

template <int BN>
struct GemmSmem {
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;  // barriers + alignment slack
};

template <int BN, uint32_t kFeat>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmArgs p) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::kBarOffset);
  uint64_t* empty_bar = full_bar + S::kStages;
  uint64_t* tmem_full = empty_bar + S::kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_kb_total = (p.K + BK - 1) / BK;
  const int kb_per_split = (num_kb_total + p.split_k - 1) / p.split_k;
  const int num_tiles = num_m * num_n * p.split_k;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 32 * kEpilogueWarps);
    }
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * BN);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mn = tile % (num_m * num_n);
        const int ks = tile / (num_m * num_n);
        const int m0 = (mn % num_m) * BM;
        const int n0 = (mn / num_m) * BN;
        const int kb_begin = ks * kb_per_split;
        const int kb_end = min(kb_begin + kb_per_split, num_kb_total);
        for (int kb = kb_begin; kb < kb_end; ++kb) {  // an empty split range issues nothing
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word, p.status, kTimeoutSmemEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          mbar_expect_tx(&full_bar[stage], S::kStageBytes);
          if (!p.a_mn_major) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tmap_a, &full_bar[stage], m0 + j * 64, kb * BK);
          }
          if (!p.b_mn_major) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tmap_b, &full_bar[stage], n0 + j * 64, kb * BK);
          }
          if (++stage == S::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- UMMA issuer ---------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, b_lbo = p.b_mn_major ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? (16 * 128) >> 4 : 32 >> 4;  // descriptor units of 16 B
      const uint32_t b_kstep = p.b_mn_major ? (16 * 128) >> 4 : 32 >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int ks = tile / (num_m * num_n);
        const int kb_begin = ks * kb_per_split;
        const int kb_end = min(kb_begin + kb_per_split, num_kb_total);
        if (kb_begin >= kb_end) continue;  // empty split range: no accumulator is produced
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_word, p.status, kTimeoutTmemEmpty)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_word, p.status, kTimeoutTmaFull)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
          const uint64_t adesc = make_smem_desc_sw128(sa, a_lbo, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sb, b_lbo, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_bf16(d_tmem, adesc + static_cast<uint64_t>(k * a_kstep), bdesc + static_cast<uint64_t>(k * b_kstep),
                      idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == S::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tmem_full[acc]);
        ++it;
      }
    }
  } else {
    // ------------------------------- epilogue (8 warps) --------------------------------------
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int chunk_par = (warp - 2) >> 2;  // 0 / 1: which interleaved half of the column chunks
    const bool do_drop = p.dropout_p > 0.f;
    const DropRng rng(p.seed + ((do_drop && p.seed_dev) ? *p.seed_dev : 0ull), p.stream_id, p.dropout_p);
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int mn = tile % (num_m * num_n);
      const int m0 = (mn % num_m) * BM;
      const int n0 = (mn / num_m) * BN;
      {
        const int kb_begin = (tile / (num_m * num_n)) * kb_per_split;
        if (kb_begin >= min(kb_begin + kb_per_split, num_kb_total)) continue;
      }
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_word, p.status, kTimeoutTmemFull)) break;
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = chunk_par; c < BN / 32; c += kEpilogueWarps / 4) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // warp-uniform
        gemm_epilogue_chunk<kFeat>(p, rng, do_drop, row, row_ok, col0,
                            tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32);
      }
      tc_fence_before_sync();
      mbar_arrive(&tmem_empty[acc]);
      ++it;
    }
  }

  // ------------------------------- teardown ------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_word) {
    // give copies that may still be in flight a bounded time to land before shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 2-D bf16 row-major tensor [rows, cols] with leading dimension ld (elements); box = [box_rows, box_cols].
static bool make_tmap_2d(CUtensorMap* out, const void* base, long rows, long cols, long ld, int box_rows, int box_cols,
                         bool f32, bool bind_context = true);
bool make_tmap_bf16_2d(CUtensorMap* out, const void* base, long rows, long cols, long ld, int box_rows,
                       int box_cols) {
  return make_tmap_2d(out, base, rows, cols, ld, box_rows, box_cols, false);
}
// Descriptor built straight into `out`: no cache, no lock, and no runtime call of its own.  The calling thread must
// already have a current context (cudaSetDevice binds the primary one).
bool make_tmap_2d_nobind(CUtensorMap* out, const void* base, long rows, long cols, long ld, int box_rows, int box_cols,
                         bool f32) {
  return make_tmap_2d(out, base, rows, cols, ld, box_rows, box_cols, f32, false);
}
static bool make_tmap_2d(CUtensorMap* out, const void* base, long rows, long cols, long ld, int box_rows, int box_cols,
                         bool f32, bool bind_context) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  // The encoder is a driver entry point and needs a current context.  A thread that has issued no runtime call yet
  // (autograd's backward thread when the first thing it does is build a descriptor) has none: bind the primary one.
  static thread_local bool context_bound = false;
  if (bind_context && !context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * (f32 ? 4 : 2)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "nmtgminor_b200: cuTensorMapEncodeTiled failed with CUresult %d (base %p, rows %ld, cols %ld, ld %ld, box %d x %d)\n",
            static_cast<int>(r), base, rows, cols, ld, box_rows, box_cols);
  return r == CUDA_SUCCESS;
}

struct TmapKey {
  const void* base;
  long rows, cols, ld;
  int br, bc;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && br == o.br && bc == o.bc;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ static_cast<size_t>(k.rows);
    h = h * 1000003u ^ static_cast<size_t>(k.cols);
    h = h * 1000003u ^ static_cast<size_t>(k.ld);
    h = h * 1000003u ^ static_cast<size_t>(k.br * 1024 + k.bc);
    return h;
  }
};

bool cached_tmap(CUtensorMap* out, const void* base, long rows, long cols, long ld, int br, int bc) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey k{base, rows, cols, ld, br, bc};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(k);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  if (!make_tmap_bf16_2d(out, base, rows, cols, ld, br, bc)) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(k, *out);
  return true;
}

// fp32 matrix, 128-byte-swizzled boxes (box_cols * 4 bytes <= 128); same cache, told apart by a negated column box
bool cached_tmap_f32(CUtensorMap* out, const void* base, long rows, long cols, long ld, int br, int bc) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey k{base, rows, cols, ld, br, -bc};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(k);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  if (!make_tmap_2d(out, base, rows, cols, ld, br, bc, true)) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(k, *out);
  return true;
}

// SMs that the persistent GEMM kernels leave free (for communication kernels that run beside them); even, set
// through nmtg_set_gemm_variant(60 + n).
static int g_gemm_sm_reserve = 0;
int gemm_sms();
static int g_num_sms = 0;
static int g_sm_reserve = 0;   // SMs that every kernel of this library leaves free (nmtg_set_sm_reserve)
// Number of SMs that the launchers size their grids for: the device's SMs minus the ones set aside for the
// communication kernels that run beside the backward pass.
int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int n = g_num_sms - g_sm_reserve;
  return n < 2 ? 2 : n;
}
void set_sm_reserve(int n) { g_sm_reserve = n < 0 ? 0 : (n & ~1); }

int gemm_sms() {
  const int n = num_sms() - g_gemm_sm_reserve;
  return n < 2 ? 2 : n;
}

template <int BN, uint32_t kFeat = kEpiAll>
static const char* launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args, int grid,
                               cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, kFeat>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GemmSmem<BN>::kTotal);
    if (e != cudaSuccess) return cudaGetErrorString(e);
    configured = true;
  }
  gemm_tcgen05_kernel<BN, kFeat><<<grid, kGemmThreads, GemmSmem<BN>::kTotal, stream>>>(ta, tb, args);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace b200

namespace b200 {
const char* launch_gemm_pair(const GemmDesc* d, const GemmArgs& a, int bn, cudaStream_t stream);
const char* launch_gather_copy(const GemmDesc* d, cudaStream_t stream);
bool plan_pair_gather(const GemmDesc* d, int bn, GatherArgs* g);
}
using namespace b200;

static int g_gemm_variant = 0;   // 0 = automatic, 1 = single-CTA kernel only, 2 = CTA-pair kernel whenever M > 128
static int g_fused_gather = 1;   // 0 (variant 50): sharded operands are always copied by a launch of their own (A/B baseline)
static long long* g_gemm_trace = nullptr;   // see nmtg_set_gemm_trace
static int g_stream_k = 1;       // gemm variant 40 switches the equal-run work split of weight gradients off, 41 on
static int g_gemm_ablate = 0;    // profiling aid, see GemmArgs::ablate; variants 10 / 11 / 12 select ablation 0 / 1 / 2
namespace b200 {
extern int g_pair_tma_store;
extern int g_pair_generic_epilogue;
}
void nmtg_set_gemm_trace(long long* buf) { g_gemm_trace = buf; }
void nmtg_set_sm_reserve(int n) { b200::set_sm_reserve(n); }

void nmtg_set_gemm_variant(int v) {
  if (v >= 60 && v < 124) b200::g_gemm_sm_reserve = (v - 60) & ~1;
  else if (v == 50 || v == 51) g_fused_gather = v - 50;
  else if (v == 40 || v == 41) g_stream_k = v - 40;
  else if (v == 30 || v == 31) b200::g_pair_generic_epilogue = v - 30;
  else if (v == 20 || v == 21) b200::g_pair_tma_store = v - 20;   // 20: per-thread stores, 21: TMA-store epilogue (default)
  else if (v >= 10) g_gemm_ablate = v - 10;
  else g_gemm_variant = v;
}

// Returns nullptr on success, else a static error string.
const char* nmtg_gemm_bf16(const GemmDesc* d, cudaStream_t stream) {
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return nullptr;
  if ((d->lda % 8) || (d->ldb % 8)) return "gemm: leading dimensions must be multiples of 8 elements";
  if ((reinterpret_cast<uintptr_t>(d->a) & 15) || (reinterpret_cast<uintptr_t>(d->b) & 15))
    return "gemm: operand base addresses must be 16-byte aligned";
  if (d->dropout_p > 0.f && (d->N % 4)) return "gemm: dropout epilogue needs N % 4 == 0";
  if ((d->ld_out % 8) || (reinterpret_cast<uintptr_t>(d->out) & 15)) return "gemm: output must be 16-byte aligned";
  GemmArgs a;
  a.M = d->M; a.N = d->N; a.K = d->K;
  a.a_mn_major = d->a_mn_major; a.b_mn_major = d->b_mn_major;
  a.alpha = d->alpha;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(d->bias);
  a.residual = reinterpret_cast<const __nv_bfloat16*>(d->residual); a.ld_res = d->ld_res;
  a.aux = reinterpret_cast<const __nv_bfloat16*>(d->aux); a.ld_aux = d->ld_aux;
  a.out = d->out; a.ld_out = d->ld_out; a.out_fp32 = d->out_fp32; a.accumulate = d->accumulate;
  a.preact = reinterpret_cast<__nv_bfloat16*>(d->preact);
  a.mask = reinterpret_cast<uint32_t*>(d->mask); a.ld_mask = d->ld_mask;
  a.colsum = d->colsum;
  a.ablate = g_gemm_ablate;
  a.stream_k = 0;
  a.trace = g_gemm_trace;
  if (d->act == kActMaskBwd && !d->mask) return "gemm: the mask-backward epilogue needs a mask";
  a.act = d->act; a.dropout_p = d->dropout_p; a.seed = d->seed; a.stream_id = d->stream_id; a.seed_dev = d->seed_dev;
  a.status = d->status;

  // A sharded B operand (d->gather) is pulled in by the CTA-pair kernel itself; every other path copies it first.
  GemmDesc unfused;
  auto gather_first = [&]() -> const char* {
    const char* e = launch_gather_copy(d, stream);
    if (e) return e;
    unfused = *d;
    unfused.gather = nullptr;
    d = &unfused;
    return nullptr;
  };
  const int sms = gemm_sms();
  const int num_kb = (d->K + BK - 1) / BK;
  auto fix_split = [&](int split) {   // largest split <= requested whose last part is not empty
    if (split > num_kb) split = num_kb;
    while (split > 1 && (split - 1) * ((num_kb + split - 1) / split) >= num_kb) --split;
    return split < 1 ? 1 : split;
  };
  // ---- skinny problems (incremental decoding: a few hundred rows): the weight matrix is streamed once, so the
  // only lever is the number of CTAs pulling it in; take the widest tile that still gives every SM a tile,
  // down to 64 columns
  const bool skinny = g_gemm_variant == 0 && d->M <= 512 && !d->out_fp32 && d->force_bn == 0 && d->split_k <= 1 && !d->colsum;
  if (skinny) {
    if (d->gather) { const char* e = gather_first(); if (e) return e; }
    const int num_m = (d->M + BM - 1) / BM;
    int bn = 64;
    if (static_cast<long>(num_m) * ((d->N + 255) / 256) >= sms) bn = 256;
    else if (static_cast<long>(num_m) * ((d->N + 127) / 128) >= sms) bn = 128;
    a.split_k = 1;
    CUtensorMap ta, tb;
    bool ok;
    if (!d->a_mn_major) ok = cached_tmap(&ta, d->a, d->M, d->K, d->lda, BM, BK);
    else ok = cached_tmap(&ta, d->a, d->K, d->M, d->lda, BK, 64);
    if (!ok) return "gemm: cuTensorMapEncodeTiled failed for A";
    if (!d->b_mn_major) ok = cached_tmap(&tb, d->b, d->N, d->K, d->ldb, bn, BK);
    else ok = cached_tmap(&tb, d->b, d->K, d->N, d->ldb, BK, 64);
    if (!ok) return "gemm: cuTensorMapEncodeTiled failed for B";
    const long tiles = static_cast<long>(num_m) * ((d->N + bn - 1) / bn);
    const int grid = static_cast<int>(tiles < sms ? tiles : sms);
    // decoding steps are latency bound: short specialised epilogues (see gemm_common.cuh) for their two shapes
    constexpr uint32_t kLinear = kEpiBf16 | kEpiBias | kEpiRes;
    constexpr uint32_t kActivated = kEpiBf16 | kEpiBias | kEpiActFwd;
    const uint32_t need = b200::g_pair_generic_epilogue ? kEpiAll : gemm_epilogue_features(a);
    if ((need & ~kLinear) == 0) {
      if (bn == 256) return launch_gemm<256, kLinear>(ta, tb, a, grid, stream);
      if (bn == 128) return launch_gemm<128, kLinear>(ta, tb, a, grid, stream);
      return launch_gemm<64, kLinear>(ta, tb, a, grid, stream);
    }
    if ((need & ~kActivated) == 0) {
      if (bn == 256) return launch_gemm<256, kActivated>(ta, tb, a, grid, stream);
      if (bn == 128) return launch_gemm<128, kActivated>(ta, tb, a, grid, stream);
      return launch_gemm<64, kActivated>(ta, tb, a, grid, stream);
    }
    if (bn == 256) return launch_gemm<256>(ta, tb, a, grid, stream);
    if (bn == 128) return launch_gemm<128>(ta, tb, a, grid, stream);
    return launch_gemm<64>(ta, tb, a, grid, stream);
  }
  // ---- CTA-pair kernel (256-row tiles): the default for everything but very small M ----------------
  if (d->colsum && d->M <= BM) return "gemm: the column-sum output needs more than 128 rows (CTA-pair kernel)";
  if ((g_gemm_variant != 1 || d->colsum) && d->M > BM) {
    int bn = (d->N > 128) ? 256 : 128;
    if (d->force_bn == 128 || d->force_bn == 256) bn = d->force_bn;
    if (d->gather) {
      GatherArgs probe;
      if (g_fused_gather == 0 || !plan_pair_gather(d, bn, &probe)) { const char* e = gather_first(); if (e) return e; }
    }
    const long tiles = static_cast<long>((d->M + 2 * BM - 1) / (2 * BM)) * ((d->N + bn - 1) / bn);
    int split = 1;
    if (d->split_k > 0) split = d->split_k;
    else if (d->out_fp32 && d->allow_split_k) {
      const int clusters = sms / 2;
      while (tiles * split * 2 <= clusters && num_kb / (split * 2) >= 8) split *= 2;
    }
    if (split > 1 && !d->out_fp32) return "gemm: split-K needs an fp32 output";
    a.split_k = fix_split(split);
    // weight gradients (fp32, accumulating): when the tiles do not fill the clusters evenly, hand every cluster an
    // equal run of k-blocks instead of whole tiles
    // (measured: a gain where whole tiles leave a fifth or more of the clusters idle, and for many-wave problems such
    // as the generator; a loss of 5-15 % from the extra partial-tile reductions where the tiles nearly fill a wave)
    const int clusters = sms / 2;
    const long units = tiles * a.split_k;
    const double wave_fill = static_cast<double>(units) / (static_cast<double>((units + clusters - 1) / clusters) * clusters);
    if (g_stream_k && d->out_fp32 && d->accumulate && d->allow_split_k && d->split_k <= 0 && (units % clusters) != 0 &&
        tiles * num_kb / clusters >= 16 && (wave_fill < 0.8 || tiles >= 4L * clusters)) {
      a.split_k = 1;
      a.stream_k = 1;
    }
    return launch_gemm_pair(d, a, bn, stream);
  }
  // ---- single-CTA kernel: tile width 256 when it does not waste a wave, else 128 -------------------
  if (d->gather) { const char* e = gather_first(); if (e) return e; }
  const int num_m = (d->M + BM - 1) / BM;
  int bn = 256;
  if (d->N <= 128 || ((d->N % 256) != 0 && (d->N % 128) == 0)) bn = 128;
  {
    long t256 = static_cast<long>(num_m) * ((d->N + 255) / 256), t128 = static_cast<long>(num_m) * ((d->N + 127) / 128);
    auto waves_eff = [&](long t) { long w = (t + sms - 1) / sms; return static_cast<double>(t) / (w * sms); };
    if (bn == 256 && waves_eff(t128) > waves_eff(t256) + 0.15) bn = 128;
  }
  if (d->force_bn == 128 || d->force_bn == 256) bn = d->force_bn;
  const int num_n = (d->N + bn - 1) / bn;
  int split = 1;
  if (d->split_k > 0) split = d->split_k;
  else if (d->out_fp32 && d->allow_split_k) {
    long tiles = static_cast<long>(num_m) * num_n;
    while (tiles * split * 2 <= sms && num_kb / (split * 2) >= 8) split *= 2;
  }
  if (split > 1 && !d->out_fp32) return "gemm: split-K needs an fp32 output";
  a.split_k = fix_split(split);

  CUtensorMap ta, tb;
  bool ok;
  if (!d->a_mn_major) ok = cached_tmap(&ta, d->a, d->M, d->K, d->lda, BM, BK);
  else ok = cached_tmap(&ta, d->a, d->K, d->M, d->lda, BK, 64);
  if (!ok) return "gemm: cuTensorMapEncodeTiled failed for A";
  if (!d->b_mn_major) ok = cached_tmap(&tb, d->b, d->N, d->K, d->ldb, bn, BK);
  else ok = cached_tmap(&tb, d->b, d->K, d->N, d->ldb, BK, 64);
  if (!ok) return "gemm: cuTensorMapEncodeTiled failed for B";

  long tiles = static_cast<long>(num_m) * num_n * split;
  int grid = static_cast<int>(tiles < sms ? tiles : sms);
  if (bn == 256) return launch_gemm<256>(ta, tb, a, grid, stream);
  return launch_gemm<128>(ta, tb, a, grid, stream);
}
