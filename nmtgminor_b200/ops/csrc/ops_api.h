// C launch interface of the sm_100a kernels.  Pointers are device pointers; every launcher enqueues on
// `stream` and returns nullptr on success or a static error string.  No launcher allocates memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

enum NmtgAct : int {
  kActNone = 0,
  kActRelu = 1,
  kActGelu = 2,   // erf form
  kActSilu = 3,
  kActReluBwd = 5,  // out = acc * 1[aux > 0]           (aux = ReLU output, after dropout)
  kActGeluBwd = 6,  // out = acc * gelu'(aux)           (aux = pre-activation)
  kActSiluBwd = 7,  // out = acc * silu'(aux)
  kActMaskBwd = 8,  // out = acc * bit(mask)              (mask = sign bits written by a forward epilogue)
};

// Where the pieces of a sharded B operand live (fully sharded parameters).  The unit that contains the matrix is
// cut into `world` pieces of `piece_len` elements; rank p keeps its piece at shards[p] + shard_off.  The matrix starts
// `unit_off` elements into the unit and must be contiguous (ldb equal to its row length); `GemmDesc::b` is its place
// in the local staging buffer.  The CTA-pair kernel pulls the pieces itself (idle epilogue warps, peer loads) and
// its TMA producer waits for per-segment completion counters; other paths run a copy launch first.
struct NmtgGather {
  int rank, world;
  const unsigned short* shards[16];
  long shard_off, piece_len, unit_off;
  int* counters;     // device ints, [2 + 128], all zero; the kernel that used them leaves them zero
};

struct GemmDesc {
  // C[M,N] = epilogue(alpha * sum_k A(m,k) B(n,k)).  K-major operand: row index = M/N, leading dimension
  // ld over K.  MN-major operand (x_mn_major = 1): stored [K, M/N] with ld over M/N.
  const void* a; int lda; int a_mn_major;
  const void* b; int ldb; int b_mn_major;
  int M, N, K;
  float alpha;
  const void* bias;       // bf16 [N] or null
  const void* residual;   // bf16 [M, ld_res] or null
  int ld_res;
  const void* aux;        // bf16 [M, ld_aux] for the *Bwd activations
  int ld_aux;
  void* out; int ld_out; int out_fp32; int accumulate;
  void* preact;           // optional bf16 [M, ld_out]
  void* mask;             // optional uint32 [M, ld_mask]: bit j of word c = (output[row, 32 c + j] > 0); written by forward
                          // epilogues (before the residual), read by kActMaskBwd
  int ld_mask;
  float* colsum;          // optional fp32 [N]: column sums of the (bf16-rounded) output are ADDED here (bias gradient of the
                          // layer whose output gradient this GEMM produces); CTA-pair kernel with the TMA-store epilogue only
  int act;
  float dropout_p; unsigned long long seed, stream_id;
  const unsigned long long* seed_dev;  // optional device word added to seed (lets graph replays draw new masks)
  int split_k;            // 0 = automatic (only when allow_split_k), else forced
  int allow_split_k;
  int force_bn;           // 0 = automatic, 128 or 256
  int* status;            // device int, 0 = ok
  const NmtgGather* gather;  // optional: B is gathered from its owners by this call (see NmtgGather)
};

const char* nmtg_gemm_bf16(const GemmDesc* d, cudaStream_t stream);
// 0 = automatic (CTA-pair kernel when M > 128), 1 = single-CTA kernel only, 2 = same as 0
void nmtg_set_gemm_variant(int v);
// n (even) SMs are left free by every launcher of this library: persistent kernels size their grids for the rest, so that
// communication kernels placed on the free SMs (nmtg_reduce_unit with a negative CTA count) never share one with them.
void nmtg_set_sm_reserve(int n);
// Timing aid for the short-sequence attention backward: bit mask of work to leave out (see the kernel); 0 = everything.
void nmtg_set_attn_bwd_ablation(int bits);
// time stamps of one CTA of the pipelined attention backward / forward kernels (timing aids, see the kernels)
int nmtg_attn_ws_trace(long long* out, int capacity);
int nmtg_attn_fws_trace(long long* out, int capacity);
// Profiling aid: device buffer of 16 int64 per CTA pair (at least 16 * #SMs / 2 entries) that the CTA-pair GEMM fills with
// cycle counters of its MMA issuer and of one epilogue warp; nullptr switches it off.
void nmtg_set_gemm_trace(long long* buf);

// LayerNorm over the last dimension of bf16 x[rows, hidden]; mean/rstd (fp32 [rows]) may be null in fwd.
const char* nmtg_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                               int rows, int hidden, float eps, cudaStream_t stream);
// dx = LN'(dy) (+ dres if given); dgamma/dbeta (fp32 [hidden]) are ACCUMULATED into.
const char* nmtg_layernorm_bwd(const void* dy, const void* x, const float* mean, const float* rstd, const void* gamma,
                               const void* dres, void* dx, float* dgamma, float* dbeta, int rows, int hidden,
                               cudaStream_t stream);

// Label-smoothed softmax cross-entropy over bf16 logits[rows, vocab] (leading dimension ld).  When
// write_grad != 0 the logits are overwritten with grad_scale * dloss/dlogit (grad_scale = *grad_scale_ptr
// * grad_scale_val, pointer optional).  row_loss / row_lse / loss_sum / correct_sum are optional; the two
// sums are ACCUMULATED into.  Rows whose label equals pad_idx contribute nothing and get a zero gradient.
const char* nmtg_xent_fused(void* logits, const int64_t* labels, float* row_loss, float* row_lse, float* loss_sum,
                            float* correct_sum, int rows, int vocab, long ld, float smoothing, int pad_idx,
                            const float* grad_scale_ptr, float grad_scale_val, int write_grad, cudaStream_t stream);

// y = (residual ? residual : 0) + dropout(x) over n bf16 elements (n % 16 == 0).  The backward of the
// dropout branch is the same call with x = dy, residual = null.
// y = dropout-mask(x) with dropout_add's mask; colsum[cols] += column sums of y.  cols = 16 * (a divisor of 256).
const char* nmtg_dropout_colsum(const void* x, void* y, float* colsum, int rows, int cols, float p, unsigned long long seed,
                                unsigned long long stream_id, const unsigned long long* seed_dev, cudaStream_t stream);
const char* nmtg_dropout_add(const void* x, const void* residual, void* y, long n, float p, unsigned long long seed,
                             unsigned long long stream_id, const unsigned long long* seed_dev, cudaStream_t stream);
// dz = dropout-mask(dy) * act'(z) over n bf16 elements (n % 8 == 0); act 1 ReLU, 2 GELU, 3 SiLU; p = 0: no mask.
const char* nmtg_act_backward(const void* dy, const void* z, void* dz, long n, int act, float p, unsigned long long seed,
                              unsigned long long stream_id, const unsigned long long* seed_dev, cudaStream_t stream);
// out[r] = dropout(table[tokens[r]] * scale + pos_table[positions[r]])  (pos_table / positions optional)
const char* nmtg_embed_fwd(const int64_t* tokens, const int64_t* positions, const void* table, const void* pos_table,
                           void* out, int rows, int hidden, int vocab, int max_pos, float scale, float p,
                           unsigned long long seed, unsigned long long stream_id, const unsigned long long* seed_dev,
                           cudaStream_t stream);
// fp32 dtable / dpos (dpos optional) are ACCUMULATED into; rows whose token is pad_idx are skipped.
const char* nmtg_embed_bwd(const int64_t* tokens, const int64_t* positions, const void* dy, float* dtable, float* dpos,
                           int rows, int hidden, int vocab, int max_pos, float scale, float p, unsigned long long seed,
                           unsigned long long stream_id, const unsigned long long* seed_dev, int pad_idx,
                           cudaStream_t stream);
// out[c] += sum over rows of bf16 x[r, c]
const char* nmtg_colsum(const void* x, float* out, int rows, int cols, long ld, cudaStream_t stream);

// Per-step optimiser scalars, kept in device memory (16 floats) so captured graphs can be replayed.
struct NmtgAdamHyper {
  float lr, beta1, beta2, eps;
  float weight_decay, bias_correction1, bias_correction2, grad_scale;
  float max_grad_norm;
  int decoupled_wd;   // 1 = AdamW, 0 = L2 added to the gradient
  int zero_grad;      // 1 = clear the gradient buffer after use
  int pad0, pad1, pad2, pad3, pad4;
};
// out_sq += sum g^2 ; *out_nonfinite |= 1 when a non-finite partial sum is met
const char* nmtg_sq_norm(const float* g, long n, float* out_sq, int* out_nonfinite, cudaStream_t stream);
// One Adam(W) step over flat fp32 buffers (n % 4 == 0); work_bf16 (optional) receives the refreshed copy.
const char* nmtg_adamw_flat(float* master, void* work_bf16, float* grad, float* m, float* v, long n,
                            const NmtgAdamHyper* hyper_dev, const float* grad_sq, const int* nonfinite,
                            cudaStream_t stream);
const char* nmtg_cast_f32_bf16(const float* src, void* dst, long n, cudaStream_t stream);
// Device-resident dynamic loss scale: state = {scale, clean steps, 1 / scale, skipped steps}.  prepare divides the
// optimiser's gradient factor by the scale; update backs off after a skipped step (nonfinite flag set, or norm < 0) and
// grows after `interval` clean ones.  Either of nonfinite / norm may be null.
const char* nmtg_loss_scale_prepare(NmtgAdamHyper* hyper_dev, const float* state, cudaStream_t stream);
const char* nmtg_loss_scale_update(float* state, const int* nonfinite, const float* norm, int interval, float growth,
                                   float backoff, float min_scale, float max_scale, cudaStream_t stream);

// Packed variable-length attention, head_dim 64.  q rows of sequence b are [cu_q[b], cu_q[b+1]) and its
// key/value rows [cu_k[b], cu_k[b+1]); head h occupies columns [64h, 64h+64) of each tensor.
struct AttnDesc {
  const void* q; int ld_q;
  const void* k; int ld_k;
  const void* v; int ld_v;
  void* out; int ld_out;              // forward output; backward input (O)
  float* lse; long lse_stride;        // [heads, lse_stride] row log-sum-exp
  const int* cu_q; const int* cu_k;   // device int32 [batch + 1]
  int batch, num_heads, head_dim;
  int max_q, max_k;                   // upper bounds on sequence lengths (grid sizing)
  int total_q, total_k;               // rows of the q / kv tensors
  int causal; float scale;
  float dropout_p; unsigned long long seed, stream_id; int kstride;
  const unsigned long long* seed_dev;
  // backward only
  const void* d_out; int ld_dout;
  void* dq; int ld_dq;
  void* dk; int ld_dk;
  void* dv; int ld_dv;
  float* dq_acc; int ld_dqacc;        // zero-initialised fp32 [total_q, heads*64]; needed when max_k > 128
  float* delta;                       // optional scratch, fp32 [heads, lse_stride]: the backward pass of sequences above 128
                                      // keys fills it with rowsum(dO * O) once instead of recomputing it per key tile
  int* status;
  // optional additive bias on the scaled scores, fp32 [batch, heads, max_q, max_k] (element strides; keys contiguous),
  // e.g. relative-position terms; dbias (same strides, zero-initialised) receives its gradient in the backward pass.
  // Calls with a bias always run the general multi-tile kernels.
  const float* bias; long bias_sb, bias_sh, bias_sq;
  float* dbias;
};
const char* nmtg_attn_fwd(const AttnDesc* d, cudaStream_t stream);
const char* nmtg_attn_bwd(const AttnDesc* d, cudaStream_t stream);
// 0 = choose automatically (persistent single-tile kernels when max_q, max_k <= 128), 1 = general kernels only
void nmtg_set_attention_variant(int v);

// ---- peer-memory data parallelism and fully sharded parameters ---------------------------------------------
// Pointers of every rank's symmetric buffers as seen from THIS process (own buffers: local pointers; peers:
// pointers obtained by opening their IPC handles).  flags[r]: int [kNmtgFlagRows][16] epochs, partials[r]:
// float [2][16].
constexpr int kNmtgFlagRows = 256;
constexpr int kNmtgMaxUnits = 96;
struct NmtgPeerTable {
  int rank, world;
  float* grads[16];            // fp32 gradient space of every rank
  unsigned short* works[16];   // bf16 parameters: full copies (data parallel) or shards (fully sharded)
  int* flags[16];
  float* partials[16];
  float* norm_out;             // optional local float: global gradient norm of the step (-1 when skipped)
  long long timeout_ns;        // wall-time bound of every cross-GPU wait
};
// The flat parameter space is cut into UNITS (one per Transformer layer, the rest merged); unit u is cut into
// `world` equal pieces and this rank owns piece `rank` of every unit: `len[u]` elements at `global_begin[u]` of the
// gradient space and at `shard_off[u]` of the shard-ordered buffers (reduced gradients, Adam moments, and - fully
// sharded mode - fp32 master weights and bf16 parameters).
struct NmtgPieces {
  int n;
  long shard_off[kNmtgMaxUnits];
  long global_begin[kNmtgMaxUnits];   // offset in the gradient space (every rank's buffer has the same layout); in
                                      // data-parallel mode this is also the offset in the flat parameter space
  long len[kNmtgMaxUnits];
};
// Reduce-scatter of ONE unit: waits (bounded) on flag row `row` until every peer has published "gradients of this
// unit are complete", then sums this rank's piece over all ranks' gradient buffers with peer loads into
// reduced[0:len) (added to the old contents when accumulate != 0).  With zero_len > 0 the kernel then waits on row
// `row + 1` until every peer has finished reading and clears its OWN gradients [zero_begin, zero_begin + zero_len)
// (rotating per-layer gradient buffers).  `counter` is one device int per launch site, zero between launches.
const char* nmtg_reduce_unit(const NmtgPeerTable* t, int row, float* reduced, long global_begin, long len, int accumulate,
                             long zero_begin, long zero_len, int* counter, const int* epoch_dev, int* status, int ctas,
                             cudaStream_t stream);
// After all units are reduced: exchange of the squared-norm partials (flag row 1), clipping coefficient, Adam(W)
// on every owned piece, refreshed bf16 parameters.  mode 0 (data parallel): master weights are indexed in the flat
// space and the bf16 values are stored into EVERY rank's full copy (the all-gather); mode 1 (fully sharded): master
// weights and bf16 parameters are shard-ordered and local.  zero_len > 0 clears the local gradient space
// [0, zero_len) afterwards (every peer has passed row 1, i.e. finished reading it).
const char* nmtg_update_pieces(const NmtgPeerTable* t, const NmtgPieces* pieces, const float* reduced, float* master, float* m,
                               float* v, const NmtgAdamHyper* hyper_dev, const float* sq, const int* nonfinite, int mode,
                               long zero_len, const int* epoch_dev, int* status, cudaStream_t stream);
// the closing barrier of a step (row 2) + epoch advance
const char* nmtg_peer_finish_step(const NmtgPeerTable* t, int* epoch_dev, int* status, cudaStream_t stream);
// dst[e0:e1) of a unit (bf16) <- pulled from the owners' shards (works[p] + shard_off, piece_len elements each)
const char* nmtg_fsdp_gather(const NmtgPeerTable* t, void* dst, long shard_off, long piece_len, long e0, long e1, int ctas,
                             cudaStream_t stream);
// waits (bounded) on one flag row; used to exercise the timeout path
const char* nmtg_peer_wait_row(const NmtgPeerTable* t, int row, int epoch, int* status, cudaStream_t stream);
