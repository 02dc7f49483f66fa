// C launch API of the sequence-model kernels (transducer joint / loss, linear-recurrence scan, Cauchy kernel
// coefficients, row softmax with mask and dropout, beam-search step, single-query decode attention).
// Every launcher returns nullptr on success or a static error string; nothing allocates.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

extern "C" {

// ---- transducer joint: h[b,t,u,:] = act(f[b,t,:] + g[b,u,:]) ------------------------------------------------
// dtype: 0 = fp32, 1 = bf16.  packed: rows of sentence b start at (b ? batch_offset[b-1] : 0) and are laid
// out [t][u] with u running over g_len[b]; dense: [B, T, U, H] with rows outside the lengths zeroed.
// relu / dropout are applied in that order; the dropout mask is a pure function of (seed, stream_id, element).
const char* nmtg_transducer_joint_fwd(const void* f, const void* g, const int* f_len, const int* g_len,
                                      const long* batch_offset, void* out, int B, int T, int U, int H, int dtype,
                                      int packed, int relu, float p, unsigned long long seed,
                                      unsigned long long stream_id, cudaStream_t stream);
// df[b,t,:] = sum_u d(out)  dg[b,u,:] = sum_t d(out); `out` (the forward result) is needed when relu or dropout is on.
const char* nmtg_transducer_joint_bwd(const void* dout, const void* out, const int* f_len, const int* g_len,
                                      const long* batch_offset, void* df, void* dg, int B, int T, int U, int H,
                                      int dtype, int packed, int relu, float p, unsigned long long seed,
                                      unsigned long long stream_id, float scale, cudaStream_t stream);

// ---- transducer loss on fp32 log-probabilities x[b,t,u,v] (dense [B,T,U,V] or packed as above) ----------------
// alpha / beta: fp32 [B, T, U]; loss[b] = -log p(label_b | audio_b).
const char* nmtg_transducer_loss_fwd(const float* x, const int* label, const int* f_len, const int* y_len,
                                     const long* batch_offset, float* alpha, float* beta, float* loss, int B, int T,
                                     int U, int V, int blank, int packed, cudaStream_t stream);
// dx has the layout of x.  fuse_softmax: x = log_softmax(z) and dx is the gradient with respect to z.
const char* nmtg_transducer_loss_bwd(const float* x, const float* loss_grad, const float* alpha, const float* beta,
                                     const int* label, const int* f_len, const int* y_len, const long* batch_offset,
                                     float* dx, int B, int T, int U, int V, int blank, int packed, int fuse_softmax,
                                     cudaStream_t stream);

// ---- diagonal linear recurrence on complex64 rows: h_t = lambda_n * h_(t-1) + x_t ------------------------------
// x, h: [B, N, L] (time innermost, interleaved re/im); lambda: [N]; lengths: [B].  direction 0 = left to right,
// 1 = right to left (starting at lengths[b]-1), 2 = first N/2 channels left to right, the rest right to left.
// Positions >= lengths[b] are written as zero.
const char* nmtg_lru_scan_fwd(const float2* lambda, const float2* x, const int* lengths, float2* h, int B, int N, int L,
                              int direction, cudaStream_t stream);
// PyTorch complex-gradient convention: dx_t = sum_s conj(lambda)^(|s-t|) g_s; dlambda[n] += sum conj(h_prev) * dx_t.
const char* nmtg_lru_scan_bwd(const float2* lambda, const float2* grad_h, const float2* h, const int* lengths,
                              float2* dx, float2* dlambda, int B, int N, int L, int direction, cudaStream_t stream);

// ---- Cauchy kernel coefficients: out[i,q,l,h] = sum_n a[i,q,h,n] / (b[q,l,h] - c[q,n])  (complex64) ------------
const char* nmtg_cauchy_fwd(const float2* a, const float2* b, const float2* c, float2* out, int I, int Q, int L, int H,
                            int N, cudaStream_t stream);
// da / db / dc must be zero on entry (db and dc are accumulated with atomics).
const char* nmtg_cauchy_bwd(const float2* a, const float2* b, const float2* c, const float2* dout, float2* da, float2* db,
                            float2* dc, int I, int Q, int L, int H, int N, cudaStream_t stream);

// ---- row softmax (+ additive/boolean key mask, + dropout) over x[rows, cols] ---------------------------------
// dtype 0 = fp32, 1 = bf16 (in and out).  pad_mask: uint8 [rows / rows_per_mask, cols], nonzero = masked out.
// y = softmax(x * scale + mask); yd = dropout(y) (yd may be null when p == 0).
const char* nmtg_softmax_dropout_fwd(const void* x, const uint8_t* pad_mask, void* y, void* yd, int rows, int cols,
                                     int rows_per_mask, int dtype, float scale, float p, unsigned long long seed,
                                     unsigned long long stream_id, cudaStream_t stream);
// dx = scale * y * (dyd_masked - sum(dyd_masked * y)) with dyd_masked = dropout-mask * dyd / (1-p)
const char* nmtg_softmax_dropout_bwd(const void* dyd, const void* y, void* dx, int rows, int cols, int dtype, float scale,
                                     float p, unsigned long long seed, unsigned long long stream_id,
                                     cudaStream_t stream);

// ---- beam search step ---------------------------------------------------------------------------------------
// logits: [R = B*K, V], rows `ld` elements apart (dtype 0 fp32 / 1 bf16).  For every row: lp = log_softmax(logits) with pad -> -inf,
// eos -> -inf when step < min_len, everything but eos -> -inf when force_eos[r]; then per sentence the best
// 2K of (scores[r] + lp[r, v]) over its K rows.  out_scores / out_index: [B, 2K]; index = k * V + v.
// row_lse: fp32 [R] scratch, cand_*: scratch [R, 2K].
const char* nmtg_beam_topk(const void* logits, long ld, int dtype, const float* scores, const uint8_t* force_eos,
                           float* row_lse, float* cand_val, int* cand_idx, float* out_scores, long* out_index, int B, int K,
                           int V, int pad, int eos, int ban_eos, cudaStream_t stream);
// dst[r, 0:copy_bytes] = src[index[r], 0:copy_bytes] for rows `row_stride_bytes` apart (both multiples of 16).
// filled_dev (optional device int): copy filled_dev[0] * unit_bytes per row instead of copy_bytes, so that a captured
// CUDA graph moves the right amount at every replay.
const char* nmtg_gather_rows(const void* src, void* dst, const long* index, int rows, int src_rows, long row_stride_bytes,
                             long copy_bytes, const int* filled_dev, long unit_bytes, cudaStream_t stream);

// ---- single-query attention over a preallocated cache ------------------------------------------------------
// q: bf16 [R, heads, 64]; k_cache / v_cache: bf16 [R / kv_div, cap, heads, 64] (kv_div > 1 shares one cache row
// between the hypotheses of a sentence, as for encoder-decoder attention); lengths: int32 [R / kv_div] or null
// (= all rows use `len`); out: bf16 [R, heads, 64].
// len_dev (optional device int, used when lengths is null): the number of valid keys is len_dev[0] + len_add.
const char* nmtg_decode_attn(const void* q, long q_ld, const void* k_cache, const void* v_cache, const int* lengths,
                             void* out, int R, int heads, int cap, int len, int kv_div, float scale, const int* len_dev,
                             int len_add, cudaStream_t stream);
// cache[r, pos, :] = new[r, :] for k and v (new rows `ld` elements apart, heads * 64 elements each).
// pos_dev (optional device int) overrides pos.
const char* nmtg_cache_append(const void* k_new, const void* v_new, long ld, void* k_cache, void* v_cache, int R, int heads,
                              int cap, int pos, const int* pos_dev, cudaStream_t stream);

// ---- relative-position (Transformer-XL) self-attention on packed sequences of at most 128 tokens ---------------
// qkv: bf16 [N, 3 * heads * 64]; r: bf16 [L, heads * 64], row r_center - d = projected embedding of distance d;
// u / w: fp32 [heads, 64] content / position biases; cu: int32 [B + 1]; out: bf16 [N, heads * 64]; lse: fp32 [heads, N].
const char* nmtg_rel_attn_fwd(const void* qkv, const void* r, const float* u, const float* w, const int* cu, void* out, float* lse,
                              int B, int N, int heads, int max_len, int r_center, int L, int causal, float scale, float p,
                              unsigned long long seed, unsigned long long stream_id, cudaStream_t stream);
// dqkv: bf16 [N, 3H] (rows of the sequences are overwritten); dr [L, H], du, dw [heads, 64]: fp32, ACCUMULATED into.
const char* nmtg_rel_attn_bwd(const void* qkv, const void* r, const float* u, const float* w, const int* cu, const float* lse,
                              const void* dctx, void* dqkv, float* dr, float* du, float* dw, int B, int N, int heads, int max_len,
                              int r_center, int L, int causal, float scale, float p, unsigned long long seed,
                              unsigned long long stream_id, cudaStream_t stream);
}
