// Python bindings: torch tensors in, raw pointers to the sm_100a launchers of ops_api.h.  Nothing here
// computes; shape / dtype / device checks fail loudly instead of falling back.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "ops_api.h"

std::vector<torch::Tensor> batch_allocate(const torch::Tensor& indices, const torch::Tensor& lengths,
                                          const c10::optional<torch::Tensor>& src_sizes,
                                          const c10::optional<torch::Tensor>& tgt_sizes, int64_t batch_size_words,
                                          int64_t batch_size_frames, int64_t batch_size_sents, int64_t multiplier,
                                          int64_t max_src_len, int64_t max_tgt_len, int64_t min_src_len,
                                          int64_t min_tgt_len, bool cleaning, bool unbalanced, int64_t cut_off_size,
                                          int64_t smallest_batch_size);

namespace {

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void ck(const char* err) {
  if (err) throw std::runtime_error(std::string("nmtgminor_b200 kernel launch failed: ") + err);
}
void need_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
}
void need_f32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kFloat, name, " must be float32");
}
void need_rowmajor2d(const Tensor& t, const char* name) {
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with unit inner stride");
}
const void* opt_ptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// per-device status word shared by all kernels
Tensor& status_tensor(int device) {
  static std::vector<Tensor> st(64);
  if (!st[device].defined())
    st[device] = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  return st[device];
}
int* status_ptr(const Tensor& like) { return status_tensor(like.get_device()).data_ptr<int>(); }

// per-device 64-bit word added to every dropout seed; advancing it (also from inside a captured graph)
// gives fresh masks without changing kernel arguments
Tensor& seed_tensor(int device) {
  static std::vector<Tensor> st(64);
  if (!st[device].defined())
    st[device] = torch::zeros({1}, torch::dtype(torch::kInt64).device(torch::kCUDA, device));
  return st[device];
}
const unsigned long long* seed_ptr(const Tensor& like) {
  return reinterpret_cast<const unsigned long long*>(seed_tensor(like.get_device()).data_ptr<int64_t>());
}
Tensor get_seed_tensor(int64_t device) { return seed_tensor(static_cast<int>(device)); }

// C[M,N] = epilogue(alpha * A B^T) ; see GemmDesc
void gemm(const Tensor& a, bool a_mn_major, const Tensor& b, bool b_mn_major, Tensor& out, const OptTensor& bias,
          const OptTensor& residual, const OptTensor& aux, const OptTensor& preact, int64_t act, double dropout_p,
          int64_t seed, int64_t stream_id, double alpha, bool accumulate, bool allow_split_k, int64_t split_k,
          int64_t force_bn, const OptTensor& mask, const OptTensor& colsum, const pybind11::object& gather) {
  need_bf16(a, "a"); need_bf16(b, "b");
  need_rowmajor2d(a, "a"); need_rowmajor2d(b, "b"); need_rowmajor2d(out, "out");
  c10::cuda::CUDAGuard guard(a.device());
  GemmDesc d = {};
  d.a = a.data_ptr(); d.lda = static_cast<int>(a.stride(0)); d.a_mn_major = a_mn_major;
  d.b = b.data_ptr(); d.ldb = static_cast<int>(b.stride(0)); d.b_mn_major = b_mn_major;
  d.M = static_cast<int>(a_mn_major ? a.size(1) : a.size(0));
  d.K = static_cast<int>(a_mn_major ? a.size(0) : a.size(1));
  d.N = static_cast<int>(b_mn_major ? b.size(1) : b.size(0));
  const int64_t kb = b_mn_major ? b.size(0) : b.size(1);
  TORCH_CHECK(kb == d.K, "gemm: reduction sizes differ (", d.K, " vs ", kb, ")");
  TORCH_CHECK(out.size(0) == d.M && out.size(1) == d.N, "gemm: output shape mismatch");
  d.alpha = static_cast<float>(alpha);
  if (bias.has_value()) { need_bf16(*bias, "bias"); TORCH_CHECK(bias->numel() == d.N && bias->is_contiguous()); }
  d.bias = opt_ptr(bias);
  if (residual.has_value()) { need_bf16(*residual, "residual"); need_rowmajor2d(*residual, "residual"); d.ld_res = static_cast<int>(residual->stride(0)); }
  d.residual = opt_ptr(residual);
  if (aux.has_value()) { need_bf16(*aux, "aux"); need_rowmajor2d(*aux, "aux"); d.ld_aux = static_cast<int>(aux->stride(0)); }
  d.aux = opt_ptr(aux);
  TORCH_CHECK(act < kActReluBwd || act == kActMaskBwd || aux.has_value(), "gemm: activation-backward epilogues need aux");
  TORCH_CHECK(act != kActMaskBwd || mask.has_value(), "gemm: the mask-backward epilogue needs a mask");
  if (mask.has_value()) {
    TORCH_CHECK(mask->is_cuda() && mask->scalar_type() == at::kInt && mask->dim() == 2 && mask->stride(1) == 1 &&
                mask->size(0) >= d.M && mask->size(1) * 32 >= d.N, "gemm: mask must be int32 [M, ceil(N / 32)]");
    d.mask = mask->data_ptr(); d.ld_mask = static_cast<int>(mask->stride(0));
  }
  if (colsum.has_value()) {
    need_f32(*colsum, "colsum");
    TORCH_CHECK(colsum->is_contiguous() && colsum->numel() >= d.N, "gemm: colsum must be fp32 [N]");
    d.colsum = colsum->data_ptr<float>();
  }
  d.out = out.data_ptr(); d.ld_out = static_cast<int>(out.stride(0));
  TORCH_CHECK(out.is_cuda());
  if (out.scalar_type() == at::kFloat) d.out_fp32 = 1;
  else TORCH_CHECK(out.scalar_type() == at::kBFloat16, "gemm: output must be bf16 or fp32");
  d.accumulate = accumulate;
  TORCH_CHECK(!accumulate || d.out_fp32, "gemm: accumulate needs an fp32 output");
  if (preact.has_value()) {
    need_bf16(*preact, "preact"); need_rowmajor2d(*preact, "preact");
    TORCH_CHECK(preact->stride(0) == out.stride(0) && !d.out_fp32, "gemm: preact must share the output layout");
  }
  d.preact = const_cast<void*>(opt_ptr(preact));
  d.act = static_cast<int>(act);
  d.dropout_p = static_cast<float>(dropout_p);
  d.seed = static_cast<unsigned long long>(seed); d.stream_id = static_cast<unsigned long long>(stream_id);
  d.split_k = static_cast<int>(split_k); d.allow_split_k = allow_split_k; d.force_bn = static_cast<int>(force_bn);
  d.seed_dev = seed_ptr(a);
  d.status = status_ptr(a);
  NmtgGather gth = {};
  if (!gather.is_none()) {
    // (rank, [shard pointer of every rank], staging buffer, shard_off, piece_len, unit_off, numel, counters): B is a view
    // of the staging buffer and its pieces are pulled from the owners' shards by this call
    auto tup = gather.cast<pybind11::tuple>();
    TORCH_CHECK(tup.size() == 8, "gemm: gather must be an 8-tuple");
    gth.rank = tup[0].cast<int>();
    auto shards = tup[1].cast<std::vector<int64_t>>();
    gth.world = static_cast<int>(shards.size());
    TORCH_CHECK(gth.world >= 1 && gth.world <= 16, "gemm: gather world size out of range");
    for (int i = 0; i < gth.world; ++i) gth.shards[i] = reinterpret_cast<const unsigned short*>(shards[i]);
    const Tensor staging = tup[2].cast<Tensor>();
    gth.shard_off = tup[3].cast<int64_t>(); gth.piece_len = tup[4].cast<int64_t>(); gth.unit_off = tup[5].cast<int64_t>();
    const int64_t numel = tup[6].cast<int64_t>();
    const Tensor counters = tup[7].cast<Tensor>();
    need_bf16(staging, "gather staging");
    TORCH_CHECK(counters.is_cuda() && counters.scalar_type() == at::kInt && counters.is_contiguous() && counters.numel() >= 2 + 128,
                "gemm: gather counters must be int32 [>= 130]");
    TORCH_CHECK(b.is_contiguous() && b.numel() == numel, "gemm: a gathered operand must be the whole contiguous matrix");
    TORCH_CHECK(reinterpret_cast<const char*>(b.data_ptr()) == reinterpret_cast<const char*>(staging.data_ptr()) + 2 * gth.unit_off,
                "gemm: the gathered operand is not at its place in the staging buffer");
    TORCH_CHECK(gth.unit_off + numel <= gth.piece_len * gth.world, "gemm: gathered operand outside its unit");
    gth.counters = counters.data_ptr<int>();
    d.gather = &gth;
  }
  ck(nmtg_gemm_bf16(&d, cur_stream()));
}

std::vector<Tensor> layernorm_fwd(const Tensor& x, const Tensor& gamma, const Tensor& beta, double eps) {
  need_bf16(x, "x"); need_bf16(gamma, "gamma"); need_bf16(beta, "beta");
  TORCH_CHECK(x.is_contiguous() && x.dim() == 2);
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = static_cast<int>(x.size(0)), hidden = static_cast<int>(x.size(1));
  Tensor y = torch::empty_like(x);
  Tensor mean = torch::empty({rows}, x.options().dtype(torch::kFloat));
  Tensor rstd = torch::empty({rows}, x.options().dtype(torch::kFloat));
  ck(nmtg_layernorm_fwd(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), mean.data_ptr<float>(),
                        rstd.data_ptr<float>(), rows, hidden, static_cast<float>(eps), cur_stream()));
  return {y, mean, rstd};
}

Tensor layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& mean, const Tensor& rstd, const Tensor& gamma,
                     const OptTensor& dres, Tensor& dgamma, Tensor& dbeta) {
  need_bf16(dy, "dy"); need_bf16(x, "x"); need_bf16(gamma, "gamma"); need_f32(dgamma, "dgamma"); need_f32(dbeta, "dbeta");
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous());
  if (dres.has_value()) { need_bf16(*dres, "dres"); TORCH_CHECK(dres->is_contiguous()); }
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty_like(x);
  ck(nmtg_layernorm_bwd(dy.data_ptr(), x.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), gamma.data_ptr(),
                        opt_ptr(dres), dx.data_ptr(), dgamma.data_ptr<float>(), dbeta.data_ptr<float>(),
                        static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), cur_stream()));
  return dx;
}

// returns row losses; loss_sum / correct_sum (fp32 scalars on device) are accumulated into when given
Tensor xent_fused(Tensor& logits, const Tensor& labels, double smoothing, int64_t pad_idx, const OptTensor& loss_sum,
                  const OptTensor& correct_sum, const OptTensor& grad_scale, double grad_scale_val, bool write_grad) {
  need_bf16(logits, "logits"); need_rowmajor2d(logits, "logits");
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.is_contiguous());
  TORCH_CHECK(labels.numel() == logits.size(0));
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor row_loss = torch::empty({logits.size(0)}, logits.options().dtype(torch::kFloat));
  ck(nmtg_xent_fused(logits.data_ptr(), labels.data_ptr<int64_t>(), row_loss.data_ptr<float>(), nullptr,
                     loss_sum.has_value() ? loss_sum->data_ptr<float>() : nullptr,
                     correct_sum.has_value() ? correct_sum->data_ptr<float>() : nullptr,
                     static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)), logits.stride(0),
                     static_cast<float>(smoothing), static_cast<int>(pad_idx),
                     grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr, static_cast<float>(grad_scale_val),
                     write_grad ? 1 : 0, cur_stream()));
  return row_loss;
}

Tensor dropout_add(const Tensor& x, const OptTensor& residual, double p, int64_t seed, int64_t stream_id) {
  need_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous());
  if (residual.has_value()) { need_bf16(*residual, "residual"); TORCH_CHECK(residual->is_contiguous() && residual->numel() == x.numel()); }
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  ck(nmtg_dropout_add(x.data_ptr(), opt_ptr(residual), y.data_ptr(), x.numel(), static_cast<float>(p),
                      static_cast<unsigned long long>(seed), static_cast<unsigned long long>(stream_id), seed_ptr(x), cur_stream()));
  return y;
}

Tensor act_backward(const Tensor& dy, const Tensor& z, int64_t act, double p, int64_t seed, int64_t stream_id) {
  need_bf16(dy, "dy"); need_bf16(z, "z");
  TORCH_CHECK(dy.is_contiguous() && z.is_contiguous() && dy.numel() == z.numel());
  c10::cuda::CUDAGuard guard(dy.device());
  Tensor dz = torch::empty_like(dy);
  ck(nmtg_act_backward(dy.data_ptr(), z.data_ptr(), dz.data_ptr(), dy.numel(), static_cast<int>(act), static_cast<float>(p),
                       static_cast<unsigned long long>(seed), static_cast<unsigned long long>(stream_id), seed_ptr(dy), cur_stream()));
  return dz;
}

Tensor dropout_colsum(const Tensor& x, double p, int64_t seed, int64_t stream_id, Tensor& colsum) {
  need_bf16(x, "x"); need_f32(colsum, "colsum");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && colsum.is_contiguous() && colsum.numel() >= x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  ck(nmtg_dropout_colsum(x.data_ptr(), y.data_ptr(), colsum.data_ptr<float>(), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)),
                         static_cast<float>(p), static_cast<unsigned long long>(seed), static_cast<unsigned long long>(stream_id),
                         seed_ptr(x), cur_stream()));
  return y;
}

Tensor embed_fwd(const Tensor& tokens, const OptTensor& positions, const Tensor& table, const OptTensor& pos_table,
                 double scale, double p, int64_t seed, int64_t stream_id) {
  need_bf16(table, "table");
  TORCH_CHECK(tokens.is_cuda() && tokens.scalar_type() == at::kLong && tokens.is_contiguous() && table.is_contiguous());
  c10::cuda::CUDAGuard guard(table.device());
  const int rows = static_cast<int>(tokens.numel()), hidden = static_cast<int>(table.size(1));
  Tensor out = torch::empty({rows, hidden}, table.options());
  int max_pos = 1;
  if (pos_table.has_value()) { need_bf16(*pos_table, "pos_table"); TORCH_CHECK(pos_table->is_contiguous() && pos_table->size(1) == hidden); max_pos = static_cast<int>(pos_table->size(0)); }
  if (positions.has_value()) TORCH_CHECK(positions->scalar_type() == at::kLong && positions->is_contiguous() && positions->numel() == rows);
  ck(nmtg_embed_fwd(tokens.data_ptr<int64_t>(), positions.has_value() ? positions->data_ptr<int64_t>() : nullptr,
                    table.data_ptr(), opt_ptr(pos_table), out.data_ptr(), rows, hidden, static_cast<int>(table.size(0)),
                    max_pos, static_cast<float>(scale), static_cast<float>(p), static_cast<unsigned long long>(seed),
                    static_cast<unsigned long long>(stream_id), seed_ptr(table), cur_stream()));
  return out;
}

void embed_bwd(const Tensor& tokens, const OptTensor& positions, const Tensor& dy, Tensor& dtable, const OptTensor& dpos,
               double scale, double p, int64_t seed, int64_t stream_id, int64_t pad_idx) {
  need_bf16(dy, "dy"); need_f32(dtable, "dtable");
  TORCH_CHECK(dy.is_contiguous() && dtable.is_contiguous() && tokens.is_contiguous());
  c10::cuda::CUDAGuard guard(dy.device());
  int max_pos = 1;
  if (dpos.has_value()) { need_f32(*dpos, "dpos"); max_pos = static_cast<int>(dpos->size(0)); }
  ck(nmtg_embed_bwd(tokens.data_ptr<int64_t>(), positions.has_value() ? positions->data_ptr<int64_t>() : nullptr,
                    dy.data_ptr(), dtable.data_ptr<float>(), dpos.has_value() ? dpos->data_ptr<float>() : nullptr,
                    static_cast<int>(tokens.numel()), static_cast<int>(dy.size(1)), static_cast<int>(dtable.size(0)), max_pos,
                    static_cast<float>(scale), static_cast<float>(p), static_cast<unsigned long long>(seed),
                    static_cast<unsigned long long>(stream_id), seed_ptr(dy), static_cast<int>(pad_idx), cur_stream()));
}

void colsum(const Tensor& x, Tensor& out) {
  need_bf16(x, "x"); need_rowmajor2d(x, "x"); need_f32(out, "out");
  TORCH_CHECK(out.numel() == x.size(1) && out.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  ck(nmtg_colsum(x.data_ptr(), out.data_ptr<float>(), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), x.stride(0),
                 cur_stream()));
}

void sq_norm(const Tensor& g, Tensor& out_sq, Tensor& nonfinite) {
  need_f32(g, "g"); need_f32(out_sq, "out_sq");
  TORCH_CHECK(g.is_contiguous() && nonfinite.scalar_type() == at::kInt && nonfinite.is_cuda());
  c10::cuda::CUDAGuard guard(g.device());
  ck(nmtg_sq_norm(g.data_ptr<float>(), g.numel(), out_sq.data_ptr<float>(), nonfinite.data_ptr<int>(), cur_stream()));
}

void loss_scale_prepare(Tensor& hyper, const Tensor& state) {
  need_f32(state, "state");
  TORCH_CHECK(hyper.is_cuda() && state.is_cuda() && state.numel() >= 4 && hyper.numel() * hyper.element_size() >= sizeof(NmtgAdamHyper));
  c10::cuda::CUDAGuard guard(state.device());
  ck(nmtg_loss_scale_prepare(reinterpret_cast<NmtgAdamHyper*>(hyper.data_ptr()), state.data_ptr<float>(), cur_stream()));
}

void loss_scale_update(Tensor& state, const OptTensor& nonfinite, const OptTensor& norm, int64_t interval, double growth,
                       double backoff, double min_scale, double max_scale) {
  need_f32(state, "state");
  TORCH_CHECK(state.is_cuda() && state.numel() >= 4);
  if (nonfinite.has_value()) TORCH_CHECK(nonfinite->scalar_type() == at::kInt && nonfinite->is_cuda());
  if (norm.has_value()) need_f32(*norm, "norm");
  c10::cuda::CUDAGuard guard(state.device());
  ck(nmtg_loss_scale_update(state.data_ptr<float>(), nonfinite.has_value() ? nonfinite->data_ptr<int>() : nullptr,
                            norm.has_value() ? norm->data_ptr<float>() : nullptr, static_cast<int>(interval),
                            static_cast<float>(growth), static_cast<float>(backoff), static_cast<float>(min_scale),
                            static_cast<float>(max_scale), cur_stream()));
}

void adamw_flat(Tensor& master, const OptTensor& work, Tensor& grad, Tensor& m, Tensor& v, const Tensor& hyper,
                const OptTensor& grad_sq, const OptTensor& nonfinite) {
  need_f32(master, "master"); need_f32(grad, "grad"); need_f32(m, "m"); need_f32(v, "v"); need_f32(hyper, "hyper");
  TORCH_CHECK(hyper.numel() >= 16 && hyper.is_contiguous());
  TORCH_CHECK(master.is_contiguous() && grad.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  TORCH_CHECK(grad.numel() == master.numel() && m.numel() == master.numel() && v.numel() == master.numel());
  if (work.has_value()) { need_bf16(*work, "work"); TORCH_CHECK(work->numel() == master.numel() && work->is_contiguous()); }
  c10::cuda::CUDAGuard guard(master.device());
  ck(nmtg_adamw_flat(master.data_ptr<float>(), const_cast<void*>(opt_ptr(work)), grad.data_ptr<float>(), m.data_ptr<float>(),
                     v.data_ptr<float>(), master.numel(), reinterpret_cast<const NmtgAdamHyper*>(hyper.data_ptr<float>()),
                     grad_sq.has_value() ? grad_sq->data_ptr<float>() : nullptr,
                     nonfinite.has_value() ? nonfinite->data_ptr<int>() : nullptr, cur_stream()));
}

void cast_f32_bf16(const Tensor& src, Tensor& dst) {
  need_f32(src, "src"); need_bf16(dst, "dst");
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.numel() == dst.numel());
  c10::cuda::CUDAGuard guard(src.device());
  ck(nmtg_cast_f32_bf16(src.data_ptr<float>(), dst.data_ptr(), src.numel(), cur_stream()));
}

void fill_attn(AttnDesc& d, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse,
               const Tensor& cu_q, const Tensor& cu_k, int64_t num_heads, int64_t max_q, int64_t max_k, bool causal,
               double scale, double dropout_p, int64_t seed, int64_t stream_id) {
  need_bf16(q, "q"); need_bf16(k, "k"); need_bf16(v, "v"); need_bf16(out, "out"); need_f32(lse, "lse");
  need_rowmajor2d(q, "q"); need_rowmajor2d(k, "k"); need_rowmajor2d(v, "v"); need_rowmajor2d(out, "out");
  TORCH_CHECK(cu_q.is_cuda() && cu_q.scalar_type() == at::kInt && cu_k.is_cuda() && cu_k.scalar_type() == at::kInt);
  TORCH_CHECK(q.size(1) == num_heads * 64 && k.size(1) == num_heads * 64 && v.size(1) == num_heads * 64,
              "attention: tensors must be [tokens, heads * 64]");
  TORCH_CHECK(lse.dim() == 2 && lse.size(0) == num_heads && lse.size(1) >= q.size(0) && lse.is_contiguous());
  d.q = q.data_ptr(); d.ld_q = static_cast<int>(q.stride(0));
  d.k = k.data_ptr(); d.ld_k = static_cast<int>(k.stride(0));
  d.v = v.data_ptr(); d.ld_v = static_cast<int>(v.stride(0));
  d.out = out.data_ptr(); d.ld_out = static_cast<int>(out.stride(0));
  d.lse = lse.data_ptr<float>(); d.lse_stride = lse.stride(0);
  d.cu_q = cu_q.data_ptr<int>(); d.cu_k = cu_k.data_ptr<int>();
  d.batch = static_cast<int>(cu_q.numel() - 1); d.num_heads = static_cast<int>(num_heads); d.head_dim = 64;
  d.max_q = static_cast<int>(max_q); d.max_k = static_cast<int>(max_k);
  d.total_q = static_cast<int>(q.size(0)); d.total_k = static_cast<int>(k.size(0));
  d.causal = causal; d.scale = static_cast<float>(scale);
  d.dropout_p = static_cast<float>(dropout_p); d.seed = static_cast<unsigned long long>(seed);
  d.stream_id = static_cast<unsigned long long>(stream_id);
  d.kstride = static_cast<int>((max_k + 15) / 16 * 16);
  d.seed_dev = seed_ptr(q);
  d.status = status_ptr(q);
}

// bias / dbias: fp32 [batch, heads, >= max_q, >= max_k], last dimension contiguous
static void fill_attn_bias(AttnDesc& d, const OptTensor& bias, const OptTensor& dbias, int64_t max_q, int64_t max_k) {
  if (!bias.has_value()) return;
  const Tensor& b = *bias;
  need_f32(b, "bias");
  TORCH_CHECK(b.is_cuda() && b.dim() == 4 && b.stride(3) == 1, "attention bias must be fp32 [batch, heads, q, k] with contiguous keys");
  TORCH_CHECK(b.size(0) == d.batch && b.size(1) == d.num_heads && b.size(2) >= max_q && b.size(3) >= max_k,
              "attention bias is smaller than [batch, heads, max_q, max_k]");
  d.bias = b.data_ptr<float>();
  d.bias_sb = b.stride(0); d.bias_sh = b.stride(1); d.bias_sq = b.stride(2);
  if (dbias.has_value()) {
    need_f32(*dbias, "dbias");
    TORCH_CHECK(dbias->sizes() == b.sizes() && dbias->strides() == b.strides(), "dbias must have the layout of bias");
    d.dbias = dbias->data_ptr<float>();
  }
}

void attn_fwd_bias(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& out, Tensor& lse, const Tensor& cu_q,
                   const Tensor& cu_k, int64_t num_heads, int64_t max_q, int64_t max_k, bool causal, double scale,
                   double dropout_p, int64_t seed, int64_t stream_id, const OptTensor& bias) {
  c10::cuda::CUDAGuard guard(q.device());
  AttnDesc d = {};
  fill_attn(d, q, k, v, out, lse, cu_q, cu_k, num_heads, max_q, max_k, causal, scale, dropout_p, seed, stream_id);
  fill_attn_bias(d, bias, c10::nullopt, max_q, max_k);
  ck(nmtg_attn_fwd(&d, cur_stream()));
}

void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& out, Tensor& lse, const Tensor& cu_q,
              const Tensor& cu_k, int64_t num_heads, int64_t max_q, int64_t max_k, bool causal, double scale,
              double dropout_p, int64_t seed, int64_t stream_id) {
  attn_fwd_bias(q, k, v, out, lse, cu_q, cu_k, num_heads, max_q, max_k, causal, scale, dropout_p, seed, stream_id, c10::nullopt);
}

void attn_bwd_bias(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse, const Tensor& d_out,
                   Tensor& dq, Tensor& dk, Tensor& dv, const OptTensor& dq_acc, const Tensor& cu_q, const Tensor& cu_k,
                   int64_t num_heads, int64_t max_q, int64_t max_k, bool causal, double scale, double dropout_p, int64_t seed,
                   int64_t stream_id, const OptTensor& bias, const OptTensor& dbias) {
  c10::cuda::CUDAGuard guard(q.device());
  AttnDesc d = {};
  fill_attn(d, q, k, v, out, lse, cu_q, cu_k, num_heads, max_q, max_k, causal, scale, dropout_p, seed, stream_id);
  fill_attn_bias(d, bias, dbias, max_q, max_k);
  need_bf16(d_out, "d_out"); need_bf16(dq, "dq"); need_bf16(dk, "dk"); need_bf16(dv, "dv");
  need_rowmajor2d(d_out, "d_out"); need_rowmajor2d(dq, "dq"); need_rowmajor2d(dk, "dk"); need_rowmajor2d(dv, "dv");
  d.d_out = d_out.data_ptr(); d.ld_dout = static_cast<int>(d_out.stride(0));
  d.dq = dq.data_ptr(); d.ld_dq = static_cast<int>(dq.stride(0));
  d.dk = dk.data_ptr(); d.ld_dk = static_cast<int>(dk.stride(0));
  d.dv = dv.data_ptr(); d.ld_dv = static_cast<int>(dv.stride(0));
  if (dq_acc.has_value()) {
    need_f32(*dq_acc, "dq_acc"); need_rowmajor2d(*dq_acc, "dq_acc");
    d.dq_acc = dq_acc->data_ptr<float>(); d.ld_dqacc = static_cast<int>(dq_acc->stride(0));
  }
  Tensor delta;
  if (max_k > 128) {
    delta = torch::empty_like(lse);
    d.delta = delta.data_ptr<float>();
  }
  ck(nmtg_attn_bwd(&d, cur_stream()));
}

void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse, const Tensor& d_out,
              Tensor& dq, Tensor& dk, Tensor& dv, const OptTensor& dq_acc, const Tensor& cu_q, const Tensor& cu_k,
              int64_t num_heads, int64_t max_q, int64_t max_k, bool causal, double scale, double dropout_p, int64_t seed,
              int64_t stream_id) {
  attn_bwd_bias(q, k, v, out, lse, d_out, dq, dk, dv, dq_acc, cu_q, cu_k, num_heads, max_q, max_k, causal, scale, dropout_p, seed,
                stream_id, c10::nullopt, c10::nullopt);
}

// ---- symmetric (IPC-exportable) memory and the peer-memory optimiser step ---------------------------------
Tensor symm_alloc(int64_t nbytes, int64_t device) {
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, static_cast<size_t>(nbytes));
  TORCH_CHECK(e == cudaSuccess, "cudaMalloc of ", nbytes, " bytes failed: ", cudaGetErrorString(e));
  cudaMemset(ptr, 0, static_cast<size_t>(nbytes));
  cudaDeviceSynchronize();
  auto opts = torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA, static_cast<c10::DeviceIndex>(device));
  return torch::from_blob(ptr, {nbytes}, [](void* p) { cudaFree(p); }, opts);
}

py::bytes ipc_get_handle(const Tensor& t) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, t.data_ptr());
  TORCH_CHECK(e == cudaSuccess, "cudaIpcGetMemHandle failed: ", cudaGetErrorString(e));
  return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
}

int64_t ipc_open_handle(const std::string& bytes, int64_t device) {
  TORCH_CHECK(bytes.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  cudaIpcMemHandle_t h;
  memcpy(&h, bytes.data(), sizeof(h));
  void* ptr = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
  TORCH_CHECK(e == cudaSuccess, "cudaIpcOpenMemHandle failed: ", cudaGetErrorString(e));
  return reinterpret_cast<int64_t>(ptr);
}

void ipc_close_handle(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }

long long g_peer_timeout_ns = 20LL * 1000 * 1000 * 1000;   // wall-time bound of every cross-GPU wait

NmtgPeerTable make_table(int64_t rank, const std::vector<int64_t>& grads, const std::vector<int64_t>& works,
                         const std::vector<int64_t>& flags, const std::vector<int64_t>& partials, const OptTensor& norm_out) {
  NmtgPeerTable t = {};
  t.rank = static_cast<int>(rank);
  t.world = static_cast<int>(grads.size());
  TORCH_CHECK(t.world >= 1 && t.world <= 16 && works.size() == grads.size() && flags.size() == grads.size() &&
              partials.size() == grads.size(), "peer table: inconsistent sizes");
  for (int i = 0; i < t.world; ++i) {
    t.grads[i] = reinterpret_cast<float*>(grads[i]);
    t.works[i] = reinterpret_cast<unsigned short*>(works[i]);
    t.flags[i] = reinterpret_cast<int*>(flags[i]);
    t.partials[i] = reinterpret_cast<float*>(partials[i]);
  }
  t.norm_out = norm_out.has_value() ? norm_out->data_ptr<float>() : nullptr;
  t.timeout_ns = g_peer_timeout_ns;
  return t;
}

// reduce-scatter of one unit (see ops_api.h); `reduced` is the unit's piece inside the shard-ordered buffer
void reduce_unit(int64_t rank, const std::vector<int64_t>& grads, const std::vector<int64_t>& flags, int64_t row, Tensor& reduced,
                 int64_t global_begin, int64_t len, bool accumulate, int64_t zero_begin, int64_t zero_len,
                 const OptTensor& counter, const Tensor& epoch, int64_t ctas) {
  need_f32(reduced, "reduced");
  TORCH_CHECK(reduced.is_contiguous() && reduced.numel() >= len, "reduce_unit: output too small");
  TORCH_CHECK(epoch.is_cuda() && epoch.scalar_type() == at::kInt);
  if (counter.has_value()) TORCH_CHECK(counter->is_cuda() && counter->scalar_type() == at::kInt);
  std::vector<int64_t> zeros(grads.size(), 0);
  c10::cuda::CUDAGuard guard(reduced.device());
  NmtgPeerTable t = make_table(rank, grads, zeros, flags, zeros, c10::nullopt);
  ck(nmtg_reduce_unit(&t, static_cast<int>(row), reduced.data_ptr<float>(), global_begin, len, accumulate ? 1 : 0, zero_begin,
                      zero_len, counter.has_value() ? counter->data_ptr<int>() : nullptr, epoch.data_ptr<int>(),
                      status_ptr(reduced), static_cast<int>(ctas), cur_stream()));
}

void update_pieces(int64_t rank, const std::vector<int64_t>& grads, const std::vector<int64_t>& works,
                   const std::vector<int64_t>& flags, const std::vector<int64_t>& partials, const std::vector<int64_t>& shard_off,
                   const std::vector<int64_t>& global_begin, const std::vector<int64_t>& piece_len, const Tensor& reduced,
                   Tensor& master, Tensor& m, Tensor& v, const Tensor& hyper, const Tensor& sq, const Tensor& nonfinite, int64_t mode,
                   int64_t zero_len, Tensor& epoch, const OptTensor& norm_out) {
  need_f32(reduced, "reduced"); need_f32(sq, "sq"); need_f32(master, "master"); need_f32(m, "m"); need_f32(v, "v");
  need_f32(hyper, "hyper");
  TORCH_CHECK(shard_off.size() == global_begin.size() && shard_off.size() == piece_len.size() &&
              shard_off.size() <= static_cast<size_t>(kNmtgMaxUnits), "update_pieces: inconsistent piece lists");
  c10::cuda::CUDAGuard guard(master.device());
  NmtgPeerTable t = make_table(rank, grads, works, flags, partials, norm_out);
  NmtgPieces pc = {};
  pc.n = static_cast<int>(shard_off.size());
  for (int u = 0; u < pc.n; ++u) {
    pc.shard_off[u] = shard_off[u]; pc.global_begin[u] = global_begin[u]; pc.len[u] = piece_len[u];
    TORCH_CHECK(shard_off[u] + piece_len[u] <= reduced.numel() && shard_off[u] + piece_len[u] <= m.numel() &&
                shard_off[u] + piece_len[u] <= v.numel(), "update_pieces: piece outside the shard-ordered buffers");
    TORCH_CHECK((mode == 0 ? global_begin[u] : shard_off[u]) + piece_len[u] <= master.numel(), "update_pieces: piece outside the master weights");
  }
  ck(nmtg_update_pieces(&t, &pc, reduced.data_ptr<float>(), master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                        reinterpret_cast<const NmtgAdamHyper*>(hyper.data_ptr<float>()), sq.data_ptr<float>(),
                        nonfinite.data_ptr<int>(), static_cast<int>(mode), zero_len, epoch.data_ptr<int>(), status_ptr(master),
                        cur_stream()));
}

void peer_finish_step(int64_t rank, const std::vector<int64_t>& flags, Tensor& epoch) {
  std::vector<int64_t> zeros(flags.size(), 0);
  c10::cuda::CUDAGuard guard(epoch.device());
  NmtgPeerTable t = make_table(rank, zeros, zeros, flags, zeros, c10::nullopt);
  ck(nmtg_peer_finish_step(&t, epoch.data_ptr<int>(), status_ptr(epoch), cur_stream()));
}

void fsdp_gather(int64_t rank, const std::vector<int64_t>& works, Tensor& dst, int64_t shard_off, int64_t piece_len,
                 int64_t e0, int64_t e1, int64_t ctas) {
  need_bf16(dst, "dst");
  TORCH_CHECK(dst.is_contiguous() && dst.numel() >= e1, "fsdp_gather: staging buffer too small");
  std::vector<int64_t> zeros(works.size(), 0);
  c10::cuda::CUDAGuard guard(dst.device());
  NmtgPeerTable t = make_table(rank, zeros, works, zeros, zeros, c10::nullopt);
  ck(nmtg_fsdp_gather(&t, dst.data_ptr(), shard_off, piece_len, e0, e1, static_cast<int>(ctas), cur_stream()));
}

void peer_wait_row(int64_t rank, const std::vector<int64_t>& flags, int64_t row, int64_t epoch, const Tensor& like) {
  std::vector<int64_t> zeros(flags.size(), 0);
  c10::cuda::CUDAGuard guard(like.device());
  NmtgPeerTable t = make_table(rank, zeros, zeros, flags, zeros, c10::nullopt);
  ck(nmtg_peer_wait_row(&t, static_cast<int>(row), static_cast<int>(epoch), status_ptr(like), cur_stream()));
}

void set_peer_timeout_ms(double ms) { g_peer_timeout_ns = static_cast<long long>(ms * 1e6); }
double get_peer_timeout_ms() { return static_cast<double>(g_peer_timeout_ns) / 1e6; }
Tensor get_status_tensor(int64_t device) { return status_tensor(static_cast<int>(device)); }

int64_t read_status(int64_t device) {
  Tensor& s = status_tensor(static_cast<int>(device));
  return s.cpu().item<int>();
}
void clear_status(int64_t device) { status_tensor(static_cast<int>(device)).zero_(); }

}  // namespace

void bind_sequence_ops(pybind11::module& m);   // bindings_seq.cpp
extern "C" long nmtg_bounds_violations();

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  bind_sequence_ops(m);
  m.def("gemm", &gemm, pybind11::arg("a"), pybind11::arg("a_mn_major"), pybind11::arg("b"), pybind11::arg("b_mn_major"), pybind11::arg("out"),
        pybind11::arg("bias"), pybind11::arg("residual"), pybind11::arg("aux"), pybind11::arg("preact"), pybind11::arg("act"),
        pybind11::arg("dropout_p"), pybind11::arg("seed"), pybind11::arg("stream_id"), pybind11::arg("alpha"), pybind11::arg("accumulate"),
        pybind11::arg("allow_split_k"), pybind11::arg("split_k"), pybind11::arg("force_bn"), pybind11::arg("mask") = pybind11::none(),
        pybind11::arg("colsum") = pybind11::none(), pybind11::arg("gather") = pybind11::none());
  m.def("set_gemm_variant", [](int64_t v) { nmtg_set_gemm_variant(static_cast<int>(v)); });
  m.def("set_sm_reserve", [](int64_t n) { nmtg_set_sm_reserve(static_cast<int>(n)); });
  m.def("set_attn_bwd_ablation", [](int64_t v) { nmtg_set_attn_bwd_ablation(static_cast<int>(v)); });
  m.def("attn_fws_trace", []() {
    Tensor t = torch::zeros({512}, torch::kInt64);
    const int n = nmtg_attn_fws_trace(reinterpret_cast<long long*>(t.data_ptr<int64_t>()), 512);
    TORCH_CHECK(n >= 0, "attn_fws_trace: copy from the device failed");
    return t.view({32, 16});
  });
  m.def("attn_ws_trace", []() {
    Tensor t = torch::zeros({512}, torch::kInt64);
    const int n = nmtg_attn_ws_trace(reinterpret_cast<long long*>(t.data_ptr<int64_t>()), 512);
    TORCH_CHECK(n >= 0, "attn_ws_trace: copy from the device failed");
    return t.view({32, 16});
  });
  m.def("set_gemm_trace", [](const OptTensor& buf) {
    if (buf.has_value()) {
      TORCH_CHECK(buf->is_cuda() && buf->scalar_type() == at::kLong && buf->is_contiguous() && buf->numel() >= 16 * 128);
      nmtg_set_gemm_trace(reinterpret_cast<long long*>(buf->data_ptr<int64_t>()));
    } else {
      nmtg_set_gemm_trace(nullptr);
    }
  });
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("xent_fused", &xent_fused);
  m.def("dropout_add", &dropout_add);
  m.def("act_backward", &act_backward);
  m.def("dropout_colsum", &dropout_colsum);
  m.def("embed_fwd", &embed_fwd);
  m.def("embed_bwd", &embed_bwd);
  m.def("colsum", &colsum);
  m.def("sq_norm", &sq_norm);
  m.def("adamw_flat", &adamw_flat);
  m.def("loss_scale_prepare", &loss_scale_prepare);
  m.def("loss_scale_update", &loss_scale_update);
  m.def("cast_f32_bf16", &cast_f32_bf16);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  m.def("attn_fwd_bias", &attn_fwd_bias);
  m.def("attn_bwd_bias", &attn_bwd_bias);
  m.def("set_attention_variant", [](int64_t v) { nmtg_set_attention_variant(static_cast<int>(v)); });
  m.def("batch_allocate", &batch_allocate);
  m.def("get_seed_tensor", &get_seed_tensor);
  m.def("symm_alloc", &symm_alloc);
  m.def("ipc_get_handle", &ipc_get_handle);
  m.def("ipc_open_handle", &ipc_open_handle);
  m.def("ipc_close_handle", &ipc_close_handle);
  m.def("reduce_unit", &reduce_unit);
  m.def("update_pieces", &update_pieces);
  m.def("peer_finish_step", &peer_finish_step);
  m.def("fsdp_gather", &fsdp_gather);
  m.def("peer_wait_row", &peer_wait_row);
  m.def("set_peer_timeout_ms", &set_peer_timeout_ms);
  m.def("get_peer_timeout_ms", &get_peer_timeout_ms);
  m.def("get_status_tensor", &get_status_tensor);
  m.def("bounds_violations", []() { return static_cast<int64_t>(nmtg_bounds_violations()); });
  m.def("read_status", &read_status);
  m.def("clear_status", &clear_status);
}
