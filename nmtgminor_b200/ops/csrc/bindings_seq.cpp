// Python bindings of the sequence / decoding kernels declared in seq_api.h.  Output tensors are allocated here;
// the launchers themselves allocate nothing.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "seq_api.h"

namespace {

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void ck(const char* err) {
  if (err) throw std::runtime_error(std::string("nmtgminor_b200 kernel launch failed: ") + err);
}
int dtype_code(const Tensor& t) {
  if (t.scalar_type() == at::kFloat) return 0;
  if (t.scalar_type() == at::kBFloat16) return 1;
  TORCH_CHECK(false, "expected a float32 or bfloat16 tensor");
  return -1;
}
void need(const Tensor& t, at::ScalarType ty, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == ty, name, ": wrong device, layout or dtype");
}
const long* off_ptr(const OptTensor& t) {
  if (!t.has_value()) return nullptr;
  need(*t, at::kLong, "batch_offset");
  return reinterpret_cast<const long*>(t->data_ptr<int64_t>());
}

Tensor joint_fwd(const Tensor& f, const Tensor& g, const Tensor& f_len, const Tensor& g_len, const OptTensor& batch_offset,
                 int64_t packed_rows, bool relu, double p, int64_t seed, int64_t stream_id) {
  TORCH_CHECK(f.is_cuda() && f.is_contiguous() && g.is_contiguous() && f.dim() == 3 && g.dim() == 3);
  TORCH_CHECK(f.scalar_type() == g.scalar_type() && f.size(0) == g.size(0) && f.size(2) == g.size(2));
  need(f_len, at::kInt, "f_len"); need(g_len, at::kInt, "g_len");
  c10::cuda::CUDAGuard guard(f.device());
  const int B = f.size(0), T = f.size(1), U = g.size(1), H = f.size(2);
  const bool packed = batch_offset.has_value();
  Tensor out = packed ? torch::empty({packed_rows, H}, f.options()) : torch::empty({B, T, U, H}, f.options());
  ck(nmtg_transducer_joint_fwd(f.data_ptr(), g.data_ptr(), f_len.data_ptr<int>(), g_len.data_ptr<int>(), off_ptr(batch_offset),
                               out.data_ptr(), B, T, U, H, dtype_code(f), packed, relu, static_cast<float>(p),
                               static_cast<unsigned long long>(seed), static_cast<unsigned long long>(stream_id), cur_stream()));
  return out;
}

std::vector<Tensor> joint_bwd(const Tensor& dout, const OptTensor& out, const Tensor& f_len, const Tensor& g_len,
                              const OptTensor& batch_offset, int64_t T, int64_t U, bool relu, double p, int64_t seed,
                              int64_t stream_id, double scale) {
  TORCH_CHECK(dout.is_cuda() && dout.is_contiguous());
  if (out.has_value()) TORCH_CHECK(out->is_contiguous() && out->scalar_type() == dout.scalar_type() && out->numel() == dout.numel());
  c10::cuda::CUDAGuard guard(dout.device());
  const int B = f_len.size(0), H = dout.size(-1);
  Tensor df = torch::empty({B, T, H}, dout.options()), dg = torch::empty({B, U, H}, dout.options());
  ck(nmtg_transducer_joint_bwd(dout.data_ptr(), out.has_value() ? out->data_ptr() : nullptr, f_len.data_ptr<int>(),
                               g_len.data_ptr<int>(), off_ptr(batch_offset), df.data_ptr(), dg.data_ptr(), B, static_cast<int>(T),
                               static_cast<int>(U), H, dtype_code(dout), batch_offset.has_value(), relu, static_cast<float>(p),
                               static_cast<unsigned long long>(seed), static_cast<unsigned long long>(stream_id),
                               static_cast<float>(scale), cur_stream()));
  return {df, dg};
}

std::vector<Tensor> rnnt_loss_fwd(const Tensor& x, const Tensor& label, const Tensor& f_len, const Tensor& y_len,
                                  const OptTensor& batch_offset, int64_t T, int64_t blank) {
  need(x, at::kFloat, "x"); need(label, at::kInt, "label"); need(f_len, at::kInt, "f_len"); need(y_len, at::kInt, "y_len");
  c10::cuda::CUDAGuard guard(x.device());
  const int B = label.size(0), U = label.size(1) + 1, V = x.size(-1);
  auto o = x.options();
  Tensor alpha = torch::zeros({B, T, U}, o), beta = torch::zeros({B, T, U}, o), loss = torch::zeros({B}, o);
  ck(nmtg_transducer_loss_fwd(x.data_ptr<float>(), label.data_ptr<int>(), f_len.data_ptr<int>(), y_len.data_ptr<int>(),
                              off_ptr(batch_offset), alpha.data_ptr<float>(), beta.data_ptr<float>(), loss.data_ptr<float>(), B,
                              static_cast<int>(T), U, V, static_cast<int>(blank), batch_offset.has_value(), cur_stream()));
  return {alpha, beta, loss};
}

Tensor rnnt_loss_bwd(const Tensor& x, const Tensor& loss_grad, const Tensor& alpha, const Tensor& beta, const Tensor& label,
                     const Tensor& f_len, const Tensor& y_len, const OptTensor& batch_offset, int64_t blank, bool fuse_softmax) {
  need(x, at::kFloat, "x"); need(loss_grad, at::kFloat, "loss_grad");
  c10::cuda::CUDAGuard guard(x.device());
  const int B = alpha.size(0), T = alpha.size(1), U = alpha.size(2), V = x.size(-1);
  Tensor dx = torch::empty_like(x);
  ck(nmtg_transducer_loss_bwd(x.data_ptr<float>(), loss_grad.data_ptr<float>(), alpha.data_ptr<float>(), beta.data_ptr<float>(),
                              label.data_ptr<int>(), f_len.data_ptr<int>(), y_len.data_ptr<int>(), off_ptr(batch_offset),
                              dx.data_ptr<float>(), B, T, U, V, static_cast<int>(blank), batch_offset.has_value(), fuse_softmax,
                              cur_stream()));
  return dx;
}

const float2* c64(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kComplexFloat, name, " must be a contiguous complex64 CUDA tensor");
  return reinterpret_cast<const float2*>(t.data_ptr());
}

Tensor lru_scan_fwd(const Tensor& lambda, const Tensor& x, const Tensor& lengths, int64_t direction) {
  need(lengths, at::kInt, "lengths");
  TORCH_CHECK(x.dim() == 3 && lambda.numel() == x.size(1) && lengths.numel() == x.size(0));
  c10::cuda::CUDAGuard guard(x.device());
  Tensor h = torch::empty_like(x);
  ck(nmtg_lru_scan_fwd(c64(lambda, "lambda"), c64(x, "x"), lengths.data_ptr<int>(), reinterpret_cast<float2*>(h.data_ptr()),
                       x.size(0), x.size(1), x.size(2), static_cast<int>(direction), cur_stream()));
  return h;
}

std::vector<Tensor> lru_scan_bwd(const Tensor& lambda, const Tensor& grad_h, const Tensor& h, const Tensor& lengths,
                                 int64_t direction) {
  need(lengths, at::kInt, "lengths");
  c10::cuda::CUDAGuard guard(h.device());
  Tensor dx = torch::empty_like(h), dl = torch::zeros_like(lambda);
  ck(nmtg_lru_scan_bwd(c64(lambda, "lambda"), c64(grad_h, "grad_h"), c64(h, "h"), lengths.data_ptr<int>(),
                       reinterpret_cast<float2*>(dx.data_ptr()), reinterpret_cast<float2*>(dl.data_ptr()), h.size(0), h.size(1),
                       h.size(2), static_cast<int>(direction), cur_stream()));
  return {dx, dl};
}

Tensor cauchy_fwd(const Tensor& a, const Tensor& b, const Tensor& c) {
  TORCH_CHECK(a.dim() == 4 && b.dim() == 3 && c.dim() == 2);
  const int I = a.size(0), Q = a.size(1), H = a.size(2), N = a.size(3), L = b.size(1);
  TORCH_CHECK(b.size(0) == Q && b.size(2) == H && c.size(0) == Q && c.size(1) == N);
  c10::cuda::CUDAGuard guard(a.device());
  Tensor out = torch::empty({I, Q, L, H}, a.options());
  ck(nmtg_cauchy_fwd(c64(a, "a"), c64(b, "b"), c64(c, "c"), reinterpret_cast<float2*>(out.data_ptr()), I, Q, L, H, N, cur_stream()));
  return out;
}

std::vector<Tensor> cauchy_bwd(const Tensor& a, const Tensor& b, const Tensor& c, const Tensor& dout) {
  const int I = a.size(0), Q = a.size(1), H = a.size(2), N = a.size(3), L = b.size(1);
  c10::cuda::CUDAGuard guard(a.device());
  Tensor da = torch::zeros_like(a), db = torch::zeros_like(b), dc = torch::zeros_like(c);
  ck(nmtg_cauchy_bwd(c64(a, "a"), c64(b, "b"), c64(c, "c"), c64(dout, "dout"), reinterpret_cast<float2*>(da.data_ptr()),
                     reinterpret_cast<float2*>(db.data_ptr()), reinterpret_cast<float2*>(dc.data_ptr()), I, Q, L, H, N, cur_stream()));
  return {da, db, dc};
}

std::vector<Tensor> softmax_dropout_fwd(const Tensor& x, const OptTensor& pad_mask, int64_t rows_per_mask, double scale, double p,
                                        int64_t seed, int64_t stream_id) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = x.size(-1), rows = x.numel() / cols;
  const uint8_t* mp = nullptr;
  if (pad_mask.has_value()) {
    TORCH_CHECK(pad_mask->is_cuda() && pad_mask->is_contiguous() && pad_mask->element_size() == 1 && pad_mask->size(-1) == cols);
    TORCH_CHECK(pad_mask->numel() / cols * rows_per_mask == rows, "mask rows * rows_per_mask must equal the number of rows");
    mp = static_cast<const uint8_t*>(pad_mask->data_ptr());
  }
  Tensor y = torch::empty_like(x);
  Tensor yd = p > 0 ? torch::empty_like(x) : y;
  ck(nmtg_softmax_dropout_fwd(x.data_ptr(), mp, y.data_ptr(), p > 0 ? yd.data_ptr() : nullptr, rows, cols,
                              static_cast<int>(rows_per_mask), dtype_code(x), static_cast<float>(scale), static_cast<float>(p),
                              static_cast<unsigned long long>(seed), static_cast<unsigned long long>(stream_id), cur_stream()));
  return {yd, y};
}

Tensor softmax_dropout_bwd(const Tensor& dyd, const Tensor& y, double scale, double p, int64_t seed, int64_t stream_id) {
  TORCH_CHECK(dyd.is_cuda() && dyd.is_contiguous() && y.is_contiguous() && dyd.scalar_type() == y.scalar_type());
  c10::cuda::CUDAGuard guard(y.device());
  const int cols = y.size(-1), rows = y.numel() / cols;
  Tensor dx = torch::empty_like(y);
  ck(nmtg_softmax_dropout_bwd(dyd.data_ptr(), y.data_ptr(), dx.data_ptr(), rows, cols, dtype_code(y), static_cast<float>(scale),
                              static_cast<float>(p), static_cast<unsigned long long>(seed),
                              static_cast<unsigned long long>(stream_id), cur_stream()));
  return dx;
}

std::vector<Tensor> beam_topk(const Tensor& logits, const Tensor& scores, const OptTensor& force_eos, int64_t K, int64_t pad,
                              int64_t eos, bool ban_eos) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  need(scores, at::kFloat, "scores");
  c10::cuda::CUDAGuard guard(logits.device());
  const int R = logits.size(0), V = logits.size(1);
  TORCH_CHECK(R % K == 0 && scores.numel() == R);
  const int B = R / K;
  const uint8_t* fe = nullptr;
  if (force_eos.has_value()) {
    TORCH_CHECK(force_eos->is_cuda() && force_eos->is_contiguous() && force_eos->element_size() == 1 && force_eos->numel() == R);
    fe = static_cast<const uint8_t*>(force_eos->data_ptr());
  }
  auto fo = torch::dtype(torch::kFloat).device(logits.device());
  Tensor lse = torch::empty({R}, fo), cv = torch::empty({R, 2 * K}, fo);
  Tensor ci = torch::empty({R, 2 * K}, fo.dtype(torch::kInt));
  Tensor os = torch::empty({B, 2 * K}, fo), oi = torch::empty({B, 2 * K}, fo.dtype(torch::kLong));
  ck(nmtg_beam_topk(logits.data_ptr(), logits.stride(0), dtype_code(logits), scores.data_ptr<float>(), fe, lse.data_ptr<float>(),
                    cv.data_ptr<float>(), ci.data_ptr<int>(), os.data_ptr<float>(), reinterpret_cast<long*>(oi.data_ptr<int64_t>()),
                    B, static_cast<int>(K), V, static_cast<int>(pad), static_cast<int>(eos), ban_eos, cur_stream()));
  return {os, oi, lse};
}

const int* dev_int(const OptTensor& t, const char* name) {
  if (!t.has_value()) return nullptr;
  need(*t, at::kInt, name);
  return t->data_ptr<int>();
}

void gather_rows(const Tensor& src, Tensor& dst, const Tensor& index, int64_t copy_elems, const OptTensor& filled_dev,
                 int64_t unit_elems) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && dst.is_contiguous() && src.sizes() == dst.sizes());
  need(index, at::kLong, "index");
  c10::cuda::CUDAGuard guard(src.device());
  const long rows = index.numel();
  TORCH_CHECK(rows <= dst.size(0));
  const long stride = src.numel() / src.size(0) * src.element_size();
  const long copy = copy_elems < 0 ? stride : copy_elems * src.element_size();
  ck(nmtg_gather_rows(src.data_ptr(), dst.data_ptr(), reinterpret_cast<const long*>(index.data_ptr<int64_t>()),
                      static_cast<int>(rows), static_cast<int>(src.size(0)), stride, copy, dev_int(filled_dev, "filled_dev"), unit_elems * src.element_size(),
                      cur_stream()));
}

Tensor decode_attn(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const OptTensor& lengths, int64_t len,
                   int64_t heads, double scale, const OptTensor& len_dev, int64_t len_add) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.dim() == 2 && q.stride(1) == 1);
  need(k_cache, at::kBFloat16, "k_cache"); need(v_cache, at::kBFloat16, "v_cache");
  TORCH_CHECK(k_cache.dim() == 3 && k_cache.sizes() == v_cache.sizes() && k_cache.size(2) == heads * 64 && q.size(1) == heads * 64);
  c10::cuda::CUDAGuard guard(q.device());
  const int R = q.size(0), cap = k_cache.size(1);
  TORCH_CHECK(R % k_cache.size(0) == 0, "query rows must be a multiple of cache rows");
  const int kv_div = R / k_cache.size(0);
  const int* lp = nullptr;
  if (lengths.has_value()) { need(*lengths, at::kInt, "lengths"); TORCH_CHECK(lengths->numel() == k_cache.size(0)); lp = lengths->data_ptr<int>(); }
  Tensor out = torch::empty({R, heads * 64}, q.options());
  ck(nmtg_decode_attn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), lp, out.data_ptr(), R,
                      static_cast<int>(heads), cap, static_cast<int>(len), kv_div, static_cast<float>(scale),
                      dev_int(len_dev, "len_dev"), static_cast<int>(len_add), cur_stream()));
  return out;
}

void cache_append(const Tensor& k_new, const Tensor& v_new, Tensor& k_cache, Tensor& v_cache, int64_t pos, const OptTensor& pos_dev) {
  TORCH_CHECK(k_new.is_cuda() && k_new.scalar_type() == at::kBFloat16 && k_new.dim() == 2 && k_new.stride(1) == 1);
  TORCH_CHECK(v_new.scalar_type() == at::kBFloat16 && v_new.stride(1) == 1 && v_new.stride(0) == k_new.stride(0) && v_new.sizes() == k_new.sizes());
  need(k_cache, at::kBFloat16, "k_cache"); need(v_cache, at::kBFloat16, "v_cache");
  TORCH_CHECK(k_cache.dim() == 3 && k_cache.size(0) >= k_new.size(0) && k_cache.size(2) == k_new.size(1) && k_new.size(1) % 64 == 0);
  c10::cuda::CUDAGuard guard(k_new.device());
  ck(nmtg_cache_append(k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                       static_cast<int>(k_new.size(0)), static_cast<int>(k_new.size(1) / 64), static_cast<int>(k_cache.size(1)),
                       static_cast<int>(pos), dev_int(pos_dev, "pos_dev"), cur_stream()));
}

std::vector<Tensor> rel_attn_fwd(const Tensor& qkv, const Tensor& r, const Tensor& u, const Tensor& w, const Tensor& cu, int64_t heads,
                                 int64_t max_len, int64_t r_center, bool causal, double scale, double p, int64_t seed, int64_t stream_id) {
  need(qkv, at::kBFloat16, "qkv"); need(r, at::kBFloat16, "r"); need(u, at::kFloat, "u"); need(w, at::kFloat, "w"); need(cu, at::kInt, "cu");
  TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) == 3 * heads * 64 && r.dim() == 2 && r.size(1) == heads * 64 && u.numel() == heads * 64 && w.numel() == heads * 64);
  c10::cuda::CUDAGuard guard(qkv.device());
  const int N = qkv.size(0), B = cu.numel() - 1;
  Tensor out = torch::zeros({N, heads * 64}, qkv.options());
  Tensor lse = torch::zeros({heads, N}, qkv.options().dtype(torch::kFloat));
  ck(nmtg_rel_attn_fwd(qkv.data_ptr(), r.data_ptr(), u.data_ptr<float>(), w.data_ptr<float>(), cu.data_ptr<int>(), out.data_ptr(),
                       lse.data_ptr<float>(), B, N, static_cast<int>(heads), static_cast<int>(max_len), static_cast<int>(r_center),
                       static_cast<int>(r.size(0)), causal, static_cast<float>(scale), static_cast<float>(p),
                       static_cast<unsigned long long>(seed), static_cast<unsigned long long>(stream_id), cur_stream()));
  return {out, lse};
}

std::vector<Tensor> rel_attn_bwd(const Tensor& qkv, const Tensor& r, const Tensor& u, const Tensor& w, const Tensor& cu, const Tensor& lse,
                                 const Tensor& dctx, int64_t heads, int64_t max_len, int64_t r_center, bool causal, double scale, double p,
                                 int64_t seed, int64_t stream_id) {
  need(dctx, at::kBFloat16, "dctx"); need(lse, at::kFloat, "lse");
  c10::cuda::CUDAGuard guard(qkv.device());
  const int N = qkv.size(0), B = cu.numel() - 1;
  auto f32 = qkv.options().dtype(torch::kFloat);
  Tensor dqkv = torch::zeros_like(qkv), dr = torch::zeros({r.size(0), r.size(1)}, f32), du = torch::zeros({heads, 64}, f32),
         dw = torch::zeros({heads, 64}, f32);
  ck(nmtg_rel_attn_bwd(qkv.data_ptr(), r.data_ptr(), u.data_ptr<float>(), w.data_ptr<float>(), cu.data_ptr<int>(), lse.data_ptr<float>(),
                       dctx.data_ptr(), dqkv.data_ptr(), dr.data_ptr<float>(), du.data_ptr<float>(), dw.data_ptr<float>(), B, N,
                       static_cast<int>(heads), static_cast<int>(max_len), static_cast<int>(r_center), static_cast<int>(r.size(0)), causal,
                       static_cast<float>(scale), static_cast<float>(p), static_cast<unsigned long long>(seed),
                       static_cast<unsigned long long>(stream_id), cur_stream()));
  return {dqkv, dr, du, dw};
}

}  // namespace

void bind_sequence_ops(pybind11::module& m) {
  m.def("rel_attn_fwd", &rel_attn_fwd);
  m.def("rel_attn_bwd", &rel_attn_bwd);
  m.def("joint_fwd", &joint_fwd);
  m.def("joint_bwd", &joint_bwd);
  m.def("rnnt_loss_fwd", &rnnt_loss_fwd);
  m.def("rnnt_loss_bwd", &rnnt_loss_bwd);
  m.def("lru_scan_fwd", &lru_scan_fwd);
  m.def("lru_scan_bwd", &lru_scan_bwd);
  m.def("cauchy_fwd", &cauchy_fwd);
  m.def("cauchy_bwd", &cauchy_bwd);
  m.def("softmax_dropout_fwd", &softmax_dropout_fwd);
  m.def("softmax_dropout_bwd", &softmax_dropout_bwd);
  m.def("beam_topk", &beam_topk);
  namespace py = pybind11;
  m.def("gather_rows", &gather_rows, py::arg("src"), py::arg("dst"), py::arg("index"), py::arg("copy_elems"),
        py::arg("filled_dev") = py::none(), py::arg("unit_elems") = 0);
  m.def("decode_attn", &decode_attn, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("lengths"), py::arg("len"),
        py::arg("heads"), py::arg("scale"), py::arg("len_dev") = py::none(), py::arg("len_add") = 0);
  m.def("cache_append", &cache_append, py::arg("k_new"), py::arg("v_new"), py::arg("k_cache"), py::arg("v_cache"), py::arg("pos"),
        py::arg("pos_dev") = py::none());
}
