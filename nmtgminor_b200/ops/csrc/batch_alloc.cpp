// Host-side greedy batch allocation over sentence sizes (the data loader's bucketing step).
//
// A batch keeps taking sentences (in the given order) while
//     max(length in batch, new length) * (count + 1) <= token budget      (and the frame budget for speech)
// and count < sentence cap; when the next sentence would overflow, the batch is cut back to a multiple of
// `multiplier` sentences (the remainder starts the next batch).  Sentences outside [min, max) source /
// target lengths are dropped when `cleaning` is set.  Returns the batches as (flat indices, offsets).
//
// Same policy as the reference's Cython allocator (onmt/data/fast_extensions.pyx:23-173) and its Python
// fallback (onmt/data/batch_utils.py:7-156).
#include <torch/extension.h>
#include <vector>
#include <algorithm>

namespace {

struct Window {
  // running maxima over the sentences currently in the batch, recomputed after a cut
  std::vector<int64_t> words, frames;
  int64_t max_words() const { return words.empty() ? 0 : *std::max_element(words.begin(), words.end()); }
  int64_t max_frames() const { return frames.empty() ? 0 : *std::max_element(frames.begin(), frames.end()); }
};

}  // namespace

std::vector<torch::Tensor> batch_allocate(const torch::Tensor& indices, const torch::Tensor& lengths,
                                          const c10::optional<torch::Tensor>& src_sizes,
                                          const c10::optional<torch::Tensor>& tgt_sizes, int64_t batch_size_words,
                                          int64_t batch_size_frames, int64_t batch_size_sents, int64_t multiplier,
                                          int64_t max_src_len, int64_t max_tgt_len, int64_t min_src_len,
                                          int64_t min_tgt_len, bool cleaning, bool unbalanced, int64_t cut_off_size,
                                          int64_t smallest_batch_size) {
  TORCH_CHECK(indices.scalar_type() == at::kLong && lengths.scalar_type() == at::kLong, "int64 arrays expected");
  auto idx = indices.contiguous();
  auto len = lengths.contiguous();
  const int64_t* ip = idx.data_ptr<int64_t>();
  const int64_t* lp = len.data_ptr<int64_t>();
  torch::Tensor ss, ts;
  const int64_t* sp = nullptr;
  const int64_t* tp = nullptr;
  if (src_sizes.has_value()) { ss = src_sizes->contiguous(); sp = ss.data_ptr<int64_t>(); }
  if (tgt_sizes.has_value()) { ts = tgt_sizes->contiguous(); tp = ts.data_ptr<int64_t>(); }
  if (multiplier < 1) multiplier = 1;

  std::vector<int64_t> flat, offsets{0};
  std::vector<int64_t> cur;
  Window w;
  int64_t mw = 0, mf = 0;  // cached maxima
  const int64_t n = idx.numel();
  for (int64_t k = 0; k < n; ++k) {
    const int64_t i = ip[k];
    const int64_t src = sp ? sp[i] : (unbalanced ? min_src_len : 0);
    const int64_t tgt = tp ? tp[i] : (unbalanced ? min_tgt_len : 0);
    if (cleaning && !(min_src_len <= src && src < max_src_len && min_tgt_len <= tgt && tgt < max_tgt_len)) continue;
    const int64_t new_words = unbalanced ? tgt : lp[i];
    const int64_t new_frames = src;
    bool over = false;
    const int64_t cnt = static_cast<int64_t>(cur.size());
    if (cnt > 0) {
      if (cnt >= batch_size_sents) over = true;
      else if (unbalanced) {
        const int64_t f = std::max(mf, new_frames);
        if (f > cut_off_size && cnt >= smallest_batch_size) over = true;
        else if (f * (cnt + 1) > batch_size_frames) over = true;
        else if (std::max(mw, new_words) * (cnt + 1) > batch_size_words) over = true;
      } else if (std::max(mw, new_words) * (cnt + 1) > batch_size_words) over = true;
    }
    if (over) {
      const int64_t keep = std::max(multiplier * (cnt / multiplier), cnt % multiplier);
      flat.insert(flat.end(), cur.begin(), cur.begin() + keep);
      offsets.push_back(static_cast<int64_t>(flat.size()));
      cur.erase(cur.begin(), cur.begin() + keep);
      w.words.erase(w.words.begin(), w.words.begin() + keep);
      w.frames.erase(w.frames.begin(), w.frames.begin() + keep);
      mw = w.max_words();
      mf = w.max_frames();
    }
    cur.push_back(i);
    w.words.push_back(new_words);
    w.frames.push_back(new_frames);
    mw = std::max(mw, new_words);
    mf = std::max(mf, new_frames);
  }
  if (!cur.empty()) {
    flat.insert(flat.end(), cur.begin(), cur.end());
    offsets.push_back(static_cast<int64_t>(flat.size()));
  }
  auto opts = torch::TensorOptions().dtype(torch::kLong);
  torch::Tensor f = torch::empty({static_cast<int64_t>(flat.size())}, opts);
  torch::Tensor o = torch::empty({static_cast<int64_t>(offsets.size())}, opts);
  std::copy(flat.begin(), flat.end(), f.data_ptr<int64_t>());
  std::copy(offsets.begin(), offsets.end(), o.data_ptr<int64_t>());
  return {f, o};
}
