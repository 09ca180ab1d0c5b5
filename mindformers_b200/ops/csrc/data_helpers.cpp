// CPU-side index builders for Megatron-style datasets (C ABI, loaded with ctypes + numpy buffers).
//
// Same five services as the reference's pybind11 module (mindformers/dataset/blended_datasets/helpers.cpp:
// build_sample_idx :142-240, build_blending_indices :75-140, build_exhaustive_blending_indices :21-73,
// build_mapping :259-555, build_blocks_mapping :557-830) and the same outputs for the same inputs, written
// against plain pointers so the library needs neither Python headers nor a per-machine `make` step.
//
// Two-call protocol for the functions whose output size depends on the data: a call with out == nullptr
// returns the number of rows, a second call fills a caller-allocated buffer.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <random>
#include <vector>

namespace {

constexpr int32_t kLongSentenceLen = 512;

inline int32_t target_sample_len(int32_t short_seq_ratio, int32_t max_length, std::mt19937& gen) {
  if (short_seq_ratio == 0) return max_length;
  const uint32_t r = gen();
  if (r % static_cast<uint32_t>(short_seq_ratio) == 0) return 2 + static_cast<int32_t>(r % static_cast<uint32_t>(max_length - 1));
  return max_length;
}

template <typename Row>
void shuffle_rows(Row* rows, int64_t n, int64_t seed) {
  std::mt19937_64 gen(static_cast<uint64_t>(seed));
  for (int64_t i = n - 1; i > 0; --i) {
    const int64_t j = static_cast<int64_t>(gen() % static_cast<uint64_t>(i + 1));
    std::swap(rows[i], rows[j]);
  }
}

struct Row3 { int64_t a, b, c; };
struct Row4 { int64_t a, b, c, d; };

}  // namespace

extern "C" {

// Number of training samples that `num_epochs` passes over `tokens_per_epoch` tokens yield.
int64_t mfb_num_samples(int64_t num_epochs, int64_t tokens_per_epoch, int32_t seq_length, int32_t drop_last,
                        int32_t extra_token) {
  const int64_t usable = num_epochs * tokens_per_epoch - extra_token;
  if (drop_last) return usable / seq_length;
  return static_cast<int64_t>(std::ceil(static_cast<float>(usable) / seq_length));
}

// out: int64 [num_samples + 1, 2] = (position in doc_idx, token offset inside that document) of every sample
// boundary when the documents listed by doc_idx are laid end to end and cut every seq_length tokens
// (+ extra_token overlap, i.e. the label of the last position is the first token of the next sample).
int mfb_build_sample_idx(const int32_t* sizes, const int32_t* doc_idx, int64_t doc_idx_len, int32_t seq_length,
                         int64_t num_epochs, int64_t tokens_per_epoch, int32_t drop_last, int32_t extra_token,
                         int64_t* out) {
  if (seq_length <= 1 || num_epochs <= 0 || tokens_per_epoch <= 1 || doc_idx_len <= 0) return 1;
  const int64_t n = mfb_num_samples(num_epochs, tokens_per_epoch, seq_length, drop_last, extra_token);
  int64_t pos = 0;       // index into doc_idx
  int32_t offset = 0;    // token offset in the current document
  out[0] = pos;
  out[1] = offset;
  for (int64_t s = 1; s <= n; ++s) {
    int32_t need = seq_length + extra_token;
    while (need != 0) {
      const int32_t avail = sizes[doc_idx[pos]] - offset;
      need -= avail;
      if (need <= 0) {
        // the sample ends inside this document; step back `extra_token` so the next sample re-reads it
        offset += need + avail - extra_token;
        need = 0;
      } else if (pos == doc_idx_len - 1) {
        // ran out of documents: only legal for the last (partial) sample
        offset = sizes[doc_idx[pos]] - extra_token;
        break;
      } else {
        ++pos;
        offset = 0;
      }
    }
    out[2 * s] = pos;
    out[2 * s + 1] = offset;
  }
  return 0;
}

// Greedy blend: at every step pick the dataset whose achieved share lags its weight the most.
int mfb_build_blending_indices(int16_t* dataset_index, int64_t* dataset_sample_index, const double* weights,
                               int32_t num_datasets, int64_t size) {
  if (num_datasets <= 0 || size < 0) return 1;
  std::vector<int64_t> taken(num_datasets, 0);
  for (int64_t i = 0; i < size; ++i) {
    const double denom = std::max(static_cast<double>(i), 1.0);
    int32_t best = 0;
    double best_err = weights[0] * denom - static_cast<double>(taken[0]);
    for (int32_t d = 1; d < num_datasets; ++d) {
      const double err = weights[d] * denom - static_cast<double>(taken[d]);
      if (err > best_err) { best_err = err; best = d; }
    }
    dataset_index[i] = static_cast<int16_t>(best);
    dataset_sample_index[i] = taken[best];
    ++taken[best];
  }
  return 0;
}

// Blend that draws exactly sizes[d] samples from dataset d, interleaved in proportion to the sizes.
int mfb_build_exhaustive_blending_indices(int16_t* dataset_index, int64_t* dataset_sample_index,
                                          const int64_t* sizes, int32_t num_datasets) {
  if (num_datasets <= 0) return 1;
  int64_t total = 0;
  for (int32_t d = 0; d < num_datasets; ++d) total += sizes[d];
  std::vector<int64_t> taken(num_datasets, 0);
  std::vector<char> open(num_datasets, 1);
  int32_t n_open = 0;
  for (int32_t d = 0; d < num_datasets; ++d) {
    if (sizes[d] > 0) ++n_open; else open[d] = 0;
  }
  int64_t i = 0;
  while (n_open > 0) {
    const double denom = std::max(static_cast<double>(i), 1.0);
    int32_t best = -1;
    double best_err = std::numeric_limits<double>::lowest();
    for (int32_t d = 0; d < num_datasets; ++d) {
      if (!open[d]) continue;
      const double err = (static_cast<double>(sizes[d]) / static_cast<double>(total)) * denom - static_cast<double>(taken[d]);
      if (err > best_err) { best_err = err; best = d; }
    }
    dataset_index[i] = static_cast<int16_t>(best);
    dataset_sample_index[i] = taken[best];
    if (++taken[best] == sizes[best]) { open[best] = 0; --n_open; }
    ++i;
  }
  return 0;
}

// Sentence-span samples for BERT-style datasets. docs: [n_docs + 1] sentence boundaries, sizes: tokens per
// sentence. Rows (first sentence, one-past-last sentence, target length). out == nullptr: count only.
int64_t mfb_build_mapping(const int64_t* docs, int64_t n_docs, const int32_t* sizes, int32_t num_epochs,
                          uint64_t max_num_samples, int32_t max_seq_length, double short_seq_prob, int32_t seed,
                          int32_t min_num_sent, int64_t* out) {
  if (num_epochs <= 0 || max_seq_length <= 1 || short_seq_prob < 0.0 || short_seq_prob > 1.0 || seed <= 0) return -1;
  const int32_t ratio = short_seq_prob > 0 ? static_cast<int32_t>(std::lround(1.0 / short_seq_prob)) : 0;
  std::mt19937 gen(static_cast<uint32_t>(seed));
  Row3* rows = reinterpret_cast<Row3*>(out);
  uint64_t count = 0;
  for (int32_t epoch = 0; epoch < num_epochs && count < max_num_samples; ++epoch) {
    for (int64_t d = 0; d < n_docs; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      int64_t remain = last - first;
      bool has_long = false;
      if (remain > 1)
        for (int64_t s = first; s < last; ++s)
          if (sizes[s] > kLongSentenceLen) { has_long = true; break; }
      if (remain < min_num_sent || has_long) continue;
      int64_t start = first;
      int32_t seq_len = 0, num_sent = 0;
      int32_t target = target_sample_len(ratio, max_seq_length, gen);
      for (int64_t s = first; s < last; ++s) {
        seq_len += sizes[s];
        ++num_sent;
        --remain;
        const bool enough = seq_len >= target && remain > 1 && num_sent >= min_num_sent;
        if (enough || remain == 0) {
          if (num_sent >= min_num_sent) {
            if (rows) rows[count] = Row3{start, s + 1, target};
            ++count;
          }
          start = s + 1;
          target = target_sample_len(ratio, max_seq_length, gen);
          seq_len = 0;
          num_sent = 0;
        }
      }
    }
  }
  if (rows) shuffle_rows(rows, static_cast<int64_t>(count), static_cast<int64_t>(seed) + 1);
  return static_cast<int64_t>(count);
}

// Block samples (ICT / retrieval style): rows (first sentence, one-past-last, document, block id).
int64_t mfb_build_blocks_mapping(const int64_t* docs, int64_t n_docs, const int32_t* sizes, const int32_t* titles_sizes,
                                 int32_t num_epochs, uint64_t max_num_samples, int32_t max_seq_length, int32_t seed,
                                 int32_t use_one_sent_blocks, int64_t* out) {
  if (num_epochs <= 0 || max_seq_length <= 1 || seed <= 0) return -1;
  const int32_t min_num_sent = use_one_sent_blocks ? 1 : 2;
  Row4* rows = reinterpret_cast<Row4*>(out);
  uint64_t count = 0;
  for (int32_t epoch = 0; epoch < num_epochs && count < max_num_samples; ++epoch) {
    int64_t block_id = 0;
    for (int64_t d = 0; d < n_docs; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      const int32_t target = max_seq_length - titles_sizes[d];
      int64_t remain = last - first;
      bool has_long = false;
      if (remain >= min_num_sent)
        for (int64_t s = first; s < last; ++s)
          if (sizes[s] > kLongSentenceLen) { has_long = true; break; }
      if (remain < min_num_sent || has_long) continue;
      int64_t start = first;
      int32_t seq_len = 0, num_sent = 0;
      for (int64_t s = first; s < last; ++s) {
        seq_len += sizes[s];
        ++num_sent;
        --remain;
        const bool enough = seq_len >= target && remain >= min_num_sent && num_sent >= min_num_sent;
        if (enough || remain == 0) {
          if (rows) rows[count] = Row4{start, s + 1, d, block_id};
          ++count;
          ++block_id;
          start = s + 1;
          seq_len = 0;
          num_sent = 0;
        }
      }
    }
  }
  if (rows) shuffle_rows(rows, static_cast<int64_t>(count), static_cast<int64_t>(seed) + 1);
  return static_cast<int64_t>(count);
}

int mfb_data_abi_version() { return 1; }

}  // extern "C"
