// CPU index builders for blended / packed token datasets (C++17, plain C ABI, called through ctypes).
//
// Same results, bit for bit, as the pybind11 helpers of the reference
// (src/nanotron/data/nemo_dataset/helpers.cpp: build_blending_indices, build_sample_idx, build_mapping,
// build_blocks_mapping); organised differently: one pass with growable vectors and a shared sentence-span walker instead of
// a counting pass plus a filling pass.  Two-step protocol for variable-size results: the *_build call returns an opaque
// handle and the row count, *_copy writes the rows into a caller-provided array and frees the handle.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <random>
#include <vector>

#define NTB_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int32_t kLongSentence = 512;  // documents holding a longer sentence are skipped by the span builders

struct Rows {
  std::vector<int64_t> data;
  int width = 0;
  int64_t rows() const { return width ? static_cast<int64_t>(data.size()) / width : 0; }
};

// Fisher-Yates with a 64-bit Mersenne twister seeded with `seed + 1`, walking from the last row down.
void shuffle_rows(Rows& r, int32_t seed) {
  std::mt19937_64 gen(static_cast<uint64_t>(seed) + 1);
  const int w = r.width;
  for (int64_t i = r.rows() - 1; i > 0; --i) {
    const int64_t j = static_cast<int64_t>(gen() % static_cast<uint64_t>(i + 1));
    for (int c = 0; c < w; ++c) std::swap(r.data[i * w + c], r.data[j * w + c]);
  }
}

// Target length of the next sample: mostly `max_len`, sometimes (1 in `ratio`) a shorter random one.
inline int32_t draw_target_len(int32_t ratio, int32_t max_len, std::mt19937& gen) {
  if (ratio == 0) return max_len;
  const auto x = gen();
  if (x % static_cast<uint32_t>(ratio) == 0) return 2 + static_cast<int32_t>(x % static_cast<uint32_t>(max_len - 1));
  return max_len;
}

inline bool has_long_sentence(const int32_t* sizes, int64_t first, int64_t last) {
  for (int64_t s = first; s < last; ++s)
    if (sizes[s] > kLongSentence) return true;
  return false;
}

}  // namespace

// dataset_index[i] = which dataset sample i comes from; dataset_sample_index[i] = its index inside that dataset.
// Greedy: at every step pick the dataset that lags most behind its target share.  `dataset_num_samples` is read as the
// starting counts and updated in place.
NTB_API void ntb_build_blending_indices(int16_t* dataset_index, int64_t* dataset_sample_index, int64_t* dataset_num_samples, const double* weights,
                                        int32_t num_datasets, int64_t size) {
  for (int64_t i = 0; i < size; ++i) {
    const double n = std::max(static_cast<double>(i), 1.0);
    int64_t best = 0;
    double best_err = weights[0] * n - static_cast<double>(dataset_num_samples[0]);
    for (int64_t d = 1; d < num_datasets; ++d) {
      const double err = weights[d] * n - static_cast<double>(dataset_num_samples[d]);
      if (err > best_err) {
        best_err = err;
        best = d;
      }
    }
    dataset_index[i] = static_cast<int16_t>(best);
    dataset_sample_index[i] = dataset_num_samples[best];
    dataset_num_samples[best] += 1;
  }
}

NTB_API int64_t ntb_sample_idx_num_samples(int32_t seq_length, int32_t num_epochs, int64_t tokens_per_epoch, int drop_last, int add_extra_token) {
  const int64_t total = static_cast<int64_t>(num_epochs) * tokens_per_epoch - add_extra_token;
  if (drop_last) return total / seq_length;
  return static_cast<int64_t>(std::ceil(static_cast<float>(total) / seq_length));
}

// out: int32 [num_samples + 1, 2] = (position in doc_idx, token offset inside that document) of every sample boundary,
// for documents flattened in `doc_idx` order and cut every `seq_length` tokens (+ `add_extra_token` overlap).
NTB_API void ntb_build_sample_idx(const int32_t* sizes, const int32_t* doc_idx, int64_t doc_idx_len, int32_t seq_length, int32_t num_epochs,
                                  int64_t tokens_per_epoch, int drop_last, int add_extra_token, int32_t* out) {
  const int64_t num_samples = ntb_sample_idx_num_samples(seq_length, num_epochs, tokens_per_epoch, drop_last, add_extra_token);
  int64_t pos = 0;      // index into doc_idx
  int32_t offset = 0;   // token offset inside the current document
  out[0] = 0;
  out[1] = 0;
  for (int64_t s = 1; s <= num_samples; ++s) {
    int32_t need = seq_length + add_extra_token;
    while (need != 0) {
      const int32_t avail = sizes[doc_idx[pos]] - offset;
      need -= avail;
      if (need <= 0) {
        offset += need + avail - add_extra_token;  // stop inside this document, one token short so samples overlap
        need = 0;
      } else if (pos == doc_idx_len - 1) {
        offset = sizes[doc_idx[pos]] - add_extra_token;  // ran out of documents (only possible without drop_last)
        break;
      } else {
        ++pos;
        offset = 0;
      }
    }
    out[2 * s] = static_cast<int32_t>(pos);
    out[2 * s + 1] = offset;
  }
}

// Rows (first sentence, one-past-last sentence, target length) covering every document with at least `min_num_sent`
// sentences and no over-long sentence; repeated for `num_epochs` or until `max_num_samples`; then shuffled.
NTB_API void* ntb_build_mapping(const int64_t* docs, int64_t num_docs_plus_one, const int32_t* sizes, int32_t num_epochs, uint64_t max_num_samples,
                                int32_t max_seq_length, double short_seq_prob, int32_t seed, int32_t min_num_sent, int64_t* out_rows) {
  auto* rows = new Rows();
  rows->width = 3;
  const int32_t ratio = short_seq_prob > 0 ? static_cast<int32_t>(std::round(1.0 / short_seq_prob)) : 0;
  std::mt19937 gen(static_cast<uint32_t>(seed));
  uint64_t count = 0;
  for (int32_t epoch = 0; epoch < num_epochs && count < max_num_samples; ++epoch) {
    for (int64_t d = 0; d + 1 < num_docs_plus_one; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      int64_t remaining = last - first;
      if (remaining < min_num_sent) continue;
      if (remaining > 1 && has_long_sentence(sizes, first, last)) continue;
      int64_t start = first;
      int32_t len = 0, nsent = 0;
      int32_t target = draw_target_len(ratio, max_seq_length, gen);
      for (int64_t s = first; s < last; ++s) {
        len += sizes[s];
        ++nsent;
        --remaining;
        const bool full = len >= target && remaining > 1 && nsent >= min_num_sent;
        if (full || remaining == 0) {
          rows->data.push_back(start);
          rows->data.push_back(s + 1);
          rows->data.push_back(target);
          ++count;
          start = s + 1;
          target = draw_target_len(ratio, max_seq_length, gen);
          len = 0;
          nsent = 0;
        }
      }
    }
  }
  shuffle_rows(*rows, seed);
  *out_rows = rows->rows();
  return rows;
}

// Rows (first sentence, one-past-last sentence, document, block id inside the epoch); the target length of a document is
// `max_seq_length - titles_sizes[doc]`.
NTB_API void* ntb_build_blocks_mapping(const int64_t* docs, int64_t num_docs_plus_one, const int32_t* sizes, const int32_t* titles_sizes, int32_t num_epochs,
                                       uint64_t max_num_samples, int32_t max_seq_length, int32_t seed, int use_one_sent_blocks, int64_t* out_rows) {
  auto* rows = new Rows();
  rows->width = 4;
  const int64_t min_num_sent = use_one_sent_blocks ? 1 : 2;
  uint64_t count = 0;
  for (int32_t epoch = 0; epoch < num_epochs && count < max_num_samples; ++epoch) {
    int64_t block_id = 0;
    for (int64_t d = 0; d + 1 < num_docs_plus_one; ++d) {
      const int64_t first = docs[d], last = docs[d + 1];
      int64_t remaining = last - first;
      if (remaining < min_num_sent || has_long_sentence(sizes, first, last)) continue;
      const int32_t target = max_seq_length - titles_sizes[d];
      int64_t start = first;
      int32_t len = 0, nsent = 0;
      for (int64_t s = first; s < last; ++s) {
        len += sizes[s];
        ++nsent;
        --remaining;
        const bool full = len >= target && remaining >= min_num_sent && nsent >= min_num_sent;
        if (full || remaining == 0) {
          rows->data.push_back(start);
          rows->data.push_back(s + 1);
          rows->data.push_back(d);
          rows->data.push_back(block_id);
          ++count;
          ++block_id;
          start = s + 1;
          len = 0;
          nsent = 0;
        }
      }
    }
  }
  shuffle_rows(*rows, seed);
  *out_rows = rows->rows();
  return rows;
}

// Copies the rows as uint32 (`as_u64 == 0`) or uint64 into `out` and releases the handle.
NTB_API void ntb_rows_copy_and_free(void* handle, void* out, int as_u64) {
  auto* rows = static_cast<Rows*>(handle);
  const size_t n = rows->data.size();
  if (as_u64) {
    auto* o = static_cast<uint64_t*>(out);
    for (size_t i = 0; i < n; ++i) o[i] = static_cast<uint64_t>(rows->data[i]);
  } else {
    auto* o = static_cast<uint32_t*>(out);
    for (size_t i = 0; i < n; ++i) o[i] = static_cast<uint32_t>(rows->data[i]);
  }
  delete rows;
}
