// Host-side dataset index builders (plain C ABI, loaded with ctypes; no Python headers needed).
//
//  * oslo_build_sample_idx      - (document, offset) start of every fixed-length training sample
//  * oslo_build_blending_indices - greedy interleave of several datasets according to weights
//  * oslo_build_mapping         - sentence-pair style samples (start sentence, end sentence, target length)
//  * oslo_build_blocks_mapping  - fixed-budget sentence blocks (start, end, document, block id)
//
// Same results as the reference's builders (oslo/fused_kernels/bindings/pybind_datasets.cpp:35-585) for
// the first two, which the Python side checks against its own NumPy statements; progress is reported
// through an optional callback instead of a terminal progress bar.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <random>
#include <vector>

extern "C" {

typedef void (*progress_fn)(int64_t done, int64_t total);

// out: [num_samples + 1, 2] int32, returns num_samples + 1 (or -1 on bad input)
int64_t oslo_build_sample_idx(const int32_t* sizes, const int32_t* doc_idx, int64_t doc_idx_len, int32_t seq_length,
                              int32_t num_epochs, int64_t tokens_per_epoch, int32_t* out, int64_t out_rows) {
  if (seq_length <= 0 || doc_idx_len <= 0) return -1;
  const int64_t num_samples = (static_cast<int64_t>(num_epochs) * tokens_per_epoch - 1) / seq_length;
  if (out_rows < num_samples + 1) return -1;
  int64_t sample = 0, di = 0;
  int32_t offset = 0;
  out[0] = 0;
  out[1] = 0;
  ++sample;
  while (sample <= num_samples) {
    int32_t remaining = seq_length + 1;
    while (remaining != 0) {
      if (di >= doc_idx_len) return -1;
      const int32_t doc_len = sizes[doc_idx[di]] - offset;
      remaining -= doc_len;
      if (remaining <= 0) {
        offset += remaining + doc_len - 1;
        remaining = 0;
      } else {
        ++di;
        offset = 0;
      }
    }
    out[2 * sample] = static_cast<int32_t>(di);
    out[2 * sample + 1] = offset;
    ++sample;
  }
  return num_samples + 1;
}

// For every output slot pick the dataset whose achieved share lags its weight the most.
void oslo_build_blending_indices(uint8_t* dataset_index, int64_t* dataset_sample_index, const double* weights,
                                 int32_t num_datasets, int64_t size, progress_fn progress) {
  std::vector<int64_t> taken(num_datasets, 0);
  for (int64_t i = 0; i < size; ++i) {
    const double denom = std::max(static_cast<double>(i), 1.0);
    int32_t best = 0;
    double best_err = weights[0] * denom - static_cast<double>(taken[0]);
    for (int32_t d = 1; d < num_datasets; ++d) {
      const double err = weights[d] * denom - static_cast<double>(taken[d]);
      if (err > best_err) { best_err = err; best = d; }
    }
    dataset_index[i] = static_cast<uint8_t>(best);
    dataset_sample_index[i] = taken[best];
    ++taken[best];
    if (progress && (i & 0xFFFFF) == 0) progress(i, size);
  }
  if (progress) progress(size, size);
}

static int32_t target_length(int32_t short_seq_ratio, int32_t max_length, std::mt19937& rng) {
  if (short_seq_ratio == 0) return max_length;
  const uint32_t r = rng();
  if (r % short_seq_ratio == 0) return 2 + static_cast<int32_t>(r % (max_length - 1));
  return max_length;
}

// Two-pass: pass 0 counts, pass 1 fills. maps: [n, 3] (start sentence, end sentence, target length).
// Call with maps == nullptr to obtain the row count.
int64_t oslo_build_mapping(const int64_t* docs, int64_t num_docs_plus1, const int32_t* sizes, int32_t num_epochs,
                           int64_t max_num_samples, int32_t max_seq_length, double short_seq_prob, int32_t seed,
                           int32_t min_num_sent, int64_t* maps, int64_t maps_rows) {
  const int32_t short_ratio = short_seq_prob > 0 ? static_cast<int32_t>(std::lround(1.0 / short_seq_prob)) : 0;
  const int64_t num_docs = num_docs_plus1 - 1;
  int64_t count = 0;
  for (int pass = 0; pass < 2; ++pass) {
    if (pass == 1 && maps == nullptr) break;
    std::mt19937 rng(static_cast<uint32_t>(seed));
    count = 0;
    bool full = false;
    for (int32_t epoch = 0; epoch < num_epochs && !full; ++epoch) {
      for (int64_t doc = 0; doc < num_docs && !full; ++doc) {
        const int64_t first = docs[doc], last = docs[doc + 1];
        int64_t remain = last - first;
        if (remain < min_num_sent) continue;
        bool too_long = false;
        for (int64_t s = first; s < last; ++s) too_long |= sizes[s] > 512;  // skip documents with a very long sentence
        if (too_long) continue;
        int64_t start = first;
        int32_t seq_len = 0, num_sent = 0;
        int32_t target = target_length(short_ratio, max_seq_length, rng);
        for (int64_t s = first; s < last; ++s) {
          seq_len += sizes[s];
          ++num_sent;
          --remain;
          if ((seq_len >= target && remain > 1 && num_sent >= min_num_sent) || remain == 0) {
            if (seq_len > max_seq_length) seq_len = max_seq_length;
            if (num_sent >= min_num_sent) {
              if (pass == 1) {
                if (count >= maps_rows) return -1;
                maps[3 * count] = start;
                maps[3 * count + 1] = s + 1;
                maps[3 * count + 2] = target;
              }
              ++count;
              if (count >= max_num_samples) { full = true; break; }
            }
            start = s + 1;
            target = target_length(short_ratio, max_seq_length, rng);
            seq_len = 0;
            num_sent = 0;
          }
        }
      }
    }
  }
  if (maps != nullptr) {  // Fisher-Yates with a 64-bit generator, deterministic in `seed`
    std::mt19937_64 rng64(static_cast<uint64_t>(seed) + 1);
    for (int64_t i = count - 1; i > 0; --i) {
      const int64_t j = static_cast<int64_t>(rng64() % static_cast<uint64_t>(i + 1));
      for (int c = 0; c < 3; ++c) std::swap(maps[3 * i + c], maps[3 * j + c]);
    }
  }
  return count;
}

// maps: [n, 4] (start sentence, end sentence, document, block id); titles_sizes[doc] tokens are reserved per block.
int64_t oslo_build_blocks_mapping(const int64_t* docs, int64_t num_docs_plus1, const int32_t* sizes,
                                  const int32_t* titles_sizes, int32_t num_epochs, int64_t max_num_samples,
                                  int32_t max_seq_length, int32_t seed, int32_t use_one_sent_blocks, int64_t* maps,
                                  int64_t maps_rows) {
  const int64_t num_docs = num_docs_plus1 - 1;
  const int32_t min_sent = use_one_sent_blocks ? 1 : 2;
  int64_t count = 0;
  for (int pass = 0; pass < 2; ++pass) {
    if (pass == 1 && maps == nullptr) break;
    count = 0;
    bool full = false;
    for (int32_t epoch = 0; epoch < num_epochs && !full; ++epoch) {
      int64_t block_id = 0;
      for (int64_t doc = 0; doc < num_docs && !full; ++doc) {
        const int64_t first = docs[doc], last = docs[doc + 1];
        const int32_t budget = max_seq_length - titles_sizes[doc];
        int64_t remain = last - first;
        if (remain < min_sent) continue;
        bool too_long = false;
        for (int64_t s = first; s < last; ++s) too_long |= sizes[s] > 512;
        if (too_long) continue;
        int64_t start = first;
        int32_t seq_len = 0, num_sent = 0;
        for (int64_t s = first; s < last; ++s) {
          seq_len += sizes[s];
          ++num_sent;
          --remain;
          if ((seq_len >= budget && remain >= min_sent && num_sent >= min_sent) || remain == 0) {
            if (pass == 1) {
              if (count >= maps_rows) return -1;
              maps[4 * count] = start;
              maps[4 * count + 1] = s + 1;
              maps[4 * count + 2] = doc;
              maps[4 * count + 3] = block_id;
            }
            ++count;
            ++block_id;
            if (count >= max_num_samples) { full = true; break; }
            start = s + 1;
            seq_len = 0;
            num_sent = 0;
          }
        }
      }
    }
  }
  if (maps != nullptr) {
    std::mt19937_64 rng64(static_cast<uint64_t>(seed) + 1);
    for (int64_t i = count - 1; i > 0; --i) {
      const int64_t j = static_cast<int64_t>(rng64() % static_cast<uint64_t>(i + 1));
      for (int c = 0; c < 4; ++c) std::swap(maps[4 * i + c], maps[4 * j + c]);
    }
  }
  return count;
}

}  // extern "C"
