// Native index builders of the data pipeline (pybind11 module `hg_dataset_helpers`).
//
//   build_sample_idx_int32 / _int64   : sample -> (position in the shuffled document list, token offset) table of a
//                                       GPT dataset that packs documents into fixed-length training samples
//   build_blending_indices            : greedy assignment of samples to datasets that follows target weights
//   build_exhaustive_blending_indices : same rule, but every dataset contributes exactly `sizes[d]` samples
//   build_mapping                     : BERT-style sentence-window samples (start sentence, end sentence, target length)
//   build_blocks_mapping              : REALM / ICT style blocks (start, end, document, block id)
//
// Same exported names and array contracts as the reference's helper module
// (galvatron/core/runtime/datasets/megatron/helpers.cpp:21-73, :75-140, :142-246, :265-560, :563-836, :838-846).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <random>
#include <stdexcept>
#include <vector>

namespace py = pybind11;

namespace {

// ---------------------------------------------------------------------------------------------------
// GPT sample index
// ---------------------------------------------------------------------------------------------------
template <typename T>
py::array build_sample_idx(const py::array_t<int32_t>& sizes_, const py::array_t<int32_t>& doc_idx_,
                           const int32_t seq_length, const int32_t num_epochs, const int64_t tokens_per_epoch,
                           const bool drop_last_partial_sequence = true, const int add_extra_token = 1) {
  if (seq_length <= 1 || num_epochs <= 0 || tokens_per_epoch <= 1) throw std::invalid_argument("bad sample-index arguments");
  auto sizes = sizes_.unchecked<1>();
  auto doc_idx = doc_idx_.unchecked<1>();
  const int64_t total_tokens = int64_t(num_epochs) * tokens_per_epoch - add_extra_token;
  int64_t num_samples = drop_last_partial_sequence ? total_tokens / seq_length
                                                   : int64_t(std::ceil(double(total_tokens) / seq_length));
  T* table = new T[2 * (num_samples + 1)];
  int64_t sample = 0;      // row being written
  int64_t cursor = 0;      // index into doc_idx
  T offset = 0;            // token offset inside the current document
  table[0] = 0;
  table[1] = 0;
  ++sample;
  const int64_t last_doc = int64_t(doc_idx.shape(0)) - 1;
  while (sample <= num_samples) {
    int32_t remaining = seq_length + add_extra_token;
    while (remaining != 0) {
      const int32_t doc_len = sizes[doc_idx[cursor]] - int32_t(offset);
      remaining -= doc_len;
      if (remaining <= 0) {
        // the sample ends inside this document: the next one starts where this one ended (minus the shared token)
        offset += T(remaining + doc_len - add_extra_token);
        remaining = 0;
      } else {
        if (cursor == last_doc) {
          // ran out of documents while filling the final (partial) sample
          offset = T(sizes[doc_idx[cursor]] - add_extra_token);
          break;
        }
        ++cursor;
        offset = 0;
      }
    }
    table[2 * sample] = T(cursor);
    table[2 * sample + 1] = offset;
    ++sample;
  }
  py::capsule owner(table, [](void* p) { delete[] reinterpret_cast<T*>(p); });
  return py::array_t<T>({size_t(num_samples + 1), size_t(2)}, {2 * sizeof(T), sizeof(T)}, table, owner);
}

// ---------------------------------------------------------------------------------------------------
// blending
// ---------------------------------------------------------------------------------------------------
void build_blending_indices(py::array_t<int16_t>& dataset_index, py::array_t<int64_t>& dataset_sample_index,
                            const py::array_t<double>& weights, const int32_t num_datasets, const int64_t size,
                            const bool verbose) {
  auto di = dataset_index.mutable_unchecked<1>();
  auto dsi = dataset_sample_index.mutable_unchecked<1>();
  auto w = weights.unchecked<1>();
  std::vector<int64_t> taken(num_datasets, 0);
  for (int64_t i = 0; i < size; ++i) {
    const double seen = std::max<double>(double(i), 1.0);
    int best = 0;
    double best_err = w[0] * seen - double(taken[0]);
    for (int d = 1; d < num_datasets; ++d) {
      const double err = w[d] * seen - double(taken[d]);
      if (err > best_err) {
        best_err = err;
        best = d;
      }
    }
    di[i] = int16_t(best);
    dsi[i] = taken[best];
    ++taken[best];
  }
  if (verbose) {
    for (int d = 0; d < num_datasets; ++d)
      py::print("dataset", d, "target weight", w[d], "achieved", double(taken[d]) / double(std::max<int64_t>(size, 1)));
  }
}

void build_exhaustive_blending_indices(py::array_t<int16_t>& dataset_index, py::array_t<int64_t>& dataset_sample_index,
                                       const py::array_t<int64_t>& sizes, const int32_t num_datasets) {
  auto di = dataset_index.mutable_unchecked<1>();
  auto dsi = dataset_sample_index.mutable_unchecked<1>();
  auto sz = sizes.unchecked<1>();
  int64_t total = 0;
  for (int d = 0; d < num_datasets; ++d) total += sz[d];
  std::vector<double> w(num_datasets);
  for (int d = 0; d < num_datasets; ++d) w[d] = double(sz[d]) / double(std::max<int64_t>(total, 1));
  std::vector<int64_t> taken(num_datasets, 0);
  std::vector<bool> retired(num_datasets, false);
  for (int64_t i = 0; i < total; ++i) {
    const double seen = std::max<double>(double(i), 1.0);
    int best = -1;
    double best_err = -std::numeric_limits<double>::infinity();
    for (int d = 0; d < num_datasets; ++d) {
      if (retired[d]) continue;
      const double err = w[d] * seen - double(taken[d]);
      if (err > best_err) {
        best_err = err;
        best = d;
      }
    }
    di[i] = int16_t(best);
    dsi[i] = taken[best];
    if (++taken[best] >= sz[best]) retired[best] = true;
  }
}

// ---------------------------------------------------------------------------------------------------
// BERT sentence-window mapping
// ---------------------------------------------------------------------------------------------------
inline int32_t pick_target_length(int32_t short_ratio, int32_t max_length, std::mt19937& gen) {
  if (short_ratio == 0) return max_length;
  const auto r = gen();
  if (r % short_ratio == 0) return 2 + int32_t(r % uint32_t(max_length - 1));
  return max_length;
}

template <typename DocIdx>
py::array build_mapping_impl(const py::array_t<int64_t>& docs_, const py::array_t<int32_t>& sizes_,
                             const int32_t num_epochs, const uint64_t max_num_samples, const int32_t max_seq_length,
                             const double short_seq_prob, const int32_t seed, const bool verbose,
                             const int32_t min_num_sent) {
  auto docs = docs_.unchecked<1>();
  auto sizes = sizes_.unchecked<1>();
  const int32_t short_ratio = short_seq_prob > 0 ? int32_t(std::lround(1.0 / short_seq_prob)) : 0;
  constexpr int32_t kLongSentence = 512;
  std::vector<DocIdx> rows;
  // two passes with the same generator seed: count, then fill (the count fixes the number of epochs used)
  for (int pass = 0; pass < 2; ++pass) {
    std::mt19937 gen(seed);
    uint64_t count = 0;
    if (pass == 1) rows.reserve(rows.capacity());
    bool full = false;
    for (int32_t epoch = 0; epoch < num_epochs && !full; ++epoch) {
      for (int64_t doc = 0; doc + 1 < docs.shape(0); ++doc) {
        const int64_t first = docs[doc], last = docs[doc + 1];
        const int64_t n_sent = last - first;
        if (n_sent < min_num_sent) continue;
        bool has_long = false;
        for (int64_t s = first; s < last; ++s)
          if (sizes[s] > kLongSentence) { has_long = true; break; }
        if (has_long) continue;
        int64_t start = first;
        int32_t seq_len = 0, sent_in_sample = 0;
        int32_t target = pick_target_length(short_ratio, max_seq_length, gen);
        int64_t remaining = n_sent;
        for (int64_t s = first; s < last; ++s) {
          seq_len += sizes[s];
          ++sent_in_sample;
          --remaining;
          const bool enough = seq_len >= target && remaining >= min_num_sent && sent_in_sample >= min_num_sent;
          if (enough || remaining == 0) {
            if (sent_in_sample >= min_num_sent || remaining == 0) {
              if (pass == 1) {
                rows.push_back(DocIdx(start));
                rows.push_back(DocIdx(s + 1));
                rows.push_back(DocIdx(target));
              }
              ++count;
              if (count >= max_num_samples) { full = true; break; }
            }
            start = s + 1;
            seq_len = 0;
            sent_in_sample = 0;
            target = pick_target_length(short_ratio, max_seq_length, gen);
          }
        }
        if (full) break;
      }
    }
    if (pass == 0) rows.reserve(size_t(count) * 3);
    if (verbose && pass == 0) py::print("build_mapping: samples", count);
  }
  const int64_t n = int64_t(rows.size() / 3);
  // Fisher-Yates on whole rows
  std::mt19937_64 gen64(uint64_t(seed) + 1);
  for (int64_t i = n - 1; i > 0; --i) {
    const int64_t j = int64_t(gen64() % uint64_t(i + 1));
    for (int c = 0; c < 3; ++c) std::swap(rows[3 * i + c], rows[3 * j + c]);
  }
  DocIdx* out = new DocIdx[std::max<int64_t>(3 * n, 1)];
  std::copy(rows.begin(), rows.end(), out);
  py::capsule owner(out, [](void* p) { delete[] reinterpret_cast<DocIdx*>(p); });
  return py::array_t<DocIdx>({size_t(n), size_t(3)}, {3 * sizeof(DocIdx), sizeof(DocIdx)}, out, owner);
}

py::array build_mapping(const py::array_t<int64_t>& docs, const py::array_t<int32_t>& sizes, const int num_epochs,
                        const uint64_t max_num_samples, const int max_seq_length, const double short_seq_prob,
                        const int seed, const bool verbose, const int32_t min_num_sent) {
  if (sizes.size() > std::numeric_limits<uint32_t>::max())
    return build_mapping_impl<uint64_t>(docs, sizes, num_epochs, max_num_samples, max_seq_length, short_seq_prob, seed,
                                        verbose, min_num_sent);
  return build_mapping_impl<uint32_t>(docs, sizes, num_epochs, max_num_samples, max_seq_length, short_seq_prob, seed,
                                      verbose, min_num_sent);
}

// ---------------------------------------------------------------------------------------------------
// REALM / ICT block mapping
// ---------------------------------------------------------------------------------------------------
template <typename DocIdx>
py::array build_blocks_mapping_impl(const py::array_t<int64_t>& docs_, const py::array_t<int32_t>& sizes_,
                                    const py::array_t<int32_t>& titles_sizes_, const int32_t num_epochs,
                                    const uint64_t max_num_samples, const int32_t max_seq_length, const int32_t seed,
                                    const bool verbose, const bool use_one_sent_blocks) {
  auto docs = docs_.unchecked<1>();
  auto sizes = sizes_.unchecked<1>();
  auto titles = titles_sizes_.unchecked<1>();
  constexpr int32_t kLongSentence = 512;
  const int32_t min_num_sent = use_one_sent_blocks ? 1 : 2;
  std::vector<DocIdx> rows;
  uint64_t count = 0;
  bool full = false;
  for (int32_t epoch = 0; epoch < num_epochs && !full; ++epoch) {
    DocIdx block_id = 0;
    for (int64_t doc = 0; doc + 1 < docs.shape(0); ++doc) {
      const int64_t first = docs[doc], last = docs[doc + 1];
      const int32_t target = max_seq_length - titles[doc];
      int64_t remaining = last - first;
      if (remaining < min_num_sent) continue;
      bool has_long = false;
      for (int64_t s = first; s < last; ++s)
        if (sizes[s] > kLongSentence) { has_long = true; break; }
      if (has_long) continue;
      int64_t start = first;
      int32_t seq_len = 0, n_in = 0;
      for (int64_t s = first; s < last; ++s) {
        seq_len += sizes[s];
        ++n_in;
        --remaining;
        const bool enough = seq_len >= target && remaining >= min_num_sent && n_in >= min_num_sent;
        if (enough || remaining == 0) {
          rows.push_back(DocIdx(start));
          rows.push_back(DocIdx(s + 1));
          rows.push_back(DocIdx(doc));
          rows.push_back(block_id);
          ++block_id;
          ++count;
          if (count >= max_num_samples) { full = true; break; }
          start = s + 1;
          seq_len = 0;
          n_in = 0;
        }
      }
      if (full) break;
    }
  }
  if (verbose) py::print("build_blocks_mapping: blocks", count);
  const int64_t n = int64_t(rows.size() / 4);
  std::mt19937_64 gen64(uint64_t(seed) + 1);
  for (int64_t i = n - 1; i > 0; --i) {
    const int64_t j = int64_t(gen64() % uint64_t(i + 1));
    for (int c = 0; c < 4; ++c) std::swap(rows[4 * i + c], rows[4 * j + c]);
  }
  DocIdx* out = new DocIdx[std::max<int64_t>(4 * n, 1)];
  std::copy(rows.begin(), rows.end(), out);
  py::capsule owner(out, [](void* p) { delete[] reinterpret_cast<DocIdx*>(p); });
  return py::array_t<DocIdx>({size_t(n), size_t(4)}, {4 * sizeof(DocIdx), sizeof(DocIdx)}, out, owner);
}

py::array build_blocks_mapping(const py::array_t<int64_t>& docs, const py::array_t<int32_t>& sizes,
                               const py::array_t<int32_t>& titles_sizes, const int num_epochs,
                               const uint64_t max_num_samples, const int max_seq_length, const int seed,
                               const bool verbose, const bool use_one_sent_blocks) {
  if (sizes.size() > std::numeric_limits<uint32_t>::max())
    return build_blocks_mapping_impl<uint64_t>(docs, sizes, titles_sizes, num_epochs, max_num_samples, max_seq_length,
                                               seed, verbose, use_one_sent_blocks);
  return build_blocks_mapping_impl<uint32_t>(docs, sizes, titles_sizes, num_epochs, max_num_samples, max_seq_length, seed,
                                             verbose, use_one_sent_blocks);
}

}  // namespace

PYBIND11_MODULE(hg_dataset_helpers, m) {
  m.doc() = "index builders of the dataset pipeline";
  m.def("build_mapping", &build_mapping);
  m.def("build_blocks_mapping", &build_blocks_mapping);
  m.def("build_sample_idx_int32", &build_sample_idx<int32_t>, py::arg("sizes"), py::arg("doc_idx"),
        py::arg("seq_length"), py::arg("num_epochs"), py::arg("tokens_per_epoch"),
        py::arg("drop_last_partial_sequence") = true, py::arg("add_extra_token_to_sequence") = 1);
  m.def("build_sample_idx_int64", &build_sample_idx<int64_t>, py::arg("sizes"), py::arg("doc_idx"),
        py::arg("seq_length"), py::arg("num_epochs"), py::arg("tokens_per_epoch"),
        py::arg("drop_last_partial_sequence") = true, py::arg("add_extra_token_to_sequence") = 1);
  m.def("build_blending_indices", &build_blending_indices);
  m.def("build_exhaustive_blending_indices", &build_exhaustive_blending_indices);
}
