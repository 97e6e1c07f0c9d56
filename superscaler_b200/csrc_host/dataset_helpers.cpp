// Host-side index builders for token datasets (no CUDA): the loops that are too slow in Python for corpora of
// hundreds of millions of documents.  Counterpart of the reference's compiled dataset helpers
// (runtime/megatron/data/helpers.cpp: build_sample_idx, build_blending_indices), written against the same
// definitions:
//
//   sample index   : training sample s covers seq_length + 1 consecutive tokens of the stream obtained by
//                    concatenating the documents in the order doc_idx; row s of the result is
//                    (position in doc_idx, token offset inside that document) of the sample's FIRST token, and
//                    consecutive samples overlap by one token (the label of the last input token).
//   blending index : for every global sample pick the dataset whose share of samples drawn so far lags furthest
//                    behind its weight, and record (dataset, running sample number inside that dataset).
//   sentence map   : (build_mapping / build_blocks_mapping of the reference's helpers.cpp) samples of whole
//                    consecutive sentences of one document for masked-LM / span-corruption / inverse-cloze
//                    training: rows (first sentence, one past the last sentence, target length) or, for blocks,
//                    (first, one past last, document, block id), shuffled with a seeded generator.  Documents
//                    with too few sentences or with a sentence longer than 512 tokens are skipped.  The random
//                    stream is splitmix64 so that the Python definition in data/sentences.py reproduces it.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <cstdint>
#include <stdexcept>
#include <utility>
#include <vector>

namespace py = pybind11;

namespace {

py::array_t<int32_t> build_sample_idx(const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& sizes,
                                      const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& doc_idx,
                                      int32_t seq_length, int32_t num_epochs, int64_t tokens_per_epoch) {
  if (seq_length < 1 || num_epochs < 1 || tokens_per_epoch < 2) throw std::invalid_argument("bad arguments");
  const auto sz = sizes.unchecked<1>();
  const auto docs = doc_idx.unchecked<1>();
  const int64_t num_samples = (static_cast<int64_t>(num_epochs) * tokens_per_epoch - 1) / seq_length;
  py::array_t<int32_t> out({num_samples + 1, static_cast<int64_t>(2)});
  auto o = out.mutable_unchecked<2>();
  int64_t pos = 0;      // index into doc_idx
  int32_t offset = 0;   // token offset inside document doc_idx[pos]
  o(0, 0) = 0;
  o(0, 1) = 0;
  for (int64_t s = 1; s <= num_samples; ++s) {
    int64_t need = static_cast<int64_t>(seq_length) + 1;  // tokens of sample s - 1
    while (need > 0) {
      if (pos >= docs.shape(0)) throw std::runtime_error("doc_idx exhausted: tokens_per_epoch does not match sizes");
      const int64_t left = static_cast<int64_t>(sz(docs(pos))) - offset;
      if (left >= need) {
        // the sample ends inside this document; its last token is the first token of the next sample
        offset += static_cast<int32_t>(need - 1);
        need = 0;
      } else {
        need -= left;
        ++pos;
        offset = 0;
      }
    }
    o(s, 0) = static_cast<int32_t>(pos);
    o(s, 1) = offset;
  }
  return out;
}

void build_blending_indices(py::array_t<uint8_t, py::array::c_style>& dataset_index,
                            py::array_t<int64_t, py::array::c_style>& dataset_sample_index,
                            const py::array_t<double, py::array::c_style | py::array::forcecast>& weights,
                            int32_t num_datasets, int64_t size) {
  auto di = dataset_index.mutable_unchecked<1>();
  auto si = dataset_sample_index.mutable_unchecked<1>();
  const auto w = weights.unchecked<1>();
  if (num_datasets < 1 || num_datasets > 255 || w.shape(0) < num_datasets || di.shape(0) < size || si.shape(0) < size)
    throw std::invalid_argument("bad arguments");
  std::vector<int64_t> drawn(num_datasets, 0);
  for (int64_t s = 0; s < size; ++s) {
    const double total = static_cast<double>(s > 0 ? s : 1);
    int best = 0;
    double best_lag = w(0) * total - static_cast<double>(drawn[0]);
    for (int d = 1; d < num_datasets; ++d) {
      const double lag = w(d) * total - static_cast<double>(drawn[d]);
      if (lag > best_lag) {
        best_lag = lag;
        best = d;
      }
    }
    di(s) = static_cast<uint8_t>(best);
    si(s) = drawn[best];
    ++drawn[best];
  }
}

struct SplitMix64 {
  uint64_t state;
  explicit SplitMix64(uint64_t seed) : state(seed) {}
  uint64_t next() {
    uint64_t z = (state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
};

constexpr int32_t kLongSentence = 512;

bool usable_document(const py::detail::unchecked_reference<int32_t, 1>& sizes, int64_t first, int64_t last,
                     int32_t min_sentences) {
  if (last - first < min_sentences) return false;
  for (int64_t i = first; i < last; ++i)
    if (sizes(i) > kLongSentence) return false;
  return true;
}

template <int W>
py::array_t<int64_t> shuffled_rows(std::vector<int64_t>& rows, uint64_t seed) {
  const int64_t n = static_cast<int64_t>(rows.size()) / W;
  SplitMix64 rng(seed);
  for (int64_t i = n - 1; i > 0; --i) {
    const int64_t j = static_cast<int64_t>(rng.next() % static_cast<uint64_t>(i + 1));
    for (int k = 0; k < W; ++k) std::swap(rows[i * W + k], rows[j * W + k]);
  }
  py::array_t<int64_t> out({n, static_cast<int64_t>(W)});
  auto o = out.mutable_unchecked<2>();
  for (int64_t i = 0; i < n; ++i)
    for (int k = 0; k < W; ++k) o(i, k) = rows[i * W + k];
  return out;
}

// One target length per sample: max_length, or with probability ~short_prob a length in [2, max_length].
int32_t draw_target(SplitMix64& rng, int32_t short_ratio, int32_t max_length) {
  if (short_ratio == 0) return max_length;
  const uint64_t r = rng.next();
  if (r % static_cast<uint64_t>(short_ratio) == 0) return 2 + static_cast<int32_t>((r >> 20) % (max_length - 1));
  return max_length;
}

py::array_t<int64_t> build_mapping(const py::array_t<int64_t, py::array::c_style | py::array::forcecast>& doc_starts,
                                   const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& sizes_,
                                   int32_t num_epochs, int64_t max_num_samples, int32_t max_seq_length,
                                   double short_seq_prob, uint64_t seed, int32_t min_num_sent) {
  if (num_epochs < 1 || max_seq_length < 2 || short_seq_prob < 0.0 || short_seq_prob > 1.0 || min_num_sent < 1)
    throw std::invalid_argument("bad arguments");
  const auto docs = doc_starts.unchecked<1>();
  const auto sizes = sizes_.unchecked<1>();
  const int32_t short_ratio = short_seq_prob > 0.0 ? static_cast<int32_t>(1.0 / short_seq_prob + 0.5) : 0;
  std::vector<int64_t> rows;
  SplitMix64 rng(seed);
  for (int32_t epoch = 0; epoch < num_epochs; ++epoch) {
    if (static_cast<int64_t>(rows.size()) / 3 >= max_num_samples) break;
    for (int64_t d = 0; d + 1 < docs.shape(0); ++d) {
      const int64_t first = docs(d), last = docs(d + 1);
      if (!usable_document(sizes, first, last, min_num_sent)) continue;
      int64_t start = first, remain = last - first;
      int32_t len = 0, count = 0, target = draw_target(rng, short_ratio, max_seq_length);
      for (int64_t i = first; i < last; ++i) {
        len += sizes(i);
        ++count;
        --remain;
        if ((len >= target && remain > 1 && count >= min_num_sent) || remain == 0) {
          rows.push_back(start);
          rows.push_back(i + 1);
          rows.push_back(target);
          start = i + 1;
          len = 0;
          count = 0;
          target = draw_target(rng, short_ratio, max_seq_length);
        }
      }
    }
  }
  return shuffled_rows<3>(rows, seed + 1);
}

py::array_t<int64_t> build_blocks_mapping(
    const py::array_t<int64_t, py::array::c_style | py::array::forcecast>& doc_starts,
    const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& sizes_,
    const py::array_t<int32_t, py::array::c_style | py::array::forcecast>& title_sizes_, int32_t num_epochs,
    int64_t max_num_samples, int32_t max_seq_length, uint64_t seed, bool use_one_sent_blocks) {
  if (num_epochs < 1 || max_seq_length < 2) throw std::invalid_argument("bad arguments");
  const auto docs = doc_starts.unchecked<1>();
  const auto sizes = sizes_.unchecked<1>();
  const auto titles = title_sizes_.unchecked<1>();
  const int32_t min_sent = use_one_sent_blocks ? 1 : 2;
  std::vector<int64_t> rows;
  for (int32_t epoch = 0; epoch < num_epochs; ++epoch) {
    if (static_cast<int64_t>(rows.size()) / 4 >= max_num_samples) break;
    int64_t block_id = 0;   // unique inside one pass over the corpus
    for (int64_t d = 0; d + 1 < docs.shape(0); ++d) {
      const int64_t first = docs(d), last = docs(d + 1);
      if (!usable_document(sizes, first, last, min_sent)) continue;
      const int32_t target = max_seq_length - titles(d);
      int64_t start = first, remain = last - first;
      int32_t len = 0, count = 0;
      for (int64_t i = first; i < last; ++i) {
        len += sizes(i);
        ++count;
        --remain;
        if ((len >= target && remain >= min_sent && count >= min_sent) || remain == 0) {
          rows.push_back(start);
          rows.push_back(i + 1);
          rows.push_back(d);
          rows.push_back(block_id++);
          start = i + 1;
          len = 0;
          count = 0;
        }
      }
    }
  }
  return shuffled_rows<4>(rows, seed + 1);
}

}  // namespace

PYBIND11_MODULE(_data_helpers, m) {
  m.def("build_sample_idx", &build_sample_idx);
  m.def("build_blending_indices", &build_blending_indices);
  m.def("build_mapping", &build_mapping);
  m.def("build_blocks_mapping", &build_blocks_mapping);
}
