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
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <cstdint>
#include <stdexcept>
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

}  // namespace

PYBIND11_MODULE(_data_helpers, m) {
  m.def("build_sample_idx", &build_sample_idx);
  m.def("build_blending_indices", &build_blending_indices);
}
