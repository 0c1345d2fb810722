// Native dataset indexing and batch assembly for token datasets stored as Megatron-style indexed files
// (<prefix>.idx + <prefix>.bin). Same role as the reference's vendored
// galvatron/site_package/megatron/core/datasets/helpers.cpp (build_sample_idx :86, build_blending_indices :19),
// plus a multi-threaded gather that assembles a [batch, seq_len + 1] int64 block straight into a caller-owned
// (pinned) host buffer, so the training loop's host side is one memcpy-speed call followed by one H2D copy.
//
//   build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch) -> int32|int64 [num_samples + 1, 2]
//       row i = (position in doc_idx, token offset inside that document) where sample i starts; sample i spans
//       seq_length + 1 tokens and shares its last token with the first token of sample i + 1.
//   build_blending_indices(weights, size) -> (dataset_index uint8 [size], dataset_sample_index int64 [size])
//       greedy error-minimising interleave of several datasets by weight.
//   gather_samples(tokens, token_width, pointers, doc_idx, sample_idx, picks, seq_length, out, threads)
//       copies the samples named in `picks` into `out`.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

template <typename Index>
py::array sample_index_impl(const int32_t* sizes, int64_t n_sizes, const int32_t* doc_idx, int64_t n_docs, int64_t seq_length,
                            int64_t num_epochs, int64_t tokens_per_epoch) {
  if (seq_length <= 0) throw std::invalid_argument("seq_length must be positive");
  const int64_t total_tokens = num_epochs * tokens_per_epoch;
  const int64_t num_samples = (total_tokens - 1) / seq_length;
  py::array_t<Index> out({num_samples + 1, static_cast<int64_t>(2)});
  Index* rows = out.mutable_data();
  int64_t pos = 0;      // position in doc_idx
  int64_t offset = 0;   // token offset inside doc_idx[pos]
  rows[0] = 0;
  rows[1] = 0;
  for (int64_t s = 1; s <= num_samples; ++s) {
    // the start of sample s is where token s * seq_length of the concatenated stream lives: walk seq_length
    // tokens on from the previous start (a start never rests on a document's end: it moves to the next document)
    int64_t need = seq_length;
    while (need > 0) {
      if (pos >= n_docs) throw std::out_of_range("sample index ran past the document index");
      const int32_t doc = doc_idx[pos];
      if (doc < 0 || doc >= n_sizes) throw std::out_of_range("document id outside the sizes array");
      const int64_t left = static_cast<int64_t>(sizes[doc]) - offset;
      if (left > need) {
        offset += need;
        need = 0;
      } else {
        need -= left;
        ++pos;
        offset = 0;
      }
    }
    rows[2 * s] = static_cast<Index>(pos);
    rows[2 * s + 1] = static_cast<Index>(offset);
  }
  return out;
}

}  // namespace

py::array build_sample_idx(py::array_t<int32_t, py::array::c_style | py::array::forcecast> sizes,
                           py::array_t<int32_t, py::array::c_style | py::array::forcecast> doc_idx, int64_t seq_length,
                           int64_t num_epochs, int64_t tokens_per_epoch) {
  const bool wide = doc_idx.size() > static_cast<py::ssize_t>(INT32_MAX);
  if (wide)
    return sample_index_impl<int64_t>(sizes.data(), sizes.size(), doc_idx.data(), doc_idx.size(), seq_length, num_epochs,
                                      tokens_per_epoch);
  return sample_index_impl<int32_t>(sizes.data(), sizes.size(), doc_idx.data(), doc_idx.size(), seq_length, num_epochs,
                                    tokens_per_epoch);
}

py::tuple build_blending_indices(py::array_t<double, py::array::c_style | py::array::forcecast> weights, int64_t size) {
  const int64_t n = weights.size();
  if (n <= 0 || n > 255) throw std::invalid_argument("between 1 and 255 datasets can be blended");
  const double* w = weights.data();
  py::array_t<uint8_t> which(size);
  py::array_t<int64_t> index(size);
  uint8_t* which_p = which.mutable_data();
  int64_t* index_p = index.mutable_data();
  std::vector<int64_t> taken(n, 0);
  for (int64_t i = 0; i < size; ++i) {
    // pick the dataset that is furthest behind its share of the first i+1 draws
    const double target = static_cast<double>(std::max<int64_t>(i, 1));
    int64_t best = 0;
    double best_err = w[0] * target - static_cast<double>(taken[0]);
    for (int64_t d = 1; d < n; ++d) {
      const double err = w[d] * target - static_cast<double>(taken[d]);
      if (err > best_err) {
        best_err = err;
        best = d;
      }
    }
    which_p[i] = static_cast<uint8_t>(best);
    index_p[i] = taken[best]++;
  }
  return py::make_tuple(which, index);
}

// tokens: raw bytes of the .bin file (memory-mapped numpy array of uint8); token_width: bytes per token (2 or 4);
// pointers: byte offset of every document; sizes: tokens per document.
void gather_samples(py::array_t<uint8_t, py::array::c_style> tokens, int token_width,
                    py::array_t<int64_t, py::array::c_style | py::array::forcecast> pointers,
                    py::array_t<int32_t, py::array::c_style | py::array::forcecast> sizes,
                    py::array_t<int32_t, py::array::c_style | py::array::forcecast> doc_idx,
                    py::array_t<int64_t, py::array::c_style | py::array::forcecast> sample_idx,
                    py::array_t<int64_t, py::array::c_style | py::array::forcecast> picks, int64_t seq_length,
                    py::array_t<int64_t, py::array::c_style> out, int threads) {
  if (token_width != 2 && token_width != 4) throw std::invalid_argument("token width must be 2 or 4 bytes");
  const int64_t n = picks.size();
  const int64_t span = seq_length + 1;
  if (out.size() < n * span) throw std::invalid_argument("output buffer too small");
  const uint8_t* tok = tokens.data();
  const int64_t tok_bytes = tokens.size();
  const int64_t* ptr = pointers.data();
  const int32_t* sz = sizes.data();
  const int32_t* docs = doc_idx.data();
  const int64_t n_docs = doc_idx.size();
  const int64_t* sidx = sample_idx.data();
  const int64_t n_samples = sample_idx.shape(0) - 1;
  const int64_t* pk = picks.data();
  int64_t* dst = out.mutable_data();
  std::vector<int> bad(std::max(threads, 1), 0);

  auto work = [&](int tid, int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
      const int64_t s = pk[i];
      if (s < 0 || s >= n_samples) { bad[tid] = 1; return; }
      int64_t pos = sidx[2 * s], off = sidx[2 * s + 1];
      int64_t filled = 0;
      int64_t* row = dst + i * span;
      while (filled < span) {
        if (pos >= n_docs) { bad[tid] = 1; return; }
        const int32_t d = docs[pos];
        const int64_t take = std::min<int64_t>(span - filled, static_cast<int64_t>(sz[d]) - off);
        const int64_t byte0 = ptr[d] + off * token_width;
        if (take < 0 || byte0 < 0 || byte0 + take * token_width > tok_bytes) { bad[tid] = 1; return; }
        if (token_width == 2) {
          const uint16_t* src = reinterpret_cast<const uint16_t*>(tok + byte0);
          for (int64_t t = 0; t < take; ++t) row[filled + t] = src[t];
        } else {
          const int32_t* src = reinterpret_cast<const int32_t*>(tok + byte0);
          for (int64_t t = 0; t < take; ++t) row[filled + t] = src[t];
        }
        filled += take;
        ++pos;
        off = 0;
      }
    }
  };
  {
    py::gil_scoped_release release;
    const int nt = std::max(1, std::min<int>(threads, static_cast<int>(n)));
    if (nt == 1) {
      work(0, 0, n);
    } else {
      std::vector<std::thread> pool;
      const int64_t per = (n + nt - 1) / nt;
      for (int t = 0; t < nt; ++t) pool.emplace_back(work, t, std::min<int64_t>(n, t * per), std::min<int64_t>(n, (t + 1) * per));
      for (auto& th : pool) th.join();
    }
  }
  for (int b : bad)
    if (b) throw std::out_of_range("a sample reaches outside the dataset files");
}

PYBIND11_MODULE(data_index, m) {
  m.doc() = "dataset sample index, blending index and batch gather";
  m.def("build_sample_idx", &build_sample_idx, py::arg("sizes"), py::arg("doc_idx"), py::arg("seq_length"),
        py::arg("num_epochs"), py::arg("tokens_per_epoch"));
  m.def("build_blending_indices", &build_blending_indices, py::arg("weights"), py::arg("size"));
  m.def("gather_samples", &gather_samples);
}
