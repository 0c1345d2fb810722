// Dynamic-programming core of the strategy search (pybind11 module `dp_core`).
//
// Call contract of the reference's native module (csrc/dp_core.cpp:24-35, bound at :122-124):
//   dynamic_programming_core(layer_num, max_mem, strategy_num, v_data[L,S] int32, mark[L,max_mem,S] int32,
//                            f[max_mem,S] float64, inter_cost[L,S,S], intra_cost[L,S],
//                            other_mem_cost{vtp: MB}, other_time_cost{vtp: ms}, res_list{vtp: int32[L]})
//     -> (total_cost{vtp}, remaining_mem{vtp});   res_list[vtp][layer] is filled in place.
// Recurrence: f_i[v][s] = min_si ( f_{i-1}[v - mem(i,s)][si] + inter(i,si,s) ) + intra(i,s), first minimum wins.
//
// Own design: the previous layer's table is kept as a separate buffer (so a layer whose memory cost is 0 MB
// reads consistent values; the reference's single rolling table is only safe for costs > 0), the tables are held
// strategy-major so the reduction over previous strategies vectorises over memory cells, tiles of cells are
// processed in parallel with OpenMP, and every index derived from caller data is bounds-checked.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <limits>
#include <map>
#include <stdexcept>
#include <utility>
#include <vector>

namespace py = pybind11;

namespace {

constexpr double kInf = std::numeric_limits<double>::infinity();

template <typename T>
T* checked_ptr(py::array_t<T>& a, size_t need, const char* name, bool writable) {
  py::buffer_info info = a.request(writable);
  if (static_cast<size_t>(info.size) < need) throw std::invalid_argument(std::string(name) + ": buffer too small");
  // C-contiguity: strides must describe a dense row-major array
  ssize_t expect = static_cast<ssize_t>(sizeof(T));
  for (ssize_t d = info.ndim - 1; d >= 0; --d) {
    if (info.shape[d] > 1 && info.strides[d] != expect) throw std::invalid_argument(std::string(name) + ": not C-contiguous");
    expect *= info.shape[d];
  }
  return static_cast<T*>(info.ptr);
}

std::pair<std::map<int, double>, std::map<int, int>> dynamic_programming_core(
    int layer_num, int max_mem, int strategy_num, py::array_t<int> v_data, py::array_t<int> mark,
    py::array_t<double> f, py::array_t<double> inter_cost, py::array_t<double> intra_cost,
    std::map<int, int> other_mem_cost, std::map<int, double> other_time_cost,
    std::map<int, py::array_t<int>> res_list) {
  if (layer_num <= 0 || max_mem <= 0 || strategy_num <= 0) throw std::invalid_argument("sizes must be positive");
  const size_t L = layer_num, V = max_mem, S = strategy_num;
  const int* v_ptr = checked_ptr(v_data, L * S, "v_data", false);
  int* mark_ptr = checked_ptr(mark, L * V * S, "mark", true);
  double* f_ptr = checked_ptr(f, V * S, "f", true);
  const double* inter_ptr = checked_ptr(inter_cost, L * S * S, "inter_cost", false);
  const double* intra_ptr = checked_ptr(intra_cost, L * S, "intra_cost", false);
  for (size_t k = 0; k < L * S; ++k)
    if (v_ptr[k] < 0) throw std::invalid_argument("v_data: negative memory cost");

  // Tables are kept strategy-major ([S][V]) so that, for one (strategy, previous strategy) pair, the candidates of a run
  // of memory cells are contiguous: the min / arg-min over previous strategies becomes S passes of an element-wise
  // compare-and-select over a tile of cells, which the compiler vectorises. Tiles are the unit of OpenMP work.
  std::vector<double> prev(S * V), cur(S * V);
  for (size_t v = 0; v < V; ++v)
    for (size_t s = 0; s < S; ++s) prev[s * V + v] = f_ptr[v * S + s];
  constexpr size_t kTile = 512;
  const long long n_tiles = static_cast<long long>((V + kTile - 1) / kTile);

  {
    py::gil_scoped_release release;
    for (size_t i = 0; i < L; ++i) {
      const double* inter_i = inter_ptr + i * S * S;
      const int* mem_i = v_ptr + i * S;
      const double* intra_i = intra_ptr + i * S;
      int* mark_i = mark_ptr + i * V * S;
#pragma omp parallel
      {
        double best[kTile], idx[kTile];
#pragma omp for schedule(static)
        for (long long t = 0; t < n_tiles; ++t) {
          const size_t v0 = static_cast<size_t>(t) * kTile, v1 = std::min(V, v0 + kTile);
          for (size_t s = 0; s < S; ++s) {
            const size_t m = static_cast<size_t>(mem_i[s]);
            const size_t lo = std::min(v1, std::max(v0, m));   // cells below `lo` cannot pay for this strategy
            for (size_t v = v0; v < lo; ++v) {
              cur[s * V + v] = kInf;
              mark_i[v * S + s] = -1;
            }
            if (lo >= v1) continue;
            const size_t n = v1 - lo;
            const double add = intra_i[s];
            {
              const double* p = prev.data() + (lo - m);
              const double w = inter_i[s];
              for (size_t k = 0; k < n; ++k) {
                best[k] = (p[k] + w) + add;
                idx[k] = 0.0;
              }
            }
            for (size_t si = 1; si < S; ++si) {
              const double* p = prev.data() + si * V + (lo - m);
              const double w = inter_i[si * S + s], tag = static_cast<double>(si);
              for (size_t k = 0; k < n; ++k) {
                const double c = (p[k] + w) + add;
                const bool lt = c < best[k];          // strict: the first minimum wins
                best[k] = lt ? c : best[k];
                idx[k] = lt ? tag : idx[k];
              }
            }
            double* out = cur.data() + s * V + lo;
            for (size_t k = 0; k < n; ++k) {
              out[k] = best[k];
              mark_i[(lo + k) * S + s] = static_cast<int>(idx[k]);
            }
          }
        }
      }
      prev.swap(cur);
    }
  }
  for (size_t v = 0; v < V; ++v)
    for (size_t s = 0; s < S; ++s) f_ptr[v * S + s] = prev[s * V + v];

  std::map<int, double> total_cost;
  std::map<int, int> remaining_mem;
  for (const auto& item : other_mem_cost) {
    const int vtp = item.first;
    const long long start_v = static_cast<long long>(max_mem) - 1 - item.second;
    if (start_v < 0 || start_v >= static_cast<long long>(V)) {
      total_cost[vtp] = kInf;
      remaining_mem[vtp] = -1;
      continue;
    }
    const double* row = f_ptr + start_v * S;
    int next_index = static_cast<int>(std::min_element(row, row + S) - row);
    long long next_v = start_v;
    double cost = row[next_index];
    if (!(cost < kInf)) {
      total_cost[vtp] = kInf;
      remaining_mem[vtp] = -1;
      continue;
    }
    auto t = other_time_cost.find(vtp);
    if (t == other_time_cost.end()) throw std::invalid_argument("other_time_cost: missing key");
    total_cost[vtp] = cost + t->second;
    auto r = res_list.find(vtp);
    if (r == res_list.end()) throw std::invalid_argument("res_list: missing key");
    int* res = checked_ptr(r->second, L, "res_list", true);
    res[L - 1] = next_index;
    for (size_t i = L - 1; i > 0; --i) {
      const int cur_index = next_index;
      if (next_v < 0) throw std::runtime_error("back-tracking left the table");
      next_index = mark_ptr[i * V * S + next_v * S + cur_index];
      next_v -= v_ptr[i * S + cur_index];
      if (next_index < 0 || next_index >= strategy_num) throw std::runtime_error("back-tracking hit an infeasible cell");
      res[i - 1] = next_index;
    }
    remaining_mem[vtp] = static_cast<int>(next_v - v_ptr[next_index]);
  }
  return {total_cost, remaining_mem};
}

}  // namespace

PYBIND11_MODULE(dp_core, m) {
  m.doc() = "Dynamic-programming core of the hybrid-parallel strategy search";
  m.def("dynamic_programming_core", &dynamic_programming_core, "Layer-wise strategy DP under a memory budget");
}
