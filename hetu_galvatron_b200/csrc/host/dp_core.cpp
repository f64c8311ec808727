// Native core of the layer-wise strategy search: a knapsack-style dynamic program over
// (layer, memory budget, strategy of this layer) with transition costs between neighbouring layers.
//
//   f_i[m][s] = min_{s'} f_{i-1}[m - mem[i][s]][s'] + inter[i][s'][s] + intra[i][s]
//
// with a back-pointer table for reconstructing the argmin path.  After the last layer, for every
// candidate of the embedding / LM-head strategy (a key with its own memory and time), the best final
// state that still fits is selected and the per-layer strategy indices are traced back.
//
// Two evaluation orders:
//   * exact    : one rolling table updated in place, memory descending -- reproduces, to the bit, the
//                order of floating-point operations (and the corner case of zero-memory strategies) of
//                the reference core (csrc/dp_core.cpp:24-120);
//   * parallel : two tables (previous / current layer) so that the memory axis can be split over
//                threads; identical results whenever every strategy needs at least 1 MB, which is how
//                budgets of 180 GB x 80 layers x 50^2 transitions stay interactive.
//
// Python interface (pybind11): dynamic_programming_core(...) with the argument list of the reference
// plus an optional thread count; search/dp.py owns the arrays.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <limits>
#include <map>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

constexpr double kInf = std::numeric_limits<double>::infinity();

struct Problem {
  int layers, mem, strat;
  const int32_t* v;      // [layers, strat]
  int32_t* mark;         // [layers, mem, strat]
  double* f;             // [mem, strat]
  const double* inter;   // [layers, strat(prev), strat(cur)]
  const double* intra;   // [layers, strat]
};

// One (layer, m) row: fills f_out[m][*] and mark[layer][m][*] reading rows of f_in.
inline void relax_row(const Problem& p, int layer, int m, const double* f_in, double* f_out) {
  const int S = p.strat;
  for (int s = 0; s < S; ++s) {
    const int need = p.v[layer * S + s];
    int32_t* mk = p.mark + (size_t(layer) * p.mem + m) * S + s;
    if (m < need) {
      *mk = -1;
      f_out[size_t(m) * S + s] = kInf;
      continue;
    }
    const double* prev = f_in + size_t(m - need) * S;
    const double* tr = p.inter + size_t(layer) * S * S + s;  // inter[layer][s'][s], stride S over s'
    const double own = p.intra[layer * S + s];
    double best = kInf;
    int arg = 0;
    for (int sp = 0; sp < S; ++sp) {
      const double c = prev[sp] + tr[size_t(sp) * S] + own;
      if (sp == 0 || c < best) {  // first argmin wins, like a forward scan with strict '<'
        best = c;
        arg = sp;
      }
    }
    *mk = arg;
    f_out[size_t(m) * S + s] = best;
  }
}

void solve_exact(const Problem& p) {
  for (int i = 0; i < p.layers; ++i)
    for (int m = p.mem - 1; m >= 0; --m) relax_row(p, i, m, p.f, p.f);
}

void solve_parallel(const Problem& p, int threads) {
  const size_t cells = size_t(p.mem) * p.strat;
  std::vector<double> other(cells);
  double* cur = p.f;            // layer i-1 lives here on entry
  double* nxt = other.data();
  threads = std::max(1, std::min(threads, p.mem));
  for (int i = 0; i < p.layers; ++i) {
    std::vector<std::thread> pool;
    const int chunk = (p.mem + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
      const int lo = t * chunk, hi = std::min(p.mem, lo + chunk);
      if (lo >= hi) break;
      pool.emplace_back([&, lo, hi, i, cur, nxt]() {
        for (int m = lo; m < hi; ++m) relax_row(p, i, m, cur, nxt);
      });
    }
    for (auto& th : pool) th.join();
    std::swap(cur, nxt);
  }
  if (cur != p.f) std::copy(cur, cur + cells, p.f);
}

bool has_zero_cost_strategy(const Problem& p) {
  for (int i = 0; i < p.layers * p.strat; ++i)
    if (p.v[i] <= 0) return true;
  return false;
}

}  // namespace

std::pair<std::map<int, double>, std::map<int, int>> dynamic_programming_core(
    int layer_num, int max_mem, int strategy_num, py::array_t<int32_t> v_data, py::array_t<int32_t> mark,
    py::array_t<double> f, py::array_t<double> inter_cost, py::array_t<double> intra_cost,
    std::map<int, int> other_mem_cost, std::map<int, double> other_time_cost,
    std::map<int, py::array_t<int32_t>> res_list, int threads) {
  Problem p;
  p.layers = layer_num;
  p.mem = max_mem;
  p.strat = strategy_num;
  p.v = static_cast<const int32_t*>(v_data.request().ptr);
  p.mark = static_cast<int32_t*>(mark.request().ptr);
  p.f = static_cast<double*>(f.request().ptr);
  p.inter = static_cast<const double*>(inter_cost.request().ptr);
  p.intra = static_cast<const double*>(intra_cost.request().ptr);

  {
    py::gil_scoped_release release;
    if (threads <= 1 || has_zero_cost_strategy(p)) solve_exact(p);
    else solve_parallel(p, threads);
  }

  std::map<int, double> total_cost;
  std::map<int, int> remaining;
  const int S = strategy_num;
  for (const auto& kv : other_mem_cost) {
    const int key = kv.first;
    const int budget = max_mem - 1 - kv.second;
    if (budget < 0) {
      total_cost[key] = kInf;
      remaining[key] = -1;
      continue;
    }
    const double* row = p.f + size_t(budget) * S;
    int s = 0;
    for (int c = 1; c < S; ++c)
      if (row[c] < row[s]) s = c;
    if (!(row[s] < kInf)) {
      total_cost[key] = kInf;
      remaining[key] = -1;
      continue;
    }
    total_cost[key] = row[s] + other_time_cost[key];
    int32_t* out = static_cast<int32_t*>(res_list[key].request().ptr);
    out[layer_num - 1] = s;
    int m = budget;
    for (int i = layer_num - 1; i > 0; --i) {
      const int cur = s;
      s = p.mark[(size_t(i) * p.mem + m) * S + cur];
      m -= p.v[i * S + cur];
      out[i - 1] = s;
    }
    remaining[key] = m - p.v[s];
  }
  return {total_cost, remaining};
}

PYBIND11_MODULE(hg_dp_core, m) {
  m.doc() = "dynamic-programming core of the layer-wise strategy search";
  m.def("dynamic_programming_core", &dynamic_programming_core, py::arg("layer_num"), py::arg("max_mem"),
        py::arg("strategy_num"), py::arg("v_data"), py::arg("mark"), py::arg("f"), py::arg("inter_cost"),
        py::arg("intra_cost"), py::arg("other_mem_cost"), py::arg("other_time_cost"), py::arg("res_list"),
        py::arg("threads") = 1);
}
