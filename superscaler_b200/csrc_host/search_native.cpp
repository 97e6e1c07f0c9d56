// Inner loops of the plan search's cost model (host only): which ops of a stage to recompute, and the two
// activation accounts that decision rests on.  Same arithmetic, in the same order, as the Python definitions in
// search/cost_model.py (`_saved_fast`, `_peak_fast`, `_choose_recompute`), so that plans and predictions are equal
// bit for bit; the search calls these hundreds of thousands of times with stages of several hundred ops
// (reference: check_recompute and the memory terms of search/aceso_cost_model.py:822-872, pure Python there).
//
// Per op of the stage:  acts[i]  activation size (MB);  kinds[i]  0 = counted, 1 = counted 1.5 times, 2 = aliases a
// neighbour (not counted);  ends[i] (i < n - 1)  the op after i starts a layer, where a recomputed segment ends.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <vector>

namespace py = pybind11;

namespace {

double saved_by_recompute(const std::vector<int>& rc, const std::vector<double>& acts, const std::vector<int>& kinds,
                          const std::vector<int>& ends) {
  const size_t n = acts.size();
  if (n <= 1) return 0.0;
  double saved = 0.0;
  for (size_t i = 0; i + 1 < n; ++i) {
    if (rc[i] == 1 && rc[i + 1] == 1) {
      if (kinds[i] == 1) {
        saved += acts[i] * 1.5;
      } else if (kinds[i] == 0 && !ends[i]) {
        saved += acts[i];
      }
    }
  }
  return saved;
}

double peak_recompute(const std::vector<int>& rc, const std::vector<double>& acts, const std::vector<int>& kinds,
                      const std::vector<int>& ends) {
  const size_t n = acts.size();
  if (n <= 1) return 0.0;
  double run = 0.0, best = 0.0;
  const size_t last = n - 1;
  for (size_t i = 0; i < last; ++i) {
    if (rc[i] == 1 && rc[i + 1] == 1) {
      if (kinds[i] == 1) {
        run += acts[i] * 1.5;
      } else if (kinds[i] == 0) {
        run += acts[i];
        if (ends[i] || i + 1 == last) {
          if (run > best) best = run;
          run = 0.0;
        }
      }
    } else if (run > 0.0) {
      if (run > best) best = run;
      run = 0.0;
    }
  }
  return best;
}

// group_of[i]: id of op i's name, ids numbered in order of first appearance; eligible[g]: the name may be chosen.
// `mem` is the stage's memory with nothing recomputed; returns the recompute flags.
std::vector<int> choose_recompute(const std::vector<double>& acts, const std::vector<int>& kinds,
                                  const std::vector<int>& ends, const std::vector<int>& group_of,
                                  const std::vector<int>& eligible, double mem, double limit, int stages_behind) {
  const size_t n = acts.size();
  const size_t num_groups = eligible.size();
  std::vector<int> rc(n, 0);
  std::vector<std::vector<int>> index(num_groups);
  std::vector<std::vector<double>> size(num_groups);
  std::vector<double> sum(num_groups, 0.0);
  std::vector<char> done(num_groups, 0);
  const double mult = static_cast<double>(stages_behind + 1);
  for (size_t i = 0; i < n; ++i) {
    const int g = group_of[i];
    const double sz = acts[i] * mult;
    index[g].push_back(static_cast<int>(i));
    size[g].push_back(sz);
    sum[g] += sz;
  }
  double saved0 = 0.0, peak0 = 0.0;
  while (mem - limit > 0.0) {
    int best = -1;
    double best_sz = 0.0;
    for (size_t g = 0; g < num_groups; ++g) {
      if (!done[g] && sum[g] > best_sz && eligible[g]) {
        best = static_cast<int>(g);
        best_sz = sum[g];
      }
    }
    if (best_sz == 0.0) break;
    done[best] = 1;
    const size_t nxt = static_cast<size_t>(index[best][0]) + 1;
    if (nxt >= n) break;
    done[group_of[nxt]] = 1;
    const double exceed = mem - limit;
    size_t take = index[best].size();
    if (!(best_sz < exceed)) {
      double acc = 0.0;
      size_t k = 0;
      while (acc <= exceed && k < size[best].size()) {
        acc += size[best][k];
        ++k;
      }
      take = k;
    }
    for (size_t j = 0; j < take; ++j) {
      const size_t i = static_cast<size_t>(index[best][j]);
      rc[i] = 1;
      if (i + 1 < n) rc[i + 1] = 1;
    }
    const double saved1 = saved_by_recompute(rc, acts, kinds, ends);
    mem -= (saved1 - saved0) * mult;
    saved0 = saved1;
    const double peak1 = peak_recompute(rc, acts, kinds, ends);
    mem += peak1 - peak0;
    peak0 = peak1;
  }
  return rc;
}

}  // namespace

PYBIND11_MODULE(_search_native, m) {
  m.def("saved_by_recompute", &saved_by_recompute);
  m.def("peak_recompute", &peak_recompute);
  m.def("choose_recompute", &choose_recompute);
}
