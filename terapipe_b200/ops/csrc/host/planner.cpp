// Slice-schedule dynamic program (host C++).
//
// Given a latency grid t[bs][s][c] (batch-slice size bs, slice length s*gap, context c*gap),
// a total batch B, a total sequence of n steps and an upper bound max_latency on any single
// slice, finds the token/batch slicing that minimises the sum of slice latencies, and reports
// the largest slice latency on that optimum so the caller can add the (K-1)*max pipeline
// fill term.  Same recurrences as the reference's numba kernel (latency_model.py:97-149);
// compiled ahead of time instead of JIT-compiled.
#include <cstdint>
#include <cmath>
#include <limits>
#include <vector>

extern "C" {

// grid: [grid_b][grid_s][grid_c] row-major doubles.
// f_step: [B+1][n+1] int64 (out), g_step: [B+1] int64 (out).
// returns sum of latencies g[B]; *max_out = largest slice latency on the optimum.
double tp_plan_slices(const double* grid, int64_t grid_b, int64_t grid_s, int64_t grid_c,
                      int64_t B, int64_t n, double max_latency,
                      int64_t* f_step, int64_t* g_step, double* max_out) {
  const double inf = std::numeric_limits<double>::infinity();
  const int64_t W = n + 1;
  std::vector<double> f((B + 1) * W, 0.0), fmax((B + 1) * W, 0.0);
  for (int64_t i = 0; i < (B + 1) * W; ++i) f_step[i] = 0;
  for (int64_t bs = 1; bs <= B; ++bs) {
    double* fb = &f[bs * W];
    double* fm = &fmax[bs * W];
    int64_t* fs = &f_step[bs * W];
    const bool have = bs < grid_b;
    for (int64_t acc = 1; acc <= n; ++acc) {
      double best = inf, best_max = 0.0;
      int64_t best_s = 0;
      if (have) {
        for (int64_t s = 1; s <= acc; ++s) {
          const int64_t c = acc - s;
          if (s >= grid_s || c >= grid_c) continue;
          const double lat = grid[(bs * grid_s + s) * grid_c + c];
          if (!(lat <= max_latency)) continue;
          const double tot = fb[c] + lat;
          if (tot < best) {
            best = tot;
            best_s = s;
            best_max = fm[c] > lat ? fm[c] : lat;
          }
        }
      }
      fb[acc] = best;
      fs[acc] = best_s;
      fm[acc] = best_max;
    }
  }
  std::vector<double> g(B + 1, 0.0), gmax(B + 1, 0.0);
  g_step[0] = 0;
  for (int64_t acc = 1; acc <= B; ++acc) {
    double best = inf, best_max = 0.0;
    int64_t best_bs = 0;
    for (int64_t bs = 1; bs <= acc; ++bs) {
      const double tot = g[acc - bs] + f[bs * W + n];
      if (tot < best) {
        best = tot;
        best_bs = bs;
        const double m = fmax[bs * W + n];
        best_max = gmax[acc - bs] > m ? gmax[acc - bs] : m;
      }
    }
    g[acc] = best;
    g_step[acc] = best_bs;
    gmax[acc] = best_max;
  }
  *max_out = gmax[B];
  return g[B];
}

}  // extern "C"
