// One FTRL minibatch on a CPU worker: margins against the pulled weights, logistic loss, the gradient of
// every unique key and how many positive / negative examples contain it (the counts feed the servers'
// per-key gradient-norm estimate).
//
// Arithmetic: FTRL::updateModel and FTRL::countKeys (src/linear_method/ftrl.cc:88-151, 154-174).  The row
// pass (margin, loss, per-row coefficient -y / (1 + e^{y Xw})) is spread over threads; the scatter into the
// per-key arrays runs in row order on one thread, so that a key's contributions are added in a fixed order.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <thread>
#include <vector>

namespace psb {

// off: rows + 1 offsets; loc: local key id per non-zero; val: values or nullptr (binary); y: +-1 per row;
// w: weight per local key (0 for keys held back by the tail filter).  g, pos, neg: one entry per local key
// (overwritten).  Returns the summed logistic loss.
inline double ftrl_minibatch(const int64_t* off, size_t rows, const int32_t* loc, const double* val, const double* y,
                             const double* w, size_t nkeys, int threads, double* g, double* pos, double* neg) {
  std::vector<double> coef(rows);
  const int T = (int)std::max<size_t>(1, std::min<size_t>((size_t)std::max(threads, 1), rows / 256));
  std::vector<double> part(T, 0.0);
  auto row_pass = [&](int t) {
    double loss = 0;
    for (size_t i = rows * t / T; i < rows * (t + 1) / T; ++i) {
      double xw = 0;
      for (int64_t p = off[i]; p < off[i + 1]; ++p) xw += w[loc[p]] * (val ? val[p] : 1.0);
      const double m = y[i] * xw;
      loss += m > 0 ? std::log1p(std::exp(-m)) : -m + std::log1p(std::exp(m));     // log(1 + e^{-m}) without overflow
      coef[i] = -y[i] / (1.0 + std::exp(m));
    }
    part[t] = loss;
  };
  if (T == 1) {
    row_pass(0);
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < T; ++t) pool.emplace_back(row_pass, t);
    for (auto& th : pool) th.join();
  }
  std::fill(g, g + nkeys, 0.0);
  std::fill(pos, pos + nkeys, 0.0);
  std::fill(neg, neg + nkeys, 0.0);
  for (size_t i = 0; i < rows; ++i) {
    const bool positive = y[i] > 0;
    for (int64_t p = off[i]; p < off[i + 1]; ++p) {
      const int32_t k = loc[p];
      g[k] += coef[i] * (val ? val[p] : 1.0);
      (positive ? pos : neg)[k] += 1.0;
    }
  }
  double loss = 0;
  for (double v : part) loss += v;
  return loss;
}

}  // namespace psb
