// DARLIN block steps for CPU nodes: the worker's block gradient and dual update and the server's
// proximal-Newton weight update over one feature block, on CSC columns in host memory.
//
// Arithmetic: Darling::computeGradients (src/linear_method/darling.cc:306-356), updateWeight (:437-477),
// updateDual (:358-435).  The gradient is threaded over columns (every column writes its own G, U);
// the dual update runs column by column, like the reference's mutex-serialised version, because two
// columns may share rows.  Inactive columns carry a NaN in (G, U), the reference's sentinel.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <limits>
#include <thread>
#include <vector>

namespace psb {

struct CscBlock {            // columns [c0, c1) of a CSC matrix with 64-bit offsets and 32-bit row ids
  const int64_t* indptr;     // offset of column j at indptr[j - col_base]
  const int32_t* indices;    // row id / value of position p at [p - pos_base]
  const double* data;        // nullptr: all values are 1 (binary features)
  int64_t c0, c1;
  int64_t col_base = 0, pos_base = 0;   // non-zero when the arrays hold a column range loaded on its own
};

// G_j = -sum_i y_i tau_i x_ij,  U_j = sum_i min(tau_i (1 - tau_i) e^{|x_ij| delta_j}, 1/4) x_ij^2,
// tau_i = 1 / (1 + dual_i).  G, U have c1 - c0 entries.
inline void darlin_block_gradient(const CscBlock& B, const double* y, const double* dual, const double* delta,
                                  const uint8_t* active, double* G, double* U, int threads) {
  const double nan = std::numeric_limits<double>::quiet_NaN();
  auto work = [&](int64_t a, int64_t b) {
    for (int64_t j = a; j < b; ++j) {
      const int64_t jj = j - B.c0;
      if (!active[j]) { G[jj] = U[jj] = nan; continue; }
      double g = 0, u = 0;
      const double d = delta[j], ed = std::exp(d);
      const int64_t* ip = B.indptr + (j - B.col_base);
      for (int64_t p = ip[0] - B.pos_base; p < ip[1] - B.pos_base; ++p) {
        const int32_t r = B.indices[p];
        const double tau = 1.0 / (1.0 + dual[r]), t2 = tau * (1.0 - tau);
        if (B.data == nullptr) {
          g += y[r] * tau;
          u += std::min(t2 * ed, 0.25);
        } else {
          const double v = B.data[p];
          g += y[r] * tau * v;
          u += std::min(t2 * std::exp(std::fabs(v) * d), 0.25) * v * v;
        }
      }
      G[jj] = -g;
      U[jj] = u;
    }
  };
  const int64_t n = B.c1 - B.c0;
  const int t = (int)std::max<int64_t>(1, std::min<int64_t>(threads, n / 64));
  if (t <= 1) { work(B.c0, B.c1); return; }
  std::vector<std::thread> pool;
  for (int i = 0; i < t; ++i) pool.emplace_back(work, B.c0 + n * i / t, B.c0 + n * (i + 1) / t);
  for (auto& th : pool) th.join();
}

// Server side: slots [0, n) of a block; w, delta, active are the block's segments (in place).
// Returns the largest KKT violation seen.
inline double darlin_update_weight(double* w, double* delta, uint8_t* active, const double* G, const double* U, int64_t n,
                                   double lambda, double eta, double kkt_threshold, double delta_max) {
  double violation = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (!active[i]) continue;
    const double g = G[i], u = U[i] / eta + 1e-10;
    if (g != g) continue;                       // every worker sent the inactive sentinel
    const double gp = g + lambda, gn = g - lambda, wk = w[i];
    double d = -wk, vio = 0;
    if (wk == 0) {
      if (gp < 0) vio = -gp;
      else if (gn > 0) vio = gn;
      else if (gp > kkt_threshold && gn < -kkt_threshold) {
        active[i] = 0;
        w[i] = std::numeric_limits<double>::quiet_NaN();
        continue;
      }
    }
    violation = std::max(violation, vio);
    if (gp <= u * wk) d = -gp / u;
    else if (gn >= u * wk) d = -gn / u;
    d = std::min(delta[i], std::max(-delta[i], d));
    delta[i] = std::min(delta_max, 2 * std::fabs(d) + 0.1);
    w[i] = wk + d;
  }
  return violation;
}

// Worker side after the pull: w_new has c1 - c0 entries (NaN = filtered by the server).
inline void darlin_update_dual(const CscBlock& B, const double* y, double* dual, double* w, double* delta, uint8_t* active,
                               const double* w_new, double delta_max) {
  for (int64_t j = B.c0; j < B.c1; ++j) {
    if (!active[j]) continue;
    const double wn = w_new[j - B.c0];
    if (wn != wn) { active[j] = 0; w[j] = 0; continue; }
    const double dw = wn - w[j];
    delta[j] = std::min(delta_max, 2 * std::fabs(dw) + 0.1);
    w[j] = wn;
    if (dw == 0) continue;
    const int64_t* ip = B.indptr + (j - B.col_base);
    for (int64_t p = ip[0] - B.pos_base; p < ip[1] - B.pos_base; ++p) {
      const int32_t r = B.indices[p];
      dual[r] *= std::exp(y[r] * (B.data ? B.data[p] : 1.0) * dw);
    }
  }
}

}  // namespace psb
