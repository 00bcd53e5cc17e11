// Deterministic single-launch sum reductions (objective values and statistics).
//
// Each block writes one fp64 partial into caller-provided scratch memory; the
// block that draws the last ticket adds the partials in index order, so the
// result does not depend on block scheduling.  Scratch layout, in bytes:
//   [0, 8*kReduceMaxBlocks)      double partial[]
//   [8*kReduceMaxBlocks, +4)     unsigned ticket   (must be 0 at launch; the
//                                kernel leaves it 0 again)
#pragma once
#include "psb_common.cuh"

namespace psb {

constexpr int kReduceMaxBlocks = 1024;
constexpr int kReduceThreads = 256;
constexpr size_t kReduceScratchBytes = 8 * (size_t)kReduceMaxBlocks + 256;

enum ReduceOp : int {
  kSumLog1pInv = 0,   // Σ log(1 + 1/x_i)      DARLIN loss from dual_i = exp(y_i·Xw_i)
  kSumAbs = 1,        // Σ |x_i| over finite, non-zero x (λ₁ penalty; NaN = filtered key)
  kCountNonZero = 2,  // #{i : x_i != 0 and x_i is not NaN}
  kSumLogistic = 3,   // Σ log(1 + exp(-x_i))  logistic loss from margins y_i·Xw_i
  kSumSquareHinge = 4,  // Σ max(0, 1 − x_i)²   square hinge loss from margins (src/linear_method/loss.h:97-99)
};

__device__ __forceinline__ double reduce_term(int op, float x) {
  switch (op) {
    case kSumLog1pInv: return log1p(1.0 / (double)x);
    case kSumAbs: return (x == x && x != 0.f) ? fabs((double)x) : 0.0;
    case kCountNonZero: return (x == x && x != 0.f) ? 1.0 : 0.0;
    case kSumSquareHinge: { const double t = 1.0 - (double)x; return t > 0 ? t * t : 0.0; }
    default: { const double m = -(double)x; return m > 0 ? m + log1p(exp(-m)) : log1p(exp(m)); }
  }
}

__device__ __forceinline__ double block_sum_d(double v, double* smem) {
  v = warp_sum_d(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) smem[wid] = v;
  __syncthreads();
  v = (threadIdx.x < (blockDim.x >> 5)) ? smem[threadIdx.x] : 0.0;
  if (wid == 0) v = warp_sum_d(v);
  __syncthreads();
  return v;  // valid in thread 0
}

static __global__ void __launch_bounds__(kReduceThreads)
reduce_sum_kernel(const float* __restrict__ x, size_t n, int op, double* partial, unsigned* ticket, double* out) {
  __shared__ double smem[kReduceThreads / 32];
  __shared__ bool last;
  double s = 0.0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    s += reduce_term(op, x[i]);
  s = block_sum_d(s, smem);
  if (threadIdx.x == 0) {
    partial[blockIdx.x] = s;
    __threadfence();
    last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  double t = 0.0;
  for (int b = threadIdx.x; b < (int)gridDim.x; b += blockDim.x) t += __ldcg(partial + b);
  t = block_sum_d(t, smem);
  if (threadIdx.x == 0) {
    out[0] = t;
    *ticket = 0u;
  }
}

inline int reduce_grid(size_t n) {
  size_t b = (n + (size_t)kReduceThreads * 8 - 1) / ((size_t)kReduceThreads * 8);
  if (b < 1) b = 1;
  if (b > (size_t)kReduceMaxBlocks) b = kReduceMaxBlocks;
  return (int)b;
}

}  // namespace psb
