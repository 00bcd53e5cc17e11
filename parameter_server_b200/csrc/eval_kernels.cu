// Evaluation kernels: the binned AUC of the reference (src/base/auc.h:69-98: a prediction falls into bin
// (int64)(p · goodness); positives and negatives are counted per bin, bins are merged over workers and
// the area is summed over the merged thresholds) and the exact AUC by sorting the scores
// (src/base/evaluation.h:18-44).  The sort / run-length steps are the radix sort and unique kernels
// of sparse_kernels.cu; this file holds the pieces specific to AUC.
#include "psb_common.cuh"

namespace psb {

// bin of every prediction as a 64-bit key whose UNSIGNED order is the signed order of the bin
// (sign bit flipped), for positives and negatives apart: keys of the other class become kEmptyKey
// and sort to the end
__global__ void k_auc_bin_keys(const float* label, const float* pred, size_t n, long long goodness, uint64_t* pos_keys,
                               uint64_t* neg_keys) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const long long bin = (long long)((double)pred[i] * (double)goodness);
    const uint64_t key = (uint64_t)bin ^ 0x8000000000000000ull;
    const bool positive = label[i] > 0.f;
    pos_keys[i] = positive ? key : kEmptyKey;
    neg_keys[i] = positive ? kEmptyKey : key;
  }
}

// scores as 64-bit keys in ascending order of the float values (NaN last)
__global__ void k_score_keys(const float* pred, size_t n, uint64_t* keys) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    uint32_t b = __float_as_uint(pred[i]);
    if (b == 0x80000000u) b = 0u;          // −0 and +0 are the same score
    keys[i] = (uint64_t)((b & 0x80000000u) ? ~b : (b | 0x80000000u));
  }
}

// Area from the runs of equal scores in ascending order: a negative counts the positives of all earlier
// runs and half of those in its own run (the tie correction of the rank-sum statistic).  `start`, `count`:
// first position and length of every run; `before`: exclusive prefix sum of the positive flags in score
// order; `total_pos`: their sum.  One thread per run, one fp64 atomic per block.
__global__ void k_auc_area(const int64_t* start, const uint32_t* count, size_t runs, const int64_t* before, size_t n,
                           const int64_t* total_pos, double* area) {
  __shared__ double smem[8];
  double s = 0.0;
  for (size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x; r < runs; r += (size_t)gridDim.x * blockDim.x) {
    const int64_t b = start[r], e = b + (int64_t)count[r];
    const int64_t pos_before = before[b];
    const int64_t pos_here = ((size_t)e < n ? before[e] : *total_pos) - pos_before;
    const int64_t neg_here = (int64_t)count[r] - pos_here;
    s += (double)neg_here * ((double)pos_before + 0.5 * (double)pos_here);
  }
  s = warp_sum_d(s);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? smem[threadIdx.x] : 0.0;
    s = warp_sum_d(s);
    if (threadIdx.x == 0 && s != 0.0) atomicAdd(area, s);
  }
}

// payload of the score sort: 1 for a positive example
__global__ void k_label_flags(const float* label, size_t n, uint32_t* flag) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    flag[i] = label[i] > 0.f ? 1u : 0u;
}

}  // namespace psb

using namespace psb;

static inline int egrid(size_t n) {
  size_t b = (n + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return (int)b;
}

extern "C" {
int psb_auc_bin_keys(const float* label, const float* pred, size_t n, long long goodness, uint64_t* pos_keys, uint64_t* neg_keys,
                     cudaStream_t s) {
  k_auc_bin_keys<<<egrid(n), 256, 0, s>>>(label, pred, n, goodness, pos_keys, neg_keys);
  return (int)cudaGetLastError();
}
int psb_score_keys(const float* pred, size_t n, uint64_t* keys, cudaStream_t s) {
  k_score_keys<<<egrid(n), 256, 0, s>>>(pred, n, keys);
  return (int)cudaGetLastError();
}
int psb_label_flags(const float* label, size_t n, uint32_t* flag, cudaStream_t s) {
  k_label_flags<<<egrid(n), 256, 0, s>>>(label, n, flag);
  return (int)cudaGetLastError();
}
int psb_auc_area(const int64_t* start, const uint32_t* count, size_t runs, const int64_t* before, size_t n,
                 const int64_t* total_pos, double* area, cudaStream_t s) {
  k_auc_area<<<egrid(runs), 256, 0, s>>>(start, count, runs, before, n, total_pos, area);
  return (int)cudaGetLastError();
}
}
