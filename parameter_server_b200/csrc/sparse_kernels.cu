// Sparse / key-set building blocks on the device: stable LSD radix sort of uint64 keys with a
// uint32 payload, run-length unique with counts, dictionary remap, bucketed scatter (CSR→CSC
// transposition and k-way key/value partition), count-min sketch, sorted-set intersection,
// plain CSR SpMV / SpMVᵀ, and parameter initialisation.
//
// Counterparts in the reference: Localizer::countUniqIndex / remapIndex (src/base/localizer.h:50-168)
// with parallelSort (src/util/parallel_sort.h), SparseMatrix::alterStorage / times
// (src/base/sparse_matrix.h:73-124, 186-241), kv_partition (src/util/kv_partition.h), CountMin
// (src/base/countmin.h:33-67), SArray set operations and setValue
// (src/base/shared_array_inl.h:108-171).  Nothing here calls a library sort or scan.
#include "psb_common.cuh"

namespace psb {

constexpr int kSortThreads = 256;
constexpr int kSortItems = 8;                         // keys per thread
constexpr int kSortTile = kSortThreads * kSortItems;  // keys per block
constexpr int kRadix = 256;

__device__ __forceinline__ uint32_t digit_of(uint64_t k, int pass) { return (uint32_t)(k >> (8 * pass)) & 0xFFu; }

// one pass over the keys: 8 histograms (one per byte) so that constant digits can be skipped
__global__ void k_digit_histograms(const uint64_t* __restrict__ keys, size_t n, unsigned long long* __restrict__ hist /*[8][256]*/) {
  __shared__ uint32_t sh[8 * kRadix];
  for (int i = threadIdx.x; i < 8 * kRadix; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t k = keys[i];
#pragma unroll
    for (int p = 0; p < 8; ++p) atomicAdd(&sh[p * kRadix + digit_of(k, p)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 8 * kRadix; i += blockDim.x)
    if (sh[i]) atomicAdd(&hist[i], (unsigned long long)sh[i]);
}

// Each warp owns a contiguous chunk of the block's tile and walks it in rounds of 32 keys, so the
// order (block, warp, round, lane) is the input order: ranks computed this way make the pass stable.
__global__ void __launch_bounds__(kSortThreads)
k_radix_count(const uint64_t* __restrict__ keys, size_t n, int pass, uint32_t* __restrict__ block_hist /*[256][nblocks]*/) {
  __shared__ uint32_t wcnt[kSortThreads / 32][kRadix];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (kSortThreads / 32) * kRadix; i += blockDim.x) (&wcnt[0][0])[i] = 0;
  __syncthreads();
  const size_t base = (size_t)blockIdx.x * kSortTile + (size_t)warp * 32 * kSortItems;
#pragma unroll
  for (int r = 0; r < kSortItems; ++r) {
    const size_t i = base + (size_t)r * 32 + lane;
    const bool valid = i < n;
    const uint32_t d = valid ? digit_of(keys[i], pass) : 0xFFFFFFFFu;
    const unsigned m = __match_any_sync(0xffffffffu, d);
    if (valid && lane == __ffs(m) - 1) wcnt[warp][d] += __popc(m);
    __syncwarp();
  }
  __syncthreads();
  for (int d = threadIdx.x; d < kRadix; d += blockDim.x) {
    uint32_t s = 0;
#pragma unroll
    for (int w = 0; w < kSortThreads / 32; ++w) s += wcnt[w][d];
    block_hist[(size_t)d * gridDim.x + blockIdx.x] = s;
  }
}
__global__ void __launch_bounds__(kSortThreads)
k_radix_scatter(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ vals, size_t n, int pass,
                const unsigned long long* __restrict__ block_off /*[256][nblocks]: first output position of (digit, block)*/,
                uint64_t* __restrict__ out_keys, uint32_t* __restrict__ out_vals) {
  __shared__ unsigned long long woff[kSortThreads / 32][kRadix];
  __shared__ uint32_t wcnt[kSortThreads / 32][kRadix];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (kSortThreads / 32) * kRadix; i += blockDim.x) (&wcnt[0][0])[i] = 0;
  __syncthreads();
  const size_t base = (size_t)blockIdx.x * kSortTile + (size_t)warp * 32 * kSortItems;
  uint64_t k[kSortItems];
#pragma unroll
  for (int r = 0; r < kSortItems; ++r) {
    const size_t i = base + (size_t)r * 32 + lane;
    const bool valid = i < n;
    k[r] = valid ? keys[i] : 0ull;
    const uint32_t d = valid ? digit_of(k[r], pass) : 0xFFFFFFFFu;
    const unsigned m = __match_any_sync(0xffffffffu, d);
    if (valid && lane == __ffs(m) - 1) wcnt[warp][d] += __popc(m);
    __syncwarp();
  }
  __syncthreads();
  // start of every (warp, digit) run: digit base + keys of this digit in earlier blocks + in earlier warps
  for (int d = threadIdx.x; d < kRadix; d += blockDim.x) {
    unsigned long long run = block_off[(size_t)d * gridDim.x + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kSortThreads / 32; ++w) { woff[w][d] = run; run += wcnt[w][d]; }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kSortItems; ++r) {
    const size_t i = base + (size_t)r * 32 + lane;
    const bool valid = i < n;
    const uint32_t d = valid ? digit_of(k[r], pass) : 0xFFFFFFFFu;
    const unsigned m = __match_any_sync(0xffffffffu, d);
    if (valid) {
      const unsigned long long pos = woff[warp][d] + __popc(m & ((1u << lane) - 1u));
      out_keys[pos] = k[r];
      if (vals) out_vals[pos] = vals[i];
    }
    __syncwarp();
    if (valid && lane == __ffs(m) - 1) woff[warp][d] += __popc(m);
    __syncwarp();
  }
}
// ---------------------------------------------------------------- scan (uint64 in, exclusive) in three kernels
constexpr int kScanThreads = 256, kScanItems = 4, kScanTile = kScanThreads * kScanItems;
__global__ void __launch_bounds__(kScanThreads)
k_scan_tiles(const uint32_t* __restrict__ in, unsigned long long* __restrict__ out, size_t n, unsigned long long* __restrict__ tile_sum) {
  __shared__ unsigned long long sh[kScanThreads];
  const size_t base = (size_t)blockIdx.x * kScanTile + (size_t)threadIdx.x * kScanItems;
  unsigned long long v[kScanItems], s = 0;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) { v[j] = base + j < n ? in[base + j] : 0; s += v[j]; }
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int off = 1; off < kScanThreads; off <<= 1) {
    unsigned long long t = threadIdx.x >= off ? sh[threadIdx.x - off] : 0;
    __syncthreads();
    sh[threadIdx.x] += t;
    __syncthreads();
  }
  unsigned long long run = sh[threadIdx.x] - s;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) { if (base + j < n) out[base + j] = run; run += v[j]; }
  if (threadIdx.x == kScanThreads - 1) tile_sum[blockIdx.x] = sh[threadIdx.x];
}
// exclusive scan of the tile sums by one block of 1024 threads: every thread owns a contiguous run of tiles
__global__ void __launch_bounds__(1024)
k_scan_sums(unsigned long long* __restrict__ tile_sum, int ntiles, unsigned long long* __restrict__ total) {
  __shared__ unsigned long long sh[1024];
  const int per = (ntiles + 1023) / 1024;
  const int b = threadIdx.x * per, e = min(b + per, ntiles);
  unsigned long long s = 0;
  for (int i = b; i < e; ++i) s += tile_sum[i];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const unsigned long long t = threadIdx.x >= off ? sh[threadIdx.x - off] : 0;
    __syncthreads();
    sh[threadIdx.x] += t;
    __syncthreads();
  }
  unsigned long long run = sh[threadIdx.x] - s;
  for (int i = b; i < e; ++i) { const unsigned long long t = tile_sum[i]; tile_sum[i] = run; run += t; }
  if (threadIdx.x == 1023) *total = sh[1023];
}
__global__ void k_scan_add(unsigned long long* __restrict__ out, size_t n, const unsigned long long* __restrict__ tile_sum) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] += tile_sum[i / kScanTile];
}

// ---------------------------------------------------------------- unique with counts on sorted keys
__global__ void k_head_flags(const uint64_t* __restrict__ keys, size_t n, uint32_t* __restrict__ flag) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    flag[i] = (i == 0 || keys[i] != keys[i - 1]) ? 1u : 0u;
}
__global__ void k_write_unique(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ flag, const unsigned long long* __restrict__ pos,
                               size_t n, uint64_t* __restrict__ ukeys, unsigned long long* __restrict__ ustart) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    if (flag[i]) { ukeys[pos[i]] = keys[i]; ustart[pos[i]] = i; }
}
__global__ void k_counts_from_starts(const unsigned long long* __restrict__ ustart, size_t nu, size_t n, uint32_t* __restrict__ counts) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nu; i += (size_t)gridDim.x * blockDim.x)
    counts[i] = (uint32_t)((i + 1 < nu ? ustart[i + 1] : n) - ustart[i]);
}

// ---------------------------------------------------------------- remap through a sorted dictionary
__global__ void k_remap(const uint64_t* __restrict__ keys, size_t n, const uint64_t* __restrict__ dict, size_t m, uint32_t* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t k = keys[i];
    size_t lo = 0, hi = m;
    while (lo < hi) { const size_t mid = (lo + hi) >> 1; if (dict[mid] < k) lo = mid + 1; else hi = mid; }
    out[i] = (lo < m && dict[lo] == k) ? (uint32_t)lo : 0xFFFFFFFFu;
  }
}

// ---------------------------------------------------------------- bucketed scatter (transpose, partition)
__global__ void k_bucket_hist(const uint32_t* __restrict__ bucket, size_t n, uint32_t nb, uint32_t* __restrict__ hist) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t b = bucket[i];
    if (b < nb) atomicAdd(&hist[b], 1u);
  }
}
// destination of every element: start[bucket] + arrival order; dropped elements (bucket >= nb) get ~0
__global__ void k_bucket_dest(const uint32_t* __restrict__ bucket, size_t n, uint32_t nb, const unsigned long long* __restrict__ start,
                              uint32_t* __restrict__ cursor, unsigned long long* __restrict__ dest) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t b = bucket[i];
    dest[i] = b < nb ? start[b] + atomicAdd(&cursor[b], 1u) : ~0ull;
  }
}
__global__ void k_owner_of_keys(const uint64_t* __restrict__ keys, size_t n, KeySeps seps, uint32_t* __restrict__ bucket) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    bucket[i] = (uint32_t)route_owner(seps, keys[i]);
}

// ---------------------------------------------------------------- count-min sketch (uint32 saturating or uint8-wrapping counters)
__global__ void k_countmin_insert(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ counts, size_t n, uint32_t* __restrict__ table,
                                  uint32_t width, int k) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    cm_insert(table, width, k, keys[i], counts ? counts[i] : 1u);
}
__global__ void k_countmin_query(const uint64_t* __restrict__ keys, size_t n, const uint32_t* __restrict__ table, uint32_t width, int k,
                                 uint32_t wrap_mask, uint32_t* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = cm_query(table, width, k, keys[i], wrap_mask);
}

// ---------------------------------------------------------------- generic CSR products and init
// y = X·w (one warp per row); vals may be null (binary)
__global__ void k_spmv_csr(const int64_t* __restrict__ off, const uint32_t* __restrict__ idx, const float* __restrict__ vals,
                           const float* __restrict__ w, float* __restrict__ y, int64_t rows) {
  const int lane = threadIdx.x & 31;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += nw) {
    float s = 0.f;
    for (int64_t i = off[r] + lane; i < off[r + 1]; i += 32) s += w[idx[i]] * (vals ? vals[i] : 1.f);
    s = warp_sum(s);
    if (lane == 0) y[r] = s;
  }
}
// out = Xᵀ·v for CSC-by-segments storage of the same arrays: one warp per outer segment, no atomics
// (given the CSC arrays of X this computes Xᵀv; given the CSR arrays it computes X·w — same kernel shape)
__global__ void k_spmv_t_scatter(const int64_t* __restrict__ off, const uint32_t* __restrict__ idx, const float* __restrict__ vals,
                                 const float* __restrict__ v, float* __restrict__ out, int64_t rows) {
  const int lane = threadIdx.x & 31;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += nw) {
    const float vr = v[r];
    if (vr == 0.f) continue;
    for (int64_t i = off[r] + lane; i < off[r + 1]; i += 32) atomicAdd(&out[idx[i]], vr * (vals ? vals[i] : 1.f));
  }
}
__global__ void k_fill_gaussian(float* __restrict__ x, size_t n, float mean, float std, uint64_t seed) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t a = mix64(seed ^ (0x9E3779B97F4A7C15ull * (i + 1))), b = mix64(a + 0x632BE59BD9B4E019ull);
    const float u1 = ((float)(a >> 40) + 1.f) * (1.f / 16777217.f), u2 = (float)(b >> 40) * (1.f / 16777216.f);
    x[i] = mean + std * sqrtf(-2.f * __logf(u1)) * __cosf(6.2831853f * u2);
  }
}
__global__ void k_set_intersect_flags(const uint64_t* __restrict__ a, size_t na, const uint64_t* __restrict__ b, size_t nb, uint32_t* __restrict__ flag) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < na; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t k = a[i];
    size_t lo = 0, hi = nb;
    while (lo < hi) { const size_t mid = (lo + hi) >> 1; if (b[mid] < k) lo = mid + 1; else hi = mid; }
    flag[i] = (lo < nb && b[lo] == k) ? 1u : 0u;
  }
}
// Sorted union of two sorted key sets without a sort (SArray::setUnion, src/base/shared_array_inl.h:146-171),
// merge by ranking: an element of `a` lands at its own index plus the number of kept elements of `b` below it,
// a kept element of `b` (one that `a` lacks; `b_pos` = how many kept ones precede it) at b_pos plus the number
// of elements of `a` below it.  Every output position is written exactly once.
__global__ void k_merge_union(const uint64_t* __restrict__ a, size_t na, const uint64_t* __restrict__ b, size_t nb,
                              const uint32_t* __restrict__ b_dup, const unsigned long long* __restrict__ b_pos,
                              uint64_t* __restrict__ out) {
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < na + nb; t += (size_t)gridDim.x * blockDim.x) {
    if (t < na) {
      const uint64_t k = a[t];
      size_t lo = 0, hi = nb;
      while (lo < hi) { const size_t mid = (lo + hi) >> 1; if (b[mid] < k) lo = mid + 1; else hi = mid; }
      // kept elements of b below k = (elements of b below k) − (duplicates among them) = b_pos at lo, where
      // b_pos counts the kept ones before an index (b_pos[nb] is not stored: all of b is below k then)
      const size_t kept_below = lo < nb ? (size_t)b_pos[lo] : (nb ? (size_t)b_pos[nb - 1] + (b_dup[nb - 1] ? 0 : 1) : 0);
      out[t + kept_below] = k;
    } else {
      const size_t j = t - na;
      if (b_dup[j]) continue;
      const uint64_t k = b[j];
      size_t lo = 0, hi = na;
      while (lo < hi) { const size_t mid = (lo + hi) >> 1; if (a[mid] < k) lo = mid + 1; else hi = mid; }
      out[(size_t)b_pos[j] + lo] = k;
    }
  }
}
// flag[i] = 1 − in[i]  (elements of b that a lacks, from the intersection flags)
__global__ void k_invert_flags(const uint32_t* __restrict__ in, size_t n, uint32_t* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = in[i] ? 0u : 1u;
}
__global__ void k_compact_u64(const uint64_t* __restrict__ in, const uint32_t* __restrict__ flag, const unsigned long long* __restrict__ pos, size_t n,
                              uint64_t* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    if (flag[i]) out[pos[i]] = in[i];
}

}  // namespace psb

using namespace psb;

namespace {
inline int g1(size_t n, int cap = 148 * 8) { size_t b = (n + 255) / 256; if (b < 1) b = 1; if (b > (size_t)cap) b = cap; return (int)b; }
}

extern "C" {

size_t psb_sort_tile() { return kSortTile; }

// 8 byte-histograms of the keys (hist: 8*256 uint64, zeroed by the caller)
int psb_digit_histograms(const uint64_t* keys, size_t n, unsigned long long* hist, cudaStream_t s) {
  k_digit_histograms<<<g1(n, 148 * 4), 256, 0, s>>>(keys, n, hist);
  return (int)cudaGetLastError();
}
// one stable radix pass on byte `pass`.  Scratch: block_hist 256*nblocks uint32, block_off 256*nblocks uint64,
// tile_sum ceil(256*nblocks / psb_scan_tile()) uint64, total 1 uint64 (nblocks = ceil(n / psb_sort_tile())).
// vals / out_vals may be null.
int psb_radix_pass(const uint64_t* keys, const uint32_t* vals, size_t n, int pass, uint32_t* block_hist, unsigned long long* block_off,
                   unsigned long long* tile_sum, unsigned long long* total, uint64_t* out_keys, uint32_t* out_vals, cudaStream_t s) {
  if (n == 0) return 0;
  const int nblocks = (int)((n + kSortTile - 1) / kSortTile);
  k_radix_count<<<nblocks, kSortThreads, 0, s>>>(keys, n, pass, block_hist);
  // flattened digit-major exclusive scan: position of the first key of every (digit, block)
  const size_t m = (size_t)kRadix * nblocks;
  const int ntiles = (int)((m + kScanTile - 1) / kScanTile);
  k_scan_tiles<<<ntiles, kScanThreads, 0, s>>>(block_hist, block_off, m, tile_sum);
  k_scan_sums<<<1, 1024, 0, s>>>(tile_sum, ntiles, total);
  k_scan_add<<<(unsigned)((m + 255) / 256), 256, 0, s>>>(block_off, m, tile_sum);
  k_radix_scatter<<<nblocks, kSortThreads, 0, s>>>(keys, vals, n, pass, block_off, out_keys, out_vals);
  return (int)cudaGetLastError();
}
size_t psb_scan_tile() { return kScanTile; }
// exclusive scan of uint32 → uint64; tile_sum: ceil(n / psb_scan_tile()) uint64; total: 1 uint64
int psb_exclusive_scan_u32(const uint32_t* in, unsigned long long* out, size_t n, unsigned long long* tile_sum, unsigned long long* total,
                           cudaStream_t s) {
  const int ntiles = (int)((n + kScanTile - 1) / kScanTile);
  if (n == 0) { cudaMemsetAsync(total, 0, 8, s); return 0; }
  k_scan_tiles<<<ntiles, kScanThreads, 0, s>>>(in, out, n, tile_sum);
  k_scan_sums<<<1, 1024, 0, s>>>(tile_sum, ntiles, total);
  k_scan_add<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(out, n, tile_sum);
  return (int)cudaGetLastError();
}
int psb_head_flags(const uint64_t* keys, size_t n, uint32_t* flag, cudaStream_t s) {
  k_head_flags<<<g1(n), 256, 0, s>>>(keys, n, flag);
  return (int)cudaGetLastError();
}
int psb_write_unique(const uint64_t* keys, const uint32_t* flag, const unsigned long long* pos, size_t n, uint64_t* ukeys,
                     unsigned long long* ustart, cudaStream_t s) {
  k_write_unique<<<g1(n), 256, 0, s>>>(keys, flag, pos, n, ukeys, ustart);
  return (int)cudaGetLastError();
}
int psb_counts_from_starts(const unsigned long long* ustart, size_t nu, size_t n, uint32_t* counts, cudaStream_t s) {
  k_counts_from_starts<<<g1(nu), 256, 0, s>>>(ustart, nu, n, counts);
  return (int)cudaGetLastError();
}
int psb_remap(const uint64_t* keys, size_t n, const uint64_t* dict, size_t m, uint32_t* out, cudaStream_t s) {
  k_remap<<<g1(n), 256, 0, s>>>(keys, n, dict, m, out);
  return (int)cudaGetLastError();
}
int psb_bucket_hist(const uint32_t* bucket, size_t n, uint32_t nb, uint32_t* hist, cudaStream_t s) {
  k_bucket_hist<<<g1(n), 256, 0, s>>>(bucket, n, nb, hist);
  return (int)cudaGetLastError();
}
int psb_bucket_dest(const uint32_t* bucket, size_t n, uint32_t nb, const unsigned long long* start, uint32_t* cursor, unsigned long long* dest,
                    cudaStream_t s) {
  k_bucket_dest<<<g1(n), 256, 0, s>>>(bucket, n, nb, start, cursor, dest);
  return (int)cudaGetLastError();
}
int psb_owner_of_keys(const uint64_t* keys, size_t n, const KeySeps* seps, uint32_t* bucket, cudaStream_t s) {
  k_owner_of_keys<<<g1(n), 256, 0, s>>>(keys, n, *seps, bucket);
  return (int)cudaGetLastError();
}
int psb_countmin_insert(const uint64_t* keys, const uint32_t* counts, size_t n, uint32_t* table, uint32_t width, int k, cudaStream_t s) {
  k_countmin_insert<<<g1(n), 256, 0, s>>>(keys, counts, n, table, width, k);
  return (int)cudaGetLastError();
}
int psb_countmin_query(const uint64_t* keys, size_t n, const uint32_t* table, uint32_t width, int k, uint32_t wrap_mask, uint32_t* out,
                       cudaStream_t s) {
  k_countmin_query<<<g1(n), 256, 0, s>>>(keys, n, table, width, k, wrap_mask, out);
  return (int)cudaGetLastError();
}
int psb_spmv_csr(const int64_t* off, const uint32_t* idx, const float* vals, const float* w, float* y, int64_t rows, cudaStream_t s) {
  k_spmv_csr<<<g1((size_t)rows * 32), 256, 0, s>>>(off, idx, vals, w, y, rows);
  return (int)cudaGetLastError();
}
int psb_spmv_t(const int64_t* off, const uint32_t* idx, const float* vals, const float* v, float* out, int64_t rows, cudaStream_t s) {
  k_spmv_t_scatter<<<g1((size_t)rows * 32), 256, 0, s>>>(off, idx, vals, v, out, rows);
  return (int)cudaGetLastError();
}
int psb_fill_gaussian(float* x, size_t n, float mean, float std, uint64_t seed, cudaStream_t s) {
  k_fill_gaussian<<<g1(n), 256, 0, s>>>(x, n, mean, std, seed);
  return (int)cudaGetLastError();
}
int psb_set_intersect_flags(const uint64_t* a, size_t na, const uint64_t* b, size_t nb, uint32_t* flag, cudaStream_t s) {
  k_set_intersect_flags<<<g1(na), 256, 0, s>>>(a, na, b, nb, flag);
  return (int)cudaGetLastError();
}
int psb_merge_union(const uint64_t* a, size_t na, const uint64_t* b, size_t nb, const uint32_t* b_dup, const unsigned long long* b_pos,
                    uint64_t* out, cudaStream_t s) {
  k_merge_union<<<g1(na + nb), 256, 0, s>>>(a, na, b, nb, b_dup, b_pos, out);
  return (int)cudaGetLastError();
}
int psb_invert_flags(const uint32_t* in, size_t n, uint32_t* out, cudaStream_t s) {
  k_invert_flags<<<g1(n), 256, 0, s>>>(in, n, out);
  return (int)cudaGetLastError();
}
int psb_compact_u64(const uint64_t* in, const uint32_t* flag, const unsigned long long* pos, size_t n, uint64_t* out, cudaStream_t s) {
  k_compact_u64<<<g1(n), 256, 0, s>>>(in, flag, pos, n, out);
  return (int)cudaGetLastError();
}

}  // extern "C"
