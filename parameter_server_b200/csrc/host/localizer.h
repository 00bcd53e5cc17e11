// Host-side localisation of sparse data: global 64-bit feature ids -> dense local column ids, and the
// row-major <-> column-major change of storage.
//
// Counterparts in the reference: Localizer::countUniqIndex (src/base/localizer.h:50-87: sort (key, position)
// pairs, unique keys with their counts), Localizer::remapIndex (:110-168: merge-join against a sorted
// dictionary, unknown keys dropped, row offsets rebuilt), SparseMatrix::alterStorage (src/base/sparse_matrix.h
// :186-241: threaded counting sort between CSR and CSC).  Here the unique keys come from a threaded sort of a
// copy of the ids and a run-length pass; ids are mapped by a binary search per non-zero, spread over threads;
// the storage change is a counting sort whose scatter runs per row range with per-thread column cursors, so
// that rows stay in ascending order inside every column without any atomic.
#pragma once
#include <algorithm>
#include <cstdint>
#include <functional>
#include <thread>
#include <vector>

#include "util.h"

namespace psb {

// Sorted unique keys of `keys` and how often each occurs.
inline void count_unique(const uint64_t* keys, size_t n, int threads, std::vector<uint64_t>* uniq, std::vector<uint32_t>* count) {
  std::vector<uint64_t> s(keys, keys + n);
  parallel_sort(s.begin(), s.end(), std::max(threads, 1), std::less<uint64_t>());
  uniq->clear();
  count->clear();
  for (size_t i = 0; i < n;) {
    size_t j = i + 1;
    while (j < n && s[j] == s[i]) ++j;
    uniq->push_back(s[i]);
    count->push_back((uint32_t)std::min<size_t>(j - i, 0xffffffffu));
    i = j;
  }
}

// Unique keys, their counts and the local id of every input position in one go: an LSD radix sort of
// (key, position) pairs, 16 bits per pass, passes whose digit is the same for every key skipped, then one
// run-length pass that hands out the ids (the reference sorts the pairs by comparison, localizer.h:50-87).
inline void localize(const uint64_t* keys, size_t n, std::vector<uint64_t>* uniq, std::vector<uint32_t>* count, int32_t* local) {
  std::vector<std::pair<uint64_t, uint32_t>> a(n), b(n);
  uint64_t all_or = 0, all_and = ~0ull;
  for (size_t i = 0; i < n; ++i) { a[i] = {keys[i], (uint32_t)i}; all_or |= keys[i]; all_and &= keys[i]; }
  std::vector<size_t> hist(1 << 16);
  for (int pass = 0; pass < 4; ++pass) {
    const int sh = 16 * pass;
    if ((((all_or ^ all_and) >> sh) & 0xffff) == 0) continue;       // every key has the same digit here
    std::fill(hist.begin(), hist.end(), 0);
    for (size_t i = 0; i < n; ++i) ++hist[(a[i].first >> sh) & 0xffff];
    size_t run = 0;
    for (auto& h : hist) { const size_t c = h; h = run; run += c; }
    for (size_t i = 0; i < n; ++i) b[hist[(a[i].first >> sh) & 0xffff]++] = a[i];
    a.swap(b);
  }
  uniq->clear();
  count->clear();
  for (size_t i = 0; i < n;) {
    size_t j = i;
    const int32_t id = (int32_t)uniq->size();
    while (j < n && a[j].first == a[i].first) { local[a[j].second] = id; ++j; }
    uniq->push_back(a[i].first);
    count->push_back((uint32_t)std::min<size_t>(j - i, 0xffffffffu));
    i = j;
  }
}

template <typename F>
inline void parallel_ranges(size_t n, int threads, size_t min_per_thread, F f) {
  const int t = (int)std::max<size_t>(1, std::min<size_t>((size_t)std::max(threads, 1), n / std::max<size_t>(min_per_thread, 1)));
  if (t <= 1) { f(0, (size_t)0, n); return; }
  std::vector<std::thread> pool;
  for (int i = 0; i < t; ++i) pool.emplace_back(f, i, n * i / t, n * (i + 1) / t);
  for (auto& th : pool) th.join();
}

// Local id (position in the sorted dictionary) of every key, -1 for keys the dictionary lacks.
inline void remap_keys(const uint64_t* keys, size_t n, const uint64_t* dict, size_t m, int threads, int32_t* out) {
  parallel_ranges(n, threads, 1 << 14, [&](int, size_t a, size_t b) {
    for (size_t i = a; i < b; ++i) {
      const uint64_t* p = std::lower_bound(dict, dict + m, keys[i]);
      out[i] = (p != dict + m && *p == keys[i]) ? (int32_t)(p - dict) : -1;
    }
  });
}

// Row-major (offsets per row, local column id per non-zero, -1 = dropped) to column-major.  vals may be null.
// indptr gets cols + 1 entries; rows / out_vals get one entry per kept non-zero.  Returns the kept count.
inline size_t csr_to_csc(const int64_t* offsets, size_t rows, const int32_t* col, const double* vals, size_t cols, int threads,
                         std::vector<int64_t>* indptr, std::vector<int32_t>* out_rows, std::vector<double>* out_vals) {
  const size_t nnz = (size_t)offsets[rows];
  int T = (int)std::max<size_t>(1, std::min<size_t>((size_t)std::max(threads, 1), rows / 1024 + 1));
  while (T > 1 && (size_t)T * cols > 4 * nnz + (1u << 20)) --T;     // the per-thread column counters must stay small beside the data
  // per-thread histogram of its row range, then cursors: column-major position = column start + what earlier
  // row ranges put into the column
  std::vector<std::vector<int64_t>> cnt(T, std::vector<int64_t>(cols, 0));
  auto rows_of = [&](int t) { return std::make_pair(rows * t / T, rows * (t + 1) / T); };
  {
    std::vector<std::thread> pool;
    for (int t = 0; t < T; ++t) pool.emplace_back([&, t] {
      auto r = rows_of(t);
      for (int64_t p = offsets[r.first]; p < offsets[r.second]; ++p) if (col[p] >= 0) ++cnt[t][col[p]];
    });
    for (auto& th : pool) th.join();
  }
  indptr->assign(cols + 1, 0);
  for (size_t c = 0; c < cols; ++c) {
    int64_t run = (*indptr)[c];
    for (int t = 0; t < T; ++t) { const int64_t k = cnt[t][c]; cnt[t][c] = run; run += k; }
    (*indptr)[c + 1] = run;
  }
  const size_t kept = (size_t)(*indptr)[cols];
  out_rows->resize(kept);
  if (vals) out_vals->resize(kept); else out_vals->clear();
  {
    std::vector<std::thread> pool;
    for (int t = 0; t < T; ++t) pool.emplace_back([&, t] {
      auto r = rows_of(t);
      auto& cur = cnt[t];
      for (size_t i = r.first; i < r.second; ++i)
        for (int64_t p = offsets[i]; p < offsets[i + 1]; ++p) {
          if (col[p] < 0) continue;
          const int64_t q = cur[col[p]]++;
          (*out_rows)[q] = (int32_t)i;
          if (vals) (*out_vals)[q] = vals[p];
        }
    });
    for (auto& th : pool) th.join();
  }
  return kept;
}

}  // namespace psb
