// Host-side numeric containers of the parameter layer: count-min sketch and key-frequency
// filter, bitmap, histogram AUC, sorted-set operations and the per-channel key/value vector.
//
// Counterparts in the reference: src/base/countmin.h, src/parameter/frequency_filter.h,
// src/base/bitmap.h, src/base/auc.h, src/base/evaluation.h, src/base/shared_array_inl.h:146-171
// (setUnion/setIntersection/findRange), src/parameter/kv_vector.h.
#pragma once
#include <unordered_map>
#include <cmath>

#include "message.h"

namespace psb {

// k probes h, h+δ, h+2δ … (δ = rotr17(h)) into n counters; insert adds, query takes the minimum.
// Counters are uint8 and wrap like the reference's (frequency_filter.h:21,29) unless `saturate`.
class CountMin {
 public:
  void resize(size_t n, int k, bool saturate = false) { data_.assign(std::max<size_t>(n, 64), 0); k_ = std::max(k, 1); sat_ = saturate; }
  bool empty() const { return data_.empty(); }
  void clear() { data_.clear(); }
  static uint32_t hash(uint64_t key) {
    const uint32_t seed = 0xbc9f1d34u, m = 0xc6a4a793u;
    uint32_t h = seed ^ (8u * m);
    h += (uint32_t)key; h *= m; h ^= (h >> 16);
    h += (uint32_t)(key >> 32); h *= m; h ^= (h >> 16);
    return h;
  }
  void insert(uint64_t key, uint32_t count) {
    uint32_t h = hash(key);
    const uint32_t d = (h >> 17) | (h << 15);
    for (int j = 0; j < k_; ++j) {
      uint8_t& c = data_[h % data_.size()];
      const uint32_t v = (uint32_t)c + count;
      c = sat_ ? (uint8_t)std::min<uint32_t>(v, 255u) : (uint8_t)v;
      h += d;
    }
  }
  uint32_t query(uint64_t key) const {
    uint32_t h = hash(key), r = 0xFFFFFFFFu;
    const uint32_t d = (h >> 17) | (h << 15);
    for (int j = 0; j < k_; ++j) { r = std::min<uint32_t>(r, data_[h % data_.size()]); h += d; }
    return r;
  }
  size_t size() const { return data_.size(); }

 private:
  std::vector<uint8_t> data_;
  int k_ = 2;
  bool sat_ = false;
};

class FrequencyFilter {
 public:
  void resize(size_t n, int k) { cm_.resize(n, k); }
  bool empty() const { return cm_.empty(); }
  void clear() { cm_.clear(); }
  void insert_keys(const Key* keys, const uint32_t* counts, size_t n) { for (size_t i = 0; i < n; ++i) cm_.insert(keys[i], counts[i]); }
  // keys whose estimated count exceeds `freq`
  std::vector<Key> query_keys(const Key* keys, size_t n, uint32_t freq) const {
    std::vector<Key> out;
    for (size_t i = 0; i < n; ++i) if (cm_.query(keys[i]) > freq) out.push_back(keys[i]);
    return out;
  }

 private:
  CountMin cm_;
};

class Bitmap {
 public:
  explicit Bitmap(size_t n = 0, bool v = false) { resize(n, v); }
  void resize(size_t n, bool v = false) { n_ = n; w_.assign((n + 63) / 64, v ? ~0ull : 0ull); trim(); }
  void set(size_t i) { w_[i >> 6] |= 1ull << (i & 63); }
  void clear(size_t i) { w_[i >> 6] &= ~(1ull << (i & 63)); }
  bool test(size_t i) const { return (w_[i >> 6] >> (i & 63)) & 1ull; }
  void fill(bool v) { std::fill(w_.begin(), w_.end(), v ? ~0ull : 0ull); trim(); }
  size_t nnz() const { size_t c = 0; for (uint64_t x : w_) c += __builtin_popcountll(x); return c; }
  size_t size() const { return n_; }

 private:
  void trim() { if (n_ & 63 && !w_.empty()) w_.back() &= (1ull << (n_ & 63)) - 1; }
  size_t n_ = 0;
  std::vector<uint64_t> w_;
};

// Mergeable AUC: histograms of int64(pred·goodness) for positive and negative labels.
class AUC {
 public:
  void set_goodness(int64_t g) { goodness_ = g; }
  void add(const float* label, const float* pred, size_t n) {
    for (size_t i = 0; i < n; ++i) {
      const int64_t k = (int64_t)((double)pred[i] * (double)goodness_);
      if (label[i] > 0) ++tp_[k]; else ++fp_[k];
    }
  }
  void merge(const AUC& o) { for (auto& kv : o.tp_) tp_[kv.first] += kv.second; for (auto& kv : o.fp_) fp_[kv.first] += kv.second; }
  void merge(const std::vector<int64_t>& tk, const std::vector<uint64_t>& tc, const std::vector<int64_t>& fk, const std::vector<uint64_t>& fc) {
    for (size_t i = 0; i < tk.size(); ++i) tp_[tk[i]] += tc[i];
    for (size_t i = 0; i < fk.size(); ++i) fp_[fk[i]] += fc[i];
  }
  void clear() { tp_.clear(); fp_.clear(); }
  const std::map<int64_t, uint64_t>& tp() const { return tp_; }
  const std::map<int64_t, uint64_t>& fp() const { return fp_; }
  // area under the ROC curve by the trapezoid rule over the merged thresholds (descending score)
  double evaluate() const {
    double tp_sum = 0, fp_sum = 0, area = 0;
    auto it = tp_.rbegin();
    auto jt = fp_.rbegin();
    while (it != tp_.rend() || jt != fp_.rend()) {
      int64_t k;
      if (jt == fp_.rend() || (it != tp_.rend() && it->first >= jt->first)) k = it->first; else k = jt->first;
      double dtp = 0, dfp = 0;
      if (it != tp_.rend() && it->first == k) { dtp = (double)it->second; ++it; }
      if (jt != fp_.rend() && jt->first == k) { dfp = (double)jt->second; ++jt; }
      area += dfp * (tp_sum + dtp / 2);
      tp_sum += dtp; fp_sum += dfp;
    }
    return (tp_sum == 0 || fp_sum == 0) ? 0.5 : area / (tp_sum * fp_sum);
  }
  double accuracy(double threshold = 0) const {
    double ok = 0, all = 0;
    const int64_t th = (int64_t)(threshold * (double)goodness_);
    for (auto& kv : tp_) { all += kv.second; if (kv.first > th) ok += kv.second; }
    for (auto& kv : fp_) { all += kv.second; if (kv.first <= th) ok += kv.second; }
    return all > 0 ? ok / all : 0;
  }

 private:
  int64_t goodness_ = 100000;
  std::map<int64_t, uint64_t> tp_, fp_;
};

// exact AUC by sorting the scores (Evaluation<V>::auc)
inline double exact_auc(const float* label, const float* pred, size_t n) {
  std::vector<size_t> idx(n);
  for (size_t i = 0; i < n; ++i) idx[i] = i;
  std::sort(idx.begin(), idx.end(), [&](size_t a, size_t b) { return pred[a] < pred[b]; });
  // Mann-Whitney U statistic with average ranks for ties
  double npos = 0, rank = 1, sum_pos_rank = 0;
  size_t i = 0;
  while (i < n) {
    size_t j = i;
    while (j < n && pred[idx[j]] == pred[idx[i]]) ++j;
    const double avg = rank + (double)(j - i - 1) / 2.0;
    for (size_t k = i; k < j; ++k) if (label[idx[k]] > 0) { sum_pos_rank += avg; ++npos; }
    rank += (double)(j - i);
    i = j;
  }
  const double nneg = (double)n - npos;
  if (npos == 0 || nneg == 0) return 0.5;
  return (sum_pos_rank - npos * (npos + 1) / 2.0) / (npos * nneg);
}

inline std::vector<Key> set_union(const Key* a, size_t na, const Key* b, size_t nb) {
  std::vector<Key> out(na + nb);
  out.resize(std::set_union(a, a + na, b, b + nb, out.begin()) - out.begin());
  return out;
}
inline std::vector<Key> set_intersection(const Key* a, size_t na, const Key* b, size_t nb) {
  std::vector<Key> out(std::min(na, nb));
  out.resize(std::set_intersection(a, a + na, b, b + nb, out.begin()) - out.begin());
  return out;
}
// positions [lo, hi) of the keys falling into `r` in a sorted array
inline std::pair<size_t, size_t> find_range(const Key* k, size_t n, const Range& r) {
  return {(size_t)(std::lower_bound(k, k + n, r.begin) - k), (size_t)(std::lower_bound(k, k + n, r.end) - k)};
}

// Per-channel sorted unique keys with aligned double values (k values per key), plus the
// per-timestamp aggregation buffers of pushes received from several senders.
class KVVector {
 public:
  explicit KVVector(int k = 1) : k_(k) {}
  int k() const { return k_; }
  std::vector<Key>& key(int ch) { return key_[ch]; }
  std::vector<double>& value(int ch) { return val_[ch]; }
  void clear(int ch) { key_.erase(ch); val_.erase(ch); }
  // key-only push: set union into key(ch)
  void merge_keys(int ch, const Key* keys, size_t n) {
    auto& cur = key_[ch];
    cur = set_union(cur.data(), cur.size(), keys, n);
  }
  // size value(ch) to the keys, filled with `init`
  void init_values(int ch, double init = 0) { val_[ch].assign(key_[ch].size() * k_, init); }
  // push with values at timestamp t over `range`: merge-join into this node's keys of the range and SUM into the
  // aggregation buffer of t (this is the server-side gradient aggregation across workers)
  size_t aggregate(int ch, int t, const Range& range, const Key* keys, size_t n, const double* vals, int nval, int threads = 1) {
    auto& mine = key_[ch];
    auto seg = find_range(mine.data(), mine.size(), range);
    auto& buf = recved_[t];
    if (buf.vals.empty()) {
      buf.lo = seg.first; buf.hi = seg.second; buf.nval = nval;
      buf.vals.assign((seg.second - seg.first) * (size_t)nval, 0.0);
    }
    return parallel_match_sorted(mine.data() + buf.lo, buf.hi - buf.lo, buf.vals.data(), keys, n, vals, (size_t)nval, MatchOp::ADD, threads);
  }
  struct Received { size_t lo = 0, hi = 0; int nval = 0; std::vector<double> vals; };
  Received received(int t) {
    Received r;
    auto it = recved_.find(t);
    if (it != recved_.end()) { r = std::move(it->second); recved_.erase(it); }
    return r;
  }
  // pull: values of the requested keys (0 for unknown keys)
  std::vector<double> lookup(int ch, const Key* keys, size_t n) {
    std::vector<double> out(n * k_, 0.0);
    auto& mine = key_[ch];
    auto& v = val_[ch];
    if (!v.empty()) match_sorted(keys, n, out.data(), mine.data(), mine.size(), v.data(), (size_t)k_, MatchOp::ASSIGN);
    return out;
  }
  std::pair<size_t, size_t> find(int ch, const Range& r) { auto& m = key_[ch]; return find_range(m.data(), m.size(), r); }

 private:
  int k_;
  std::map<int, std::vector<Key>> key_;
  std::map<int, std::vector<double>> val_;
  std::map<int, Received> recved_;
};

// Open-addressing hash map from 64-bit keys to small records (linear probing, power-of-two capacity, grows at
// 60 % load; no erase).  The host form of the hash-map store that the reference only declares (KVMap,
// src/parameter/kv_map.h); the online solver's model lives in it: one cache line per probe instead of the
// node allocation and pointer chase of std::unordered_map.
template <typename V>
class KeyMap {
 public:
  explicit KeyMap(size_t capacity = 1024) { rehash(capacity); }
  size_t size() const { return size_; }
  V& operator[](Key k) {
    if ((size_ + 1) * 5 > slots_.size() * 3) rehash(slots_.size() * 2);
    size_t i = index(k);
    while (used_[i] && slots_[i].first != k) i = (i + 1) & mask_;
    if (!used_[i]) { used_[i] = 1; slots_[i].first = k; slots_[i].second = V(); ++size_; }
    return slots_[i].second;
  }
  const V* find(Key k) const {
    size_t i = index(k);
    while (used_[i]) {
      if (slots_[i].first == k) return &slots_[i].second;
      i = (i + 1) & mask_;
    }
    return nullptr;
  }
  template <typename F> void for_each(F f) const {
    for (size_t i = 0; i < slots_.size(); ++i) if (used_[i]) f(slots_[i].first, slots_[i].second);
  }

 private:
  size_t index(Key k) const {                 // Fibonacci hashing: the top bits of k * 2^64 / phi
    return (size_t)((k * 0x9E3779B97F4A7C15ull) >> shift_) & mask_;
  }
  void rehash(size_t want) {
    size_t cap = 16;
    int bits = 4;
    while (cap < want) { cap <<= 1; ++bits; }
    std::vector<std::pair<Key, V>> old_slots;
    std::vector<uint8_t> old_used;
    old_slots.swap(slots_);
    old_used.swap(used_);
    slots_.assign(cap, std::pair<Key, V>());
    used_.assign(cap, 0);
    mask_ = cap - 1;
    shift_ = 64 - bits;
    size_ = 0;
    for (size_t i = 0; i < old_slots.size(); ++i) if (old_used[i]) (*this)[old_slots[i].first] = old_slots[i].second;
  }
  std::vector<std::pair<Key, V>> slots_;
  std::vector<uint8_t> used_;
  size_t mask_ = 0, size_ = 0;
  int shift_ = 60;
};

// Server-side state of the online solver on CPU nodes: key -> {pos, neg, w, z} with the per-key
// FTRL-proximal update and the count-based estimate of the gradient norm, plus running |w|_1, |w|_2^2
// and nnz(w) (FTRLModel::setValue / getValue / objv, src/linear_method/ftrl_model.h:60-127).
class FTRLModel {
 public:
  struct Entry { double pos = 0, neg = 0, w = 0, z = 0; };
  FTRLModel(double alpha, double beta, double lambda1, double lambda2) : alpha_(alpha), beta_(beta), l1_(lambda1), l2_(lambda2) {}
  static double sqrt_n(double pos, double neg) {
    const double all = pos + neg;
    return all == 0 ? 0 : std::sqrt(pos * neg / all);
  }
  void update(const Key* keys, size_t n, const double* grad, const double* pos, const double* neg) {
    for (size_t i = 0; i < n; ++i) {
      Entry& e = model_[keys[i]];
      const double sq = sqrt_n(e.pos, e.neg);
      e.pos += pos[i];
      e.neg += neg[i];
      const double sq_new = sqrt_n(e.pos, e.neg);
      const double sigma = (sq_new - sq) / alpha_;
      e.z += grad[i] - sigma * e.w;
      const double l2 = l2_ + (beta_ + sq_new) / alpha_;
      const double w_old = e.w, az = std::fabs(e.z) - l1_;
      e.w = az > 0 ? -std::copysign(az, e.z) / l2 : 0.0;
      norm1_ += std::fabs(e.w) - std::fabs(w_old);
      norm2_ += e.w * e.w - w_old * w_old;
      nnz_ += (e.w != 0 && w_old == 0) - (e.w == 0 && w_old != 0);
    }
  }
  std::vector<double> get(const Key* keys, size_t n) const {
    std::vector<double> out(n, 0.0);
    for (size_t i = 0; i < n; ++i) {
      const Entry* e = model_.find(keys[i]);
      if (e) out[i] = e->w;
    }
    return out;
  }
  double norm1() const { return norm1_; }
  double norm2() const { return norm2_; }
  long long nnz() const { return nnz_; }
  size_t size() const { return model_.size(); }
  // non-zero weights in ascending key order
  void nonzero(std::vector<Key>* keys, std::vector<double>* w) const {
    std::vector<std::pair<Key, double>> v;
    model_.for_each([&](Key k, const Entry& e) { if (e.w != 0) v.emplace_back(k, e.w); });
    std::sort(v.begin(), v.end());
    keys->clear(); w->clear();
    for (auto& p : v) { keys->push_back(p.first); w->push_back(p.second); }
  }

 private:
  double alpha_, beta_, l1_, l2_;
  double norm1_ = 0, norm2_ = 0;
  long long nnz_ = 0;
  KeyMap<Entry> model_;
};

inline double soft_thresholding(double x, double l1, double l2) {
  // argmin_y x·y + ½ l2 y² + l1 |y|   (src/base/soft_thresholding.h:7-13)
  if (x > l1) return -(x - l1) / l2;
  if (x < -l1) return -(x + l1) / l2;
  return 0;
}

}  // namespace psb
