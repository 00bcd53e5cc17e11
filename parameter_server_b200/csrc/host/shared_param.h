// The shared parameter of the batch solvers as a customer of the native runtime: it serves push and pull on a
// KVVector (server side) and collects pull replies (worker side) on its executor thread, without entering
// the interpreter.
//
// Counterpart in the reference: SharedParameter<K>::process (src/parameter/shared_parameter.h:90-149) over
// KVVector (src/parameter/kv_vector.h) and FreqencyFilter (src/parameter/frequency_filter.h).  A push is one of
//   * key counts for the tail-feature filter (flag kInsertKeyFreq): inserted into the count-min sketch, which is
//     sized by the first push: n = workers * keys * countmin_n_ratio / log(workers + 1);
//   * keys only: set union into the channel's key list;
//   * keys with values at a timestamp: merge-joined into this node's keys of the message's key range and summed
//     over the senders (the server-side aggregation of the workers' gradients).
// A pull with aux > 0 answers the keys whose sketch count exceeds aux, any other pull answers the values of the keys.
// The reference guards its maps by protocol order alone; here one mutex covers every access, from the executor
// thread and from the application threads that read what was aggregated and write the updated weights.
#pragma once
#include <cmath>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "kv.h"
#include "runtime.h"

namespace psb {

template <class Base = Customer>      // Base: Customer, or a subclass of it that a language binding adds methods to
class SharedParamCustomerT : public Base {
 public:
  using Base::key_ordered_slice;
  using Base::process;
  using Base::reply;
  static constexpr int kPush = 1, kPull = 2;
  static constexpr uint32_t kInsertKeyFreq = 1, kInsertKey = 2;

  SharedParamCustomerT(Postoffice* po, std::string name, int match_threads, int num_workers, int countmin_k, double countmin_n_ratio)
      : Base(po, std::move(name)), threads_(std::max(match_threads, 1)), workers_(std::max(num_workers, 1)), cm_k_(countmin_k),
        cm_ratio_(countmin_n_ratio) {
    key_ordered_slice = true;
    process = [this](const MessagePtr& m) { handle(m); };
  }

  // ---- application side (any thread)
  std::vector<Key> keys(int ch) { std::lock_guard<std::mutex> l(mu_); return kv_.key(ch); }
  std::vector<double> values(int ch) { std::lock_guard<std::mutex> l(mu_); return kv_.value(ch); }
  void set_values(int ch, const double* v, size_t n) { std::lock_guard<std::mutex> l(mu_); kv_.value(ch).assign(v, v + n); }
  void set_values_range(int ch, size_t lo, const double* v, size_t n) {
    std::lock_guard<std::mutex> l(mu_);
    auto& dst = kv_.value(ch);
    if ((lo + n) > dst.size()) throw std::out_of_range("shared parameter: value range outside the channel");
    std::copy(v, v + n, dst.begin() + lo);
  }
  void init_values(int ch, double init) { std::lock_guard<std::mutex> l(mu_); kv_.init_values(ch, init); }
  KVVector::Received received(int t) { std::lock_guard<std::mutex> l(mu_); return kv_.received(t); }
  void clear_filter() { std::lock_guard<std::mutex> l(mu_); filter_.clear(); }
  // replies of pull `t`, concatenated in the order of `servers` (= key order): (key bytes, value bytes)
  std::pair<std::string, std::string> take_pulled(int t, const std::vector<std::string>& servers) {
    std::map<std::string, std::pair<std::string, std::string>> parts;
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = pulled_.find(t);
      if (it != pulled_.end()) { parts.swap(it->second); pulled_.erase(it); }
    }
    std::pair<std::string, std::string> out;
    for (auto& s : servers) {
      auto it = parts.find(s);
      if (it == parts.end()) continue;
      out.first += it->second.first;
      out.second += it->second.second;
    }
    return out;
  }

 private:
  void handle(const MessagePtr& msg) {
    const Task& t = msg->task;
    const Key* keys = reinterpret_cast<const Key*>(msg->key.data());
    const size_t n = msg->key.size() / sizeof(Key);
    if (t.request && t.cmd == kPush) {
      std::lock_guard<std::mutex> l(mu_);
      if (t.flags & kInsertKeyFreq) {
        if (msg->value.empty() || msg->value[0].size() != n * sizeof(uint32_t)) return;
        if (filter_.empty()) {
          const double want = workers_ * (double)n * cm_ratio_ / std::log(workers_ + 1.0);
          filter_.resize((size_t)std::max(want, 64.0), cm_k_);
        }
        filter_.insert_keys(keys, reinterpret_cast<const uint32_t*>(msg->value[0].data()), n);
      } else if (msg->value.empty()) {
        kv_.merge_keys(t.key_channel, keys, n);
      } else {
        const std::string& v = msg->value[0];
        const size_t nd = v.size() / sizeof(double);
        const int nval = n ? (int)(nd / n) : 2;
        const Range r = t.has_key_range ? t.key_range : Range::all();
        kv_.aggregate(t.key_channel, t.time, r, keys, n, reinterpret_cast<const double*>(v.data()), nval, threads_);
      }
    } else if (t.request && t.cmd == kPull) {
      std::string rk, rv;
      {
        std::lock_guard<std::mutex> l(mu_);
        if (t.aux > 0) {
          auto kept = filter_.query_keys(keys, n, (uint32_t)t.aux);
          rk.assign(reinterpret_cast<const char*>(kept.data()), kept.size() * sizeof(Key));
        } else {
          auto vals = kv_.lookup(t.key_channel, keys, n);
          rv.assign(reinterpret_cast<const char*>(vals.data()), vals.size() * sizeof(double));
        }
      }
      reply(msg, std::move(rk), {std::move(rv)});
    } else if (!t.request && t.cmd == kPull) {
      std::lock_guard<std::mutex> l(mu_);
      pulled_[t.time][msg->sender] = {msg->key, msg->value.empty() ? std::string() : msg->value[0]};
    }
  }

  std::mutex mu_;
  KVVector kv_{1};
  FrequencyFilter filter_;
  std::map<int, std::map<std::string, std::pair<std::string, std::string>>> pulled_;
  int threads_, workers_, cm_k_;
  double cm_ratio_;
};

using SharedParamCustomer = SharedParamCustomerT<Customer>;

// The shared parameter of the online solver: the server keeps an FTRLModel (key -> {pos, neg, w, z}), a push
// carries (gradient, positive count, negative count) per key and is applied on arrival, a pull answers the
// current weights; key counts go through the tail-feature sketch like above, whose width is countmin_n divided
// over the servers.  Counterpart: FTRLModel as the store of SharedParameter (src/linear_method/ftrl_model.h
// :72-112, src/parameter/shared_parameter.h:90-149).
template <class Base = Customer>
class FTRLParamCustomerT : public Base {
 public:
  using Base::key_ordered_slice;
  using Base::process;
  using Base::reply;
  static constexpr int kPush = 1, kPull = 2;
  static constexpr uint32_t kInsertKeyFreq = 1;

  FTRLParamCustomerT(Postoffice* po, std::string name, double alpha, double beta, double lambda1, double lambda2, size_t sketch_width,
                     int countmin_k)
      : Base(po, std::move(name)), store_(alpha, beta, lambda1, lambda2), width_(std::max<size_t>(sketch_width, 64)), cm_k_(countmin_k) {
    key_ordered_slice = true;
    process = [this](const MessagePtr& m) { handle(m); };
  }
  // (|w|_1, |w|_2^2, non-zero weights) of this shard
  void stats(double* n1, double* n2, size_t* nnz) { std::lock_guard<std::mutex> l(mu_); *n1 = store_.norm1(); *n2 = store_.norm2(); *nnz = store_.nnz(); }
  void nonzero(std::vector<Key>* k, std::vector<double>* w) { std::lock_guard<std::mutex> l(mu_); store_.nonzero(k, w); }
  size_t size() { std::lock_guard<std::mutex> l(mu_); return store_.size(); }
  std::pair<std::string, std::string> take_pulled(int t, const std::vector<std::string>& servers) {
    std::map<std::string, std::pair<std::string, std::string>> parts;
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = pulled_.find(t);
      if (it != pulled_.end()) { parts.swap(it->second); pulled_.erase(it); }
    }
    std::pair<std::string, std::string> out;
    for (auto& s : servers) {
      auto it = parts.find(s);
      if (it == parts.end()) continue;
      out.first += it->second.first;
      out.second += it->second.second;
    }
    return out;
  }

 private:
  void handle(const MessagePtr& msg) {
    const Task& t = msg->task;
    const Key* keys = reinterpret_cast<const Key*>(msg->key.data());
    const size_t n = msg->key.size() / sizeof(Key);
    if (t.request && t.cmd == kPush) {
      std::lock_guard<std::mutex> l(mu_);
      if (t.flags & kInsertKeyFreq) {
        if (msg->value.empty() || msg->value[0].size() != n * sizeof(uint32_t)) return;
        if (filter_.empty()) filter_.resize(width_, cm_k_);
        filter_.insert_keys(keys, reinterpret_cast<const uint32_t*>(msg->value[0].data()), n);
      } else {
        if (msg->value.size() < 3) return;
        for (int i = 0; i < 3; ++i) if (msg->value[i].size() != n * sizeof(double)) return;
        store_.update(keys, n, reinterpret_cast<const double*>(msg->value[0].data()), reinterpret_cast<const double*>(msg->value[1].data()),
                      reinterpret_cast<const double*>(msg->value[2].data()));
      }
    } else if (t.request && t.cmd == kPull) {
      std::string rk, rv;
      {
        std::lock_guard<std::mutex> l(mu_);
        if (t.aux > 0) {
          auto kept = filter_.query_keys(keys, n, (uint32_t)t.aux);
          rk.assign(reinterpret_cast<const char*>(kept.data()), kept.size() * sizeof(Key));
        } else {
          auto w = store_.get(keys, n);
          rv.assign(reinterpret_cast<const char*>(w.data()), w.size() * sizeof(double));
        }
      }
      reply(msg, std::move(rk), {std::move(rv)});
    } else if (!t.request && t.cmd == kPull) {
      std::lock_guard<std::mutex> l(mu_);
      pulled_[t.time][msg->sender] = {msg->key, msg->value.empty() ? std::string() : msg->value[0]};
    }
  }

  std::mutex mu_;
  FTRLModel store_;
  FrequencyFilter filter_;
  std::map<int, std::map<std::string, std::pair<std::string, std::string>>> pulled_;
  size_t width_;
  int cm_k_;
};
using FTRLParamCustomer = FTRLParamCustomerT<Customer>;

}  // namespace psb
