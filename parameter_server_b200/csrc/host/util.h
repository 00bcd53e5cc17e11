// Host utilities of the runtime: hashing (crc32c, MurmurHash3 x64-128, DJB), timers, process
// resource usage, thread pool, blocking queues/maps, parallel sort, k-way key/value partition,
// record IO and (gz) file access.
//
// Counterparts in the reference: src/util/crc32c.{h,cc}, MurmurHash3.{h,cc}, common.h (DJBHash32),
// resource_usage.h, threadpool.{h,cc}, threadsafe_queue.h, threadsafe_limited_queue.h,
// threadsafe_limited_set.h, threadsafe_map.h, parallel_sort.h, kv_partition.h, recordio.h,
// file.{h,cc}, filelinereader.{h,cc}, status.h.
#pragma once
#include <arpa/inet.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <zlib.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <fstream>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace psb {

using Key = uint64_t;
constexpr Key kMaxKey = 0xFFFFFFFFFFFFFFFFull;

// ------------------------------------------------------------------ Status
class Status {
 public:
  enum Code { kOk = 0, kNotFound, kInvalidArgument, kIOError, kNetError, kTimeout };
  Status() = default;
  Status(Code c, std::string m) : code_(c), msg_(std::move(m)) {}
  static Status OK() { return Status(); }
  static Status NotFound(const std::string& m) { return Status(kNotFound, m); }
  static Status InvalidArgument(const std::string& m) { return Status(kInvalidArgument, m); }
  static Status IOError(const std::string& m) { return Status(kIOError, m); }
  static Status NetError(const std::string& m) { return Status(kNetError, m); }
  static Status Timeout(const std::string& m) { return Status(kTimeout, m); }
  bool ok() const { return code_ == kOk; }
  Code code() const { return code_; }
  std::string ToString() const {
    static const char* names[] = {"OK", "NotFound", "InvalidArgument", "IOError", "NetError", "Timeout"};
    return ok() ? "OK" : std::string(names[code_]) + ": " + msg_;
  }

 private:
  Code code_ = kOk;
  std::string msg_;
};

// ------------------------------------------------------------------ hashing
// CRC-32C (Castagnoli, reflected polynomial 0x82F63B78), slice-by-1 table built on first use.
inline uint32_t crc32c_extend(uint32_t crc, const char* data, size_t n) {
  static uint32_t table[256];
  static std::once_flag once;
  std::call_once(once, [] {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : c >> 1;
      table[i] = c;
    }
  });
  uint32_t c = crc ^ 0xFFFFFFFFu;
  const unsigned char* p = reinterpret_cast<const unsigned char*>(data);
  for (size_t i = 0; i < n; ++i) c = table[(c ^ p[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}
inline uint32_t crc32c_value(const char* data, size_t n) { return crc32c_extend(0, data, n); }
inline uint32_t crc32c_mask(uint32_t crc) { return ((crc >> 15) | (crc << 17)) + 0xa282ead8u; }
inline uint32_t crc32c_unmask(uint32_t m) { uint32_t r = m - 0xa282ead8u; return (r >> 17) | (r << 15); }

inline uint64_t rotl64(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
inline uint64_t fmix64(uint64_t k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdull; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ull; k ^= k >> 33;
  return k;
}
// MurmurHash3_x64_128 (Austin Appleby's public-domain algorithm)
inline void murmur3_x64_128(const void* key, int len, uint32_t seed, uint64_t out[2]) {
  const uint8_t* data = static_cast<const uint8_t*>(key);
  const int nblocks = len / 16;
  uint64_t h1 = seed, h2 = seed;
  const uint64_t c1 = 0x87c37b91114253d5ull, c2 = 0x4cf5ad432745937full;
  for (int i = 0; i < nblocks; ++i) {
    uint64_t k1, k2;
    std::memcpy(&k1, data + i * 16, 8);
    std::memcpy(&k2, data + i * 16 + 8, 8);
    k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
    h1 = rotl64(h1, 27); h1 += h2; h1 = h1 * 5 + 0x52dce729;
    k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2;
    h2 = rotl64(h2, 31); h2 += h1; h2 = h2 * 5 + 0x38495ab5;
  }
  const uint8_t* tail = data + nblocks * 16;
  uint64_t k1 = 0, k2 = 0;
  switch (len & 15) {
    case 15: k2 ^= uint64_t(tail[14]) << 48; [[fallthrough]];
    case 14: k2 ^= uint64_t(tail[13]) << 40; [[fallthrough]];
    case 13: k2 ^= uint64_t(tail[12]) << 32; [[fallthrough]];
    case 12: k2 ^= uint64_t(tail[11]) << 24; [[fallthrough]];
    case 11: k2 ^= uint64_t(tail[10]) << 16; [[fallthrough]];
    case 10: k2 ^= uint64_t(tail[9]) << 8; [[fallthrough]];
    case 9: k2 ^= uint64_t(tail[8]);
      k2 *= c2; k2 = rotl64(k2, 33); k2 *= c1; h2 ^= k2; [[fallthrough]];
    case 8: k1 ^= uint64_t(tail[7]) << 56; [[fallthrough]];
    case 7: k1 ^= uint64_t(tail[6]) << 48; [[fallthrough]];
    case 6: k1 ^= uint64_t(tail[5]) << 40; [[fallthrough]];
    case 5: k1 ^= uint64_t(tail[4]) << 32; [[fallthrough]];
    case 4: k1 ^= uint64_t(tail[3]) << 24; [[fallthrough]];
    case 3: k1 ^= uint64_t(tail[2]) << 16; [[fallthrough]];
    case 2: k1 ^= uint64_t(tail[1]) << 8; [[fallthrough]];
    case 1: k1 ^= uint64_t(tail[0]);
      k1 *= c1; k1 = rotl64(k1, 31); k1 *= c2; h1 ^= k1;
  }
  h1 ^= (uint64_t)len; h2 ^= (uint64_t)len;
  h1 += h2; h2 += h1;
  h1 = fmix64(h1); h2 = fmix64(h2);
  h1 += h2; h2 += h1;
  out[0] = h1; out[1] = h2;
}
// feature-id shuffle used by the TERAFEA parser (src/data/example_parser.cc:205-209)
inline uint64_t shuffle_feature_id(uint64_t id) {
  uint64_t h[2];
  murmur3_x64_128(&id, 8, 512927377u, h);
  return h[0] ^ h[1];
}
inline uint32_t djb_hash32(const std::string& s) {
  uint32_t h = 5381;
  for (unsigned char c : s) h = ((h << 5) + h) + c;
  return h;
}

// ------------------------------------------------------------------ time / resources
inline double now_seconds() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
class Timer {
 public:
  void start() { t0_ = now_seconds(); running_ = true; }
  double stop() { if (running_) { total_ += now_seconds() - t0_; running_ = false; } return total_; }
  void restart() { total_ = 0; start(); }
  void reset() { total_ = 0; running_ = false; }
  double get() const { return total_ + (running_ ? now_seconds() - t0_ : 0.0); }

 private:
  double t0_ = 0, total_ = 0;
  bool running_ = false;
};
struct ResUsage {
  // resident / virtual memory of this process in MB, from /proc/self/statm
  static void memory_mb(double* rss, double* virt) {
    *rss = *virt = 0;
    std::ifstream f("/proc/self/statm");
    uint64_t v = 0, r = 0;
    if (f >> v >> r) { *virt = v * 4096.0 / 1e6; *rss = r * 4096.0 / 1e6; }
  }
  // user+system jiffies of this process and of the host, from /proc/self/stat and /proc/stat
  static void cpu_jiffies(uint64_t* proc, uint64_t* host) {
    *proc = *host = 0;
    std::ifstream f("/proc/self/stat");
    std::string tok;
    for (int i = 1; f >> tok; ++i) {
      if (i == 14 || i == 15) *proc += std::strtoull(tok.c_str(), nullptr, 10);
      if (i > 15) break;
    }
    std::ifstream h("/proc/stat");
    std::string cpu;
    h >> cpu;
    for (int i = 0; i < 8; ++i) { uint64_t v = 0; if (h >> v) *host += (i == 3 || i == 4) ? 0 : v; }
  }
  // total received / transmitted bytes over all interfaces, from /proc/net/dev
  static void net_bytes(uint64_t* in, uint64_t* out) {
    *in = *out = 0;
    std::ifstream f("/proc/net/dev");
    std::string line;
    while (std::getline(f, line)) {
      auto c = line.find(':');
      if (c == std::string::npos) continue;
      std::istringstream is(line.substr(c + 1));
      uint64_t v[16] = {0};
      for (int i = 0; i < 16 && (is >> v[i]); ++i) {}
      *in += v[0]; *out += v[8];
    }
  }
};

// ------------------------------------------------------------------ concurrency
class Barrier {
 public:
  explicit Barrier(int n) : n_(n) {}
  bool wait() {
    std::unique_lock<std::mutex> l(mu_);
    int gen = gen_;
    if (++count_ == n_) { count_ = 0; ++gen_; cv_.notify_all(); return true; }
    cv_.wait(l, [&] { return gen != gen_; });
    return false;
  }

 private:
  std::mutex mu_; std::condition_variable cv_; int n_, count_ = 0, gen_ = 0;
};

// Tasks are queued with add() and run by `n` threads after start(); the destructor (or join())
// waits for completion — the semantics of the reference's ThreadPool.
class ThreadPool {
 public:
  explicit ThreadPool(int n) : n_(std::max(n, 1)) {}
  ~ThreadPool() { join(); }
  void add(std::function<void()> f) { std::lock_guard<std::mutex> l(mu_); tasks_.push_back(std::move(f)); }
  void start() {
    started_ = true;
    for (int i = 0; i < n_; ++i) threads_.emplace_back([this] {
      for (;;) {
        std::function<void()> f;
        { std::lock_guard<std::mutex> l(mu_); if (tasks_.empty()) return; f = std::move(tasks_.front()); tasks_.pop_front(); }
        f();
      }
    });
  }
  void join() { if (!started_) start(); for (auto& t : threads_) if (t.joinable()) t.join(); threads_.clear(); }

 private:
  int n_; bool started_ = false;
  std::mutex mu_; std::deque<std::function<void()>> tasks_; std::vector<std::thread> threads_;
};

template <typename T>
class ThreadsafeQueue {
 public:
  void push(T v) { { std::lock_guard<std::mutex> l(mu_); q_.push_back(std::move(v)); } cv_.notify_one(); }
  void wait_and_pop(T& v) {
    std::unique_lock<std::mutex> l(mu_);
    cv_.wait(l, [&] { return !q_.empty(); });
    v = std::move(q_.front()); q_.pop_front();
  }
  bool wait_and_pop_for(T& v, double seconds) {
    std::unique_lock<std::mutex> l(mu_);
    if (!cv_.wait_for(l, std::chrono::duration<double>(seconds), [&] { return !q_.empty(); })) return false;
    v = std::move(q_.front()); q_.pop_front();
    return true;
  }
  bool try_pop(T& v) {
    std::lock_guard<std::mutex> l(mu_);
    if (q_.empty()) return false;
    v = std::move(q_.front()); q_.pop_front();
    return true;
  }
  size_t size() const { std::lock_guard<std::mutex> l(mu_); return q_.size(); }
  bool empty() const { return size() == 0; }

 private:
  mutable std::mutex mu_; std::condition_variable cv_; std::deque<T> q_;
};

// Queue bounded by the total *capacity units* (e.g. bytes) of the queued items; producers block
// while full; setFinished() lets consumers drain and then return false.
template <typename T>
class ThreadsafeLimitedQueue {
 public:
  explicit ThreadsafeLimitedQueue(size_t capacity = 0) : cap_(capacity) {}
  void set_capacity(size_t c) { cap_ = c; }
  void push(T v, size_t cost, bool finished = false) {
    std::unique_lock<std::mutex> l(mu_);
    full_.wait(l, [&] { return cur_ == 0 || cur_ + cost <= cap_; });
    q_.emplace_back(std::move(v), cost); cur_ += cost; done_ = done_ || finished;
    empty_.notify_all();
  }
  void set_finished() { std::lock_guard<std::mutex> l(mu_); done_ = true; empty_.notify_all(); }
  bool pop(T& v) {
    std::unique_lock<std::mutex> l(mu_);
    empty_.wait(l, [&] { return !q_.empty() || done_; });
    if (q_.empty()) return false;
    v = std::move(q_.front().first); cur_ -= q_.front().second; q_.pop_front();
    full_.notify_all();
    return true;
  }
  size_t size() const { std::lock_guard<std::mutex> l(mu_); return q_.size(); }

 private:
  mutable std::mutex mu_; std::condition_variable full_, empty_;
  std::deque<std::pair<T, size_t>> q_; size_t cap_, cur_ = 0; bool done_ = false;
};

// Set bounded by total cost; insert blocks (up to a deadline) while full.  Used as the memory
// allowance of prefetch jobs.
template <typename T>
class ThreadsafeLimitedSet {
 public:
  explicit ThreadsafeLimitedSet(size_t capacity = 0) : cap_(capacity) {}
  void set_capacity(size_t c) { cap_ = c; }
  bool insert(const T& v, size_t cost, double timeout_s = 1e9) {
    std::unique_lock<std::mutex> l(mu_);
    if (items_.count(v)) return true;
    if (!cv_.wait_for(l, std::chrono::duration<double>(timeout_s), [&] { return cur_ == 0 || cur_ + cost <= cap_; })) return false;
    items_[v] = cost; cur_ += cost;
    return true;
  }
  void erase(const T& v) {
    std::lock_guard<std::mutex> l(mu_);
    auto it = items_.find(v);
    if (it != items_.end()) { cur_ -= it->second; items_.erase(it); cv_.notify_all(); }
  }
  bool contains(const T& v) const { std::lock_guard<std::mutex> l(mu_); return items_.count(v) > 0; }
  size_t cost() const { std::lock_guard<std::mutex> l(mu_); return cur_; }

 private:
  mutable std::mutex mu_; std::condition_variable cv_; std::map<T, size_t> items_; size_t cap_, cur_ = 0;
};

template <typename K, typename V>
class ThreadsafeMap {
 public:
  void insert(const K& k, V v) { { std::lock_guard<std::mutex> l(mu_); m_[k] = std::move(v); } cv_.notify_all(); }
  bool try_get(const K& k, V& v) const { std::lock_guard<std::mutex> l(mu_); auto it = m_.find(k); if (it == m_.end()) return false; v = it->second; return true; }
  bool wait_and_get(const K& k, V& v, double timeout_s = 1e9) {
    std::unique_lock<std::mutex> l(mu_);
    if (!cv_.wait_for(l, std::chrono::duration<double>(timeout_s), [&] { return m_.count(k) > 0; })) return false;
    v = m_[k]; return true;
  }
  bool wait_and_pop(const K& k, V& v, double timeout_s = 1e9) {
    std::unique_lock<std::mutex> l(mu_);
    if (!cv_.wait_for(l, std::chrono::duration<double>(timeout_s), [&] { return m_.count(k) > 0; })) return false;
    v = std::move(m_[k]); m_.erase(k); return true;
  }
  void erase(const K& k) { std::lock_guard<std::mutex> l(mu_); m_.erase(k); }
  size_t size() const { std::lock_guard<std::mutex> l(mu_); return m_.size(); }

 private:
  mutable std::mutex mu_; std::condition_variable cv_; std::map<K, V> m_;
};

// recursive split + inplace_merge over up to `threads` threads
template <typename It, typename Cmp>
void parallel_sort(It b, It e, int threads, Cmp cmp) {
  const size_t n = e - b;
  if (threads <= 1 || n < (1u << 14)) { std::sort(b, e, cmp); return; }
  It m = b + n / 2;
  std::thread t([&] { parallel_sort(b, m, threads / 2, cmp); });
  parallel_sort(m, e, threads - threads / 2, cmp);
  t.join();
  std::inplace_merge(b, m, e, cmp);
}

// In-place k-way partition of (key,value) pairs by ascending pivots: on return the pairs of
// part p (keys in [pivot[p-1], pivot[p])) are contiguous; returns the k+1 part offsets.
template <typename K, typename V>
std::vector<size_t> kv_partition(K* keys, V* vals, size_t n, const std::vector<K>& pivots) {
  const size_t k = pivots.size() + 1;
  auto part = [&](K x) { return (size_t)(std::upper_bound(pivots.begin(), pivots.end(), x) - pivots.begin()); };
  std::vector<size_t> cnt(k + 1, 0);
  for (size_t i = 0; i < n; ++i) ++cnt[part(keys[i]) + 1];
  for (size_t p = 0; p < k; ++p) cnt[p + 1] += cnt[p];
  std::vector<size_t> cur(cnt.begin(), cnt.end() - 1);
  for (size_t p = 0; p < k; ++p) {
    while (cur[p] < cnt[p + 1]) {
      size_t q = part(keys[cur[p]]);
      if (q == p) { ++cur[p]; continue; }
      std::swap(keys[cur[p]], keys[cur[q]]);
      if (vals) std::swap(vals[cur[p]], vals[cur[q]]);
      ++cur[q];
    }
  }
  return cnt;
}

// ------------------------------------------------------------------ files
// Sequential reader over plain or gzip files (zlib's gz layer reads both transparently).
// Network interfaces of this machine (src/util/local_machine.h: IP(interface), pickupAvailableInterfaceAndIP).
// A node of a job that spans machines advertises the address of -interface, or of the first interface that
// is up and not the loopback.
struct LocalMachine {
  // (name, IPv4 address) of every interface that is up, loopback last
  static std::vector<std::pair<std::string, std::string>> interfaces() {
    std::vector<std::pair<std::string, std::string>> out, lo;
    ifaddrs* list = nullptr;
    if (getifaddrs(&list) != 0) return out;
    for (ifaddrs* a = list; a; a = a->ifa_next) {
      if (!a->ifa_addr || a->ifa_addr->sa_family != AF_INET || !(a->ifa_flags & IFF_UP)) continue;
      char buf[INET_ADDRSTRLEN] = {0};
      inet_ntop(AF_INET, &reinterpret_cast<sockaddr_in*>(a->ifa_addr)->sin_addr, buf, sizeof(buf));
      ((a->ifa_flags & IFF_LOOPBACK) ? lo : out).emplace_back(a->ifa_name, buf);
    }
    freeifaddrs(list);
    out.insert(out.end(), lo.begin(), lo.end());
    return out;
  }
  // address of `interface`; empty name: the first interface that is not the loopback, else the loopback; "" if none
  static std::string ip(const std::string& interface = std::string()) {
    for (auto& kv : interfaces()) if (interface.empty() || kv.first == interface) return kv.second;
    return std::string();
  }
};

// Files on HDFS.  A path "hdfs:<path>" is read through a pipe from `<hadoop fs command> -cat <path>` and a
// directory "hdfs:<dir>" is listed with `-ls`, like the reference (src/util/file.cc:50-66, 270-300; its
// hadoopFS() hard-codes a user name, here the command is set from the job's HDFSConfig).  Read-only.
inline std::string& hadoop_fs_command() { static std::string c = "hadoop fs"; return c; }
inline bool is_hdfs_path(const std::string& p) { return p.compare(0, 5, "hdfs:") == 0; }
inline std::string shell_quote(const std::string& s) {
  std::string q = "'";
  for (char c : s) { if (c == '\'') q += "'\\''"; else q += c; }
  return q + "'";
}

class File {
 public:
  // Plain and gzip files alike (zlib reads both); "hdfs:" paths through a pipe, gzip or not.
  static std::unique_ptr<File> open(const std::string& path, const char* mode) {
    if (is_hdfs_path(path)) {
      if (mode[0] != 'r') return nullptr;
      FILE* p = ::popen((hadoop_fs_command() + " -cat " + shell_quote(path.substr(5))).c_str(), "r");
      if (!p) return nullptr;
      gzFile f = gzdopen(::dup(fileno(p)), "r");
      if (!f) { ::pclose(p); return nullptr; }
      gzbuffer(f, 1 << 20);
      auto out = std::unique_ptr<File>(new File(f));
      out->pipe_ = p;
      return out;
    }
    gzFile f = gzopen(path.c_str(), mode);
    if (!f) return nullptr;
    gzbuffer(f, 1 << 20);
    return std::unique_ptr<File>(new File(f));
  }
  ~File() {
    if (f_) gzclose(f_);
    if (pipe_) ::pclose(pipe_);
  }
  int read(void* buf, size_t n) { return gzread(f_, buf, (unsigned)n); }
  bool write(const void* buf, size_t n) { return gzwrite(f_, buf, (unsigned)n) == (int)n; }
  char* read_line(char* buf, int n) { return gzgets(f_, buf, n); }
  bool seek(size_t pos) { return gzseek(f_, (z_off_t)pos, SEEK_SET) >= 0; }
  bool eof() { return gzeof(f_); }

 private:
  explicit File(gzFile f) : f_(f) {}
  gzFile f_;
  FILE* pipe_ = nullptr;
};

// Record stream: [magic u32 = 0x3ed7230a][size u32][payload]
class RecordWriter {
 public:
  explicit RecordWriter(File* f) : f_(f) {}
  bool write(const std::string& rec) {
    const uint32_t magic = 0x3ed7230a, sz = (uint32_t)rec.size();
    return f_->write(&magic, 4) && f_->write(&sz, 4) && f_->write(rec.data(), rec.size());
  }

 private:
  File* f_;
};
class RecordReader {
 public:
  explicit RecordReader(File* f) : f_(f) {}
  bool read(std::string* rec) {
    uint32_t magic = 0, sz = 0;
    if (f_->read(&magic, 4) != 4 || magic != 0x3ed7230a) return false;
    if (f_->read(&sz, 4) != 4) return false;
    rec->resize(sz);
    return sz == 0 || f_->read(&(*rec)[0], sz) == (int)sz;
  }

 private:
  File* f_;
};

inline std::string zlib_compress(const char* data, size_t n, int level = 1) {
  uLongf cap = compressBound((uLong)n);
  std::string out(cap, '\0');
  if (compress2(reinterpret_cast<Bytef*>(&out[0]), &cap, reinterpret_cast<const Bytef*>(data), (uLong)n, level) != Z_OK)
    throw std::runtime_error("zlib compress failed");
  out.resize(cap);
  return out;
}
inline bool zlib_uncompress(const char* data, size_t n, char* out, size_t out_n) {
  uLongf len = (uLongf)out_n;
  return uncompress(reinterpret_cast<Bytef*>(out), &len, reinterpret_cast<const Bytef*>(data), (uLong)n) == Z_OK && len == out_n;
}

}  // namespace psb
