// Worker-side store of the training features of a batch solver, by feature group, in column-major order.
//
// Two modes.  In memory: a group's arrays stay resident and a column range is a view.  On disk
// (-mmap_training_data): a group is written once to <dir>/<name>_grp<g>.{info,offset,index,value} in the binary
// matrix layout and its index / value arrays leave memory; column ranges come back through a pool of prefetch
// threads that read ahead of the solver, keyed by the task that will use the range, under a memory limit
// (-prefetch_mem_limit_kb) and a limit on queued jobs (-prefetch_job_limit); a range is released when its
// task is done.  The column offsets (8 bytes per column) stay resident in both modes, so a range's size is
// known without touching the disk.
//
// Counterpart in the reference: FeatureStation (src/linear_method/feature_station.{h,cc}: addFeatureGrp
// :70-109, prefetch :212-230, prefetchThreadFunc :232-279, getFeature :374-431, dropFeature :433-465) and
// the generic block store Ocean (src/system/ocean.{h,cc}; here csrc/host/ocean.h).  Differences: ranges are read with
// pread() into plain buffers instead of through SArray file reads, a task that was not prefetched, or whose
// read-ahead is still queued while the readers wait for room under the limit, is loaded by the caller itself
// (counted as a miss) instead of waiting, and a range larger than the
// whole limit is admitted when nothing else is resident so that it cannot block the queue.
#pragma once
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <fstream>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "data.h"

namespace psb {

// Columns [c0, c1) of one group.  Offsets are positions within the whole group; the row ids and values of
// position p sit at index p - pos0.
struct FeatureBlock {
  int grp = 0;
  int64_t c0 = 0, c1 = 0;
  std::vector<int64_t> indptr_own;     // disk mode: the range's own copies; memory mode: empty (views below)
  std::vector<int32_t> indices_own;
  std::vector<double> values_own;
  const int64_t* indptr = nullptr;     // c1 - c0 + 1 entries; indptr[j - c0] is the first position of column j
  const int32_t* indices = nullptr;
  const double* values = nullptr;      // nullptr: binary features
  int64_t pos0 = 0;                    // position of indices[0] / values[0] within the group
  size_t bytes() const { return indices_own.size() * 4 + values_own.size() * 8 + indptr_own.size() * 8; }
};
using FeatureBlockPtr = std::shared_ptr<FeatureBlock>;

class FeatureStation {
 public:
  struct Stats {
    uint64_t bytes_written = 0, bytes_read = 0, prefetched = 0, hits = 0, misses = 0, peak_resident = 0, limit_waits = 0;
  };

  // dir empty: in-memory mode.  threads: prefetch threads (disk mode).  mem_limit_kb: bytes that resident ranges may take.
  FeatureStation(std::string dir, std::string name, size_t mem_limit_kb, int threads, size_t job_limit = 64, bool detail = false)
      : dir_(std::move(dir)), name_(std::move(name)), limit_(mem_limit_kb * 1024), job_limit_(job_limit), detail_(detail) {
    if (disk()) {
      make_dirs(dir_);
      for (int i = 0; i < std::max(threads, 1); ++i) pool_.emplace_back([this] { prefetch_loop(); });
    }
  }
  ~FeatureStation() {
    { std::lock_guard<std::mutex> l(mu_); done_ = true; }
    cv_.notify_all();
    for (auto& t : pool_) t.join();
    for (auto& g : groups_) {
      if (g.second.fd_index >= 0) ::close(g.second.fd_index);
      if (g.second.fd_value >= 0) ::close(g.second.fd_value);
    }
  }
  bool disk() const { return !dir_.empty(); }

  // Takes a column-major group (indptr has cols + 1 entries).  Disk mode writes it out and keeps the offsets only.
  void add_group(int grp, uint64_t rows, const int64_t* indptr, int64_t cols, const int32_t* indices, const double* values) {
    Group g;
    g.rows = rows;
    g.cols = cols;
    g.binary = values == nullptr;
    g.indptr.assign(indptr, indptr + cols + 1);
    const int64_t nnz = g.indptr[cols];
    if (!disk()) {
      g.indices.assign(indices, indices + nnz);
      if (values) g.values.assign(values, values + nnz);
    } else {
      const std::string base = dir_ + "/" + name_ + "_grp" + std::to_string(grp);
      BinMatrix m;
      m.sparse = true; m.binary = g.binary; m.row_major = false; m.rows = rows; m.cols = (uint64_t)cols; m.nnz = (uint64_t)nnz;
      m.sizeof_index = 4;
      write_info(base, m);
      write_raw(base + ".offset", indptr, (size_t)(cols + 1) * 8);
      write_raw(base + ".index", indices, (size_t)nnz * 4);
      if (values) write_raw(base + ".value", values, (size_t)nnz * 8);
      g.fd_index = ::open((base + ".index").c_str(), O_RDONLY);
      g.fd_value = values ? ::open((base + ".value").c_str(), O_RDONLY) : -1;
      if (g.fd_index < 0 || (values && g.fd_value < 0)) throw std::runtime_error("feature station: cannot reopen " + base);
      stats_.bytes_written += (uint64_t)(cols + 1) * 8 + (uint64_t)nnz * (values ? 12 : 4);
      g.base = base;
    }
    std::lock_guard<std::mutex> l(mu_);
    total_bytes_ += (uint64_t)nnz * (values ? 12 : 4) + (uint64_t)(cols + 1) * 8;
    groups_[grp] = std::move(g);
  }

  uint64_t mem_size() const { std::lock_guard<std::mutex> l(mu_); return total_bytes_; }
  int64_t cols(int grp) const { std::lock_guard<std::mutex> l(mu_); return groups_.at(grp).cols; }
  uint64_t rows(int grp) const { std::lock_guard<std::mutex> l(mu_); return groups_.at(grp).rows; }
  std::string file_base(int grp) const { std::lock_guard<std::mutex> l(mu_); return groups_.at(grp).base; }

  // Bytes a column range will occupy once loaded.
  size_t range_bytes(int grp, int64_t c0, int64_t c1) const {
    std::lock_guard<std::mutex> l(mu_);
    return range_bytes_nolock(groups_.at(grp), c0, c1);
  }

  // Queue a read of columns [c0, c1) for `task`.  False: the task id was used already, or the queue is full.
  bool prefetch(int task, int grp, int64_t c0, int64_t c1) {
    if (!disk()) return false;
    std::lock_guard<std::mutex> l(mu_);
    if (used_.count(task) || jobs_.size() >= job_limit_) return false;
    used_.insert(task);
    max_task_ = std::max(max_task_, task);
    jobs_.push_back({task, grp, c0, c1});
    cv_.notify_all();
    return true;
  }
  size_t pending() const { std::lock_guard<std::mutex> l(mu_); return jobs_.size() + in_flight_; }
  bool task_used(int task) const { std::lock_guard<std::mutex> l(mu_); return used_.count(task) > 0; }
  int max_task() const { std::lock_guard<std::mutex> l(mu_); return max_task_; }
  size_t resident_bytes() const { std::lock_guard<std::mutex> l(mu_); return resident_; }

  // The range for `task`.  Waits for a prefetch that is queued or running; loads the range itself when the
  // task was never queued.  The block stays resident until drop(task).
  FeatureBlockPtr get(int task, int grp, int64_t c0, int64_t c1) {
    std::unique_lock<std::mutex> l(mu_);
    const Group& g = groups_.at(grp);
    check_range(g, c0, c1);
    if (!disk()) {
      auto b = std::make_shared<FeatureBlock>();
      b->grp = grp; b->c0 = c0; b->c1 = c1;
      b->indptr = g.indptr.data() + c0;
      b->pos0 = 0;
      b->indices = g.indices.data();
      b->values = g.binary ? nullptr : g.values.data();
      return b;
    }
    if (used_.count(task)) {
      // queued, being read, or resident; a failed prefetch takes the task out of used_ again.  While the readers are
      // held back by the memory limit (the job at the head of the queue does not fit beside what is resident) a job
      // that is still queued is taken over by the caller: what fills the limit may be ranges that only the caller's
      // progress releases, so the solver must not wait behind it.
      while (!ready_.count(task) && used_.count(task) && !done_) {
        if (limit_waiters_ > 0 && !jobs_.empty() && !fits_nolock(jobs_.front())) {
          auto it = jobs_.begin();
          while (it != jobs_.end() && it->task != task) ++it;
          if (it != jobs_.end()) {
            jobs_.erase(it);
            used_.erase(task);
            cv_.notify_all();
            break;
          }
        }
        cv_.wait(l);
      }
      auto it = ready_.find(task);
      if (it != ready_.end()) {
        FeatureBlockPtr b = it->second;
        if (b->grp != grp || b->c0 != c0 || b->c1 != c1) throw std::runtime_error("feature station: task was prefetched with another range");
        ++stats_.hits;
        return b;
      }
      if (done_) throw std::runtime_error("feature station: stopped while a range was awaited");
    }
    used_.insert(task);
    max_task_ = std::max(max_task_, task);
    ++stats_.misses;
    const size_t cost = range_bytes_nolock(g, c0, c1);
    l.unlock();
    FeatureBlockPtr b = load(g, grp, c0, c1);      // without waiting for room under the limit: the solver needs it now
    l.lock();
    resident_ += cost;
    stats_.peak_resident = std::max<uint64_t>(stats_.peak_resident, resident_);
    ready_[task] = b;
    cv_.notify_all();              // what is resident changed: callers that wait behind the limit look again
    return b;
  }

  // Releases the range of a finished task.
  void drop(int task) {
    std::lock_guard<std::mutex> l(mu_);
    auto it = ready_.find(task);
    if (it == ready_.end()) return;
    resident_ -= std::min(resident_, it->second->bytes());
    ready_.erase(it);
    used_.erase(task);             // a later get(task) loads the range again instead of waiting for nothing
    cv_.notify_all();
  }

  Stats stats() const { std::lock_guard<std::mutex> l(mu_); return stats_; }

 private:
  struct Group {
    uint64_t rows = 0;
    int64_t cols = 0;
    bool binary = false;
    std::vector<int64_t> indptr;
    std::vector<int32_t> indices;      // memory mode only
    std::vector<double> values;
    int fd_index = -1, fd_value = -1;  // disk mode
    std::string base;
  };
  struct Job { int task, grp; int64_t c0, c1; };

  // whether a queued job could be read now under the memory limit (an oversized one may when nothing is resident)
  bool fits_nolock(const Job& j) const {
    const size_t cost = range_bytes_nolock(groups_.at(j.grp), j.c0, j.c1);
    return resident_ + reserved_ == 0 || resident_ + reserved_ + cost <= limit_;
  }

  static void make_dirs(const std::string& d) {
    for (size_t i = 1; i <= d.size(); ++i)
      if (i == d.size() || d[i] == '/') ::mkdir(d.substr(0, i).c_str(), 0755);
  }
  static void write_raw(const std::string& path, const void* p, size_t n) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f || (n && std::fwrite(p, 1, n, f) != n)) { if (f) std::fclose(f); throw std::runtime_error("feature station: cannot write " + path); }
    std::fclose(f);
  }
  static void write_info(const std::string& base, const BinMatrix& m) {
    std::ofstream info(base + ".info");
    info << "type: " << (m.binary ? "SPARSE_BINARY" : "SPARSE") << "\nrow_major: false\nrow { begin: 0 end: " << m.rows
         << " }\ncol { begin: 0 end: " << m.cols << " }\nnnz: " << m.nnz << "\nsizeof_index: " << m.sizeof_index
         << "\nsizeof_value: " << (m.binary ? 0 : 8) << "\n";
    if (!info.good()) throw std::runtime_error("feature station: cannot write " + base + ".info");
  }
  static void read_fully(int fd, void* dst, size_t n, off_t at) {
    char* p = static_cast<char*>(dst);
    while (n) {
      ssize_t r = ::pread(fd, p, n, at);
      if (r < 0 && errno == EINTR) continue;
      if (r <= 0) throw std::runtime_error("feature station: short read");
      p += r; n -= (size_t)r; at += r;
    }
  }
  static void check_range(const Group& g, int64_t c0, int64_t c1) {
    if (c0 < 0 || c1 < c0 || c1 > g.cols) throw std::out_of_range("feature station: column range outside the group");
  }
  static size_t range_bytes_nolock(const Group& g, int64_t c0, int64_t c1) {
    check_range(g, c0, c1);
    const int64_t n = g.indptr[c1] - g.indptr[c0];
    return (size_t)n * (g.binary ? 4 : 12) + (size_t)(c1 - c0 + 1) * 8;
  }

  // Reads one range from the group's files.  Touches only immutable members of g.
  FeatureBlockPtr load(const Group& g, int grp, int64_t c0, int64_t c1) {
    auto b = std::make_shared<FeatureBlock>();
    b->grp = grp; b->c0 = c0; b->c1 = c1;
    const int64_t p0 = g.indptr[c0], n = g.indptr[c1] - p0;
    b->indptr_own.assign(g.indptr.begin() + c0, g.indptr.begin() + c1 + 1);
    b->indices_own.resize((size_t)n);
    if (n) read_fully(g.fd_index, b->indices_own.data(), (size_t)n * 4, (off_t)p0 * 4);
    if (!g.binary) {
      b->values_own.resize((size_t)n);
      if (n) read_fully(g.fd_value, b->values_own.data(), (size_t)n * 8, (off_t)p0 * 8);
    }
    b->indptr = b->indptr_own.data();
    b->indices = b->indices_own.data();
    b->values = g.binary ? nullptr : b->values_own.data();
    b->pos0 = p0;
    std::lock_guard<std::mutex> l(mu_);
    stats_.bytes_read += (uint64_t)n * (g.binary ? 4 : 12);
    return b;
  }

  void prefetch_loop() {
    for (;;) {
      Job j;
      const Group* g = nullptr;
      size_t cost = 0;
      {
        std::unique_lock<std::mutex> l(mu_);
        cv_.wait(l, [&] { return done_ || !jobs_.empty(); });
        if (done_) return;
        j = jobs_.front();
        g = &groups_.at(j.grp);
        cost = range_bytes_nolock(*g, j.c0, j.c1);
        // the memory limit: wait until the range fits, or nothing else is resident (an oversized range must not block)
        if (resident_ + reserved_ != 0 && resident_ + reserved_ + cost > limit_) {
          ++stats_.limit_waits;
          ++limit_waiters_;
          cv_.notify_all();          // callers that wait for a queued job look again
          cv_.wait(l, [&] { return done_ || resident_ + reserved_ == 0 || resident_ + reserved_ + cost <= limit_; });
          --limit_waiters_;
          if (done_) return;
          if (jobs_.empty() || jobs_.front().task != j.task) continue;   // another thread took it meanwhile
        }
        jobs_.pop_front();
        reserved_ += cost;
        ++in_flight_;
      }
      FeatureBlockPtr b;
      std::string err;
      try { b = load(*g, j.grp, j.c0, j.c1); } catch (const std::exception& e) { err = e.what(); }
      {
        std::lock_guard<std::mutex> l(mu_);
        reserved_ -= cost;
        --in_flight_;
        if (b) {
          resident_ += cost;
          stats_.peak_resident = std::max<uint64_t>(stats_.peak_resident, resident_);
          ++stats_.prefetched;
          ready_[j.task] = b;
          if (detail_) std::fprintf(stderr, "[feature station %s] task %d: columns [%lld, %lld) of group %d, %zu KB, %zu KB resident\n",
                                    name_.c_str(), j.task, (long long)j.c0, (long long)j.c1, j.grp, cost >> 10, resident_ >> 10);
        } else {
          used_.erase(j.task);      // get() will load it itself and report the error there
          std::fprintf(stderr, "[feature station %s] prefetch of task %d failed: %s\n", name_.c_str(), j.task, err.c_str());
        }
      }
      cv_.notify_all();
    }
  }

  std::string dir_, name_;
  size_t limit_, job_limit_;
  bool detail_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::map<int, Group> groups_;          // nodes are stable: threads hold pointers to groups while they read
  std::deque<Job> jobs_;
  std::map<int, FeatureBlockPtr> ready_;
  std::set<int> used_;
  std::vector<std::thread> pool_;
  size_t resident_ = 0, reserved_ = 0, in_flight_ = 0, limit_waiters_ = 0;
  uint64_t total_bytes_ = 0;
  int max_task_ = -1;
  bool done_ = false;
  Stats stats_;
};

}  // namespace psb
