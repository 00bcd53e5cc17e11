// A node's block store for everything a block-coordinate solver touches per feature block: the features of the
// block (column offsets, row ids, values) and the column state that goes with it (parameter keys and values, trust
// regions).  Arrays are handed over whole, cut along the node's column partition, written to one file per
// (group, block, kind) and dropped from memory; blocks come back through prefetch threads ahead of the solver,
// are handed out by reference count and leave memory when the last user drops them.
//
// Counterpart in the reference: Ocean (src/system/ocean.{h,cc}: dump :102-193, prefetch :195-208, the loader
// threads :210-239, get* :278-354, drop :356-368, load on demand :370-382), which nothing in the reference calls.
// Here the feature part of the job is done by FeatureStation for the solvers; this class covers the general form
// (six kinds of arrays, a partition given up front, a limit on the number of blocks that prefetching keeps
// loaded, load on demand for a block that was not prefetched).  Differences: blocks are addressed by group and
// block number instead of by key range, a second dump of the same (group, kind) is refused before anything is
// written, a prefetch counts as one future get + drop so that a block prefetched twice survives its first drop
// (unless -less_memory), and the files are removed with the store.
#pragma once
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <array>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

namespace psb {

class Ocean {
 public:
  enum Kind : int { FEATURE_KEY = 0, FEATURE_OFFSET, FEATURE_VALUE, PARAMETER_KEY, PARAMETER_VALUE, DELTA, NUM_KINDS };
  using Bytes = std::vector<char>;
  using BytesPtr = std::shared_ptr<const Bytes>;
  struct Stats {
    uint64_t bytes_written = 0, bytes_read = 0, prefetched = 0, hits = 0, misses = 0, loaded_now = 0, peak_loaded = 0;
  };

  // job_limit: most blocks loaded or loading at a time through prefetch (-prefetch_job_limit); less_memory: a block
  // leaves memory as soon as its count reaches zero even if it was prefetched more than once (-less_memory)
  Ocean(std::string dir, std::string identity, int threads, int job_limit, bool less_memory)
      : dir_(std::move(dir)), id_(std::move(identity)), job_limit_(job_limit > 0 ? job_limit : 1), less_memory_(less_memory) {
    ::mkdir(dir_.c_str(), 0755);
    for (int i = 0; i < (threads > 0 ? threads : 1); ++i) pool_.emplace_back([this] { loader(); });
  }
  ~Ocean() {
    { std::lock_guard<std::mutex> l(mu_); done_ = true; }
    cv_.notify_all();
    for (auto& t : pool_) t.join();
    for (auto& f : files_) ::unlink(f.c_str());
  }
  Ocean(const Ocean&) = delete;
  Ocean& operator=(const Ocean&) = delete;

  // columns [cuts[i], cuts[i+1]) of group grp form block i; must be set before the group's first dump
  bool set_partition(int grp, std::vector<uint64_t> cuts) {
    std::lock_guard<std::mutex> l(mu_);
    if (cuts.size() < 2 || part_.count(grp)) return false;
    for (size_t i = 1; i < cuts.size(); ++i) if (cuts[i] < cuts[i - 1]) return false;
    part_[grp] = std::move(cuts);
    return true;
  }
  size_t num_blocks(int grp) const {
    std::lock_guard<std::mutex> l(mu_);
    auto it = part_.find(grp);
    return it == part_.end() ? 0 : it->second.size() - 1;
  }

  // Hands an array of n elements of `elem` bytes over to the store.  Per-column kinds (PARAMETER_KEY,
  // PARAMETER_VALUE, DELTA) hold one element per column of the partition; FEATURE_OFFSET holds one uint64 per column
  // plus one (positions of the columns' non-zeros) and is stored per block rebased to the block's first position;
  // FEATURE_KEY / FEATURE_VALUE hold one element per non-zero and need the group's offsets dumped first.
  // false: unknown group, wrong length, (grp, kind) already there, or a write failed (a full disk).
  bool dump(int grp, Kind kind, const void* data, size_t n, size_t elem) {
    std::vector<uint64_t> cuts, off;
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = part_.find(grp);
      if (it == part_.end() || kind < 0 || kind >= NUM_KINDS || elem == 0 || have_.count({grp, (int)kind})) return false;
      cuts = it->second;
      const uint64_t cols = cuts.back() - cuts.front();
      if (kind == FEATURE_OFFSET) {
        if (n != cols + 1 || elem != sizeof(uint64_t)) return false;
      } else if (kind == FEATURE_KEY || kind == FEATURE_VALUE) {
        auto o = offsets_.find(grp);
        if (o == offsets_.end() || n != o->second.back() - o->second.front()) return false;
        off = o->second;
      } else if (n != cols) {
        return false;
      }
      have_.insert({grp, (int)kind});          // claimed under the lock: a concurrent second dump is refused
    }
    const char* p = static_cast<const char*>(data);
    bool ok = true;
    if (kind == FEATURE_OFFSET) off.assign(reinterpret_cast<const uint64_t*>(p), reinterpret_cast<const uint64_t*>(p) + n);
    for (size_t b = 0; b + 1 < cuts.size() && ok; ++b) {
      const uint64_t c0 = cuts[b] - cuts.front(), c1 = cuts[b + 1] - cuts.front();
      if (kind == FEATURE_OFFSET) {
        std::vector<uint64_t> rebased(off.begin() + c0, off.begin() + c1 + 1);
        const uint64_t base = rebased.front();
        for (auto& v : rebased) v -= base;
        ok = write_file(grp, b, kind, rebased.data(), rebased.size() * sizeof(uint64_t));
      } else if (kind == FEATURE_KEY || kind == FEATURE_VALUE) {
        const uint64_t p0 = off[c0] - off.front(), p1 = off[c1] - off.front();
        ok = write_file(grp, b, kind, p + p0 * elem, (p1 - p0) * elem);
      } else {
        ok = write_file(grp, b, kind, p + c0 * elem, (c1 - c0) * elem);
      }
    }
    std::lock_guard<std::mutex> l(mu_);
    if (!ok) { have_.erase({grp, (int)kind}); return false; }
    if (kind == FEATURE_OFFSET) offsets_[grp] = std::move(off);
    return true;
  }

  // Queues block `blk` of group grp for loading (all kinds that were dumped).  It starts when fewer than the job
  // limit are loaded or loading.  Every prefetch is one future get + drop.
  void prefetch(int grp, size_t blk) {
    {
      std::lock_guard<std::mutex> l(mu_);
      auto& e = entry(grp, blk);
      ++e.expected;
      if (e.state == Entry::ABSENT) { e.state = Entry::QUEUED; queue_.push_back({grp, blk}); ++stats_.prefetched; }
    }
    cv_.notify_all();
  }

  // The block's array of one kind (nullptr if that kind was never dumped).  Counts one user; pair with drop().
  BytesPtr get(int grp, size_t blk, Kind kind) {
    std::unique_lock<std::mutex> l(mu_);
    auto& e = entry(grp, blk);
    ++e.users;            // counted before any wait: the block cannot leave memory under a thread that waits for it
    if (e.state == Entry::LOADED || e.state == Entry::LOADING) ++stats_.hits; else ++stats_.misses;
    if (e.state == Entry::ABSENT || e.state == Entry::QUEUED) {
      // not loaded and no loader has it: the caller loads it itself instead of waiting for a free job slot
      if (e.state == Entry::QUEUED) {
        for (auto it = queue_.begin(); it != queue_.end(); ++it)
          if (it->first == grp && it->second == blk) { queue_.erase(it); break; }
      }
      e.state = Entry::LOADING;
      note_loaded(+1);
      l.unlock();
      auto data = read_block(grp, blk);
      l.lock();
      auto& e2 = entry(grp, blk);
      e2.data = std::move(data);
      e2.state = Entry::LOADED;
      cv_.notify_all();
    } else {
      cv_.wait(l, [&] { return entry(grp, blk).state == Entry::LOADED; });
    }
    return entry(grp, blk).data[kind];
  }

  // One user less; the block leaves memory when nobody uses it and no prefetch is still to be consumed
  void drop(int grp, size_t blk) {
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = blocks_.find({grp, blk});
      if (it == blocks_.end()) return;
      auto& e = it->second;
      if (e.users > 0) --e.users;
      if (e.expected > 0) --e.expected;
      if (e.users == 0 && e.state == Entry::LOADED && (e.expected == 0 || less_memory_)) {
        blocks_.erase(it);
        note_loaded(-1);
      }
    }
    cv_.notify_all();
  }

  Stats stats() const { std::lock_guard<std::mutex> l(mu_); return stats_; }
  size_t pending() const { std::lock_guard<std::mutex> l(mu_); return queue_.size(); }

 private:
  struct Entry {
    enum State { ABSENT, QUEUED, LOADING, LOADED } state = ABSENT;
    int users = 0, expected = 0;
    std::array<BytesPtr, NUM_KINDS> data;
  };
  Entry& entry(int grp, size_t blk) { return blocks_[{grp, blk}]; }
  void note_loaded(int d) {
    stats_.loaded_now += d;
    if (stats_.loaded_now > stats_.peak_loaded) stats_.peak_loaded = stats_.loaded_now;
  }
  std::string path(int grp, size_t blk, int kind) const {
    return dir_ + "/" + id_ + "_g" + std::to_string(grp) + "_b" + std::to_string(blk) + "_k" + std::to_string(kind);
  }
  bool write_file(int grp, size_t blk, int kind, const void* p, size_t bytes) {
    const std::string f = path(grp, blk, kind);
    const int fd = ::open(f.c_str(), O_CREAT | O_TRUNC | O_WRONLY, 0644);
    if (fd < 0) return false;
    const char* c = static_cast<const char*>(p);
    size_t done = 0;
    while (done < bytes) {
      const ssize_t w = ::write(fd, c + done, bytes - done);
      if (w <= 0) { ::close(fd); ::unlink(f.c_str()); return false; }
      done += (size_t)w;
    }
    ::close(fd);
    std::lock_guard<std::mutex> l(mu_);
    files_.insert(f);
    stats_.bytes_written += bytes;
    return true;
  }
  std::array<BytesPtr, NUM_KINDS> read_block(int grp, size_t blk) {
    std::array<BytesPtr, NUM_KINDS> out;
    uint64_t total = 0;
    for (int k = 0; k < NUM_KINDS; ++k) {
      { std::lock_guard<std::mutex> l(mu_); if (!have_.count({grp, k})) continue; }
      const std::string f = path(grp, blk, k);
      const int fd = ::open(f.c_str(), O_RDONLY);
      if (fd < 0) continue;
      struct stat st;
      auto buf = std::make_shared<Bytes>();
      if (::fstat(fd, &st) == 0) {
        buf->resize((size_t)st.st_size);
        size_t done = 0;
        while (done < buf->size()) {
          const ssize_t r = ::pread(fd, buf->data() + done, buf->size() - done, (off_t)done);
          if (r <= 0) break;
          done += (size_t)r;
        }
        buf->resize(done);
        total += done;
      }
      ::close(fd);
      out[k] = buf;
    }
    std::lock_guard<std::mutex> l(mu_);
    stats_.bytes_read += total;
    return out;
  }
  void loader() {
    std::unique_lock<std::mutex> l(mu_);
    while (true) {
      cv_.wait(l, [&] { return done_ || (!queue_.empty() && stats_.loaded_now < (uint64_t)job_limit_); });
      if (done_) return;
      const auto job = queue_.front();
      queue_.pop_front();
      auto& e = entry(job.first, job.second);
      if (e.state != Entry::QUEUED) continue;      // a caller took it meanwhile
      e.state = Entry::LOADING;
      note_loaded(+1);
      l.unlock();
      auto data = read_block(job.first, job.second);
      l.lock();
      auto& e2 = entry(job.first, job.second);
      e2.data = std::move(data);
      e2.state = Entry::LOADED;
      if (e2.users == 0 && e2.expected == 0) {     // dropped while it was queued or loading: nobody will come for it
        blocks_.erase({job.first, job.second});
        note_loaded(-1);
      }
      cv_.notify_all();
    }
  }

  const std::string dir_, id_;
  const int job_limit_;
  const bool less_memory_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  bool done_ = false;
  std::map<int, std::vector<uint64_t>> part_, offsets_;
  std::set<std::pair<int, int>> have_;
  std::map<std::pair<int, size_t>, Entry> blocks_;
  std::deque<std::pair<int, size_t>> queue_;
  std::set<std::string> files_;
  Stats stats_;
  std::vector<std::thread> pool_;
};

}  // namespace psb
