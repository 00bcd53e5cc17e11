// Control-plane transport ("Van").  Two interchangeable backends carry encoded messages
// between nodes:
//   * InprocVan — nodes are threads of one process and exchange frames through a shared hub
//                 (used by tests and by single-process multi-role runs);
//   * TcpVan    — one listening socket per node, one outgoing connection per peer, frames
//                 prefixed by their length (multi-process runs on localhost or a LAN).
// Bulk parameter data never travels here: on the GPU box it moves through peer memory from
// inside kernels.  This layer replaces the ZeroMQ ROUTER/DEALER van of the reference
// (src/system/van.{h,cc}): same send/recv/connect surface, per-frame compression flag, byte
// counters and the optional message log (-print_van).
//
// Fault injection for tests lives here too, on the host only: a per-van filter may drop, delay
// or duplicate outgoing messages.
#pragma once
#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include "message.h"

namespace psb {

class Van {
 public:
  virtual ~Van() = default;
  virtual Status connect(const Node& node) = 0;
  virtual Status send_frame(const std::string& to, std::string frame) = 0;
  // blocks up to timeout_s; returns false on timeout or after close()
  virtual bool recv_frame(std::string* frame, double timeout_s) = 0;
  virtual void close() = 0;

  Status send(const Message& m) {
    if (filter_) {
      const int verdict = filter_(m);          // 0 pass, 1 drop, 2 duplicate, >2: delay in ms
      if (verdict == 1) { ++dropped_; return Status::OK(); }
      if (verdict == 2) { Status s = do_send(m); if (!s.ok()) return s; }
      if (verdict > 2) std::this_thread::sleep_for(std::chrono::milliseconds(verdict));
    }
    return do_send(m);
  }
  bool recv(MessagePtr* m, double timeout_s) {
    std::string frame;
    if (!recv_frame(&frame, timeout_s)) return false;
    *m = decode_message(frame.data(), frame.size());
    recv_bytes_ += frame.size();
    log("RCV", **m);
    return true;
  }
  void set_compress(bool c) { compress_ = c; }
  void set_filter(std::function<int(const Message&)> f) { filter_ = std::move(f); }
  void set_log(const std::string& path) { log_.open(path); }
  uint64_t sent_bytes() const { return sent_bytes_; }
  uint64_t recv_bytes() const { return recv_bytes_; }
  uint64_t dropped() const { return dropped_; }
  Node my_node;

 protected:
  Status do_send(const Message& m) {
    std::string frame = encode_message(m, compress_);
    sent_bytes_ += frame.size();
    log("SND", m);
    return send_frame(m.recver, std::move(frame));
  }
  void log(const char* dir, const Message& m) {
    if (!log_.is_open()) return;
    std::lock_guard<std::mutex> l(log_mu_);
    log_ << dir << " " << m.short_debug() << "\n";
    log_.flush();
  }
  bool compress_ = false;
  std::atomic<uint64_t> sent_bytes_{0}, recv_bytes_{0}, dropped_{0};
  std::function<int(const Message&)> filter_;
  std::ofstream log_;
  std::mutex log_mu_;
};

// ------------------------------------------------------------------ in-process
class InprocHub {
 public:
  std::shared_ptr<ThreadsafeQueue<std::string>> queue(const std::string& id) {
    std::lock_guard<std::mutex> l(mu_);
    auto& q = queues_[id];
    if (!q) q = std::make_shared<ThreadsafeQueue<std::string>>();
    return q;
  }

 private:
  std::mutex mu_;
  std::map<std::string, std::shared_ptr<ThreadsafeQueue<std::string>>> queues_;
};

class InprocVan : public Van {
 public:
  InprocVan(std::shared_ptr<InprocHub> hub, const Node& me) : hub_(std::move(hub)) {
    my_node = me;
    inbox_ = hub_->queue(me.id);
  }
  Status connect(const Node&) override { return Status::OK(); }
  Status send_frame(const std::string& to, std::string frame) override {
    if (closed_) return Status::NetError("van closed");
    hub_->queue(to)->push(std::move(frame));
    return Status::OK();
  }
  bool recv_frame(std::string* frame, double timeout_s) override {
    const double deadline = now_seconds() + timeout_s;
    while (!closed_) {
      if (inbox_->wait_and_pop_for(*frame, 0.05)) return true;
      if (now_seconds() > deadline) return false;
    }
    return false;
  }
  void close() override { closed_ = true; }

 private:
  std::shared_ptr<InprocHub> hub_;
  std::shared_ptr<ThreadsafeQueue<std::string>> inbox_;
  std::atomic<bool> closed_{false};
};

// ------------------------------------------------------------------ TCP
class TcpVan : public Van {
 public:
  explicit TcpVan(const Node& me) { my_node = me; }
  ~TcpVan() override { close(); }

  // bind + listen on my_node.port (0 = pick a free port, written back to my_node.port)
  Status bind() {
    listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (listen_fd_ < 0) return Status::NetError("socket() failed");
    int one = 1;
    setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_addr.s_addr = htonl(INADDR_ANY);
    a.sin_port = htons((uint16_t)my_node.port);
    if (::bind(listen_fd_, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0) return Status::NetError("bind() failed on port " + std::to_string(my_node.port));
    socklen_t len = sizeof(a);
    getsockname(listen_fd_, reinterpret_cast<sockaddr*>(&a), &len);
    my_node.port = ntohs(a.sin_port);
    if (::listen(listen_fd_, 64) != 0) return Status::NetError("listen() failed");
    accept_thread_ = std::thread([this] { accept_loop(); });
    return Status::OK();
  }
  Status connect(const Node& node) override {
    std::lock_guard<std::mutex> l(mu_);
    peers_[node.id] = node;
    return Status::OK();
  }
  Status send_frame(const std::string& to, std::string frame) override {
    // one lock per peer: frames to one peer go out whole and in order, a peer that is slow to accept
    // a connection holds up nobody else's traffic
    std::mutex* peer_mu;
    {
      std::lock_guard<std::mutex> l2(mu_);
      auto& slot = peer_mu_[to];
      if (!slot) slot.reset(new std::mutex);
      peer_mu = slot.get();
    }
    std::lock_guard<std::mutex> l(*peer_mu);
    int fd = -1;
    {
      std::lock_guard<std::mutex> l2(mu_);
      auto it = out_fd_.find(to);
      if (it != out_fd_.end()) fd = it->second;
    }
    if (fd < 0) {
      Node peer;
      {
        std::lock_guard<std::mutex> l2(mu_);
        auto it = peers_.find(to);
        if (it == peers_.end()) return Status::NetError("unknown peer " + to);
        peer = it->second;
      }
      // numeric address or host name (the reference's tcp://host:port accepts both)
      const std::string host = peer.hostname.empty() ? "127.0.0.1" : peer.hostname;
      addrinfo hints{}, *res = nullptr;
      hints.ai_family = AF_INET;
      hints.ai_socktype = SOCK_STREAM;
      if (getaddrinfo(host.c_str(), std::to_string(peer.port).c_str(), &hints, &res) != 0 || res == nullptr)
        return Status::NetError("cannot resolve " + host + " (node " + to + ")");
      // The long retry schedule is for the start of a job, when a peer may not be listening yet.  A peer that was
      // reached before and is gone now (its process ended) is given three quick attempts: senders must not sit
      // for most of a minute on every message to a dead node.
      bool reached_before;
      { std::lock_guard<std::mutex> l2(mu_); reached_before = reached_.count(to) > 0; }
      const int attempts = reached_before ? std::min(retries_, 3) : retries_;
      for (int attempt = 0; attempt < attempts && fd < 0; ++attempt) {
        fd = ::socket(AF_INET, SOCK_STREAM, 0);
        if (fd < 0 || ::connect(fd, res->ai_addr, res->ai_addrlen) != 0) {
          if (fd >= 0) ::close(fd);
          fd = -1;
          std::this_thread::sleep_for(std::chrono::milliseconds(50 * (attempt + 1)));
        }
      }
      freeaddrinfo(res);
      if (fd < 0) return Status::NetError("cannot connect to " + to);
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      std::lock_guard<std::mutex> l2(mu_);
      if (closed_) { ::close(fd); return Status::NetError("van closed"); }
      out_fd_[to] = fd;
      reached_.insert(to);
    }
    const uint64_t n = frame.size();
    if (!write_all(fd, &n, 8) || !write_all(fd, frame.data(), n)) {
      std::lock_guard<std::mutex> l2(mu_);
      auto it = out_fd_.find(to);
      if (it != out_fd_.end() && it->second == fd) { ::close(fd); out_fd_.erase(it); }
      return Status::NetError("send to " + to + " failed");
    }
    return Status::OK();
  }
  bool recv_frame(std::string* frame, double timeout_s) override {
    const double deadline = now_seconds() + timeout_s;
    while (!closed_) {
      if (inbox_.wait_and_pop_for(*frame, 0.05)) return true;
      if (now_seconds() > deadline) return false;
    }
    return false;
  }
  void close() override {
    if (closed_.exchange(true)) return;
    if (listen_fd_ >= 0) { ::shutdown(listen_fd_, SHUT_RDWR); ::close(listen_fd_); }
    if (accept_thread_.joinable()) accept_thread_.join();
    {
      std::lock_guard<std::mutex> l(mu_);
      for (auto& kv : out_fd_) ::close(kv.second);
      for (int fd : in_fd_) ::shutdown(fd, SHUT_RDWR);
      out_fd_.clear();
    }
    for (auto& t : readers_) if (t.joinable()) t.join();
  }
  void set_retries(int n) { retries_ = std::max(1, n); }

 private:
  static bool write_all(int fd, const void* p, size_t n) {
    const char* c = static_cast<const char*>(p);
    while (n > 0) {
      ssize_t w = ::send(fd, c, n, MSG_NOSIGNAL);
      if (w < 0) { if (errno == EINTR) continue; return false; }
      c += w; n -= (size_t)w;
    }
    return true;
  }
  static bool read_all(int fd, void* p, size_t n) {
    char* c = static_cast<char*>(p);
    while (n > 0) {
      ssize_t r = ::recv(fd, c, n, 0);
      if (r == 0) return false;
      if (r < 0) { if (errno == EINTR) continue; return false; }
      c += r; n -= (size_t)r;
    }
    return true;
  }
  void accept_loop() {
    while (!closed_) {
      int fd = ::accept(listen_fd_, nullptr, nullptr);
      if (fd < 0) { if (closed_) return; continue; }
      std::lock_guard<std::mutex> l(mu_);
      in_fd_.push_back(fd);
      readers_.emplace_back([this, fd] {
        for (;;) {
          uint64_t n = 0;
          if (!read_all(fd, &n, 8) || n > (1ull << 34)) break;
          std::string frame(n, '\0');
          if (n && !read_all(fd, &frame[0], n)) break;
          inbox_.push(std::move(frame));
        }
        // forget the descriptor before closing it: its number may be handed to any other socket of
        // the process right away, and close() must not shut that one down
        std::lock_guard<std::mutex> l2(mu_);
        in_fd_.erase(std::remove(in_fd_.begin(), in_fd_.end(), fd), in_fd_.end());
        ::close(fd);
      });
    }
  }
  int listen_fd_ = -1, retries_ = 3;
  std::set<std::string> reached_;      // peers that a connection was made to at least once (guarded by mu_)
  std::atomic<bool> closed_{false};
  std::mutex mu_;
  std::map<std::string, Node> peers_;
  std::map<std::string, std::unique_ptr<std::mutex>> peer_mu_;
  std::map<std::string, int> out_fd_;
  std::vector<int> in_fd_;
  std::vector<std::thread> readers_;
  std::thread accept_thread_;
  ThreadsafeQueue<std::string> inbox_;
};

}  // namespace psb
