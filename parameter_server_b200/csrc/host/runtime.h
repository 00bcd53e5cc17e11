// The control-plane runtime: logical-clock task tracking, remote-node proxies with key-range
// slicing and key caching, the per-customer dependency (DAG) executor, and the per-process
// post office with its send/receive threads, membership management, heartbeats and a
// deadline-based failure detector.
//
// Counterparts in the reference: src/system/task_tracker.h, remote_node.{h,cc}, executor.{h,cc},
// customer.h, postoffice.{h,cc}, yellow_pages.{h,cc}, heartbeat_info.{h,cc}.  Semantics kept:
//   * a request carries (time, wait_time); it becomes runnable once the sender's incoming task
//     `wait_time` is finished (or wait_time < 0); replies are always runnable;
//   * after process() the incoming task is marked finished and an empty ack is sent unless the
//     customer deferred it (msg->finished = false) or already replied with data;
//   * a submit to a group is sliced by the group's key partition; the finish callback fires
//     when every member has replied;
//   * sender/receiver key caches keyed by (channel, key range) with a crc32c signature.
#pragma once
#include "van.h"

namespace psb {

// -verbose: every executor narrates the messages it picks and those it holds back for a dependency
// (src/system/executor.cc:95-133).
inline std::atomic<bool>& verbose_flag() { static std::atomic<bool> v{false}; return v; }

class TaskTracker {
 public:
  void start(int t) { std::lock_guard<std::mutex> l(mu_); task_.emplace(t, false); }
  void finish(int t) { { std::lock_guard<std::mutex> l(mu_); task_[t] = true; } cv_.notify_all(); }
  bool try_wait(int t) const { std::lock_guard<std::mutex> l(mu_); auto it = task_.find(t); return it != task_.end() && it->second; }
  // false: the time ran out, or the waits were called off (abort) before t finished
  bool wait(int t, double timeout_s = 1e9) {
    std::unique_lock<std::mutex> l(mu_);
    auto done = [&] { auto it = task_.find(t); return it != task_.end() && it->second; };
    cv_.wait_for(l, std::chrono::duration<double>(timeout_s), [&] { return aborted_ || done(); });
    return done();
  }
  bool has_started(int t) const { std::lock_guard<std::mutex> l(mu_); return task_.count(t) > 0; }
  // The job is over (TERMINATE while a node still waits for a peer that is gone): every wait, now and later, returns.
  void abort() { { std::lock_guard<std::mutex> l(mu_); aborted_ = true; } cv_.notify_all(); }

 private:
  mutable std::mutex mu_; std::condition_variable cv_; std::map<int, bool> task_; bool aborted_ = false;
};

class Postoffice;
class Executor;
class Customer;

class RNode {
 public:
  RNode(const Node& n, Executor* e) : node(n), exec_(e) {}
  Node node;
  TaskTracker incoming, outgoing;
  int time = 0;                         // newest timestamp used with this node (guarded by Executor::clock_mu)
  std::mutex mu;
  std::mutex send_mu;                   // orders key-cache decisions with the send queue
  std::atomic<uint64_t> key_cache_misses{0};   // requests that named a key list this node no longer caches
  std::map<int, MessagePtr> pending;    // sent, not yet acknowledged
  std::map<int, std::function<void()>> recv_handles, fin_handles;
  // key caches: (channel, range) -> (signature, keys)
  std::map<std::pair<int, Range>, std::pair<uint32_t, std::string>> key_cache;

  void cache_key_sender(const MessagePtr& m, bool enabled);
  void cache_key_recver(const MessagePtr& m, bool enabled);

 private:
  Executor* exec_;
};
using RNodePtr = std::shared_ptr<RNode>;

inline uint32_t key_signature(const std::string& key) {
  return crc32c_value(key.data(), std::min<size_t>(key.size(), 2048)) + (uint32_t)key.size();
}
inline void RNode::cache_key_sender(const MessagePtr& m, bool enabled) {
  if (!enabled || !m->task.has_key_range) return;
  std::lock_guard<std::mutex> l(mu);
  auto ck = std::make_pair(m->task.key_channel, m->task.key_range);
  if (m->task.erase_key_cache) { key_cache.erase(ck); return; }
  if (!m->task.has_key) return;
  const uint32_t sig = key_signature(m->key);
  auto it = key_cache.find(ck);
  if (it != key_cache.end() && it->second.first == sig) {
    m->key.clear();               // receiver restores the keys from its cache
    m->task.has_key = false;
  } else {
    key_cache[ck] = {sig, std::string()};
  }
  m->task.key_signature = sig;
}
inline void RNode::cache_key_recver(const MessagePtr& m, bool enabled) {
  if (!enabled || !m->task.has_key_range || !m->task.request) return;
  std::lock_guard<std::mutex> l(mu);
  auto ck = std::make_pair(m->task.key_channel, m->task.key_range);
  if (m->task.erase_key_cache) { key_cache.erase(ck); return; }
  if (m->task.has_key) {
    key_cache[ck] = {m->task.key_signature, m->key};
  } else if (m->task.key_signature != 0) {
    auto it = key_cache.find(ck);
    if (it != key_cache.end() && it->second.first == m->task.key_signature) {
      m->key = it->second.second;
      m->task.has_key = true;
    } else if (key_cache_misses++ == 0) {
      std::fprintf(stderr, "key cache miss: %s sent signature %u on channel %d that is not cached here\n",
                   m->sender.c_str(), m->task.key_signature, m->task.key_channel);
    }
  }
}

class Customer {
 public:
  Customer(Postoffice* po, std::string name);
  virtual ~Customer();
  const std::string& name() const { return name_; }
  Postoffice* po() { return po_; }
  Executor* exec() { return exec_.get(); }
  // user hooks
  std::function<void(const MessagePtr&)> process;     // every request and every data reply
  bool key_ordered_slice = true;                      // false: every receiver gets a full copy
  std::vector<MessagePtr> slice(const MessagePtr& m, const std::vector<Key>& sep) {
    if (key_ordered_slice) return slice_key_ordered(m, sep);
    std::vector<MessagePtr> out;
    for (size_t i = 0; i + 1 < sep.size(); ++i) out.push_back(std::make_shared<Message>(*m));
    return out;
  }
  // submit `m` (m->recver = node or group id); returns its timestamp
  int submit(const MessagePtr& m);
  bool wait_out(const std::string& node, int t, double timeout_s = 1e9);
  bool wait_in(const std::string& node, int t, double timeout_s = 1e9);
  bool try_wait_out(const std::string& node, int t);
  void finish_in(const std::string& node, int t);
  void finish_out(const std::string& node, int t);
  // reply to request `req`, optionally with data (pull replies)
  void reply(const MessagePtr& req, std::string key = std::string(), std::vector<std::string> values = {}, std::string payload = std::string());

 private:
  Postoffice* po_;
  std::string name_;
  std::unique_ptr<Executor> exec_;
};

class Executor {
 public:
  Executor(Customer* c, Postoffice* po) : obj_(c), po_(po) {}
  ~Executor() { stop(); }
  void init(const std::vector<Node>& nodes, const Node& me, int num_replicas);
  void start() { if (!thread_.joinable()) thread_ = std::thread([this] { run(); }); }
  void stop() {
    { std::lock_guard<std::mutex> l(mu_); done_ = true; }
    cv_.notify_all();
    if (thread_.joinable()) thread_.join();
  }
  void accept(const MessagePtr& m) {
    {
      std::lock_guard<std::mutex> l(mu_);
      auto s = rnode_nolock(m->sender);
      if (s) s->cache_key_recver(m, key_cache_enabled);
      recved_.push_back(m);
    }
    cv_.notify_all();
  }
  void notify() { cv_.notify_all(); }
  // calls off every wait on this customer's nodes (wait_in / wait_out of application threads and handlers)
  void abort_waits() {
    std::vector<RNodePtr> all;
    { std::lock_guard<std::mutex> l(mu_); for (auto& kv : nodes_) all.push_back(kv.second); }
    for (auto& n : all) { n->incoming.abort(); n->outgoing.abort(); }
  }
  RNodePtr rnode(const std::string& id) { std::lock_guard<std::mutex> l(mu_); return rnode_nolock(id); }
  std::vector<RNodePtr> group(const std::string& id) {
    std::lock_guard<std::mutex> l(mu_);
    auto it = groups_.find(id);
    return it == groups_.end() ? std::vector<RNodePtr>() : it->second;
  }
  std::vector<Key> partition(const std::string& id) {
    std::lock_guard<std::mutex> l(mu_);
    auto it = partitions_.find(id);
    return it == partitions_.end() ? std::vector<Key>() : it->second;
  }
  bool initialized() const { return inited_; }
  int last_task() const { return last_task_; }
  // Requests that have arrived but not started yet, in arrival order (a worker looks ahead in them to
  // prefetch the data of coming tasks; the reference walks its queue with Executor::forEach,
  // src/system/executor.cc:262-272).
  std::vector<MessagePtr> pending_requests() {
    std::lock_guard<std::mutex> l(mu_);
    std::vector<MessagePtr> out;
    for (auto& m : recved_) if (m->task.request) out.push_back(m);
    return out;
  }
  bool key_cache_enabled = true;
  std::atomic<uint64_t> processed{0};
  std::mutex clock_mu;   // guards RNode::time of every node and group of this executor
  // payloads (task.msg) of the replies to outgoing task t, by replying node
  std::map<std::string, std::string> take_replies(int t) {
    std::lock_guard<std::mutex> l(mu_);
    std::map<std::string, std::string> out;
    auto it = replies_.find(t);
    if (it != replies_.end()) { out.swap(it->second); replies_.erase(it); }
    return out;
  }

 private:
  RNodePtr rnode_nolock(const std::string& id) { auto it = nodes_.find(id); return it == nodes_.end() ? nullptr : it->second; }
  void add(const Node& n) {
    auto r = std::make_shared<RNode>(n, this);
    nodes_[n.id] = r;
    if (n.role != Node::GROUP) {
      groups_[n.id] = {r};
      groups_[kLiveGroup].push_back(r);
      if (n.role == Node::SERVER) { groups_[kServerGroup].push_back(r); groups_[kActiveGroup].push_back(r); }
      if (n.role == Node::WORKER) { groups_[kWorkerGroup].push_back(r); groups_[kActiveGroup].push_back(r); }
    }
  }
  void run();
  Customer* obj_;
  Postoffice* po_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<MessagePtr> recved_;
  std::map<std::string, RNodePtr> nodes_;
  std::map<std::string, std::vector<RNodePtr>> groups_;
  std::map<std::string, std::vector<Key>> partitions_;
  std::thread thread_;
  bool done_ = false;
  std::atomic<bool> inited_{false};
  std::atomic<int> last_task_{0};
  std::map<int, std::map<std::string, std::string>> replies_;
};

struct HeartbeatRecord {
  double when = 0;
  int task_id = 0;
  std::string report;   // text-format HeartbeatReport
};

class Postoffice {
 public:
  Postoffice(std::shared_ptr<Van> van, int num_workers, int num_servers, int num_replicas = 0)
      : van_(std::move(van)), num_workers_(num_workers), num_servers_(num_servers), num_replicas_(num_replicas) {}
  ~Postoffice() { stop(); }
  Node& my_node() { return van_->my_node; }
  Van* van() { return van_.get(); }
  void set_scheduler(const Node& s) { scheduler_ = s; van_->connect(s); }
  const Node& scheduler() const { return scheduler_; }

  void start() {
    if (recv_thread_.joinable()) return;
    recv_thread_ = std::thread([this] { recv_loop(); });
    send_thread_ = std::thread([this] { send_loop(); });
  }
  void stop() {
    if (done_.exchange(true)) return;
    hb_cv_.notify_all();
    send_q_.push(nullptr);
    van_->close();
    if (recv_thread_.joinable()) recv_thread_.join();
    if (send_thread_.joinable()) send_thread_.join();
    if (hb_thread_.joinable()) hb_thread_.join();
  }
  bool done() const { return done_; }

  // ---- customers
  void add_customer(Customer* c) {
    std::vector<MessagePtr> backlog;
    {
      std::lock_guard<std::mutex> l(mu_);
      customers_[c->name()] = c;
      if (!nodes_.empty()) c->exec()->init(nodes_, my_node(), num_replicas_);
      auto it = orphan_.find(c->name());
      if (it != orphan_.end()) { backlog.swap(it->second); orphan_.erase(it); }
    }
    c->exec()->key_cache_enabled = key_cache_;
    c->exec()->start();
    for (auto& m : backlog) c->exec()->accept(m);
  }
  // A customer that goes away is first taken out of the table, then waits until no message is being handed to
  // it: dispatch() calls into the customer's executor after it let go of the table's lock.
  void remove_customer(Customer* c) {
    std::unique_lock<std::mutex> l(mu_);
    customers_.erase(c->name());
    deliver_cv_.wait(l, [&] { return delivering_.count(c) == 0; });
  }

  // ---- membership (src/system/postoffice.cc:185-243)
  // non-scheduler: announce myself to the scheduler
  void register_with_scheduler() {
    auto m = std::make_shared<Message>();
    m->task.type = Task::MANAGE;
    m->task.request = true;
    m->task.customer = "default";
    m->task.msg = "ADD " + encode_node(my_node());
    m->sender = my_node().id;
    m->recver = scheduler_.id;
    queue(m);
  }
  // scheduler: block until all workers and servers announced themselves, assign server key
  // ranges, broadcast the node table
  bool wait_nodes_and_init(double timeout_s) {
    {
      std::unique_lock<std::mutex> l(mu_);
      // every worker and every server must have registered; stand-by nodes (role UNUSED) join the table if they
      // are there by then, they are not waited for
      auto complete = [&] {
        int w = 0, s = 0;
        for (auto& n : pending_nodes_) { w += n.role == Node::WORKER; s += n.role == Node::SERVER; }
        return w >= num_workers_ && s >= num_servers_;
      };
      if (!nodes_cv_.wait_for(l, std::chrono::duration<double>(timeout_s), complete)) return false;
    }
    std::vector<Node> nodes;
    {
      std::lock_guard<std::mutex> l(mu_);
      int si = 0;
      // by role letter, then by number: S2 before S10, so that server i owns the i-th key range
      auto num = [](const std::string& id) { return id.size() > 1 ? std::atoi(id.c_str() + 1) : 0; };
      std::sort(pending_nodes_.begin(), pending_nodes_.end(), [&](const Node& a, const Node& b) {
        if (a.id.empty() || b.id.empty() || a.id[0] != b.id[0]) return a.id < b.id;
        return num(a.id) != num(b.id) ? num(a.id) < num(b.id) : a.id < b.id;
      });
      for (auto n : pending_nodes_) {
        if (n.role == Node::SERVER) n.key = Range::all().even_divide(num_servers_, si++);
        else n.key = Range::all();
        nodes.push_back(n);
      }
      Node me = my_node();
      me.key = Range::all();
      nodes.push_back(me);
      // table_sent_ flips under the same lock as the copy of the table that goes out and nodes_ is
      // filled before the lock is dropped, so a registration is either in that copy or handled as
      // a late one (never both, never neither)
      nodes_ = nodes;
      table_sent_ = true;
    }
    std::string table = "INIT";
    set_nodes(nodes);
    for (auto& n : nodes) table += " " + encode_node(n);
    for (auto& n : nodes) {
      if (n.id == my_node().id) continue;
      auto m = std::make_shared<Message>();
      m->task.type = Task::MANAGE;
      m->task.request = true;
      m->task.customer = "default";
      m->task.msg = table;
      m->sender = my_node().id;
      m->recver = n.id;
      queue(m);
    }
    return true;
  }
  void set_nodes(const std::vector<Node>& nodes) {
    std::lock_guard<std::mutex> l(mu_);
    nodes_ = nodes;
    for (auto& n : nodes) {
      van_->connect(n);
      if (n.id == my_node().id) my_node().key = n.key;
    }
    for (auto& kv : customers_) kv.second->exec()->init(nodes_, my_node(), num_replicas_);
    nodes_ready_ = true;
    nodes_cv_.notify_all();
  }
  bool wait_nodes_ready(double timeout_s) {
    std::unique_lock<std::mutex> l(mu_);
    return nodes_cv_.wait_for(l, std::chrono::duration<double>(timeout_s), [&] { return nodes_ready_; });
  }
  std::vector<Node> nodes() { std::lock_guard<std::mutex> l(mu_); return nodes_; }
  // broadcast TERMINATE to every other node (App::stopAll)
  void stop_all() {
    for (auto& n : nodes()) {
      if (n.id == my_node().id) continue;
      auto m = std::make_shared<Message>();
      m->task.type = Task::TERMINATE;
      m->task.customer = "default";
      m->sender = my_node().id;
      m->recver = n.id;
      van_->send(*m);
    }
  }
  bool wait_terminate(double timeout_s) {
    std::unique_lock<std::mutex> l(mu_);
    return term_cv_.wait_for(l, std::chrono::duration<double>(timeout_s), [&] { return terminated_; });
  }

  // ---- sending
  void queue(const MessagePtr& m) {
    if (!m->valid) {
      // nothing to send to this receiver: fake its acknowledgement locally
      auto ack = std::make_shared<Message>();
      ack->task = m->task;
      ack->task.type = Task::REPLY;
      ack->task.request = false;
      ack->sender = m->recver;
      ack->recver = m->sender;
      dispatch(ack);
      return;
    }
    send_q_.push(m);
  }
  void on_manage_app(std::function<void(const std::string&)> f) { manage_app_ = std::move(f); }
  void set_key_cache(bool on) { key_cache_ = on; }

  // ---- heartbeats and failure detection (host side only)
  void start_heartbeat(double interval_s, std::function<std::string()> make_report) {
    if (interval_s <= 0 || hb_thread_.joinable()) return;
    hb_thread_ = std::thread([this, interval_s, make_report] {
      std::unique_lock<std::mutex> l(hb_mu_);
      while (!done_) {
        hb_cv_.wait_for(l, std::chrono::duration<double>(interval_s));
        if (done_) break;
        auto m = std::make_shared<Message>();
        m->task.type = Task::HEARTBEATING;
        m->task.customer = "default";
        m->task.msg = make_report ? make_report() : std::string();
        m->sender = my_node().id;
        m->recver = scheduler_.id;
        queue(m);
      }
    });
  }
  std::map<std::string, HeartbeatRecord> heartbeats() { std::lock_guard<std::mutex> l(mu_); return hb_; }
  // nodes whose last heartbeat (or registration) is older than deadline_s
  std::vector<std::string> dead_nodes(double deadline_s) {
    std::vector<std::string> out;
    std::lock_guard<std::mutex> l(mu_);
    const double now = now_seconds();
    for (auto& n : nodes_) {
      if (n.id == my_node().id || n.role == Node::SCHEDULER) continue;
      auto it = hb_.find(n.id);
      const double last = it == hb_.end() ? start_time_ : it->second.when;
      if (now - last > deadline_s) out.push_back(n.id);
    }
    return out;
  }
  int last_task_of(const std::string& customer) {
    std::lock_guard<std::mutex> l(mu_);
    auto it = customers_.find(customer);
    return it == customers_.end() ? 0 : it->second->exec()->last_task();
  }

  static std::string encode_node(const Node& n) {
    std::ostringstream os;
    os << n.role << "," << n.id << "," << (n.hostname.empty() ? "127.0.0.1" : n.hostname) << "," << n.port << "," << n.key.begin << "," << n.key.end;
    return os.str();
  }
  static Node decode_node(const std::string& s) {
    Node n;
    std::istringstream is(s);
    std::string f;
    std::getline(is, f, ','); n.role = std::stoi(f);
    std::getline(is, n.id, ',');
    std::getline(is, n.hostname, ',');
    std::getline(is, f, ','); n.port = std::stoi(f);
    std::getline(is, f, ','); n.key.begin = std::stoull(f);
    std::getline(is, f, ','); n.key.end = std::stoull(f);
    return n;
  }

 private:
  void send_loop() {
    for (;;) {
      MessagePtr m;
      send_q_.wait_and_pop(m);
      if (!m || done_) return;
      Status s = van_->send(*m);
      if (!s.ok()) std::fprintf(stderr, "[%s] send failed: %s (%s)\n", my_node().id.c_str(), s.ToString().c_str(), m->short_debug().c_str());
    }
  }
  void recv_loop() {
    while (!done_) {
      MessagePtr m;
      try {
        if (!van_->recv(&m, 0.2)) continue;
      } catch (const std::exception& e) {
        std::fprintf(stderr, "[%s] bad frame dropped: %s\n", my_node().id.c_str(), e.what());
        continue;
      }
      dispatch(m);
    }
  }
  void dispatch(const MessagePtr& m) {
    const Task& t = m->task;
    if (t.type == Task::TERMINATE) {
      { std::lock_guard<std::mutex> l(mu_); terminated_ = true; }
      term_cv_.notify_all();
      return;
    }
    if (t.type == Task::HEARTBEATING) {
      std::lock_guard<std::mutex> l(mu_);
      auto& r = hb_[m->sender];
      r.when = now_seconds();
      r.report = t.msg;
      return;
    }
    if (t.type == Task::MANAGE && t.request) {
      std::istringstream is(t.msg);
      std::string cmd, tok;
      is >> cmd;
      if (cmd == "ADD") {
        is >> tok;
        MessagePtr late;
        {
          std::lock_guard<std::mutex> l(mu_);
          Node n = decode_node(tok);
          hb_[n.id].when = now_seconds();
          if (!table_sent_) {
            pending_nodes_.push_back(n);
            nodes_cv_.notify_all();
          } else {
            // A node that registers after the table went out (a stand-by node started last, a slow
            // machine): it joins the scheduler's table and receives the table itself, so that it is
            // told when the job ends.  Workers and servers are never late: the broadcast waits for them.
            bool known = false;
            for (auto& o : nodes_) known |= o.id == n.id;
            if (!known) {
              n.key = Range::all();
              nodes_.push_back(n);
              van_->connect(n);
            }
            late = std::make_shared<Message>();
            late->task.type = Task::MANAGE;
            late->task.request = true;
            late->task.customer = "default";
            late->task.msg = "INIT";
            for (auto& o : nodes_) late->task.msg += " " + encode_node(o);
            late->sender = my_node().id;
            late->recver = n.id;
          }
        }
        if (late) queue(late);
      } else if (cmd == "INIT") {
        std::vector<Node> nodes;
        while (is >> tok) nodes.push_back(decode_node(tok));
        set_nodes(nodes);
      } else if (cmd == "APP") {
        std::string rest;
        std::getline(is, rest, '\0');
        if (manage_app_) manage_app_(rest);
      }
      return;
    }
    Customer* c = nullptr;
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = customers_.find(t.customer);
      if (it == customers_.end() || !it->second->exec()->initialized()) {
        orphan_[t.customer].push_back(m);     // customer not created yet: keep until it registers
        return;
      }
      c = it->second;
      ++delivering_[c];
    }
    c->exec()->accept(m);
    {
      std::lock_guard<std::mutex> l(mu_);
      if (--delivering_[c] == 0) delivering_.erase(c);
    }
    deliver_cv_.notify_all();
  }

  std::shared_ptr<Van> van_;
  Node scheduler_;
  int num_workers_, num_servers_, num_replicas_;
  std::atomic<bool> done_{false};
  std::thread recv_thread_, send_thread_, hb_thread_;
  ThreadsafeQueue<MessagePtr> send_q_;
  std::mutex mu_, hb_mu_;
  std::condition_variable nodes_cv_, term_cv_, hb_cv_;
  std::map<std::string, Customer*> customers_;
  std::map<Customer*, int> delivering_;      // customers whose executor is being handed a message right now
  std::condition_variable deliver_cv_;
  std::map<std::string, std::vector<MessagePtr>> orphan_;
  std::vector<Node> nodes_, pending_nodes_;
  bool nodes_ready_ = false, table_sent_ = false, terminated_ = false, key_cache_ = true;
  std::map<std::string, HeartbeatRecord> hb_;
  std::function<void(const std::string&)> manage_app_;
  double start_time_ = now_seconds();
  friend class Customer;
  friend class Executor;
};

// ------------------------------------------------------------------ Executor
inline void Executor::init(const std::vector<Node>& nodes, const Node& me, int num_replicas) {
  std::lock_guard<std::mutex> l(mu_);
  std::map<std::string, RNodePtr> old;
  old.swap(nodes_);
  groups_.clear();
  partitions_.clear();
  for (const char* g : {kServerGroup, kWorkerGroup, kActiveGroup, kReplicaGroup, kOwnerGroup, kLiveGroup}) {
    Node n;
    n.role = Node::GROUP;
    n.id = g;
    add(n);
    groups_[g];
  }
  for (auto& n : nodes) {
    add(n);
    auto it = old.find(n.id);
    if (it != old.end()) {   // keep clocks and pending state of nodes we already knew
      nodes_[n.id] = it->second;
      it->second->node = n;
      for (auto& g : groups_) for (auto& r : g.second) if (r->node.id == n.id) r = it->second;
    }
  }
  for (auto& g : groups_) {
    if (nodes_.count(g.first) && nodes_[g.first]->node.role != Node::GROUP) continue;
    std::stable_sort(g.second.begin(), g.second.end(), [](const RNodePtr& a, const RNodePtr& b) { return a->node.key.begin < b->node.key.begin; });
  }
  if (me.role == Node::SERVER && num_replicas > 0) {
    auto& servers = groups_[kServerGroup];
    const int n = (int)servers.size();
    int pos = 0;
    for (; pos < n; ++pos) if (servers[pos]->node.id == me.id) break;
    if (pos < n && num_replicas < n) {
      for (int i = 1; i <= num_replicas; ++i) {
        groups_[kReplicaGroup].push_back(servers[(pos - i + n) % n]);   // ring neighbours before me
        groups_[kOwnerGroup].push_back(servers[(pos + i) % n]);         // and after me
      }
    }
  }
  for (auto& g : groups_) {
    auto& p = partitions_[g.first];
    for (auto& r : g.second) p.push_back(r->node.key.begin);
    p.push_back(g.second.empty() ? 0 : g.second.back()->node.key.end);
  }
  inited_ = true;
  cv_.notify_all();
}

inline void Executor::run() {
  for (;;) {
    MessagePtr msg;
    size_t queued = 0;
    {
      std::unique_lock<std::mutex> l(mu_);
      for (;;) {
        if (done_) return;
        bool dropped = false;
        for (auto it = recved_.begin(); it != recved_.end(); ++it) {
          auto s = rnode_nolock((*it)->sender);
          if (!s) {
            std::fprintf(stderr, "[%s] message from unknown node %s ignored\n", obj_->name().c_str(), (*it)->sender.c_str());
            recved_.erase(it);
            dropped = true;
            break;
          }
          const int w = (*it)->task.wait_time;
          if (!(*it)->task.request || w <= kInvalidTime || s->incoming.try_wait(w)) {
            msg = *it;
            recved_.erase(it);
            queued = recved_.size();
            break;
          }
        }
        if (msg) break;
        if (!dropped) cv_.wait_for(l, std::chrono::milliseconds(50));
      }
    }
    const bool req = msg->task.request;
    const int t = msg->task.time;
    RNodePtr sender = rnode(msg->sender);
    if (verbose_flag())
      std::fprintf(stderr, "[%s@%s] %s t=%d wait=%d from %s (%zu queued)\n", obj_->name().c_str(), po_->my_node().id.c_str(),
                   req ? "request" : "reply", t, msg->task.wait_time, msg->sender.c_str(), queued);
    if (req) { sender->incoming.start(t); last_task_ = t; }
    if (msg->task.type != Task::REPLY && obj_->process) obj_->process(msg);
    ++processed;
    if (req) {
      if (msg->finished) {
        sender->incoming.finish(t);
        notify();
        if (!msg->replied) obj_->reply(msg);
      }
    } else {
      std::function<void()> h;
      std::string orig;
      if (!msg->task.msg.empty()) {
        std::lock_guard<std::mutex> l(mu_);
        replies_[t][msg->sender] = msg->task.msg;
      }
      {
        std::lock_guard<std::mutex> l(sender->mu);
        auto b = sender->recv_handles.find(t);
        if (b != sender->recv_handles.end()) h = b->second;
      }
      if (h) h();
      sender->outgoing.finish(t);
      {
        std::lock_guard<std::mutex> l(sender->mu);
        auto it = sender->pending.find(t);
        if (it == sender->pending.end()) continue;     // duplicate or unsolicited reply
        orig = it->second->original_recver;
        sender->pending.erase(it);
        sender->recv_handles.erase(t);
      }
      auto members = group(orig);
      bool all = !members.empty();
      for (auto& m : members) all = all && m->outgoing.try_wait(t);
      if (all) {
        RNodePtr o = rnode(orig);
        std::function<void()> f;
        if (o) {
          std::lock_guard<std::mutex> l(o->mu);
          auto a = o->fin_handles.find(t);
          if (a != o->fin_handles.end()) { f = a->second; o->fin_handles.erase(a); }
        }
        if (f) f();
      }
    }
  }
}

// ------------------------------------------------------------------ Customer
inline Customer::Customer(Postoffice* po, std::string name) : po_(po), name_(std::move(name)) {
  exec_.reset(new Executor(this, po));
  po_->add_customer(this);
}
inline Customer::~Customer() {
  po_->remove_customer(this);
  exec_->stop();
}
inline int Customer::submit(const MessagePtr& msg) {
  Task& task = msg->task;
  task.request = true;
  task.customer = name_;
  RNodePtr dst = exec_->rnode(msg->recver);
  if (!dst) throw std::runtime_error(name_ + ": unknown receiver " + msg->recver);
  msg->original_recver = msg->recver;
  auto members = exec_->group(msg->recver);
  {
    // the logical clocks of all remote nodes of this customer advance under one lock: a group's clock
    // reads its members' clocks, and several application threads may submit at the same time
    std::lock_guard<std::mutex> lc(exec_->clock_mu);
    if (task.time > kInvalidTime) {
      dst->time = std::max(task.time, dst->time);
    } else {
      for (auto& w : members) dst->time = std::max(dst->time, w->time);
      task.time = ++dst->time;
    }
    for (auto& w : members) w->time = std::max(task.time, w->time);
  }
  if (msg->fin_handle) {
    std::lock_guard<std::mutex> l(dst->mu);
    dst->fin_handles[task.time] = msg->fin_handle;
  }
  const int t = task.time;
  for (auto& w : members) w->outgoing.start(t);
  auto pieces = slice(msg, exec_->partition(msg->recver));
  if (pieces.size() != members.size()) throw std::runtime_error(name_ + ": slice size mismatch");
  for (size_t i = 0; i < members.size(); ++i) {
    auto& w = members[i];
    pieces[i]->sender = po_->my_node().id;
    pieces[i]->recver = w->node.id;
    pieces[i]->original_recver = msg->recver;
    {
      std::lock_guard<std::mutex> l(w->mu);
      w->pending[t] = pieces[i];
      if (msg->recv_handle) w->recv_handles[t] = msg->recv_handle;
    }
    if (pieces[i]->valid) {
      // the key-cache decision and the place in the send queue are taken together: the receiver
      // replays the same sequence of cache updates, so two threads must not interleave here
      std::lock_guard<std::mutex> ls(w->send_mu);
      w->cache_key_sender(pieces[i], exec_->key_cache_enabled);
      po_->queue(pieces[i]);
    } else {
      po_->queue(pieces[i]);
    }
  }
  if (members.empty() && msg->fin_handle) msg->fin_handle();
  if (msg->wait) wait_out(msg->recver, t);
  return t;
}
inline bool Customer::wait_out(const std::string& node, int t, double timeout_s) {
  bool ok = true;
  for (auto& w : exec_->group(node)) ok = w->outgoing.wait(t, timeout_s) && ok;
  return ok;
}
inline bool Customer::try_wait_out(const std::string& node, int t) {
  for (auto& w : exec_->group(node)) if (!w->outgoing.try_wait(t)) return false;
  return true;
}
inline bool Customer::wait_in(const std::string& node, int t, double timeout_s) {
  bool ok = true;
  for (auto& w : exec_->group(node)) ok = w->incoming.wait(t, timeout_s) && ok;
  return ok;
}
inline void Customer::finish_in(const std::string& node, int t) {
  for (auto& w : exec_->group(node)) w->incoming.finish(t);
  exec_->notify();
}
inline void Customer::finish_out(const std::string& node, int t) {
  for (auto& w : exec_->group(node)) w->outgoing.finish(t);
}
inline void Customer::reply(const MessagePtr& req, std::string key, std::vector<std::string> values, std::string payload) {
  auto m = std::make_shared<Message>();
  m->task = req->task;
  m->task.request = false;
  m->task.msg = std::move(payload);
  const bool data = !key.empty() || !values.empty();
  m->task.type = data ? req->task.type : Task::REPLY;
  if (!m->task.msg.empty() && !data) m->task.type = Task::REPLY;
  m->task.has_key = !key.empty();
  m->key = std::move(key);
  m->value = std::move(values);
  m->sender = po_->my_node().id;
  m->recver = req->sender;
  req->replied = true;
  po_->queue(m);
}

}  // namespace psb
