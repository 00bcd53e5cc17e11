// Native self-test of the host runtime, meant to be built with -fsanitize=thread or
// -fsanitize=address,undefined and run on a machine without a GPU.
//
// The reference has no sanitizer builds and a few documented hazards ("Van::send is not thread
// safe", src/system/van.cc:106-108; key/value maps shared between the app thread and the executor
// thread, guarded only by protocol order).  This program drives the same code paths from several
// threads at once so that a sanitizer can see them: 1 scheduler + 2 servers + 2 workers over the
// in-process van, membership, concurrent pushes from two threads per worker, pulls with a
// wait_time dependency on the push, heartbeats and the deadline-based failure detector, shutdown
// while traffic is still queued; then the thread pool, the slot reader's parser threads and the feature
// store's prefetch threads against two solver threads.  Exit code 0 = every check passed (the sanitizer adds its own
// non-zero exit code when it finds something).
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "../darlin_cpu.h"
#include "../feature_station.h"
#include "../ocean.h"
#include "../data.h"
#include "../kv.h"
#include "../runtime.h"
#include "../shared_param.h"

using namespace psb;

namespace {

int g_failed = 0;
#define CHECK_TRUE(cond)                                                          \
  do {                                                                            \
    if (!(cond)) {                                                                \
      std::fprintf(stderr, "selftest: %s failed (line %d)\n", #cond, __LINE__);   \
      ++g_failed;                                                                 \
    }                                                                             \
  } while (0)

std::string bytes_of(const std::vector<uint64_t>& v) {
  return std::string(reinterpret_cast<const char*>(v.data()), v.size() * sizeof(uint64_t));
}
std::string bytes_of(const std::vector<double>& v) {
  return std::string(reinterpret_cast<const char*>(v.data()), v.size() * sizeof(double));
}

struct NodeRt {  // one node of the in-process cluster
  std::shared_ptr<Van> van;
  std::unique_ptr<Postoffice> po;
  std::unique_ptr<Customer> cust;
  std::mutex mu;
  std::map<uint64_t, double> store;   // server: key -> summed value
  std::atomic<int> pushes{0};
};

}  // namespace

// PSB_SELFTEST_TRACE=1: name every section on stderr as it starts (to see where a run stopped)
#define SECTION(name) do { if (std::getenv("PSB_SELFTEST_TRACE")) std::fprintf(stderr, "selftest: section %s\n", name); } while (0)

int main(int argc, char** argv) {
  const bool tcp = argc > 1 && std::strcmp(argv[1], "tcp") == 0;   // loopback TCP van instead of the in-process hub
  const int W = 2, S = 2, kRounds = 40, kThreadsPerWorker = 2;
  auto hub = std::make_shared<InprocHub>();
  std::vector<std::pair<std::string, int>> ids = {{"H", Node::SCHEDULER}, {"W0", Node::WORKER}, {"W1", Node::WORKER},
                                                   {"S0", Node::SERVER}, {"S1", Node::SERVER}};
  std::map<std::string, std::unique_ptr<NodeRt>> rt;
  Node sched;
  for (auto& id : ids) {
    Node n;
    n.role = id.second;
    n.id = id.first;
    n.hostname = "127.0.0.1";
    auto r = std::make_unique<NodeRt>();
    if (tcp) {
      auto tv = std::make_shared<TcpVan>(n);
      CHECK_TRUE(tv->bind().ok());
      tv->set_compress(true);
      r->van = tv;
    } else {
      r->van = std::make_shared<InprocVan>(hub, n);
    }
    r->po = std::make_unique<Postoffice>(r->van, W, S);
    if (id.first == "H") sched = r->van->my_node;
    r->po->set_scheduler(sched);
    r->po->start();
    rt[id.first] = std::move(r);
  }
  for (auto& id : ids)
    if (id.first != "H") rt[id.first]->po->register_with_scheduler();
  CHECK_TRUE(rt["H"]->po->wait_nodes_and_init(10.0));
  for (auto& id : ids)
    if (id.first != "H") CHECK_TRUE(rt[id.first]->po->wait_nodes_ready(10.0));

  SECTION("customers");
  // customers: servers sum pushed values per key and answer pulls with the current sums
  std::atomic<int> pulled_ok{0};
  for (auto& id : ids) {
    NodeRt* r = rt[id.first].get();
    r->cust = std::make_unique<Customer>(r->po.get(), "w");
    if (id.second == Node::SERVER) {
      r->cust->process = [r](const MessagePtr& m) {
        if (!m->task.request) return;
        const size_t n = m->key.size() / sizeof(uint64_t);
        const uint64_t* k = reinterpret_cast<const uint64_t*>(m->key.data());
        if (m->task.cmd == 1) {
          const double* v = reinterpret_cast<const double*>(m->value.at(0).data());
          std::lock_guard<std::mutex> l(r->mu);
          for (size_t i = 0; i < n; ++i) r->store[k[i]] += v[i];
          ++r->pushes;
        } else if (m->task.cmd == 2) {
          std::vector<double> out(n);
          {
            std::lock_guard<std::mutex> l(r->mu);
            for (size_t i = 0; i < n; ++i) out[i] = r->store[k[i]];
          }
          r->cust->reply(m, m->key, {bytes_of(out)});
        }
      };
    } else if (id.second == Node::WORKER) {
      r->cust->process = [&pulled_ok](const MessagePtr& m) {
        if (!m->task.request && m->task.cmd == 2 && !m->value.empty()) ++pulled_ok;
      };
    }
  }

  SECTION("heartbeats");
  // heartbeats from every non-scheduler node
  for (auto& id : ids)
    if (id.first != "H") {
      std::string who = id.first;
      rt[id.first]->po->start_heartbeat(0.02, [who] { return "alive " + who; });
    }

  SECTION("concurrent pushes");
  // concurrent pushes (two threads per worker), each followed by a pull that waits for it
  const uint64_t half = (~0ull - 1) / 2;
  std::vector<std::thread> threads;
  for (int w = 0; w < W; ++w)
    for (int t = 0; t < kThreadsPerWorker; ++t)
      threads.emplace_back([&, w, t] {
        Customer* c = rt["W" + std::to_string(w)]->cust.get();
        for (int r = 0; r < kRounds; ++r) {
          std::vector<uint64_t> keys = {3, 7 + (uint64_t)t, half + 5, half + 9 + (uint64_t)r % 3};
          std::vector<double> vals = {1.0, 2.0, 3.0, 4.0};
          auto push = std::make_shared<Message>();
          push->recver = kServerGroup;
          push->task.cmd = 1;
          push->task.has_key = true;
          push->key = bytes_of(keys);
          push->value.push_back(bytes_of(vals));
          push->task.has_key_range = true;
          push->task.key_range = Range::all();
          const int tp = c->submit(push);
          auto pull = std::make_shared<Message>();
          pull->recver = kServerGroup;
          pull->task.cmd = 2;
          pull->task.has_key = true;
          pull->key = bytes_of(keys);
          pull->task.has_key_range = true;
          pull->task.key_range = Range::all();
          pull->task.wait_time = tp;
          const int tl = c->submit(pull);
          if (!c->wait_out(kServerGroup, tl, 20.0)) ++g_failed;
        }
      });
  for (auto& th : threads) th.join();

  SECTION("push sums");
  // every push arrived exactly once at both servers; sums are what the workers sent
  const int total_pushes = W * kThreadsPerWorker * kRounds;
  CHECK_TRUE(rt["S0"]->pushes == total_pushes && rt["S1"]->pushes == total_pushes);
  {
    std::lock_guard<std::mutex> l(rt["S0"]->mu);
    CHECK_TRUE(rt["S0"]->store[3] == 1.0 * total_pushes);
  }
  {
    std::lock_guard<std::mutex> l(rt["S1"]->mu);
    CHECK_TRUE(rt["S1"]->store[half + 5] == 3.0 * total_pushes);
  }
  CHECK_TRUE(pulled_ok == 2 * total_pushes);   // one data reply per server and pull

  SECTION("batch shared parameter");
  // the native shared-parameter customer under the batch solvers' protocol: workers push keys, then per round
  // values at time t; a solver thread on every server waits for both pushes, takes the aggregate, writes the new
  // weights and releases t + 1; the workers' pulls (time t + 2, waiting for t + 1) must see exactly those weights.
  // The servers' executor threads (push / pull handling) and solver threads (received / set_values_range) run
  // at the same time, rounds overlap between the two workers.
  {
    std::map<std::string, std::unique_ptr<SharedParamCustomer>> sp;
    for (auto& id : ids)
      if (id.first != "H") sp[id.first] = std::make_unique<SharedParamCustomer>(rt[id.first]->po.get(), "p", 2, W, 2, 2.0);
    const std::vector<uint64_t> wk[2] = {{2, 4, 6, half + 2, half + 4}, {4, 6, 8, half + 4, half + 8}};
    const int kR = 20;
    std::atomic<int> bad{0};
    std::vector<std::thread> ts;
    for (int w = 0; w < W; ++w)
      ts.emplace_back([&, w] {
        auto* c = sp["W" + std::to_string(w)].get();
        auto mk = [&](int cmd, int time, int wait) {
          auto m = std::make_shared<Message>();
          m->recver = kServerGroup;
          m->task.cmd = cmd;
          m->task.time = time;
          m->task.wait_time = wait;
          m->task.has_key = true;
          m->key = bytes_of(wk[w]);
          m->task.has_key_range = true;
          m->task.key_range = Range::all();
          return m;
        };
        c->submit(mk(1, 10, -1));                                   // keys only
        if (!c->wait_out(kServerGroup, 10, 20.0)) ++bad;
        for (int r = 0; r < kR; ++r) {
          const int t = 20 + 10 * r;
          // the first values wait for the servers' time 11 (all workers' keys merged, values initialised): nothing else
          // keeps a fast worker's values from reaching a server before a slow worker's keys
          auto push = mk(1, t, r == 0 ? 11 : -1);
          std::vector<double> v(wk[w].size(), (double)(w + 1));     // every key of worker w carries w + 1
          push->value.push_back(bytes_of(v));
          c->submit(push);
          c->submit(mk(2, t + 2, t + 1));
          if (!c->wait_out(kServerGroup, t + 2, 20.0)) {
            std::fprintf(stderr, "selftest: worker %d round %d: no reply to the pull at %d (S0 %d, S1 %d)\n", w, r, t + 2,
                         (int)c->try_wait_out("S0", t + 2), (int)c->try_wait_out("S1", t + 2));
            for (const char* sid : {"S0", "S1"}) {                   // what the servers hold for this worker
              auto* sc = sp[sid].get();
              auto me = sc->exec()->rnode("W" + std::to_string(w));
              std::fprintf(stderr, "selftest:   %s: time %d of W%d finished: %d, started %d; waiting requests:", sid, t + 1, w,
                           me ? (int)me->incoming.try_wait(t + 1) : -1, me ? (int)me->incoming.try_wait(t) : -1);
              for (auto& q : sc->exec()->pending_requests())
                std::fprintf(stderr, " [%s cmd %d t %d wait %d]", q->sender.c_str(), q->task.cmd, q->task.time, q->task.wait_time);
              std::fprintf(stderr, " processed %d\n", (int)sc->exec()->processed);
            }
            ++bad;
            break;                                                   // the later rounds would only time out as well
          }
          auto got = c->take_pulled(t + 2, {"S0", "S1"});
          const double* x = reinterpret_cast<const double*>(got.second.data());     // values only: a value reply carries no keys
          if (got.second.size() != wk[w].size() * 8) { ++bad; continue; }
          for (size_t i = 0; i < wk[w].size(); ++i) {
            const uint64_t k = wk[w][i];
            const bool both = k == 4 || k == 6 || k == half + 4;               // keys that the two workers share
            if (x[i] != (r + 1) * (both ? 3.0 : (double)(w + 1))) ++bad;
          }
        }
      });
    for (int sv = 0; sv < S; ++sv)
      ts.emplace_back([&, sv] {
        auto* c = sp["S" + std::to_string(sv)].get();
        if (!c->wait_in(kWorkerGroup, 10, 20.0)) ++bad;
        c->init_values(0, 0.0);
        c->finish_in(kWorkerGroup, 11);
        for (int r = 0; r < kR; ++r) {
          const int t = 20 + 10 * r;
          if (!c->wait_in(kWorkerGroup, t, 20.0)) {
            std::fprintf(stderr, "selftest: server %d round %d: the pushes at %d did not both arrive\n", sv, r, t);
            ++bad;
            break;
          }
          auto agg = c->received(t);
          auto w = c->values(0);
          if (agg.nval != 1 || agg.hi - agg.lo != w.size()) {
            std::fprintf(stderr, "selftest: server %d round %d: aggregate of %d values per key over [%zu, %zu), %zu values, %zu keys here\n",
                         sv, r, agg.nval, agg.lo, agg.hi, w.size(), c->keys(0).size());
            ++bad;
            break;
          }
          for (size_t i = 0; i < w.size(); ++i) w[i] += agg.vals[i];
          c->set_values_range(0, agg.lo, w.data(), w.size());
          c->finish_in(kWorkerGroup, t + 1);
        }
      });
    for (auto& th : ts) th.join();
    CHECK_TRUE(bad == 0);
    CHECK_TRUE(sp["S0"]->keys(0) == (std::vector<uint64_t>{2, 4, 6, 8}));
    for (auto& kv : sp) kv.second->exec()->stop();
  }

  SECTION("online shared parameter");
  // the online solver's parameter customer: two workers push (gradient, positive, negative) per key without
  // waiting and pull in between, the servers update their FTRL models on arrival; stats are read meanwhile
  {
    std::map<std::string, std::unique_ptr<FTRLParamCustomer>> fp;
    for (auto& id : ids)
      if (id.first != "H") fp[id.first] = std::make_unique<FTRLParamCustomer>(rt[id.first]->po.get(), "f", 0.1, 1.0, 0.01, 0.0, 4096, 2);
    std::atomic<int> bad{0};
    std::vector<std::thread> ts;
    for (int w = 0; w < W; ++w)
      ts.emplace_back([&, w] {
        auto* c = fp["W" + std::to_string(w)].get();
        int last = -1;
        for (int r = 0; r < 30; ++r) {
          std::vector<uint64_t> keys = {5, 9 + (uint64_t)w, half + 1, half + 7 + (uint64_t)(r % 2)};
          std::vector<double> g = {0.5, -0.25, 1.0, -1.5}, pos = {1, 0, 1, 0}, neg = {0, 1, 0, 1};
          auto push = std::make_shared<Message>();
          push->recver = kServerGroup;
          push->task.cmd = 1;
          push->task.has_key = true;
          push->key = bytes_of(keys);
          push->value = {bytes_of(g), bytes_of(pos), bytes_of(neg)};
          push->task.has_key_range = true;
          push->task.key_range = Range::all();
          last = c->submit(push);
          auto pull = std::make_shared<Message>();
          pull->recver = kServerGroup;
          pull->task.cmd = 2;
          pull->task.has_key = true;
          pull->key = bytes_of(keys);
          pull->task.has_key_range = true;
          pull->task.key_range = Range::all();
          const int tl = c->submit(pull);
          if (!c->wait_out(kServerGroup, tl, 20.0)) { ++bad; continue; }
          if (c->take_pulled(tl, {"S0", "S1"}).second.size() != keys.size() * 8) ++bad;
        }
        if (!c->wait_out(kServerGroup, last, 20.0)) ++bad;
      });
    ts.emplace_back([&] {
      for (int i = 0; i < 200; ++i) { double a, b; size_t n; fp["S0"]->stats(&a, &b, &n); fp["S1"]->size(); }
    });
    for (auto& th : ts) th.join();
    CHECK_TRUE(bad == 0);
    CHECK_TRUE(fp["S0"]->size() == 3 && fp["S1"]->size() == 3);       // {5, 9, 10} and {half + 1, half + 7, half + 8}
    std::vector<Key> k; std::vector<double> wv;
    fp["S0"]->nonzero(&k, &wv);
    CHECK_TRUE(!k.empty());
    for (auto& kv : fp) kv.second->exec()->stop();
  }

  SECTION("failure detector");
  // failure detector: everybody reported recently; after S1 stops, it shows up as dead
  std::this_thread::sleep_for(std::chrono::milliseconds(100));
  CHECK_TRUE(rt["H"]->po->dead_nodes(5.0).empty());
  rt["S1"]->cust->exec()->stop();
  rt["S1"]->po->stop();
  std::this_thread::sleep_for(std::chrono::milliseconds(300));
  auto dead = rt["H"]->po->dead_nodes(0.2);
  CHECK_TRUE(dead.size() == 1 && dead[0] == "S1");

  SECTION("containers");
  // host containers touched from several threads
  {
    ThreadsafeQueue<int> q;
    std::atomic<long> sum{0};
    std::vector<std::thread> ts;
    for (int p = 0; p < 3; ++p) ts.emplace_back([&q] { for (int i = 1; i <= 1000; ++i) q.push(i); });
    for (int cns = 0; cns < 3; ++cns) ts.emplace_back([&q, &sum] { int v; for (int i = 0; i < 1000; ++i) { q.wait_and_pop(v); sum += v; } });
    for (auto& t : ts) t.join();
    CHECK_TRUE(sum == 3L * 500500);
    ThreadPool pool(4);
    std::atomic<int> done{0};
    for (int i = 0; i < 64; ++i) pool.add([&done] { ++done; });
    pool.join();
    CHECK_TRUE(done == 64);
  }

  SECTION("data ingest");
  // data ingest: four LIBSVM files parsed by four threads into the slot cache, then served from it
  if (argc > 2) {
    const std::string dir = argv[2];
    std::vector<std::string> files;
    size_t nnz = 0;
    for (int f = 0; f < 4; ++f) {
      files.push_back(dir + "/part-" + std::to_string(f));
      std::ofstream out(files.back());
      for (int i = 0; i < 500; ++i) {
        out << (i % 3 ? "+1" : "-1");
        for (int k = 0; k < 1 + (i + f) % 7; ++k) { out << " " << (10 * k + f + 1) << ":" << (0.5 + k); ++nnz; }
        out << "\n";
      }
    }
    for (int round = 0; round < 2; ++round) {
      SlotReader rd;
      rd.init(files, TextFormat::LIBSVM, dir + "/cache", true);
      ExampleInfo info;
      const int hits = rd.read(4, &info);
      CHECK_TRUE(hits == (round == 0 ? 0 : 4));
      CHECK_TRUE(info.num_ex == 2000);
      CHECK_TRUE(rd.index(1).size() == nnz && rd.value(1).size() == nnz && rd.offset(1).back() == nnz);
    }
  }

  SECTION("feature store");
  // feature store on disk: one thread queues read-ahead, two solver threads take, use and release ranges under a
  // memory limit that holds about two of them; then the block gradient on a loaded range against the resident arrays
  if (argc > 2) {
    const std::string dir = argv[2];
    const int64_t cols = 240, rows = 300;
    std::vector<int64_t> indptr(1, 0);
    std::vector<int32_t> indices;
    std::vector<double> values;
    for (int64_t j = 0; j < cols; ++j) {
      for (int64_t r = j % 5; r < rows; r += 3 + j % 11) { indices.push_back((int32_t)r); values.push_back(0.25 + (r + j) % 7); }
      indptr.push_back((int64_t)indices.size());
    }
    FeatureStation st(dir + "/features", "T0", 12, 3, 64, false);
    st.add_group(1, rows, indptr.data(), cols, indices.data(), values.data());
    CHECK_TRUE(st.mem_size() == indices.size() * 12 + (cols + 1) * 8);
    const int tasks = 24;
    std::thread ahead([&] { for (int t = 0; t < tasks; t += 2) st.prefetch(t, 1, t * 10, t * 10 + 10); });   // even tasks only
    std::atomic<int> bad{0};
    auto solver = [&](int first) {
      for (int t = first; t < tasks; t += 2) {
        auto b = st.get(t, 1, t * 10, t * 10 + 10);
        for (int64_t j = 0; j < 10; ++j) {
          const int64_t c = t * 10 + j;
          if (b->indptr[j + 1] - b->indptr[j] != indptr[c + 1] - indptr[c]) ++bad;
          for (int64_t p = b->indptr[j]; p < b->indptr[j + 1]; ++p)
            if (b->indices[p - b->pos0] != indices[p] || b->values[p - b->pos0] != values[p]) ++bad;
        }
        st.drop(t);
      }
    };
    std::thread s0(solver, 0), s1(solver, 1);
    ahead.join(); s0.join(); s1.join();
    CHECK_TRUE(bad == 0);
    // a read-ahead that lost the race against its solver thread (the task was taken, used and dropped before the
    // read-ahead was queued) stays until somebody drops it: release those before looking at the totals
    for (int k = 0; k < 400 && !(st.resident_bytes() == 0 && st.pending() == 0); ++k) {
      for (int t = 0; t < tasks; ++t) st.drop(t);
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    CHECK_TRUE(st.resident_bytes() == 0 && st.pending() == 0);
    auto stats = st.stats();
    CHECK_TRUE(stats.hits + stats.misses == (uint64_t)tasks && stats.misses >= (uint64_t)tasks / 2);

    std::vector<double> y(rows), dual(rows), delta(cols, 1.0), G0(40), U0(40), G1(40), U1(40);
    std::vector<uint8_t> active(cols, 1);
    for (int64_t r = 0; r < rows; ++r) { y[r] = r % 2 ? 1 : -1; dual[r] = 0.5 + (r % 9) * 0.2; }
    active[105] = 0;
    CscBlock whole{indptr.data(), indices.data(), values.data(), 100, 140};
    darlin_block_gradient(whole, y.data(), dual.data(), delta.data(), active.data(), G0.data(), U0.data(), 1);
    auto b = st.get(1000, 1, 100, 140);
    CscBlock part{b->indptr, b->indices, b->values, 100, 140, 100, b->pos0};
    darlin_block_gradient(part, y.data(), dual.data(), delta.data(), active.data(), G1.data(), U1.data(), 2);
    for (int i = 0; i < 40; ++i)
      CHECK_TRUE((G0[i] == G1[i] && U0[i] == U1[i]) || (i == 5 && G0[i] != G0[i] && G1[i] != G1[i]));
    st.drop(1000);

    SECTION("block store");
    // the general block store under concurrent prefetchers and users
    {
      Ocean oc(dir + "/ocean", "T0", 3, 4, false);
      std::vector<uint64_t> cuts;
      for (uint64_t c = 0; c <= (uint64_t)cols; c += 20) cuts.push_back(c);
      CHECK_TRUE(oc.set_partition(1, cuts));
      std::vector<uint64_t> off(indptr.begin(), indptr.end());
      CHECK_TRUE(oc.dump(1, Ocean::FEATURE_OFFSET, off.data(), off.size(), 8));
      CHECK_TRUE(oc.dump(1, Ocean::FEATURE_KEY, indices.data(), indices.size(), 4));
      CHECK_TRUE(oc.dump(1, Ocean::FEATURE_VALUE, values.data(), values.size(), 8));
      CHECK_TRUE(!oc.dump(1, Ocean::FEATURE_VALUE, values.data(), values.size(), 8));
      const size_t nb = oc.num_blocks(1);
      std::atomic<int> wrong{0};
      std::thread pre([&] { for (size_t b = 0; b < nb; ++b) { oc.prefetch(1, b); oc.prefetch(1, b); } });
      auto user = [&] {
        for (size_t b = 0; b < nb; ++b) {
          auto k = oc.get(1, b, Ocean::FEATURE_KEY);
          auto o = oc.get(1, b, Ocean::FEATURE_OFFSET);
          const int64_t p0 = indptr[20 * b], p1 = indptr[20 * b + 20];
          if (!k || !o || k->size() != (size_t)(p1 - p0) * 4 || o->size() != 21 * 8) { ++wrong; continue; }
          if (std::memcmp(k->data(), indices.data() + p0, k->size()) != 0) ++wrong;
          oc.drop(1, b);
          oc.drop(1, b);
        }
      };
      std::thread u0(user), u1(user);
      pre.join(); u0.join(); u1.join();
      CHECK_TRUE(wrong == 0);
      CHECK_TRUE(oc.pending() == 0);
    }
  }

  SECTION("shutdown");
  // shutdown with traffic possibly still queued
  for (auto& id : ids) {
    rt[id.first]->cust->exec()->stop();
    rt[id.first]->po->stop();
  }
  for (auto& id : ids) rt[id.first]->cust.reset();
  std::printf("selftest (%s van): %s\n", tcp ? "tcp" : "in-process", g_failed == 0 ? "ok" : "FAILED");
  return g_failed == 0 ? 0 : 1;
}
