// Control-plane message model: Range, Node, Task, Message, the wire encoding, key-range
// slicing of key-ordered messages and the sorted merge-join (`match`) used by KVVector.
//
// Counterparts in the reference: src/base/range.h, src/proto/{node,task,range}.proto,
// src/system/message.{h,cc} (Message, sliceKeyOrderedMsg :89-123, match :134-226).
// Keys travel as raw little-endian uint64 bytes, values as raw bytes of k arrays whose length
// is a multiple of the number of keys.
#pragma once
#include "util.h"

namespace psb {

struct Range {
  uint64_t begin = 0, end = 0;
  Range() = default;
  Range(uint64_t b, uint64_t e) : begin(b), end(e) {}
  static Range all() { return Range(0, kMaxKey); }
  uint64_t size() const { return end - begin; }
  bool valid() const { return end >= begin; }
  bool empty() const { return begin >= end; }
  bool contains(uint64_t v) const { return begin <= v && v < end; }
  Range intersect(const Range& o) const { return Range(std::max(begin, o.begin), std::min(end, o.end)); }
  Range set_union(const Range& o) const { return Range(std::min(begin, o.begin), std::max(end, o.end)); }
  bool operator==(const Range& o) const { return begin == o.begin && end == o.end; }
  bool operator<(const Range& o) const { return begin != o.begin ? begin < o.begin : end < o.end; }
  // i-th of n even parts, exact 128-bit integer arithmetic
  Range even_divide(size_t n, size_t i) const {
    const unsigned __int128 sz = end - begin;
    const uint64_t b = begin + (uint64_t)(sz * i / n);
    const uint64_t e = (i + 1 == n) ? end : begin + (uint64_t)(sz * (i + 1) / n);
    return Range(b, e);
  }
  std::string str() const { return "[" + std::to_string(begin) + "," + std::to_string(end) + ")"; }
};

struct Node {
  enum Role { SERVER = 0, WORKER = 1, MANAGER = 2, SCHEDULER = 3, GROUP = 4, UNUSED = 5 };
  int role = WORKER;
  std::string id, hostname;
  int port = 0;
  Range key;
};

// group ids (src/system/executor.h:7-18)
static const char* const kServerGroup = "all_servers";
static const char* const kWorkerGroup = "all_workers";
static const char* const kActiveGroup = "all_actives";   // servers + workers
static const char* const kReplicaGroup = "all_replicas";
static const char* const kOwnerGroup = "all_owners";
static const char* const kLiveGroup = "all_lives";       // everything but the scheduler's own id

struct Task {
  enum Type { TERMINATE = 1, TERMINATE_CONFIRM = 2, REPLY = 3, MANAGE = 4, CALL_CUSTOMER = 5, HEARTBEATING = 6 };
  int type = CALL_CUSTOMER;
  bool request = false;
  std::string customer;
  int time = -1;
  int wait_time = -1;
  bool has_key = false;
  bool has_key_range = false;
  Range key_range;
  uint32_t key_signature = 0;
  int key_channel = 0;
  bool erase_key_cache = false;
  std::vector<uint64_t> uncompressed_size;
  std::string msg;      // opaque application payload (text-format call descriptor, report, ...)
  int cmd = 0;          // shared-parameter command: 1 push, 2 pull (0 = application call)
  uint32_t flags = 0;   // CallSharedPara bits: 1 insert_key_freq, 2 insert_key, 4 replica; query_key_freq in aux
  int aux = 0;
};
constexpr int kInvalidTime = -1;

struct Message;
using MessagePtr = std::shared_ptr<Message>;
struct Message {
  Task task;
  std::string sender, recver, original_recver;
  std::string key;                  // raw uint64 keys (sorted ascending when has_key)
  std::vector<std::string> value;   // raw value arrays
  bool valid = true;      // false: no need to send (empty slice); a local reply is faked
  bool finished = true;   // set false inside process() to defer the completion mark + ack
  bool replied = false;
  bool wait = false;      // submit blocks until every receiver replied
  std::function<void()> recv_handle, fin_handle;

  size_t num_keys() const { return key.size() / sizeof(Key); }
  const Key* keys() const { return reinterpret_cast<const Key*>(key.data()); }
  size_t bytes() const { size_t n = key.size(); for (auto& v : value) n += v.size(); return n; }
  std::string short_debug() const {
    std::ostringstream os;
    os << (task.request ? "REQ " : "ACK ") << sender << "=>" << recver << " T=" << task.time << " wait=" << task.wait_time
       << " cust=" << task.customer << " type=" << task.type << " cmd=" << task.cmd << " keys=" << num_keys()
       << " vals=" << value.size();
    if (task.has_key_range) os << " range=" << task.key_range.str();
    return os.str();
  }
};

// ------------------------------------------------------------------ wire encoding
class Encoder {
 public:
  template <typename T> void put(const T& v) { buf_.append(reinterpret_cast<const char*>(&v), sizeof(T)); }
  void put_str(const std::string& s) { put<uint64_t>(s.size()); buf_.append(s); }
  std::string take() { return std::move(buf_); }

 private:
  std::string buf_;
};
class Decoder {
 public:
  Decoder(const char* p, size_t n) : p_(p), e_(p + n) {}
  template <typename T> T get() {
    if (p_ + sizeof(T) > e_) throw std::runtime_error("message truncated");
    T v; std::memcpy(&v, p_, sizeof(T)); p_ += sizeof(T); return v;
  }
  std::string get_str() {
    const uint64_t n = get<uint64_t>();
    if (p_ + n > e_) throw std::runtime_error("message truncated");
    std::string s(p_, n); p_ += n; return s;
  }

 private:
  const char* p_; const char* e_;
};

// frame = header | key | value...; data parts optionally zlib-compressed with the original sizes
// carried in task.uncompressed_size (the reference does the same with snappy, van.cc:123-132)
inline std::string encode_message(const Message& m, bool compress) {
  Encoder e;
  const Task& t = m.task;
  e.put<uint32_t>(0x50534232u);  // "PSB2"
  e.put<int32_t>(t.type); e.put<uint8_t>(t.request); e.put_str(t.customer);
  e.put<int32_t>(t.time); e.put<int32_t>(t.wait_time); e.put<uint8_t>(t.has_key); e.put<uint8_t>(t.has_key_range);
  e.put<uint64_t>(t.key_range.begin); e.put<uint64_t>(t.key_range.end); e.put<uint32_t>(t.key_signature);
  e.put<int32_t>(t.key_channel); e.put<uint8_t>(t.erase_key_cache); e.put_str(t.msg); e.put<int32_t>(t.cmd);
  e.put<uint32_t>(t.flags); e.put<int32_t>(t.aux);
  e.put_str(m.sender); e.put_str(m.recver);
  e.put<uint8_t>(compress);
  const size_t nparts = 1 + m.value.size();
  e.put<uint32_t>((uint32_t)nparts);
  for (size_t i = 0; i < nparts; ++i) {
    const std::string& part = i == 0 ? m.key : m.value[i - 1];
    e.put<uint64_t>(part.size());
    if (compress && !part.empty()) e.put_str(zlib_compress(part.data(), part.size()));
    else e.put_str(part);
  }
  return e.take();
}
inline MessagePtr decode_message(const char* data, size_t n) {
  Decoder d(data, n);
  if (d.get<uint32_t>() != 0x50534232u) throw std::runtime_error("bad message magic");
  auto m = std::make_shared<Message>();
  Task& t = m->task;
  t.type = d.get<int32_t>(); t.request = d.get<uint8_t>(); t.customer = d.get_str();
  t.time = d.get<int32_t>(); t.wait_time = d.get<int32_t>(); t.has_key = d.get<uint8_t>(); t.has_key_range = d.get<uint8_t>();
  t.key_range.begin = d.get<uint64_t>(); t.key_range.end = d.get<uint64_t>(); t.key_signature = d.get<uint32_t>();
  t.key_channel = d.get<int32_t>(); t.erase_key_cache = d.get<uint8_t>(); t.msg = d.get_str(); t.cmd = d.get<int32_t>();
  t.flags = d.get<uint32_t>(); t.aux = d.get<int32_t>();
  m->sender = d.get_str(); m->recver = d.get_str();
  const bool compressed = d.get<uint8_t>();
  const uint32_t nparts = d.get<uint32_t>();
  for (uint32_t i = 0; i < nparts; ++i) {
    const uint64_t raw = d.get<uint64_t>();
    std::string part = d.get_str();
    if (compressed && raw > 0) {
      std::string out(raw, '\0');
      if (!zlib_uncompress(part.data(), part.size(), &out[0], raw)) throw std::runtime_error("bad compressed frame");
      part.swap(out);
    }
    t.uncompressed_size.push_back(raw);
    if (i == 0) m->key.swap(part); else m->value.push_back(std::move(part));
  }
  return m;
}

// ------------------------------------------------------------------ slicing and matching
// Split a message whose keys are sorted ascending at the n+1 separators `sep` into n messages;
// values are split proportionally (each value array holds a whole number of entries per key).
// A piece outside the message's key_range (or, for keyed messages, without keys) is marked
// invalid so that it is not sent.
inline std::vector<MessagePtr> slice_key_ordered(const MessagePtr& msg, const std::vector<Key>& sep) {
  const size_t n = sep.size() - 1;
  std::vector<MessagePtr> out(n);
  const Key* k = msg->keys();
  const size_t nk = msg->num_keys();
  std::vector<size_t> pos(n + 1, 0);
  if (msg->task.has_key)
    for (size_t i = 0; i <= n; ++i) pos[i] = std::lower_bound(k, k + nk, sep[i]) - k;
  Range msg_range = msg->task.has_key_range ? msg->task.key_range : Range::all();
  for (size_t i = 0; i < n; ++i) {
    auto p = std::make_shared<Message>(*msg);
    p->key.clear();
    p->value.clear();
    if (msg->task.has_key) {
      if (Range(sep[i], sep[i + 1]).intersect(msg_range).empty()) {
        p->valid = false;
      } else {
        p->key.assign(msg->key.data() + pos[i] * sizeof(Key), (pos[i + 1] - pos[i]) * sizeof(Key));
        for (const auto& v : msg->value) {
          const size_t per = nk ? v.size() / nk : 0;
          p->value.emplace_back(v.data() + pos[i] * per, (pos[i + 1] - pos[i]) * per);
        }
      }
      if (msg->task.has_key_range) {
        p->task.key_range = Range(sep[i], sep[i + 1]).intersect(msg_range);
      } else {
        p->task.key_range = Range(sep[i], sep[i + 1]);
        p->task.has_key_range = true;
      }
    } else {
      p->key = msg->key;
      p->value = msg->value;
    }
    out[i] = p;
  }
  return out;
}

enum class MatchOp { ASSIGN, ADD };
// Align (src_key, src_val) onto dst_key: for every key present in both, dst_val[j] (op)= src_val[i]
// (k values per key).  Both key lists sorted ascending and unique.  Returns the number of matches.
template <typename V>
size_t match_sorted(const Key* dst_key, size_t nd, V* dst_val, const Key* src_key, size_t ns, const V* src_val,
                    size_t k, MatchOp op) {
  size_t i = 0, j = 0, hits = 0;
  while (i < ns && j < nd) {
    if (src_key[i] < dst_key[j]) ++i;
    else if (src_key[i] > dst_key[j]) ++j;
    else {
      for (size_t c = 0; c < k; ++c) {
        if (op == MatchOp::ASSIGN) dst_val[j * k + c] = src_val[i * k + c];
        else dst_val[j * k + c] += src_val[i * k + c];
      }
      ++i; ++j; ++hits;
    }
  }
  return hits;
}
// multi-threaded variant: dst is cut into `threads` ranges, each joined with the matching src range
template <typename V>
size_t parallel_match_sorted(const Key* dst_key, size_t nd, V* dst_val, const Key* src_key, size_t ns,
                             const V* src_val, size_t k, MatchOp op, int threads) {
  if (threads <= 1 || nd < 4096) return match_sorted(dst_key, nd, dst_val, src_key, ns, src_val, k, op);
  std::vector<size_t> hits(threads, 0);
  std::vector<std::thread> th;
  for (int t = 0; t < threads; ++t) {
    th.emplace_back([&, t] {
      const size_t d0 = nd * t / threads, d1 = nd * (t + 1) / threads;
      if (d1 <= d0) return;
      const size_t s0 = std::lower_bound(src_key, src_key + ns, dst_key[d0]) - src_key;
      const size_t s1 = d1 < nd ? std::lower_bound(src_key, src_key + ns, dst_key[d1]) - src_key : ns;
      hits[t] = match_sorted(dst_key + d0, d1 - d0, dst_val + d0 * k, src_key + s0, s1 - s0, src_val + s0 * k, k, op);
    });
  }
  size_t total = 0;
  for (int t = 0; t < threads; ++t) { th[t].join(); total += hits[t]; }
  return total;
}

}  // namespace psb
