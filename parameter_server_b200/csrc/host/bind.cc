// pybind11 surface of the host runtime (module `_psb_host`).  Python sees nodes, vans, the post
// office, customers and messages (control plane), the data-ingest classes and the host numeric
// containers.  Blocking calls release the GIL; callbacks from executor threads take it.
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "darlin_cpu.h"
#include "data.h"
#include "feature_station.h"
#include "ocean.h"
#include "ftrl_cpu.h"
#include "kv.h"
#include "localizer.h"
#include "runtime.h"
#include "shared_param.h"

namespace py = pybind11;
using namespace psb;

namespace {

template <typename T>
py::array_t<T> to_array(const std::vector<T>& v) {
  py::array_t<T> a((py::ssize_t)v.size());
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}
template <typename T>
using carray = py::array_t<T, py::array::c_style | py::array::forcecast>;

py::dict slot_info_dict(const SlotInfo& s) {
  py::dict d;
  d["id"] = s.id;
  d["format"] = s.format == SlotFormat::DENSE ? "DENSE" : s.format == SlotFormat::SPARSE ? "SPARSE" : "SPARSE_BINARY";
  d["min_key"] = s.min_key; d["max_key"] = s.max_key; d["nnz_ele"] = s.nnz_ele; d["nnz_ex"] = s.nnz_ex;
  return d;
}
py::dict example_info_dict(const ExampleInfo& e) {
  py::dict d, slots;
  for (auto& kv : e.slot) slots[py::int_(kv.first)] = slot_info_dict(kv.second);
  d["num_ex"] = e.num_ex;
  d["slot"] = slots;
  d["text"] = e.to_text();
  return d;
}
py::dict slots_to_dict(const std::map<int, SlotData>& slots, uint64_t num_ex) {
  py::dict out;
  for (auto& kv : slots) {
    py::dict s;
    const SlotData& sd = kv.second;
    if (kv.first == 0) {
      s["value"] = to_array(sd.val);
    } else {
      std::vector<uint64_t> off(num_ex + 1, 0);
      for (size_t i = 0; i < sd.row_siz.size() && i < num_ex; ++i) off[i + 1] = off[i] + sd.row_siz[i];
      for (size_t i = sd.row_siz.size(); i < num_ex; ++i) off[i + 1] = off[i];
      s["offset"] = to_array(off);
      s["index"] = to_array(sd.col_idx);
      s["value"] = to_array(sd.val);
    }
    out[py::int_(kv.first)] = s;
  }
  return out;
}

// A Python callable that may be copied and destroyed on threads that do not hold the GIL.
inline std::shared_ptr<py::object> hold(py::object o) {
  return std::shared_ptr<py::object>(new py::object(std::move(o)), [](py::object* p) { py::gil_scoped_acquire g; delete p; });
}

struct PyCustomer : public Customer {
  using Customer::Customer;
};

// (keys, values) arrays of concatenated pull replies
py::tuple pulled_arrays(const std::pair<std::string, std::string>& p) {
  py::array_t<uint64_t> k((py::ssize_t)(p.first.size() / 8));
  py::array_t<double> v((py::ssize_t)(p.second.size() / 8));
  if (p.first.size() >= 8) std::memcpy(k.mutable_data(), p.first.data(), p.first.size() / 8 * 8);
  if (p.second.size() >= 8) std::memcpy(v.mutable_data(), p.second.data(), p.second.size() / 8 * 8);
  return py::make_tuple(k, v);
}

MessagePtr make_message(const std::string& recver, int type, int cmd, const std::string& payload, py::object key,
                        const std::vector<py::bytes>& values, int time, int wait_time, int channel, py::object key_range,
                        uint32_t flags, int aux, bool erase_key_cache) {
  auto m = std::make_shared<Message>();
  m->recver = recver;
  m->task.type = type;
  m->task.cmd = cmd;
  m->task.msg = payload;
  m->task.time = time;
  m->task.wait_time = wait_time;
  m->task.key_channel = channel;
  m->task.flags = flags;
  m->task.aux = aux;
  m->task.erase_key_cache = erase_key_cache;
  if (!key.is_none()) {
    m->key = key.cast<std::string>();
    m->task.has_key = true;
  }
  if (!key_range.is_none()) {
    auto r = key_range.cast<std::pair<uint64_t, uint64_t>>();
    m->task.key_range = Range(r.first, r.second);
    m->task.has_key_range = true;
  }
  for (auto& v : values) m->value.push_back(v);
  return m;
}

}  // namespace

PYBIND11_MODULE(_psb_host, m) {
  m.doc() = "host runtime of parameter_server_b200 (control plane, data ingest, host containers)";

  // ---------------------------------------------------------------- hashing / util
  m.def("crc32c", [](py::bytes b) { std::string s = b; return crc32c_value(s.data(), s.size()); });
  m.def("crc32c_extend", [](uint32_t c, py::bytes b) { std::string s = b; return crc32c_extend(c, s.data(), s.size()); });
  m.def("crc32c_mask", &crc32c_mask);
  m.def("crc32c_unmask", &crc32c_unmask);
  m.def("murmur3_x64_128", [](py::bytes b, uint32_t seed) { std::string s = b; uint64_t o[2]; murmur3_x64_128(s.data(), (int)s.size(), seed, o); return std::make_pair(o[0], o[1]); });
  m.def("shuffle_feature_id", &shuffle_feature_id);
  m.def("djb_hash32", &djb_hash32);
  m.def("key_signature", [](py::bytes b) { return key_signature(b); });
  m.def("set_verbose", [](bool on) { verbose_flag() = on; }, "executors narrate the messages they process (-verbose)");
  m.def("interfaces", &LocalMachine::interfaces, "(name, IPv4 address) of every interface that is up, loopback last");
  m.def("local_ip", &LocalMachine::ip, py::arg("interface") = std::string());
  m.def("resource_usage", [] {
    double rss, virt; uint64_t pj, hj, in, out;
    ResUsage::memory_mb(&rss, &virt); ResUsage::cpu_jiffies(&pj, &hj); ResUsage::net_bytes(&in, &out);
    py::dict d; d["rss_mb"] = rss; d["virt_mb"] = virt; d["proc_jiffies"] = pj; d["host_jiffies"] = hj; d["net_in"] = in; d["net_out"] = out;
    return d;
  });
  m.def("parallel_sort_u64", [](carray<uint64_t> a, int threads) {
    std::vector<uint64_t> v(a.data(), a.data() + a.size());
    { py::gil_scoped_release r; parallel_sort(v.begin(), v.end(), threads, std::less<uint64_t>()); }
    return to_array(v);
  });
  // ---- localisation: unique keys with counts, global -> local ids, row-major -> column-major
  m.def("count_unique", [](carray<uint64_t> keys, int threads) {
    std::vector<uint64_t> u; std::vector<uint32_t> c;
    { py::gil_scoped_release r; count_unique(keys.data(), (size_t)keys.size(), threads, &u, &c); }
    return py::make_tuple(to_array(u), to_array(c));
  }, py::arg("keys"), py::arg("threads") = 1, "(sorted unique keys, their counts)");
  m.def("localize", [](carray<uint64_t> keys) {
    if (keys.size() >= (py::ssize_t)1 << 31) throw std::invalid_argument("localize: more than 2^31 positions");
    std::vector<uint64_t> u; std::vector<uint32_t> c;
    py::array_t<int32_t> local(keys.size());
    { py::gil_scoped_release r; localize(keys.data(), (size_t)keys.size(), &u, &c, local.mutable_data()); }
    return py::make_tuple(to_array(u), to_array(c), local);
  }, "(sorted unique keys, their counts, local id of every position)");
  m.def("remap_keys", [](carray<uint64_t> keys, carray<uint64_t> dict, int threads) {
    py::array_t<int32_t> out(keys.size());
    { py::gil_scoped_release r; remap_keys(keys.data(), (size_t)keys.size(), dict.data(), (size_t)dict.size(), threads, out.mutable_data()); }
    return out;
  }, py::arg("keys"), py::arg("dict"), py::arg("threads") = 1, "position of every key in the sorted dictionary, -1 where absent");
  m.def("csr_to_csc", [](carray<int64_t> offsets, carray<int32_t> col, py::object vals, size_t cols, int threads) {
    carray<double> dv;
    const double* dp = nullptr;
    if (!vals.is_none()) { dv = vals.cast<carray<double>>(); dp = dv.data(); }
    if (offsets.size() < 1 || offsets.data()[offsets.size() - 1] != col.size() || (dp && dv.size() != col.size()))
      throw std::invalid_argument("offsets, column ids and values do not fit together");
    for (py::ssize_t i = 0; i < col.size(); ++i) if (col.data()[i] >= (int64_t)cols) throw std::invalid_argument("column id out of range");
    std::vector<int64_t> ip; std::vector<int32_t> rows; std::vector<double> ov;
    { py::gil_scoped_release r; csr_to_csc(offsets.data(), (size_t)offsets.size() - 1, col.data(), dp, cols, threads, &ip, &rows, &ov); }
    return py::make_tuple(to_array(ip), to_array(rows), dp ? py::object(to_array(ov)) : py::object(py::none()));
  }, py::arg("offsets"), py::arg("col"), py::arg("vals"), py::arg("cols"), py::arg("threads") = 1,
     "(indptr, row ids, values or None) of the column-major form; column id -1 drops a non-zero");
  m.def("kv_partition", [](carray<uint64_t> keys, carray<double> vals, std::vector<uint64_t> pivots) {
    std::vector<uint64_t> k(keys.data(), keys.data() + keys.size());
    std::vector<double> v(vals.data(), vals.data() + vals.size());
    auto off = kv_partition(k.data(), v.empty() ? (double*)nullptr : v.data(), k.size(), pivots);
    return py::make_tuple(to_array(k), to_array(v), off);
  });
  m.def("zlib_roundtrip", [](py::bytes b) { std::string s = b; std::string z = zlib_compress(s.data(), s.size()); std::string o(s.size(), '\0'); bool ok = zlib_uncompress(z.data(), z.size(), &o[0], o.size()); return py::make_tuple(ok, z.size(), py::bytes(o)); });
  m.def("record_write", [](const std::string& path, const std::vector<py::bytes>& recs) {
    auto f = File::open(path, "w"); if (!f) return false; RecordWriter w(f.get());
    for (auto& r : recs) if (!w.write(r)) return false;
    return true;
  });
  m.def("record_read", [](const std::string& path) {
    std::vector<py::bytes> out; auto f = File::open(path, "r"); if (!f) return out; RecordReader r(f.get()); std::string s;
    while (r.read(&s)) out.emplace_back(s);
    return out;
  });

  // ---------------------------------------------------------------- sorted-key algorithms
  m.def("set_union", [](carray<uint64_t> a, carray<uint64_t> b) { return to_array(set_union(a.data(), a.size(), b.data(), b.size())); });
  m.def("set_intersection", [](carray<uint64_t> a, carray<uint64_t> b) { return to_array(set_intersection(a.data(), a.size(), b.data(), b.size())); });
  m.def("find_range", [](carray<uint64_t> a, uint64_t lo, uint64_t hi) { return find_range(a.data(), a.size(), Range(lo, hi)); });
  m.def("match", [](carray<uint64_t> dst_key, py::array_t<double> dst_val, carray<uint64_t> src_key, carray<double> src_val, int k, bool add, int threads) {
    return parallel_match_sorted(dst_key.data(), dst_key.size(), dst_val.mutable_data(), src_key.data(), src_key.size(), src_val.data(), (size_t)k,
                                 add ? MatchOp::ADD : MatchOp::ASSIGN, threads);
  }, py::arg("dst_key"), py::arg("dst_val"), py::arg("src_key"), py::arg("src_val"), py::arg("k") = 1, py::arg("add") = false, py::arg("threads") = 1);
  m.def("even_divide", [](uint64_t b, uint64_t e, size_t n, size_t i) { Range r = Range(b, e).even_divide(n, i); return std::make_pair(r.begin, r.end); });
  m.def("soft_thresholding", &soft_thresholding);
  m.def("exact_auc", [](carray<float> label, carray<float> pred) { return exact_auc(label.data(), pred.data(), label.size()); });

  py::class_<CountMin>(m, "CountMin")
      .def(py::init<>())
      .def("resize", &CountMin::resize, py::arg("n"), py::arg("k"), py::arg("saturate") = false)
      .def("insert", [](CountMin& c, carray<uint64_t> k, carray<uint32_t> cnt) { for (py::ssize_t i = 0; i < k.size(); ++i) c.insert(k.data()[i], cnt.data()[i]); })
      .def("query", [](const CountMin& c, carray<uint64_t> k) { std::vector<uint32_t> o(k.size()); for (py::ssize_t i = 0; i < k.size(); ++i) o[i] = c.query(k.data()[i]); return to_array(o); })
      .def_static("hash", &CountMin::hash)
      .def("size", &CountMin::size);
  py::class_<FrequencyFilter>(m, "FrequencyFilter")
      .def(py::init<>())
      .def("resize", &FrequencyFilter::resize)
      .def("empty", &FrequencyFilter::empty)
      .def("clear", &FrequencyFilter::clear)
      .def("insert_keys", [](FrequencyFilter& f, carray<uint64_t> k, carray<uint32_t> c) { f.insert_keys(k.data(), c.data(), k.size()); })
      .def("query_keys", [](const FrequencyFilter& f, carray<uint64_t> k, uint32_t freq) { return to_array(f.query_keys(k.data(), k.size(), freq)); });
  py::class_<Bitmap>(m, "Bitmap")
      .def(py::init<size_t, bool>(), py::arg("n") = 0, py::arg("value") = false)
      .def("resize", &Bitmap::resize, py::arg("n"), py::arg("value") = false)
      .def("set", &Bitmap::set).def("clear", &Bitmap::clear).def("test", &Bitmap::test).def("fill", &Bitmap::fill)
      .def("nnz", &Bitmap::nnz).def("size", &Bitmap::size);
  py::class_<AUC>(m, "AUC")
      .def(py::init<>())
      .def("set_goodness", &AUC::set_goodness)
      .def("add", [](AUC& a, carray<float> label, carray<float> pred) { a.add(label.data(), pred.data(), label.size()); })
      .def("merge", [](AUC& a, const AUC& o) { a.merge(o); })
      .def("merge_data", [](AUC& a, std::vector<int64_t> tk, std::vector<uint64_t> tc, std::vector<int64_t> fk, std::vector<uint64_t> fc) { a.merge(tk, tc, fk, fc); })
      .def("data", [](const AUC& a) {
        std::vector<int64_t> tk, fk; std::vector<uint64_t> tc, fc;
        for (auto& kv : a.tp()) { tk.push_back(kv.first); tc.push_back(kv.second); }
        for (auto& kv : a.fp()) { fk.push_back(kv.first); fc.push_back(kv.second); }
        return py::make_tuple(tk, tc, fk, fc);
      })
      .def("clear", &AUC::clear).def("evaluate", &AUC::evaluate).def("accuracy", &AUC::accuracy, py::arg("threshold") = 0.0);
  // ---- DARLIN block steps on CPU nodes (in-place arrays must be C-contiguous, writeable and of the exact dtype)
  using marray_d = py::array_t<double, py::array::c_style>;
  using marray_b = py::array_t<uint8_t, py::array::c_style>;
  auto need_rw = [](const py::array& a, const char* what) {
    if (!a.writeable()) throw std::invalid_argument(std::string(what) + " must be writeable");
  };
  m.def("darlin_block_gradient", [](carray<int64_t> indptr, carray<int32_t> indices, py::object data, carray<double> y,
                                    carray<double> dual, carray<double> delta, carray<uint8_t> active, int64_t c0, int64_t c1,
                                    int threads) {
    carray<double> dv;
    const double* dp = nullptr;
    if (!data.is_none()) { dv = data.cast<carray<double>>(); dp = dv.data(); }
    if (c0 < 0 || c1 < c0 || c1 + 1 > indptr.size() || c1 > delta.size() || c1 > active.size()) throw std::invalid_argument("bad column range");
    py::array_t<double> G(c1 - c0), U(c1 - c0);
    CscBlock B{indptr.data(), indices.data(), dp, c0, c1};
    {
      py::gil_scoped_release rel;
      darlin_block_gradient(B, y.data(), dual.data(), delta.data(), active.data(), G.mutable_data(), U.mutable_data(), threads);
    }
    return py::make_tuple(G, U);
  }, py::arg("indptr"), py::arg("indices"), py::arg("data"), py::arg("y"), py::arg("dual"), py::arg("delta"), py::arg("active"),
     py::arg("c0"), py::arg("c1"), py::arg("threads") = 1);
  m.def("darlin_update_weight", [need_rw](marray_d w, marray_d delta, marray_b active, carray<double> G, carray<double> U,
                                          double lambda, double eta, double kkt_threshold, double delta_max) {
    need_rw(w, "w"); need_rw(delta, "delta"); need_rw(active, "active");
    const py::ssize_t n = w.size();
    if (delta.size() != n || active.size() != n || G.size() != n || U.size() != n) throw std::invalid_argument("segment sizes differ");
    return darlin_update_weight(w.mutable_data(), delta.mutable_data(), active.mutable_data(), G.data(), U.data(), n, lambda, eta,
                                kkt_threshold, delta_max);
  });
  m.def("darlin_update_dual", [need_rw](carray<int64_t> indptr, carray<int32_t> indices, py::object data, carray<double> y,
                                        marray_d dual, marray_d w, marray_d delta, marray_b active, carray<double> w_new,
                                        int64_t c0, int64_t c1, double delta_max) {
    need_rw(dual, "dual"); need_rw(w, "w"); need_rw(delta, "delta"); need_rw(active, "active");
    carray<double> dv;
    const double* dp = nullptr;
    if (!data.is_none()) { dv = data.cast<carray<double>>(); dp = dv.data(); }
    if (c0 < 0 || c1 < c0 || c1 + 1 > indptr.size() || c1 > w.size() || w_new.size() != c1 - c0) throw std::invalid_argument("bad column range");
    CscBlock B{indptr.data(), indices.data(), dp, c0, c1};
    darlin_update_dual(B, y.data(), dual.mutable_data(), w.mutable_data(), delta.mutable_data(), active.mutable_data(), w_new.data(),
                       delta_max);
  });
  // ---- general block store: arrays cut along a column partition, spilled per block, prefetched by block
  {
    py::class_<Ocean> oc(m, "Ocean");
    oc.def(py::init<std::string, std::string, int, int, bool>(), py::arg("dir"), py::arg("identity"), py::arg("threads") = 2,
           py::arg("job_limit") = 64, py::arg("less_memory") = false)
        .def("set_partition", &Ocean::set_partition)
        .def("num_blocks", &Ocean::num_blocks)
        .def("dump", [](Ocean& o, int grp, int kind, py::array a) {
          py::array c = py::array::ensure(a, py::array::c_style);
          if (!c) return false;
          const void* p = c.data(); const size_t n = (size_t)c.size(), elem = (size_t)c.itemsize();
          py::gil_scoped_release rel;
          return o.dump(grp, (Ocean::Kind)kind, p, n, elem);
        })
        .def("prefetch", &Ocean::prefetch)
        .def("get", [](Ocean& o, int grp, size_t blk, int kind, const std::string& dtype) -> py::object {
          if (kind < 0 || kind >= Ocean::NUM_KINDS) throw std::invalid_argument("unknown kind");
          Ocean::BytesPtr b;
          { py::gil_scoped_release rel; b = o.get(grp, blk, (Ocean::Kind)kind); }
          if (!b) return py::none();
          py::dtype dt = py::dtype::from_args(py::str(dtype));
          if (b->size() % (size_t)dt.itemsize() != 0) throw std::invalid_argument("block size is not a multiple of the element size");
          const std::vector<py::ssize_t> shape{(py::ssize_t)(b->size() / (size_t)dt.itemsize())};
          py::array out(dt, shape);
          if (!b->empty()) std::memcpy(out.mutable_data(), b->data(), b->size());
          return py::object(std::move(out));
        }, py::arg("grp"), py::arg("blk"), py::arg("kind"), py::arg("dtype"))
        .def("drop", &Ocean::drop, py::call_guard<py::gil_scoped_release>())
        .def("pending", &Ocean::pending)
        .def("stats", [](Ocean& o) {
          auto s = o.stats(); py::dict d;
          d["bytes_written"] = s.bytes_written; d["bytes_read"] = s.bytes_read; d["prefetched"] = s.prefetched; d["hits"] = s.hits;
          d["misses"] = s.misses; d["loaded_now"] = s.loaded_now; d["peak_loaded"] = s.peak_loaded;
          return d;
        });
    oc.attr("FEATURE_KEY") = (int)Ocean::FEATURE_KEY; oc.attr("FEATURE_OFFSET") = (int)Ocean::FEATURE_OFFSET;
    oc.attr("FEATURE_VALUE") = (int)Ocean::FEATURE_VALUE; oc.attr("PARAMETER_KEY") = (int)Ocean::PARAMETER_KEY;
    oc.attr("PARAMETER_VALUE") = (int)Ocean::PARAMETER_VALUE; oc.attr("DELTA") = (int)Ocean::DELTA;
  }
  // ---- worker-side feature store (memory or disk with prefetch) and the block steps on its ranges
  py::class_<FeatureStation>(m, "FeatureStation")
      .def(py::init<std::string, std::string, size_t, int, size_t, bool>(), py::arg("dir"), py::arg("name"), py::arg("mem_limit_kb") = 1048576,
           py::arg("threads") = 2, py::arg("job_limit") = 64, py::arg("detail") = false)
      .def_property_readonly("disk", &FeatureStation::disk)
      .def("add_group", [](FeatureStation& f, int grp, uint64_t rows, carray<int64_t> indptr, carray<int32_t> indices, py::object data) {
        carray<double> dv;
        const double* dp = nullptr;
        if (!data.is_none()) { dv = data.cast<carray<double>>(); dp = dv.data(); }
        if (indptr.size() < 1 || indptr.data()[indptr.size() - 1] != indices.size() || (dp && dv.size() != indices.size()))
          throw std::invalid_argument("offsets, row ids and values do not fit together");
        py::gil_scoped_release rel;
        f.add_group(grp, rows, indptr.data(), indptr.size() - 1, indices.data(), dp);
      }, py::arg("grp"), py::arg("rows"), py::arg("indptr"), py::arg("indices"), py::arg("data"))
      .def("mem_size", &FeatureStation::mem_size)
      .def("cols", &FeatureStation::cols)
      .def("file_base", &FeatureStation::file_base)
      .def("range_bytes", &FeatureStation::range_bytes)
      .def("prefetch", &FeatureStation::prefetch)
      .def("pending", &FeatureStation::pending)
      .def("task_used", &FeatureStation::task_used)
      .def("max_task", &FeatureStation::max_task)
      .def("resident_bytes", &FeatureStation::resident_bytes)
      .def("drop", &FeatureStation::drop)
      .def("get", [](FeatureStation& f, int task, int grp, int64_t c0, int64_t c1) {
        FeatureBlockPtr b;
        { py::gil_scoped_release rel; b = f.get(task, grp, c0, c1); }
        const int64_t p0 = b->indptr[0], n = b->indptr[c1 - c0] - p0;
        py::array_t<int64_t> ip(c1 - c0 + 1);
        for (int64_t j = 0; j <= c1 - c0; ++j) ip.mutable_data()[j] = b->indptr[j] - p0;
        py::array_t<int32_t> idx(n);
        if (n) std::memcpy(idx.mutable_data(), b->indices + (p0 - b->pos0), (size_t)n * 4);
        py::object val = py::none();
        if (b->values) { py::array_t<double> v(n); if (n) std::memcpy(v.mutable_data(), b->values + (p0 - b->pos0), (size_t)n * 8); val = v; }
        return py::make_tuple(ip, idx, val);
      }, "copies of columns [c0, c1): (offsets from 0, row ids, values or None)")
      .def("block_gradient", [](FeatureStation& f, int task, int grp, int64_t c0, int64_t c1, carray<double> y, carray<double> dual,
                                carray<double> delta, carray<uint8_t> active, int threads) {
        if (c1 > delta.size() || c1 > active.size()) throw std::invalid_argument("bad column range");
        py::array_t<double> G(c1 - c0), U(c1 - c0);
        {
          py::gil_scoped_release rel;
          FeatureBlockPtr b = f.get(task, grp, c0, c1);
          CscBlock B{b->indptr, b->indices, b->values, c0, c1, c0, b->pos0};
          darlin_block_gradient(B, y.data(), dual.data(), delta.data(), active.data(), G.mutable_data(), U.mutable_data(), threads);
        }
        return py::make_tuple(G, U);
      })
      .def("block_update_dual", [need_rw](FeatureStation& f, int task, int grp, int64_t c0, int64_t c1, carray<double> y, marray_d dual, marray_d w,
                                          marray_d delta, marray_b active, carray<double> w_new, double delta_max) {
        need_rw(dual, "dual"); need_rw(w, "w"); need_rw(delta, "delta"); need_rw(active, "active");
        if (c1 > w.size() || w_new.size() != c1 - c0) throw std::invalid_argument("bad column range");
        py::gil_scoped_release rel;
        FeatureBlockPtr b = f.get(task, grp, c0, c1);
        CscBlock B{b->indptr, b->indices, b->values, c0, c1, c0, b->pos0};
        darlin_update_dual(B, y.data(), dual.mutable_data(), w.mutable_data(), delta.mutable_data(), active.mutable_data(), w_new.data(), delta_max);
      })
      .def("stats", [](FeatureStation& f) {
        auto s = f.stats();
        py::dict d;
        d["bytes_written"] = s.bytes_written; d["bytes_read"] = s.bytes_read; d["prefetched"] = s.prefetched; d["hits"] = s.hits;
        d["misses"] = s.misses; d["peak_resident"] = s.peak_resident; d["limit_waits"] = s.limit_waits;
        return d;
      });
  m.def("ftrl_minibatch", [](carray<int64_t> off, carray<int32_t> loc, py::object vals, carray<double> y, carray<double> w, int threads) {
    carray<double> dv;
    const double* dp = nullptr;
    if (!vals.is_none()) { dv = vals.cast<carray<double>>(); dp = dv.data(); }
    const py::ssize_t rows = off.size() - 1, nk = w.size();
    if (rows < 0 || y.size() != rows || off.data()[rows] != loc.size() || (dp && dv.size() != loc.size())) throw std::invalid_argument("minibatch arrays do not fit together");
    for (py::ssize_t i = 0; i < loc.size(); ++i) if (loc.data()[i] < 0 || loc.data()[i] >= nk) throw std::invalid_argument("local key id out of range");
    py::array_t<double> g(nk), pos(nk), neg(nk);
    double loss;
    { py::gil_scoped_release r; loss = ftrl_minibatch(off.data(), (size_t)rows, loc.data(), dp, y.data(), w.data(), (size_t)nk, threads, g.mutable_data(), pos.mutable_data(), neg.mutable_data()); }
    return py::make_tuple(loss, g, pos, neg);
  }, py::arg("offsets"), py::arg("loc"), py::arg("vals"), py::arg("y"), py::arg("w"), py::arg("threads") = 1,
     "(summed logistic loss, gradient, positive count, negative count per local key) of one minibatch");
  py::class_<FTRLModel>(m, "FTRLModel")
      .def(py::init<double, double, double, double>(), py::arg("alpha"), py::arg("beta"), py::arg("lambda1"), py::arg("lambda2"))
      .def("update", [](FTRLModel& f, carray<uint64_t> k, carray<double> g, carray<double> pos, carray<double> neg) {
        if (g.size() != k.size() || pos.size() != k.size() || neg.size() != k.size()) throw std::invalid_argument("FTRLModel.update: array sizes differ");
        f.update(k.data(), (size_t)k.size(), g.data(), pos.data(), neg.data());
      })
      .def("get", [](const FTRLModel& f, carray<uint64_t> k) { return to_array(f.get(k.data(), (size_t)k.size())); })
      .def("stats", [](const FTRLModel& f) { return py::make_tuple(f.norm1(), f.norm2(), f.nnz()); })
      .def("size", &FTRLModel::size)
      .def("nonzero", [](const FTRLModel& f) {
        std::vector<Key> k; std::vector<double> w;
        f.nonzero(&k, &w);
        return py::make_tuple(to_array(k), to_array(w));
      });
  py::class_<KVVector>(m, "KVVector")
      .def(py::init<int>(), py::arg("k") = 1)
      .def("k", &KVVector::k)
      .def("keys", [](KVVector& v, int ch) { return to_array(v.key(ch)); })
      .def("values", [](KVVector& v, int ch) { return to_array(v.value(ch)); })
      .def("set_keys", [](KVVector& v, int ch, carray<uint64_t> k) { v.key(ch).assign(k.data(), k.data() + k.size()); })
      .def("set_values", [](KVVector& v, int ch, carray<double> a) { v.value(ch).assign(a.data(), a.data() + a.size()); })
      .def("set_values_range", [](KVVector& v, int ch, size_t lo, carray<double> a) { std::copy(a.data(), a.data() + a.size(), v.value(ch).begin() + lo * v.k()); })
      .def("merge_keys", [](KVVector& v, int ch, carray<uint64_t> k) { v.merge_keys(ch, k.data(), k.size()); })
      .def("init_values", &KVVector::init_values, py::arg("ch"), py::arg("init") = 0.0)
      .def("aggregate", [](KVVector& v, int ch, int t, uint64_t lo, uint64_t hi, carray<uint64_t> k, carray<double> a, int nval, int threads) {
        return v.aggregate(ch, t, Range(lo, hi), k.data(), k.size(), a.data(), nval, threads);
      })
      .def("received", [](KVVector& v, int t) { auto r = v.received(t); return py::make_tuple(r.lo, r.hi, r.nval, to_array(r.vals)); })
      .def("lookup", [](KVVector& v, int ch, carray<uint64_t> k) { return to_array(v.lookup(ch, k.data(), k.size())); })
      .def("find", [](KVVector& v, int ch, uint64_t lo, uint64_t hi) { return v.find(ch, Range(lo, hi)); })
      .def("clear", &KVVector::clear);

  // ---------------------------------------------------------------- data ingest
  py::enum_<TextFormat>(m, "TextFormat")
      .value("PS_DENSE", TextFormat::PS_DENSE).value("PS_SPARSE", TextFormat::PS_SPARSE).value("PS_SPARSE_BINARY", TextFormat::PS_SPARSE_BINARY)
      .value("ADFEA", TextFormat::ADFEA).value("LIBSVM", TextFormat::LIBSVM).value("TERAFEA", TextFormat::TERAFEA);
  m.def("set_hadoop_fs", [](const std::string& cmd) { hadoop_fs_command() = cmd; }, "command that stands for `hadoop fs` when \"hdfs:\" paths are read");
  m.def("hadoop_fs", [] { return hadoop_fs_command(); });
  m.def("search_files", &search_files);
  m.def("divide_files", &divide_files, py::arg("files"), py::arg("num_workers"), py::arg("load_limit") = 0);
  m.def("parse_text", [](const std::string& text, TextFormat fmt, bool ignore_grp, bool shuffle, bool beta) {
    ExampleParser p; p.init(fmt, ignore_grp, shuffle, beta);
    std::map<int, SlotData> slots; ExampleInfo info; size_t bad = 0;
    std::istringstream is(text); std::string line;
    while (std::getline(is, line)) { if (line.empty()) continue; std::vector<char> buf(line.begin(), line.end()); buf.push_back(0); if (!p.parse_line(buf.data(), &slots, &info)) ++bad; }
    ExampleParser::finish(&slots, info.num_ex);
    return py::make_tuple(slots_to_dict(slots, info.num_ex), example_info_dict(info), bad);
  }, py::arg("text"), py::arg("format"), py::arg("ignore_feature_group") = false, py::arg("shuffle_fea_id") = false, py::arg("add_beta_feature") = false);
  py::class_<SlotReader>(m, "SlotReader")
      .def(py::init<>())
      .def("init", &SlotReader::init, py::arg("files"), py::arg("format"), py::arg("cache_dir"), py::arg("ignore_feature_group") = false,
           py::arg("shuffle_fea_id") = false, py::arg("add_beta_feature") = false, py::arg("line_limit") = 0, py::arg("max_mb_per_thread") = 2048)
      .def("read", [](SlotReader& r, int threads) { ExampleInfo info; int hits; { py::gil_scoped_release rel; hits = r.read(threads, &info); } return py::make_tuple(example_info_dict(info), hits); })
      .def("index", [](SlotReader& r, int slot) { return to_array(r.index(slot)); })
      .def("offset", [](SlotReader& r, int slot) { return to_array(r.offset(slot)); })
      .def("value", [](SlotReader& r, int slot) { return to_array(r.value(slot)); })
      .def("cache_name", &SlotReader::cache_name);
  py::class_<StreamReader>(m, "StreamReader")
      .def(py::init<>())
      .def("init", &StreamReader::init, py::arg("files"), py::arg("format"), py::arg("ignore_feature_group") = false, py::arg("shuffle_fea_id") = false)
      .def("read", [](StreamReader& r, size_t n) -> py::object {
        std::map<int, SlotData> slots; ExampleInfo info; bool ok;
        { py::gil_scoped_release rel; ok = r.read(n, &slots, &info); }
        if (!ok) return py::none();
        return py::make_tuple(slots_to_dict(slots, info.num_ex), example_info_dict(info));
      });
  m.def("write_bin_matrix", [](const std::string& name, bool row_major, uint64_t rows, uint64_t cols, carray<uint64_t> offset, carray<uint64_t> index, py::object value, int sizeof_index) {
    BinMatrix b; b.row_major = row_major; b.rows = rows; b.cols = cols; b.sizeof_index = sizeof_index;
    b.offset.assign(offset.data(), offset.data() + offset.size()); b.index.assign(index.data(), index.data() + index.size());
    b.nnz = b.index.size(); b.binary = value.is_none();
    if (!b.binary) { auto v = value.cast<carray<float>>(); b.value.assign(v.data(), v.data() + v.size()); }
    return write_bin_matrix(name, b);
  }, py::arg("name"), py::arg("row_major"), py::arg("rows"), py::arg("cols"), py::arg("offset"), py::arg("index"), py::arg("value") = py::none(), py::arg("sizeof_index") = 8);
  m.def("read_bin_matrix", [](const std::string& name, uint64_t row_begin, uint64_t row_end) -> py::object {
    BinMatrix b;
    if (!read_bin_matrix(name, &b, row_begin, row_end)) return py::none();
    py::dict d; d["row_major"] = b.row_major; d["rows"] = b.rows; d["cols"] = b.cols; d["nnz"] = b.nnz; d["binary"] = b.binary; d["sparse"] = b.sparse;
    d["offset"] = to_array(b.offset); d["index"] = to_array(b.index); d["value"] = to_array(b.value);
    return d;
  }, py::arg("name"), py::arg("row_begin") = 0, py::arg("row_end") = ~0ull);

  // ---------------------------------------------------------------- control plane
  py::class_<Node>(m, "Node")
      .def(py::init([](int role, std::string id, std::string host, int port) { Node n; n.role = role; n.id = id; n.hostname = host; n.port = port; n.key = Range::all(); return n; }),
           py::arg("role"), py::arg("id"), py::arg("hostname") = "127.0.0.1", py::arg("port") = 0)
      .def_readwrite("role", &Node::role).def_readwrite("id", &Node::id).def_readwrite("hostname", &Node::hostname).def_readwrite("port", &Node::port)
      .def_property("key", [](const Node& n) { return std::make_pair(n.key.begin, n.key.end); }, [](Node& n, std::pair<uint64_t, uint64_t> r) { n.key = Range(r.first, r.second); })
      .def("__repr__", [](const Node& n) { return "<Node " + n.id + " role=" + std::to_string(n.role) + " " + n.hostname + ":" + std::to_string(n.port) + " " + n.key.str() + ">"; });
  m.attr("SERVER") = (int)Node::SERVER; m.attr("WORKER") = (int)Node::WORKER; m.attr("SCHEDULER") = (int)Node::SCHEDULER; m.attr("UNUSED") = (int)Node::UNUSED;
  m.attr("kServerGroup") = kServerGroup; m.attr("kWorkerGroup") = kWorkerGroup; m.attr("kActiveGroup") = kActiveGroup;
  m.attr("kReplicaGroup") = kReplicaGroup; m.attr("kOwnerGroup") = kOwnerGroup; m.attr("kLiveGroup") = kLiveGroup;
  m.attr("TERMINATE") = (int)Task::TERMINATE; m.attr("REPLY") = (int)Task::REPLY; m.attr("MANAGE") = (int)Task::MANAGE;
  m.attr("CALL_CUSTOMER") = (int)Task::CALL_CUSTOMER; m.attr("HEARTBEATING") = (int)Task::HEARTBEATING;

  py::class_<InprocHub, std::shared_ptr<InprocHub>>(m, "InprocHub").def(py::init<>());
  py::class_<Van, std::shared_ptr<Van>>(m, "Van")
      .def("set_compress", &Van::set_compress)
      .def("set_log", &Van::set_log)
      .def("set_filter", [](Van& v, py::object f) {
        if (f.is_none()) { v.set_filter(nullptr); return; }
        v.set_filter([h = hold(f)](const Message& msg) { py::gil_scoped_acquire g; return (*h)(msg.sender, msg.recver, msg.task.type, msg.task.request, msg.task.time, msg.task.customer).cast<int>(); });
      })
      .def("sent_bytes", &Van::sent_bytes).def("recv_bytes", &Van::recv_bytes).def("dropped", &Van::dropped)
      .def_property_readonly("my_node", [](Van& v) { return v.my_node; })
      .def("close", &Van::close, py::call_guard<py::gil_scoped_release>());
  py::class_<InprocVan, Van, std::shared_ptr<InprocVan>>(m, "InprocVan").def(py::init<std::shared_ptr<InprocHub>, const Node&>());
  py::class_<TcpVan, Van, std::shared_ptr<TcpVan>>(m, "TcpVan")
      .def(py::init<const Node&>())
      .def("bind", [](TcpVan& v) { Status s = v.bind(); if (!s.ok()) throw std::runtime_error(s.ToString()); return v.my_node.port; })
      .def("set_retries", &TcpVan::set_retries);

  py::class_<Message, MessagePtr>(m, "Message")
      .def_readonly("sender", &Message::sender).def_readonly("recver", &Message::recver)
      .def_property_readonly("request", [](const Message& x) { return x.task.request; })
      .def_property_readonly("type", [](const Message& x) { return x.task.type; })
      .def_property_readonly("cmd", [](const Message& x) { return x.task.cmd; })
      .def_property_readonly("time", [](const Message& x) { return x.task.time; })
      .def_property_readonly("wait_time", [](const Message& x) { return x.task.wait_time; })
      .def_property_readonly("payload", [](const Message& x) { return py::bytes(x.task.msg); })
      .def_property_readonly("channel", [](const Message& x) { return x.task.key_channel; })
      .def_property_readonly("flags", [](const Message& x) { return x.task.flags; })
      .def_property_readonly("aux", [](const Message& x) { return x.task.aux; })
      .def_property_readonly("has_key", [](const Message& x) { return x.task.has_key; })
      .def_property_readonly("key_signature", [](const Message& x) { return x.task.key_signature; })
      .def_property_readonly("key_range", [](const Message& x) -> py::object { if (!x.task.has_key_range) return py::none(); return py::cast(std::make_pair(x.task.key_range.begin, x.task.key_range.end)); })
      .def_property_readonly("key", [](const Message& x) { return py::bytes(x.key); })
      .def_property_readonly("values", [](const Message& x) { std::vector<py::bytes> v; for (auto& s : x.value) v.emplace_back(s); return v; })
      .def_property_readonly("valid", [](const Message& x) { return x.valid; })
      .def("defer", [](Message& x) { x.finished = false; }, "do not mark the task finished / ack it when process() returns")
      .def("__repr__", [](const Message& x) { return "<Message " + x.short_debug() + ">"; });
  m.def("slice_key_ordered", [](py::bytes key, std::vector<py::bytes> values, std::vector<uint64_t> sep, py::object key_range) {
    auto msg = std::make_shared<Message>();
    msg->key = key; msg->task.has_key = true;
    for (auto& v : values) msg->value.push_back(v);
    if (!key_range.is_none()) { auto r = key_range.cast<std::pair<uint64_t, uint64_t>>(); msg->task.key_range = Range(r.first, r.second); msg->task.has_key_range = true; }
    return slice_key_ordered(msg, sep);
  }, py::arg("key"), py::arg("values"), py::arg("separators"), py::arg("key_range") = py::none());
  m.def("encode_decode", [](MessagePtr msg, bool compress) { std::string f = encode_message(*msg, compress); return py::make_tuple(f.size(), decode_message(f.data(), f.size())); });

  py::class_<Postoffice>(m, "Postoffice")
      .def(py::init<std::shared_ptr<Van>, int, int, int>(), py::arg("van"), py::arg("num_workers"), py::arg("num_servers"), py::arg("num_replicas") = 0)
      .def_property_readonly("my_node", [](Postoffice& p) { return p.my_node(); })
      .def("set_scheduler", &Postoffice::set_scheduler)
      .def("start", &Postoffice::start)
      .def("stop", &Postoffice::stop, py::call_guard<py::gil_scoped_release>())
      .def("register_with_scheduler", &Postoffice::register_with_scheduler)
      .def("wait_nodes_and_init", &Postoffice::wait_nodes_and_init, py::call_guard<py::gil_scoped_release>())
      .def("wait_nodes_ready", &Postoffice::wait_nodes_ready, py::call_guard<py::gil_scoped_release>())
      .def("set_nodes", &Postoffice::set_nodes)
      .def("nodes", &Postoffice::nodes)
      .def("stop_all", &Postoffice::stop_all, py::call_guard<py::gil_scoped_release>())
      .def("wait_terminate", &Postoffice::wait_terminate, py::call_guard<py::gil_scoped_release>())
      .def("set_key_cache", &Postoffice::set_key_cache)
      .def("on_manage_app", [](Postoffice& p, py::function f) { p.on_manage_app([h = hold(f)](const std::string& s) { py::gil_scoped_acquire g; (*h)(py::bytes(s)); }); })
      .def("start_heartbeat", [](Postoffice& p, double interval, py::object f) {
        if (f.is_none()) { p.start_heartbeat(interval, nullptr); return; }
        p.start_heartbeat(interval, [h = hold(f)]() { py::gil_scoped_acquire g; return (*h)().cast<std::string>(); });
      })
      .def("heartbeats", [](Postoffice& p) { py::dict d; const double now = now_seconds(); for (auto& kv : p.heartbeats()) d[py::str(kv.first)] = py::make_tuple(now - kv.second.when, py::bytes(kv.second.report)); return d; })
      .def("dead_nodes", &Postoffice::dead_nodes)
      .def("last_task_of", &Postoffice::last_task_of)
      .def("sent_bytes", [](Postoffice& p) { return p.van()->sent_bytes(); })
      .def("recv_bytes", [](Postoffice& p) { return p.van()->recv_bytes(); });

  py::class_<PyCustomer>(m, "Customer")
      .def(py::init([](Postoffice* po, std::string name, py::object process, bool key_ordered_slice) {
        auto c = new PyCustomer(po, name);
        c->key_ordered_slice = key_ordered_slice;
        if (!process.is_none()) c->process = [h = hold(process)](const MessagePtr& msg) {
          py::gil_scoped_acquire g;
          try { (*h)(msg); } catch (py::error_already_set& e) { std::fprintf(stderr, "exception in process(): %s\n", e.what()); }
        };
        return c;
      }), py::arg("postoffice"), py::arg("name"), py::arg("process") = py::none(), py::arg("key_ordered_slice") = true, py::keep_alive<1, 2>())
      .def_property_readonly("name", &PyCustomer::name)
      .def("submit", [](PyCustomer& c, const std::string& recver, int cmd, py::bytes payload, py::object key, std::vector<py::bytes> values, int time, int wait_time,
                        int channel, py::object key_range, uint32_t flags, int aux, bool erase_key_cache, bool wait, py::object on_finish, int type) {
        auto msg = make_message(recver, type, cmd, payload, key, values, time, wait_time, channel, key_range, flags, aux, erase_key_cache);
        msg->wait = wait;
        if (!on_finish.is_none()) msg->fin_handle = [h = hold(on_finish)]() {
          py::gil_scoped_acquire g;
          try { (*h)(); } catch (py::error_already_set& e) { std::fprintf(stderr, "exception in finish callback: %s\n", e.what()); }
        };
        py::gil_scoped_release rel;
        return c.submit(msg);
      }, py::arg("recver"), py::arg("cmd") = 0, py::arg("payload") = py::bytes(), py::arg("key") = py::none(), py::arg("values") = std::vector<py::bytes>(),
         py::arg("time") = -1, py::arg("wait_time") = -1, py::arg("channel") = 0, py::arg("key_range") = py::none(), py::arg("flags") = 0, py::arg("aux") = 0,
         py::arg("erase_key_cache") = false, py::arg("wait") = false, py::arg("on_finish") = py::none(), py::arg("type") = (int)Task::CALL_CUSTOMER)
      .def("wait_out", &PyCustomer::wait_out, py::arg("node"), py::arg("time"), py::arg("timeout_s") = 1e9, py::call_guard<py::gil_scoped_release>())
      .def("wait_in", &PyCustomer::wait_in, py::arg("node"), py::arg("time"), py::arg("timeout_s") = 1e9, py::call_guard<py::gil_scoped_release>())
      .def("try_wait_out", &PyCustomer::try_wait_out)
      .def("finish_in", &PyCustomer::finish_in)
      .def("finish_out", &PyCustomer::finish_out)
      .def("reply", [](PyCustomer& c, MessagePtr req, py::object key, std::vector<py::bytes> values, py::bytes payload) {
        std::vector<std::string> v; for (auto& b : values) v.push_back(b);
        c.reply(req, key.is_none() ? std::string() : key.cast<std::string>(), std::move(v), payload);
      }, py::arg("request"), py::arg("key") = py::none(), py::arg("values") = std::vector<py::bytes>(), py::arg("payload") = py::bytes())
      .def("take_replies", [](PyCustomer& c, int t) { py::dict d; for (auto& kv : c.exec()->take_replies(t)) d[py::str(kv.first)] = py::bytes(kv.second); return d; })
      .def("group", [](PyCustomer& c, const std::string& id) { std::vector<std::string> ids; for (auto& r : c.exec()->group(id)) ids.push_back(r->node.id); return ids; })
      .def("partition", [](PyCustomer& c, const std::string& id) { return c.exec()->partition(id); })
      .def("processed", [](PyCustomer& c) { return (uint64_t)c.exec()->processed; })
      .def("pending_requests", [](PyCustomer& c) { return c.exec()->pending_requests(); })
      .def("abort_waits", [](PyCustomer& c) { c.exec()->abort_waits(); }, "calls off every wait_in / wait_out on this customer (the job is over)")
      .def("stop", [](PyCustomer& c) {
        c.exec()->stop();
        // the callback usually is a bound method of the object that owns this customer: dropping it breaks that cycle,
        // which the interpreter's collector cannot see through
        if (!dynamic_cast<SharedParamCustomerT<PyCustomer>*>(&c) && !dynamic_cast<FTRLParamCustomerT<PyCustomer>*>(&c)) c.process = nullptr;
      }, py::call_guard<py::gil_scoped_release>());

  // the shared parameter of the batch solvers: push / pull served natively on the executor thread
  using PyShared = SharedParamCustomerT<PyCustomer>;
  py::class_<PyShared, PyCustomer>(m, "SharedParamCustomer")
      .def(py::init([](Postoffice* po, std::string name, int match_threads, int num_workers, int countmin_k, double countmin_n_ratio) {
        return new PyShared(po, std::move(name), match_threads, num_workers, countmin_k, countmin_n_ratio);
      }), py::arg("postoffice"), py::arg("name"), py::arg("match_threads") = 1, py::arg("num_workers") = 1, py::arg("countmin_k") = 2,
          py::arg("countmin_n_ratio") = 2.0, py::keep_alive<1, 2>())
      .def("keys", [](PyShared& c, int ch) { return to_array(c.keys(ch)); })
      .def("values", [](PyShared& c, int ch) { return to_array(c.values(ch)); })
      .def("set_values", [](PyShared& c, int ch, carray<double> a) { c.set_values(ch, a.data(), (size_t)a.size()); })
      .def("set_values_range", [](PyShared& c, int ch, size_t lo, carray<double> a) { c.set_values_range(ch, lo, a.data(), (size_t)a.size()); })
      .def("init_values", [](PyShared& c, int ch, double init) { c.init_values(ch, init); }, py::arg("ch"), py::arg("init") = 0.0)
      .def("received", [](PyShared& c, int t) { auto r = c.received(t); return py::make_tuple(r.lo, r.hi, r.nval, to_array(r.vals)); })
      .def("clear_filter", [](PyShared& c) { c.clear_filter(); })
      .def("take_pulled", [](PyShared& c, int t, const std::vector<std::string>& servers) { return pulled_arrays(c.take_pulled(t, servers)); });

  // the shared parameter of the online solver: an FTRL model per server, updated as pushes arrive
  using PyFtrlParam = FTRLParamCustomerT<PyCustomer>;
  py::class_<PyFtrlParam, PyCustomer>(m, "FTRLParamCustomer")
      .def(py::init([](Postoffice* po, std::string name, double alpha, double beta, double l1, double l2, size_t width, int k) {
        return new PyFtrlParam(po, std::move(name), alpha, beta, l1, l2, width, k);
      }), py::arg("postoffice"), py::arg("name"), py::arg("alpha"), py::arg("beta"), py::arg("lambda1"), py::arg("lambda2"),
          py::arg("sketch_width") = 1 << 20, py::arg("countmin_k") = 2, py::keep_alive<1, 2>())
      .def("stats", [](PyFtrlParam& c) { double a, b; size_t n; c.stats(&a, &b, &n); return py::make_tuple(a, b, n); })
      .def("size", &PyFtrlParam::size)
      .def("nonzero", [](PyFtrlParam& c) { std::vector<Key> k; std::vector<double> w; c.nonzero(&k, &w); return py::make_tuple(to_array(k), to_array(w)); })
      .def("take_pulled", [](PyFtrlParam& c, int t, const std::vector<std::string>& servers) { return pulled_arrays(c.take_pulled(t, servers)); });
}
