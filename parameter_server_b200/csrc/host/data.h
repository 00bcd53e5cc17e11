// Data ingest on the host: file search/assignment, text parsers (LIBSVM, ADFEA, TERAFEA) that
// emit column arrays per feature slot, the multi-threaded slot reader with its on-disk cache,
// the streaming minibatch reader and the binary matrix format.
//
// Counterparts in the reference: src/data/common.{h,cc} (searchFiles :96-146, divideFiles
// :148-166), src/data/example_parser.{h,cc}, src/data/slot_reader.{h,cc},
// src/data/stream_reader.h, src/base/matrix_io_inl.h (binary matrices :117-213),
// src/util/filelinereader.{h,cc}.  Cache partitions are zlib-compressed (the reference used
// snappy, which is not available here); the file layout is otherwise the reference's:
// <cache><DJBHash32(path)>-<name>_slot_<id>.{colidx,value,rowsiz} + .partition + .info.
#pragma once
#include <dirent.h>
#include <sys/stat.h>

#include <regex>
#include <sstream>

#include "message.h"

namespace psb {

enum class TextFormat { PS_DENSE = 1, PS_SPARSE = 2, PS_SPARSE_BINARY = 3, ADFEA = 4, LIBSVM = 5, TERAFEA = 6 };
enum class SlotFormat { DENSE = 1, SPARSE = 2, SPARSE_BINARY = 3 };

struct SlotInfo {
  int id = 0;
  SlotFormat format = SlotFormat::SPARSE;
  uint64_t min_key = kMaxKey, max_key = 0, nnz_ele = 0, nnz_ex = 0;   // max_key is exclusive (max + 1)
  void merge(const SlotInfo& o) {
    format = o.format;
    min_key = std::min(min_key, o.min_key);
    max_key = std::max(max_key, o.max_key);
    nnz_ele += o.nnz_ele;
    nnz_ex += o.nnz_ex;
  }
};
struct ExampleInfo {
  std::map<int, SlotInfo> slot;
  uint64_t num_ex = 0;
  void merge(const ExampleInfo& o) {
    num_ex += o.num_ex;
    for (auto& kv : o.slot) { auto& s = slot[kv.first]; s.id = kv.first; s.merge(kv.second); }
  }
  std::string to_text() const {
    std::ostringstream os;
    for (auto& kv : slot) {
      const SlotInfo& s = kv.second;
      os << "slot { format: " << (s.format == SlotFormat::DENSE ? "DENSE" : s.format == SlotFormat::SPARSE ? "SPARSE" : "SPARSE_BINARY")
         << " id: " << s.id << " min_key: " << s.min_key << " max_key: " << s.max_key << " nnz_ele: " << s.nnz_ele
         << " nnz_ex: " << s.nnz_ex << " }\n";
    }
    os << "num_ex: " << num_ex << "\n";
    return os.str();
  }
  static bool from_text(const std::string& text, ExampleInfo* out) {
    std::istringstream is(text);
    std::string tok;
    SlotInfo cur;
    bool in_slot = false;
    while (is >> tok) {
      if (tok == "slot") { is >> tok; cur = SlotInfo(); in_slot = true; }
      else if (tok == "}") { out->slot[cur.id] = cur; in_slot = false; }
      else if (tok == "format:") { is >> tok; cur.format = tok == "DENSE" ? SlotFormat::DENSE : tok == "SPARSE" ? SlotFormat::SPARSE : SlotFormat::SPARSE_BINARY; }
      else if (tok == "id:") is >> cur.id;
      else if (tok == "min_key:") is >> cur.min_key;
      else if (tok == "max_key:") is >> cur.max_key;
      else if (tok == "nnz_ele:") is >> cur.nnz_ele;
      else if (tok == "nnz_ex:") is >> cur.nnz_ex;
      else if (tok == "num_ex:") is >> out->num_ex;
      else return false;
    }
    return !in_slot;
  }
};

// Column arrays of one slot for a run of examples.  Slot 0 is the label (one value per row).
struct SlotData {
  std::vector<uint64_t> col_idx;
  std::vector<float> val;
  std::vector<uint32_t> row_siz;   // one entry per example (0 when the example lacks the slot)
  void clear() { col_idx.clear(); val.clear(); row_siz.clear(); }
  size_t mem() const { return col_idx.size() * 8 + val.size() * 4 + row_siz.size() * 4; }
};

// ------------------------------------------------------------------ files
inline bool file_exists(const std::string& p) {
  if (is_hdfs_path(p)) return std::system((hadoop_fs_command() + " -test -e " + shell_quote(p.substr(5)) + " >/dev/null 2>&1").c_str()) == 0;
  struct stat st;
  return ::stat(p.c_str(), &st) == 0;
}
inline std::string path_dir(const std::string& p) { auto s = p.find_last_of('/'); return s == std::string::npos ? "." : (s == 0 ? "/" : p.substr(0, s)); }
inline std::string path_name(const std::string& p) { auto s = p.find_last_of('/'); return s == std::string::npos ? p : p.substr(s + 1); }
inline bool make_dirs(const std::string& dir) {
  std::string cur;
  for (size_t i = 0; i <= dir.size(); ++i) {
    if (i == dir.size() || dir[i] == '/') { if (!cur.empty() && !file_exists(cur)) ::mkdir(cur.c_str(), 0755); }
    if (i < dir.size()) cur += dir[i];
  }
  return file_exists(dir);
}
// Names of the files in a directory "hdfs:<dir>": the last of the eight columns of `hadoop fs -ls`, directories left out.
inline std::vector<std::string> list_hdfs_dir(const std::string& dir) {
  std::vector<std::string> out;
  FILE* p = ::popen((hadoop_fs_command() + " -ls " + shell_quote(dir.substr(5)) + " 2>/dev/null").c_str(), "r");
  if (!p) return out;
  char line[10000];
  while (std::fgets(line, sizeof(line), p)) {
    std::vector<std::string> col;
    std::istringstream in(line);
    for (std::string t; in >> t;) col.push_back(t);
    if (col.size() != 8 || col[0][0] == 'd') continue;
    auto s = col.back().find_last_of('/');
    out.push_back(s == std::string::npos ? col.back() : col.back().substr(s + 1));
  }
  ::pclose(p);
  std::sort(out.begin(), out.end());
  return out;
}
inline std::vector<std::string> list_dir(const std::string& dir) {
  if (is_hdfs_path(dir)) return list_hdfs_dir(dir);
  std::vector<std::string> out;
  DIR* d = ::opendir(dir.c_str());
  if (!d) return out;
  while (dirent* e = ::readdir(d)) { std::string n = e->d_name; if (n != "." && n != "..") out.push_back(n); }
  ::closedir(d);
  std::sort(out.begin(), out.end());
  return out;
}
// Every pattern's file-name part is a regular expression matched against the names in its
// directory; results are de-duplicated and sorted.
inline std::vector<std::string> search_files(const std::vector<std::string>& patterns) {
  std::set<std::string> found;
  for (const auto& p : patterns) {
    const std::string dir = path_dir(p), pat = path_name(p);
    std::regex re;
    try { re = std::regex(pat); } catch (const std::regex_error&) { if (file_exists(p)) found.insert(p); continue; }
    for (const auto& n : list_dir(dir)) if (std::regex_match(n, re)) found.insert(dir + "/" + n);
  }
  return std::vector<std::string>(found.begin(), found.end());
}
// file j goes to worker j % num_workers; at most `load_limit` files per worker when > 0
inline std::vector<std::vector<std::string>> divide_files(const std::vector<std::string>& files, int num_workers, int load_limit) {
  std::vector<std::vector<std::string>> out(std::max(num_workers, 1));
  for (size_t j = 0; j < files.size(); ++j) {
    auto& mine = out[j % out.size()];
    if (load_limit > 0 && (int)mine.size() >= load_limit) continue;
    mine.push_back(files[j]);
  }
  return out;
}

// ------------------------------------------------------------------ number parsing
inline bool parse_u64(const char* s, uint64_t* v) { if (!s || !*s) return false; char* e; errno = 0; *v = std::strtoull(s, &e, 10); return errno == 0 && *e == 0 && e != s; }
inline bool parse_i32(const char* s, int32_t* v) { if (!s || !*s) return false; char* e; errno = 0; long x = std::strtol(s, &e, 10); *v = (int32_t)x; return errno == 0 && *e == 0 && e != s; }
inline bool parse_f32(const char* s, float* v) { if (!s || !*s) return false; char* e; errno = 0; *v = std::strtof(s, &e); return *e == 0 && e != s; }

// ------------------------------------------------------------------ example parser
// Parses one text line and appends the example to per-slot column arrays.
class ExampleParser {
 public:
  void init(TextFormat f, bool ignore_feature_group, bool shuffle_fea_id = false, bool add_beta_feature = false) {
    fmt_ = f; ignore_grp_ = ignore_feature_group; shuffle_ = shuffle_fea_id; beta_ = add_beta_feature;
  }
  // returns false (and leaves `out` untouched) on a malformed line
  bool parse_line(char* line, std::map<int, SlotData>* out, ExampleInfo* info) {
    tmp_.clear();
    label_ = 0;
    bool ok = false;
    switch (fmt_) {
      case TextFormat::LIBSVM: ok = parse_libsvm(line); break;
      case TextFormat::ADFEA: ok = parse_adfea(line); break;
      case TextFormat::TERAFEA: ok = parse_terafea(line); break;
      default: ok = false;
    }
    if (!ok) return false;
    const size_t row = info->num_ex;
    auto& lab = (*out)[0];
    lab.val.push_back(label_);
    auto& li = info->slot[0];
    li.id = 0; li.format = SlotFormat::DENSE; li.nnz_ele += 1; li.nnz_ex += 1;
    for (auto& kv : tmp_) {
      const int id = ignore_grp_ ? 1 : kv.first;
      auto& sd = (*out)[id];
      if (sd.row_siz.size() < row) sd.row_siz.resize(row, 0);            // examples that lacked this slot
      if (sd.row_siz.size() == row) sd.row_siz.push_back(0);
      auto& si = info->slot[id];
      si.id = id;
      si.format = binary_ ? SlotFormat::SPARSE_BINARY : SlotFormat::SPARSE;
      if (!kv.second.first.empty()) si.nnz_ex += (sd.row_siz[row] == 0);
      for (size_t i = 0; i < kv.second.first.size(); ++i) {
        const uint64_t k = kv.second.first[i];
        sd.col_idx.push_back(k);
        if (!binary_) sd.val.push_back(kv.second.second[i]);
        si.min_key = std::min(si.min_key, k);
        si.max_key = std::max(si.max_key, k + 1);
      }
      sd.row_siz[row] += (uint32_t)kv.second.first.size();
      si.nnz_ele += kv.second.first.size();
    }
    ++info->num_ex;
    return true;
  }
  // pad every slot's row_siz to num_ex rows (call once after the last line of a block)
  static void finish(std::map<int, SlotData>* out, uint64_t num_ex) {
    for (auto& kv : *out) if (kv.first != 0) kv.second.row_siz.resize(num_ex, 0);
  }

 private:
  bool parse_libsvm(char* buf) {   // label idx:val idx:val ...   (ascending idx)
    binary_ = false;
    char* save;
    char* p = strtok_r(buf, " \t\r\n", &save);
    if (!parse_f32(p, &label_)) return false;
    auto& s = tmp_[1];
    uint64_t last = 0;
    for (p = strtok_r(nullptr, " \t\r\n", &save); p; p = strtok_r(nullptr, " \t\r\n", &save)) {
      char* c = std::strchr(p, ':');
      if (!c) return false;
      *c = 0;
      uint64_t idx; float v;
      if (!parse_u64(p, &idx) || !parse_f32(c + 1, &v) || last > idx) return false;
      last = idx;
      s.first.push_back(idx);
      s.second.push_back(v);
    }
    return true;
  }
  bool parse_adfea(char* line) {   // line_id 1 clicked key:grp key:grp ...
    binary_ = true;
    char* save;
    uint64_t key = 0;
    int i = 0;
    for (char* t = strtok_r(line, " :\t\r\n", &save); t; t = strtok_r(nullptr, " :\t\r\n", &save), ++i) {
      if (i < 2) continue;
      if (i == 2) { int32_t l; if (!parse_i32(t, &l)) return false; label_ = l > 0 ? 1.f : -1.f; }
      else if (i % 2 == 1) { if (!parse_u64(t, &key)) return false; }
      else { int32_t g = 1; if (!ignore_grp_ && !parse_i32(t, &g)) return false; tmp_[g].first.push_back(key); }
    }
    return i >= 3;
  }
  bool parse_terafea(char* line) {   // clicked line_id | u64 u64 ...   (group = top 10 bits)
    binary_ = true;
    char* save;
    std::vector<uint64_t> keys;
    int i = 0;
    for (char* t = strtok_r(line, " |\t\r\n", &save); t; t = strtok_r(nullptr, " |\t\r\n", &save), ++i) {
      if (i == 0) { int32_t l; if (!parse_i32(t, &l)) return false; label_ = l > 0 ? 1.f : -1.f; }
      else if (i == 1) continue;
      else { uint64_t k; if (!parse_u64(t, &k)) return false; keys.push_back(k); }
    }
    if (i < 1) return false;
    std::sort(keys.begin(), keys.end());
    for (uint64_t k : keys) tmp_[(int)(k >> 54)].first.push_back(shuffle_ ? shuffle_feature_id(k) : k);
    if (beta_) tmp_[1023].first.push_back(0);
    return true;
  }
  TextFormat fmt_ = TextFormat::LIBSVM;
  bool ignore_grp_ = false, shuffle_ = false, beta_ = false, binary_ = false;
  float label_ = 0;
  std::map<int, std::pair<std::vector<uint64_t>, std::vector<float>>> tmp_;
};

// ------------------------------------------------------------------ slot reader
// Parses every file once (one task per file, `threads` at a time) into per-slot column arrays kept
// as compressed partitions in cache files; later calls re-assemble a slot from the cache.  A file
// whose `.info` exists in the cache directory is not parsed again.
class SlotReader {
 public:
  void init(std::vector<std::string> files, TextFormat fmt, std::string cache_dir, bool ignore_feature_group,
            bool shuffle_fea_id = false, bool add_beta_feature = false, size_t line_limit = 0, size_t max_mb_per_thread = 2048) {
    files_ = std::move(files); fmt_ = fmt; cache_ = std::move(cache_dir);
    if (!cache_.empty() && cache_.back() != '/') cache_ += '/';
    ignore_grp_ = ignore_feature_group; shuffle_ = shuffle_fea_id; beta_ = add_beta_feature;
    line_limit_ = line_limit; max_bytes_ = max_mb_per_thread << 20;
    make_dirs(cache_.substr(0, cache_.size() - 1));
  }
  // returns the number of files served from the cache
  int read(int threads, ExampleInfo* info) {
    std::vector<ExampleInfo> infos(files_.size());
    std::vector<int> hit(files_.size(), 0);
    std::vector<std::string> err(files_.size());
    {
      ThreadPool pool(threads);
      for (size_t i = 0; i < files_.size(); ++i) pool.add([this, i, &infos, &hit, &err] {
        try { hit[i] = read_one(files_[i], &infos[i]); } catch (const std::exception& e) { err[i] = e.what(); }
      });
      pool.start();
    }
    int hits = 0;
    info_ = ExampleInfo();
    file_rows_.clear();
    for (size_t i = 0; i < files_.size(); ++i) {
      if (!err[i].empty()) throw std::runtime_error(files_[i] + ": " + err[i]);
      info_.merge(infos[i]);
      file_rows_.push_back(infos[i].num_ex);
      hits += hit[i];
    }
    *info = info_;
    return hits;
  }
  const ExampleInfo& info() const { return info_; }
  std::vector<uint64_t> index(int slot) { return assemble<uint64_t>(slot, "colidx"); }
  std::vector<float> value(int slot) { return assemble<float>(slot, "value"); }
  // CSR offsets (num_ex + 1) of a slot over all files
  std::vector<uint64_t> offset(int slot) {
    auto siz = assemble<uint32_t>(slot, "rowsiz");
    std::vector<uint64_t> off(siz.size() + 1, 0);
    for (size_t i = 0; i < siz.size(); ++i) off[i + 1] = off[i] + siz[i];
    return off;
  }
  std::string cache_name(const std::string& file, int slot) const {
    return cache_ + std::to_string(djb_hash32(file)) + "-" + path_name(file) + "_slot_" + std::to_string(slot);
  }

 private:
  std::string info_name(const std::string& file) const { return cache_ + std::to_string(djb_hash32(file)) + "-" + path_name(file) + ".info"; }
  static void append_partition(const std::string& name, const char* ext, const void* data, size_t bytes) {
    const std::string z = bytes ? zlib_compress(static_cast<const char*>(data), bytes) : std::string();
    const std::string f = name + "." + ext;
    uint64_t start = 0;
    { std::ifstream in(f, std::ios::binary | std::ios::ate); if (in) start = (uint64_t)in.tellg(); }
    { std::ofstream out(f, std::ios::binary | std::ios::app); out.write(z.data(), (std::streamsize)z.size()); }
    std::ofstream idx(f + ".partition", std::ios::app);
    idx << start << "\t" << z.size() << "\t" << bytes << "\n";
  }
  void spill(const std::string& file, std::map<int, SlotData>* slots, uint64_t rows) {
    ExampleParser::finish(slots, rows);
    for (auto& kv : *slots) {
      const std::string name = cache_name(file, kv.first);
      auto& s = kv.second;
      if (kv.first == 0) {
        append_partition(name, "value", s.val.data(), s.val.size() * 4);
      } else {
        // rows of this spill that precede the first row of the slot were padded by finish(); rows of
        // earlier spills are padded by the per-spill row base
        append_partition(name, "colidx", s.col_idx.data(), s.col_idx.size() * 8);
        append_partition(name, "value", s.val.data(), s.val.size() * 4);
        append_partition(name, "rowsiz", s.row_siz.data(), s.row_siz.size() * 4);
      }
      s.clear();
    }
  }
  int read_one(const std::string& file, ExampleInfo* info) {
    const std::string inf = info_name(file);
    if (file_exists(inf)) {
      std::ifstream in(inf);
      std::stringstream ss; ss << in.rdbuf();
      if (ExampleInfo::from_text(ss.str(), info)) return 1;
      *info = ExampleInfo();
    }
    auto f = File::open(file, "r");
    if (!f) throw std::runtime_error("cannot open");
    ExampleParser parser;
    parser.init(fmt_, ignore_grp_, shuffle_, beta_);
    std::map<int, SlotData> slots;
    std::vector<char> line(1 << 20);
    uint64_t rows_in_spill = 0, spills = 0;
    ExampleInfo spill_info;           // row counter local to the current spill
    std::set<int> seen;
    size_t nline = 0;
    while (f->read_line(line.data(), (int)line.size())) {
      if (line_limit_ && nline >= line_limit_) break;
      ++nline;
      if (line[0] == 0 || line[0] == '\n' || line[0] == '#') continue;
      if (!parser.parse_line(line.data(), &slots, &spill_info)) continue;
      ++rows_in_spill;
      size_t mem = 0;
      for (auto& kv : slots) mem += kv.second.mem();
      if (mem > max_bytes_) {
        pad_new_slots(file, slots, &seen, info->num_ex);
        spill(file, &slots, rows_in_spill);
        info->merge(spill_info);
        spill_info = ExampleInfo();
        rows_in_spill = 0;
        ++spills;
      }
    }
    pad_new_slots(file, slots, &seen, info->num_ex);
    spill(file, &slots, rows_in_spill);
    info->merge(spill_info);
    // slots that appeared only in early spills need zero rows for the later ones
    for (int id : seen) {
      if (id == 0) continue;
      const uint64_t have = rows_in_cache(cache_name(file, id));
      if (have < info->num_ex) {
        std::vector<uint32_t> z(info->num_ex - have, 0);
        append_partition(cache_name(file, id), "rowsiz", z.data(), z.size() * 4);
      }
    }
    std::ofstream out(inf);
    out << info->to_text();
    return 0;
  }
  // a slot first seen in a later spill gets zero rows for the examples of the earlier spills
  void pad_new_slots(const std::string& file, const std::map<int, SlotData>& slots, std::set<int>* seen, uint64_t rows_before) {
    for (auto& kv : slots) {
      if (seen->insert(kv.first).second && kv.first != 0 && rows_before > 0) {
        std::vector<uint32_t> z(rows_before, 0);
        append_partition(cache_name(file, kv.first), "rowsiz", z.data(), z.size() * 4);
      }
    }
  }
  static uint64_t rows_in_cache(const std::string& name) {
    std::ifstream idx(name + ".rowsiz.partition");
    uint64_t start, zs, raw, rows = 0;
    while (idx >> start >> zs >> raw) rows += raw / 4;
    return rows;
  }
  template <typename T>
  std::vector<T> assemble(int slot, const char* ext) {
    std::vector<T> out;
    for (size_t fi = 0; fi < files_.size(); ++fi) {
      const std::string name = cache_name(files_[fi], slot) + "." + ext;
      std::ifstream idx(name + ".partition");
      std::ifstream in(name, std::ios::binary);
      uint64_t start, zs, raw;
      size_t got = 0;
      while (idx >> start >> zs >> raw) {
        const size_t at = out.size();
        out.resize(at + raw / sizeof(T));
        got += raw / sizeof(T);
        if (raw == 0) continue;
        std::string z(zs, '\0');
        in.seekg((std::streamoff)start);
        in.read(&z[0], (std::streamsize)zs);
        if (!zlib_uncompress(z.data(), zs, reinterpret_cast<char*>(out.data() + at), raw)) throw std::runtime_error("corrupt cache " + name);
      }
      // a file in which the slot never occurs contributes empty rows
      if (std::string(ext) == "rowsiz" && got < file_rows_[fi]) out.resize(out.size() + (file_rows_[fi] - got), 0);
    }
    return out;
  }
  std::vector<std::string> files_;
  std::vector<uint64_t> file_rows_;
  TextFormat fmt_ = TextFormat::LIBSVM;
  std::string cache_;
  bool ignore_grp_ = false, shuffle_ = false, beta_ = false;
  size_t line_limit_ = 0, max_bytes_ = 2048ull << 20;
  ExampleInfo info_;
};

// ------------------------------------------------------------------ stream reader
// Sequential minibatches over a list of text files: labels + one CSR matrix per slot.
class StreamReader {
 public:
  void init(std::vector<std::string> files, TextFormat fmt, bool ignore_feature_group, bool shuffle_fea_id = false) {
    files_ = std::move(files);
    parser_.init(fmt, ignore_feature_group, shuffle_fea_id, false);
    next_ = 0;
    cur_.reset();
    line_.resize(1 << 20);
  }
  // reads up to n examples; returns false when no example is left
  bool read(size_t n, std::map<int, SlotData>* slots, ExampleInfo* info) {
    slots->clear();
    *info = ExampleInfo();
    while (info->num_ex < n) {
      if (!cur_) {
        if (next_ >= files_.size()) break;
        cur_ = File::open(files_[next_++], "r");
        if (!cur_) continue;
      }
      if (!cur_->read_line(line_.data(), (int)line_.size())) { cur_.reset(); continue; }
      if (line_[0] == 0 || line_[0] == '\n' || line_[0] == '#') continue;
      parser_.parse_line(line_.data(), slots, info);
    }
    ExampleParser::finish(slots, info->num_ex);
    return info->num_ex > 0;
  }

 private:
  std::vector<std::string> files_;
  size_t next_ = 0;
  std::unique_ptr<File> cur_;
  ExampleParser parser_;
  std::vector<char> line_;
};

// ------------------------------------------------------------------ binary matrices
// name.info (text) + name.offset (u64) + name.index (u32|u64) + name.value (float)
struct BinMatrix {
  bool sparse = true, binary = false, row_major = true;
  uint64_t rows = 0, cols = 0, nnz = 0;
  int sizeof_index = 8;
  std::vector<uint64_t> offset;
  std::vector<uint64_t> index;
  std::vector<float> value;
};
template <typename T> inline bool write_array(const std::string& path, const std::vector<T>& v) {
  std::ofstream f(path, std::ios::binary);
  f.write(reinterpret_cast<const char*>(v.data()), (std::streamsize)(v.size() * sizeof(T)));
  return f.good();
}
template <typename T> inline bool read_array(const std::string& path, std::vector<T>* v, uint64_t first = 0, uint64_t count = ~0ull) {
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f) return false;
  const uint64_t total = (uint64_t)f.tellg() / sizeof(T);
  if (first > total) return false;
  count = std::min<uint64_t>(count, total - first);
  v->resize(count);
  f.seekg((std::streamoff)(first * sizeof(T)));
  f.read(reinterpret_cast<char*>(v->data()), (std::streamsize)(count * sizeof(T)));
  return f.good() || count == 0;
}
inline bool write_bin_matrix(const std::string& name, const BinMatrix& m) {
  std::ofstream info(name + ".info");
  info << "type: " << (!m.sparse ? "DENSE" : m.binary ? "SPARSE_BINARY" : "SPARSE") << "\nrow_major: " << (m.row_major ? "true" : "false")
       << "\nrow { begin: 0 end: " << m.rows << " }\ncol { begin: 0 end: " << m.cols << " }\nnnz: " << m.nnz
       << "\nsizeof_index: " << m.sizeof_index << "\nsizeof_value: 4\n";
  bool ok = info.good();
  if (m.sparse) {
    ok = write_array(name + ".offset", m.offset) && ok;
    if (m.sizeof_index == 4) { std::vector<uint32_t> i32(m.index.begin(), m.index.end()); ok = write_array(name + ".index", i32) && ok; }
    else ok = write_array(name + ".index", m.index) && ok;
  }
  if (!m.binary) ok = write_array(name + ".value", m.value) && ok;
  return ok;
}
// reads outer rows [row_begin, row_end) (the whole matrix when row_end = ~0)
inline bool read_bin_matrix(const std::string& name, BinMatrix* m, uint64_t row_begin = 0, uint64_t row_end = ~0ull) {
  std::ifstream info(name + ".info");
  if (!info) return false;
  std::string tok;
  while (info >> tok) {
    if (tok == "type:") { info >> tok; m->sparse = tok != "DENSE"; m->binary = tok == "SPARSE_BINARY"; }
    else if (tok == "row_major:") { info >> tok; m->row_major = tok == "true"; }
    else if (tok == "row" || tok == "col") {
      const bool is_row = tok == "row";
      std::string b; uint64_t lo = 0, hi = 0;
      info >> b >> b >> lo >> b >> hi >> b;
      (is_row ? m->rows : m->cols) = hi - lo;
    }
    else if (tok == "nnz:") info >> m->nnz;
    else if (tok == "sizeof_index:") info >> m->sizeof_index;
    else if (tok == "sizeof_value:") { int v; info >> v; }
  }
  const uint64_t outer = m->row_major ? m->rows : m->cols;
  row_end = std::min(row_end, outer);
  if (row_begin > row_end) return false;
  if (!m->sparse) {
    const uint64_t inner = m->row_major ? m->cols : m->rows;
    return read_array(name + ".value", &m->value, row_begin * inner, (row_end - row_begin) * inner);
  }
  if (!read_array(name + ".offset", &m->offset, row_begin, row_end - row_begin + 1)) return false;
  const uint64_t p0 = m->offset.front(), p1 = m->offset.back();
  for (auto& o : m->offset) o -= p0;
  if (m->sizeof_index == 4) {
    std::vector<uint32_t> i32;
    if (!read_array(name + ".index", &i32, p0, p1 - p0)) return false;
    m->index.assign(i32.begin(), i32.end());
  } else if (!read_array(name + ".index", &m->index, p0, p1 - p0)) return false;
  if (!m->binary && !read_array(name + ".value", &m->value, p0, p1 - p0)) return false;
  if (m->row_major) m->rows = row_end - row_begin; else m->cols = row_end - row_begin;
  m->nnz = p1 - p0;
  return true;
}

}  // namespace psb
