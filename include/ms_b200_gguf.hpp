// GGUF reader for the host side of the drop-in: typed metadata, the tensor table with ABSOLUTE file offsets across all
// splits, ggml type sizes, and the per-layer expert layout -- the interface of the reference's src/gguf/gguf.hpp:38-96
// and ExpertLayout::from_gguf (src/store/experts.hpp:35-42, experts.mm:36-54), without its SSD streaming machinery:
// with the experts resident in HBM the file is read once, range by range, at load time (ms_b200_expert_shard.hpp).
// Pure host code: no CUDA, no dependency on the kernel library.  Errors throw std::runtime_error (the reference aborts).
#pragma once
#include <algorithm>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace ms {

enum class GType : uint32_t {
  F32 = 0, F16 = 1, Q4_0 = 2, Q4_1 = 3, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q8_1 = 9, Q2_K = 10, Q3_K = 11, Q4_K = 12,
  Q5_K = 13, Q6_K = 14, Q8_K = 15, IQ2_XXS = 16, IQ2_XS = 17, IQ3_XXS = 18, IQ1_S = 19, IQ4_NL = 20, IQ3_S = 21,
  IQ2_S = 22, IQ4_XS = 23, I8 = 24, I16 = 25, I32 = 26, I64 = 27, F64 = 28, IQ1_M = 29, BF16 = 30, TQ1_0 = 34,
  TQ2_0 = 35, MXFP4 = 39,
};
struct TypeInfo { const char* name; uint32_t blck; uint32_t bytes; };   // elements per block, bytes per block

inline const TypeInfo* type_info(GType t) {
  struct Row { GType t; TypeInfo i; };
  static const Row rows[] = {
      {GType::F32, {"F32", 1, 4}},         {GType::F16, {"F16", 1, 2}},         {GType::Q4_0, {"Q4_0", 32, 18}},
      {GType::Q4_1, {"Q4_1", 32, 20}},     {GType::Q5_0, {"Q5_0", 32, 22}},     {GType::Q5_1, {"Q5_1", 32, 24}},
      {GType::Q8_0, {"Q8_0", 32, 34}},     {GType::Q8_1, {"Q8_1", 32, 36}},     {GType::Q2_K, {"Q2_K", 256, 84}},
      {GType::Q3_K, {"Q3_K", 256, 110}},   {GType::Q4_K, {"Q4_K", 256, 144}},   {GType::Q5_K, {"Q5_K", 256, 176}},
      {GType::Q6_K, {"Q6_K", 256, 210}},   {GType::Q8_K, {"Q8_K", 256, 292}},   {GType::IQ2_XXS, {"IQ2_XXS", 256, 66}},
      {GType::IQ2_XS, {"IQ2_XS", 256, 74}}, {GType::IQ3_XXS, {"IQ3_XXS", 256, 98}}, {GType::IQ1_S, {"IQ1_S", 256, 50}},
      {GType::IQ4_NL, {"IQ4_NL", 32, 18}}, {GType::IQ3_S, {"IQ3_S", 256, 110}}, {GType::IQ2_S, {"IQ2_S", 256, 82}},
      {GType::IQ4_XS, {"IQ4_XS", 256, 136}}, {GType::I8, {"I8", 1, 1}},          {GType::I16, {"I16", 1, 2}},
      {GType::I32, {"I32", 1, 4}},         {GType::I64, {"I64", 1, 8}},         {GType::F64, {"F64", 1, 8}},
      {GType::IQ1_M, {"IQ1_M", 256, 56}},  {GType::BF16, {"BF16", 1, 2}},       {GType::TQ1_0, {"TQ1_0", 256, 54}},
      {GType::TQ2_0, {"TQ2_0", 256, 66}},  {GType::MXFP4, {"MXFP4", 32, 17}},
  };
  for (const Row& r : rows)
    if (r.t == t) return &r.i;
  return nullptr;
}
inline const char* type_name(GType t) { const TypeInfo* i = type_info(t); return i ? i->name : "?"; }
inline uint64_t type_bytes(GType t, uint64_t nelem) {
  const TypeInfo* i = type_info(t);
  if (!i || nelem % i->blck) throw std::runtime_error("gguf: element count is not a multiple of the type's block");
  return nelem / i->blck * i->bytes;
}

enum class KvType : uint32_t { U8 = 0, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 };

struct KvValue {
  KvType type = KvType::U8;
  KvType arr_type = KvType::U8;       // element type when type == ARR
  // scalars: integers / bools fill i and u (same bits), floats fill f (integers are mirrored into f), strings fill s
  int64_t i = 0; uint64_t u = 0; double f = 0; std::string s;
  // arrays by element type: integer / bool -> ai, float -> af, string -> as, nested array -> aa
  std::vector<int64_t> ai; std::vector<double> af; std::vector<std::string> as; std::vector<KvValue> aa;
  size_t size() const { return type != KvType::ARR ? 0 : !ai.empty() ? ai.size() : !af.empty() ? af.size() : !as.empty() ? as.size() : aa.size(); }
  bool is_int() const { return type != KvType::F32 && type != KvType::F64 && type != KvType::STR && type != KvType::ARR; }
  bool is_float() const { return type == KvType::F32 || type == KvType::F64; }
};

struct TensorInfo {
  std::string name;
  GType type = GType::F32;
  int n_dims = 0;
  int64_t ne[4] = {1, 1, 1, 1};       // ggml order: ne[0] contiguous
  uint64_t nbytes = 0;
  int split = 0;                      // index into Gguf::path()
  uint64_t offset = 0;                // ABSOLUTE byte offset of the data in that split file
  int64_t nelements() const { return ne[0] * ne[1] * ne[2] * ne[3]; }
  uint64_t row_bytes() const { return type_bytes(type, (uint64_t)ne[0]); }
};

// pread until len bytes or EOF, retrying interrupted and short reads; bytes read, or -1 on error
inline long long pread_full(int fd, void* dst, size_t len, uint64_t off) {
  size_t got = 0;
  while (got < len) {
    const ssize_t n = ::pread(fd, static_cast<char*>(dst) + got, len - got, (off_t)(off + got));
    if (n < 0) { if (errno == EINTR) continue; return -1; }
    if (n == 0) break;
    got += (size_t)n;
  }
  return (long long)got;
}

class Gguf {
 public:
  // One path: if it matches "*-0000N-of-0000M.gguf" all M splits are opened, else just that file.
  explicit Gguf(const std::string& path) : Gguf(expand_splits(path)) {}
  explicit Gguf(const std::vector<std::string>& paths) {
    files_.resize(paths.size());
    for (size_t k = 0; k < paths.size(); k++) {
      File& f = files_[k];
      f.path = paths[k];
      f.fd = ::open(f.path.c_str(), O_RDONLY);
      if (f.fd < 0) throw std::runtime_error("gguf: cannot open " + f.path);
      struct stat st;
      if (::fstat(f.fd, &st) != 0) throw std::runtime_error("gguf: cannot stat " + f.path);
      f.size = (uint64_t)st.st_size;
      parse_file((int)k);
    }
    for (size_t k = 0; k < tensors_.size(); k++) tindex_[tensors_[k].name] = k;
  }
  ~Gguf() { for (File& f : files_) if (f.fd >= 0) ::close(f.fd); }
  Gguf(const Gguf&) = delete;
  Gguf& operator=(const Gguf&) = delete;

  static std::vector<std::string> expand_splits(const std::string& path) {
    // <stem>-NNNNN-of-MMMMM.gguf, five digits each
    const size_t n = path.size();
    auto digits = [&](size_t at) { for (size_t k = 0; k < 5; k++) if (at + k >= n || path[at + k] < '0' || path[at + k] > '9') return false; return true; };
    if (n < 20 || path.compare(n - 5, 5, ".gguf") != 0 || path.compare(n - 14, 4, "-of-") != 0 || path[n - 20] != '-' ||
        !digits(n - 19) || !digits(n - 10))
      return {path};
    const int total = std::stoi(path.substr(n - 10, 5));
    std::vector<std::string> out;
    char tail[40];
    for (int k = 1; k <= total; k++) {
      std::snprintf(tail, sizeof tail, "-%05d-of-%05d.gguf", k, total);
      out.push_back(path.substr(0, n - 20) + tail);
    }
    return out;
  }
  static bool exists(const std::string& path) { struct stat st; return ::stat(path.c_str(), &st) == 0; }

  // metadata (merged across splits, first occurrence wins; insertion order kept in keys())
  const KvValue* kv(const std::string& key) const { auto it = kv_.find(key); return it == kv_.end() ? nullptr : &it->second; }
  const std::vector<std::string>& keys() const { return kv_order_; }
  int64_t get_i64(const std::string& key, int64_t dflt = 0) const {
    const KvValue* v = kv(key);
    return !v || v->type == KvType::STR || v->type == KvType::ARR ? dflt : v->is_float() ? (int64_t)v->f : v->i;
  }
  double get_f64(const std::string& key, double dflt = 0) const {
    const KvValue* v = kv(key);
    return !v || v->type == KvType::STR || v->type == KvType::ARR ? dflt : v->f;
  }
  std::string get_str(const std::string& key, const std::string& dflt = "") const {
    const KvValue* v = kv(key);
    return v && v->type == KvType::STR ? v->s : dflt;
  }
  std::vector<int64_t> get_arr_i64(const std::string& key) const {
    const KvValue* v = kv(key);
    if (!v || v->type != KvType::ARR) return {};
    if (!v->ai.empty()) return v->ai;
    return std::vector<int64_t>(v->af.begin(), v->af.end());
  }
  std::vector<float> get_arr_f32(const std::string& key) const {
    const KvValue* v = kv(key);
    if (!v || v->type != KvType::ARR) return {};
    if (!v->af.empty()) return std::vector<float>(v->af.begin(), v->af.end());
    return std::vector<float>(v->ai.begin(), v->ai.end());
  }
  const std::vector<std::string>& get_arr_str(const std::string& key) const {
    static const std::vector<std::string> none;
    const KvValue* v = kv(key);
    return v && v->type == KvType::ARR ? v->as : none;
  }

  // tensors (in file order, split by split)
  const std::vector<TensorInfo>& tensors() const { return tensors_; }
  const TensorInfo* find(const std::string& name) const { auto it = tindex_.find(name); return it == tindex_.end() ? nullptr : &tensors_[it->second]; }
  const TensorInfo& at(const std::string& name) const {
    const TensorInfo* t = find(name);
    if (!t) throw std::runtime_error("gguf: no tensor " + name);
    return *t;
  }
  int n_splits() const { return (int)files_.size(); }
  const std::string& path(int split) const { return files_[split].path; }
  std::string basename(int split) const { const std::string& p = files_[split].path; const size_t s = p.rfind('/'); return s == std::string::npos ? p : p.substr(s + 1); }
  int fd(int split) const { return files_[split].fd; }
  uint64_t file_size(int split) const { return files_[split].size; }
  uint64_t data_offset(int split) const { return files_[split].data_off; }
  uint32_t alignment() const { return align_; }
  uint32_t version() const { return version_; }
  // tensor bytes [begin, begin + len) of tensor t into dst
  void read(const TensorInfo& t, uint64_t begin, void* dst, size_t len) const {
    if (begin + len > t.nbytes) throw std::runtime_error("gguf: read past the end of " + t.name);
    if (pread_full(files_[t.split].fd, dst, len, t.offset + begin) != (long long)len) throw std::runtime_error("gguf: short read of " + t.name);
  }

 private:
  struct File { std::string path; int fd = -1; uint64_t size = 0, data_off = 0; };
  // sequential reader over a file's header region, refilled in 1 MB windows
  struct Reader {
    int fd; const std::string& path; uint64_t size; uint64_t pos = 0;
    std::vector<char> win; uint64_t win_off = 0;
    Reader(int fd_, const std::string& p, uint64_t sz) : fd(fd_), path(p), size(sz) {}
    [[noreturn]] void fail(const char* what) const { throw std::runtime_error("gguf: " + path + ": " + what); }
    void read(void* dst, size_t n) {
      if (pos + n > size) fail("header runs past the end of the file");
      char* d = static_cast<char*>(dst);
      while (n) {
        if (pos < win_off || pos >= win_off + win.size()) {
          win.resize((size_t)std::min<uint64_t>(1u << 20, size - pos));
          win_off = pos;
          if (pread_full(fd, win.data(), win.size(), pos) != (long long)win.size()) fail("read error");
        }
        const size_t take = (size_t)std::min<uint64_t>(n, win_off + win.size() - pos);
        std::memcpy(d, win.data() + (pos - win_off), take);
        d += take; pos += take; n -= take;
      }
    }
    template <typename T> T get() { T v; read(&v, sizeof v); return v; }
    std::string str() {
      const uint64_t n = get<uint64_t>();
      if (n > size - pos) fail("string length past the end of the file");
      std::string s((size_t)n, '\0');
      if (n) read(&s[0], (size_t)n);
      return s;
    }
  };
  static void read_scalar(Reader& r, KvType t, KvValue& v) {
    switch (t) {
      case KvType::U8: v.u = r.get<uint8_t>(); v.i = (int64_t)v.u; v.f = (double)v.u; break;
      case KvType::I8: v.i = r.get<int8_t>(); v.u = (uint64_t)v.i; v.f = (double)v.i; break;
      case KvType::U16: v.u = r.get<uint16_t>(); v.i = (int64_t)v.u; v.f = (double)v.u; break;
      case KvType::I16: v.i = r.get<int16_t>(); v.u = (uint64_t)v.i; v.f = (double)v.i; break;
      case KvType::U32: v.u = r.get<uint32_t>(); v.i = (int64_t)v.u; v.f = (double)v.u; break;
      case KvType::I32: v.i = r.get<int32_t>(); v.u = (uint64_t)v.i; v.f = (double)v.i; break;
      case KvType::U64: v.u = r.get<uint64_t>(); v.i = (int64_t)v.u; v.f = (double)v.u; break;
      case KvType::I64: v.i = r.get<int64_t>(); v.u = (uint64_t)v.i; v.f = (double)v.i; break;
      case KvType::BOOL: v.u = r.get<uint8_t>() ? 1 : 0; v.i = (int64_t)v.u; v.f = (double)v.u; break;
      case KvType::F32: v.f = r.get<float>(); break;
      case KvType::F64: v.f = r.get<double>(); break;
      case KvType::STR: v.s = r.str(); break;
      default: r.fail("unknown metadata value type");
    }
  }
  static void read_value(Reader& r, KvType t, KvValue& v, int depth = 0) {
    v.type = t;
    if (t != KvType::ARR) { read_scalar(r, t, v); return; }
    if (depth > 4) r.fail("metadata arrays nested too deep");
    v.arr_type = (KvType)r.get<uint32_t>();
    const uint64_t n = r.get<uint64_t>();
    if (n > r.size) r.fail("array length past the end of the file");
    for (uint64_t k = 0; k < n; k++) {
      KvValue e;
      read_value(r, v.arr_type, e, depth + 1);
      if (v.arr_type == KvType::ARR) v.aa.push_back(std::move(e));
      else if (v.arr_type == KvType::STR) v.as.push_back(std::move(e.s));
      else if (e.is_float()) v.af.push_back(e.f);
      else v.ai.push_back(e.i);
    }
  }
  void parse_file(int split) {
    File& f = files_[split];
    Reader r(f.fd, f.path, f.size);
    char magic[4];
    r.read(magic, 4);
    if (std::memcmp(magic, "GGUF", 4) != 0) r.fail("bad magic");
    const uint32_t ver = r.get<uint32_t>();
    if (ver < 2) r.fail("unsupported version");
    if (split == 0) version_ = ver;
    const uint64_t nt = r.get<uint64_t>(), nkv = r.get<uint64_t>();
    uint32_t align = 32;
    for (uint64_t k = 0; k < nkv; k++) {
      std::string key = r.str();
      const KvType t = (KvType)r.get<uint32_t>();
      KvValue v;
      read_value(r, t, v);
      if (key == "general.alignment") align = (uint32_t)v.u;
      if (!kv_.count(key)) { kv_order_.push_back(key); kv_.emplace(std::move(key), std::move(v)); }
    }
    if (align == 0 || (align & (align - 1))) r.fail("alignment is not a power of two");
    if (split == 0) align_ = align;
    const size_t first = tensors_.size();
    for (uint64_t k = 0; k < nt; k++) {
      TensorInfo ti;
      ti.name = r.str();
      ti.n_dims = (int)r.get<uint32_t>();
      if (ti.n_dims < 1 || ti.n_dims > 4) r.fail("bad number of dimensions");
      for (int d = 0; d < ti.n_dims; d++) ti.ne[d] = (int64_t)r.get<uint64_t>();
      ti.type = (GType)r.get<uint32_t>();
      if (!type_info(ti.type)) r.fail("unknown tensor type");
      ti.offset = r.get<uint64_t>();          // relative to the data section until the header is complete
      ti.split = split;
      ti.nbytes = type_bytes(ti.type, (uint64_t)ti.nelements());
      tensors_.push_back(std::move(ti));
    }
    f.data_off = (r.pos + align - 1) / align * align;
    for (size_t k = first; k < tensors_.size(); k++) {
      tensors_[k].offset += f.data_off;
      if (tensors_[k].offset + tensors_[k].nbytes > f.size) r.fail("tensor data past the end of the file");
    }
  }

  std::vector<File> files_;
  std::unordered_map<std::string, KvValue> kv_;
  std::vector<std::string> kv_order_;
  std::vector<TensorInfo> tensors_;
  std::unordered_map<std::string, size_t> tindex_;
  uint32_t align_ = 32, version_ = 0;
};

// Where each layer's stacked expert tensors live in the files: expert e of matrix k is the byte range
// [base + e * stride, + len) of one split (src/store/experts.hpp:35-42).  mat: 0 = gate (w1), 1 = up (w3), 2 = down (w2).
struct ExpertMat { int split = 0; uint64_t base = 0, stride = 0, file_size = 0; uint32_t len = 0; GType type = GType::F32; int64_t rows = 0, cols = 0; };
struct ExpertLayerLayout { ExpertMat mat[3]; };
struct ExpertLayout {
  int n_layers = 0, n_experts = 0;
  std::vector<ExpertLayerLayout> layers;
  // block_count / expert_count are read under the file's own architecture prefix (general.architecture)
  static ExpertLayout from_gguf(const Gguf& g) {
    ExpertLayout L;
    const std::string arch = g.get_str("general.architecture");
    L.n_layers = (int)g.get_i64(arch + ".block_count", 0);
    L.n_experts = (int)g.get_i64(arch + ".expert_count", 0);
    if (L.n_layers <= 0 || L.n_experts <= 0) throw std::runtime_error("gguf: no block_count / expert_count under '" + arch + "'");
    static const char* names[3] = {"ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"};
    for (int l = 0; l < L.n_layers; l++) {
      ExpertLayerLayout ll;
      for (int k = 0; k < 3; k++) {
        const TensorInfo& t = g.at("blk." + std::to_string(l) + "." + names[k] + ".weight");
        if (t.ne[2] != L.n_experts || t.nbytes % (uint64_t)L.n_experts) throw std::runtime_error("gguf: bad expert tensor " + t.name);
        ExpertMat& m = ll.mat[k];
        m.split = t.split; m.base = t.offset; m.stride = t.nbytes / (uint64_t)L.n_experts; m.len = (uint32_t)m.stride;
        m.type = t.type; m.file_size = g.file_size(t.split); m.cols = t.ne[0]; m.rows = t.ne[1];
      }
      L.layers.push_back(ll);
    }
    return L;
  }
  uint64_t expert_bytes(int layer) const { const ExpertLayerLayout& l = layers[layer]; return (uint64_t)l.mat[0].len + l.mat[1].len + l.mat[2].len; }
};

}  // namespace ms
