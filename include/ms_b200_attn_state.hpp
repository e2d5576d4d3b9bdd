// ms::attn::State and the decode-side attention calls with the reference's own signatures
// (src/kernels/attn.hpp:62-129): encode_kv_window / encode_compress / encode_index_decode / encode_sparse /
// encode_layer take (Enc&, State&, int layer, ...), State owns every cache and scratch buffer and the layer -> source maps.
// Header-only over libmacseek_b200's C ABI; no CUDA header is needed.
//
// Differences from the reference, all additive: the shapes the reference fixes at compile time (kD, kH, kIH, kTopk, the
// layer roles) are fields of attn::Shape / attn::Roles with the reference's values as defaults, so the same State serves
// the benchmark's shapes (576-wide bf16 rows, 64 index heads, FP8 keys, top-2048, an indexer on every layer); buffers
// live in device memory (ms::Device::alloc -> msb_device_alloc), host access goes through ms::upload / ms::download.
// Prefill (n > 1) entry points are not part of this header.
#pragma once
#include <algorithm>
#include <cmath>
#include <functional>
#include <vector>
#include "ms_b200_shim.hpp"

namespace ms {

class Device {            // src/core/metal.hpp:20-40: zero-filled allocations owned by the caller
 public:
  static Device& get() { static Device d; return d; }
  Buffer alloc(size_t bytes, const char* /*label*/ = nullptr) {
    void* p = nullptr;
    check(msb_device_alloc(bytes, &p), "Device::alloc");
    return Buffer{p, 0, bytes};
  }
  void release(Buffer& b) { if (b.buf && b.off == 0) msb_device_free(b.buf); b = Buffer{}; }
};
inline void upload(const Buffer& dst, const void* src, size_t bytes, void* stream = nullptr) {
  check(msb_copy_to_device(dst.ptr(), src, bytes, stream), "upload");
}
inline void download(void* dst, const Buffer& src, size_t bytes, void* stream = nullptr) {
  check(msb_copy_to_host(dst, src.ptr(), bytes, stream), "download");
}

namespace q {
// Prefill projections with the reference's exact signatures (src/kernels/quant.hpp:41-46): the half copies of X and W
// live in module-owned scratch that grows on demand (quant.mm:175-184), so callers pass no scratch.  Not thread-safe,
// like the reference's: one stream per model instance.
inline Buffer& module_scratch(size_t bytes) {
  static Buffer buf;
  if (buf.size < bytes) { Device::get().release(buf); buf = Device::get().alloc(bytes, "quant module scratch"); }
  return buf;
}
inline void encode_matmul(Enc& e, QType t, const Buffer& W, int rows, int cols, const Buffer& X, const Buffer& Y, int n,
                          bool accumulate = false) {
  encode_matmul(e, t, W, rows, cols, X, Y, n, module_scratch(matmul_scratch_bytes(t, rows, cols, n, true)), accumulate);
}
inline void encode_matmul_h(Enc& e, QType t, const Buffer& W, int rows, int cols, const Buffer& X16, const Buffer& Y, int n,
                            bool accumulate = false, int x_stride = 0) {
  encode_matmul_h(e, t, W, rows, cols, X16, Y, n, module_scratch(matmul_scratch_bytes(t, rows, cols, n, false)), accumulate, x_stride);
}
}  // namespace q

namespace attn {

constexpr int kLayers = 40, kD = 512, kRD = 64, kH = 64, kWin = 128;
constexpr int kIH = 32, kID = 128, kTopk = 512, kCandBlocks = 2048, kCandBS = 8;
constexpr int kRowPad = 128;

// ---- layer roles of the reference model (attn.hpp:17-24)
inline int ratio_of(int L) { return L < 2 ? 0 : (L < 20 ? 2 : 1); }
inline bool is_kv_source(int L) { return L == 2 || L == 8 || L == 14 || L == 20; }
inline int kv_source_of(int L) { return L < 2 ? -1 : L < 8 ? 2 : L < 14 ? 8 : L < 20 ? 14 : 20; }
inline int src_slot(int s) { return s == 2 ? 0 : s == 8 ? 1 : s == 14 ? 2 : 3; }
inline bool is_index_source(int L) { return is_kv_source(L) || L == 24 || L == 28 || L == 32 || L == 36; }
inline int index_source_of(int L) { if (L < 20) return kv_source_of(L); return L < 24 ? 20 : 24 + 4 * ((L - 24) / 4); }
inline bool is_cand_source(int L) { return L == 20; }
inline bool uses_cand(int L) { return L > 20 && is_index_source(L); }

struct Options {          // the decode-relevant switches of attn.hpp:26-60
  bool actq = true;
  int max_pos = 262144;
  bool fused_combine = false;
  int max_chunk = 1;      // tokens per encode_layer call: the state keeps one top-k list (and candidate list) per token of a chunk
};

struct Shape {
  int layers = kLayers, D = kD, heads = kH, window = kWin, index_heads = kIH, index_dim = kID, topk = kTopk;
  int cand_blocks = kCandBlocks, cand_bs = kCandBS;
  int key_type = MSB_F16, elem_type = MSB_F16;
};

// Layer -> source maps.  reference(): the model's own roles.  every_layer(n): each layer is its own KV and index source
// with ratio 1 and no candidate hand-off (the benchmark's synthetic step).
struct Roles {
  std::vector<int> kv_source;      // [layers] layer whose caches this layer attends to (-1: window only)
  std::vector<int> index_source;   // [layers] layer whose top-k this layer uses (-1: none)
  std::vector<int> ratio;          // [layers] compression ratio of the layer's source (0: none)
  int cand_source = -1;            // layer that also produces candidate blocks; later index sources score only those
  static Roles reference() {
    Roles r;
    for (int L = 0; L < kLayers; L++) {
      r.kv_source.push_back(kv_source_of(L));
      r.index_source.push_back(L < 2 ? -1 : index_source_of(L));
      r.ratio.push_back(ratio_of(L));
    }
    r.cand_source = 20;
    return r;
  }
  static Roles every_layer(int n) {
    Roles r;
    for (int L = 0; L < n; L++) { r.kv_source.push_back(L); r.index_source.push_back(L); r.ratio.push_back(1); }
    return r;
  }
};

struct State {
  Options opt;
  Shape shape;
  Roles roles;
  Buffer rope_plain, rope_yarn;            // float2 [max_pos][32]
  std::vector<Buffer> win;                 // [layers] elem [window][D]
  std::vector<Buffer> ckv, ikey, cst;      // per KV source slot: elem [cap + 128][D], key [cap + 128][index_dim], f32 [2][ratio][D]
  std::vector<int> cap, slot_layer;        // per slot: capacity in rows, the source layer
  std::vector<int> slot_of_layer;          // [layers] -> slot (-1)
  // ---- scratch / per-token work buffers
  Buffer dec_scores, dec_bscores, q_prep, w_prep, topk_scratch, sparse_scratch;
  std::vector<Buffer> topk;                // per index source layer: int [max_chunk][topk], row t = token t of the current chunk
  std::vector<int> topk_of_layer;          // [layers] -> index into topk (-1)
  Buffer cand_list;                        // int [max_chunk][cand_blocks]
  bool is_kv_src(int L) const { return roles.kv_source[L] == L; }
  bool is_index_src(int L) const { return roles.index_source[L] == L; }
  bool uses_candidates(int L) const { return roles.cand_source >= 0 && L > roles.cand_source && is_index_src(L); }
  int elem_bytes() const { return 2; }
  int key_bytes() const { return shape.key_type == MSB_KEY_FP8_E4M3 ? 1 : 2; }
  const float* rope_row(int L, int pos) const {
    const Buffer& t = roles.ratio[L] == 0 ? rope_plain : rope_yarn;
    return (const float*)t.ptr() + (size_t)pos * 64;
  }
};

// rope tables on the CPU, float2 [max_pos][32] = (cos, sin): theta 1e4 plain, theta 1.6e5 + YaRN(16, 65536, 32, 1)
// otherwise, with the float rounding steps of the reference's table (tests/ref/attn_ref.cpp:15-46)
inline void make_rope_table(float* dst, int max_pos, bool yarn) {
  const int dim = 64;
  const double base = yarn ? 160000.0 : 10000.0;
  float f[32];
  for (int i = 0; i < 32; i++) f[i] = (float)(1.0 / std::pow(base, (double)(float)(2 * i) / dim));
  if (yarn) {
    const double factor = 16.0, orig = 65536.0, bf = 32.0, bs = 1.0, pi = 3.14159265358979323846;
    auto corr = [&](double rot) { return dim * std::log(orig / (rot * 2 * pi)) / (2 * std::log(base)); };
    const double low = std::max(std::floor(corr(bf)), 0.0), high = std::min(std::ceil(corr(bs)), dim - 1.0);
    for (int i = 0; i < 32; i++) {
      float ramp = (float)((i - low) / std::max(high - low, 1e-3));
      ramp = std::min(std::max(ramp, 0.0f), 1.0f);
      const float smooth = 1.0f - ramp;
      f[i] = f[i] / (float)factor * (1.0f - smooth) + f[i] * smooth;
    }
  }
  for (int p = 0; p < max_pos; p++)
    for (int i = 0; i < 32; i++) {
      const double a = (double)((float)p * f[i]);
      dst[((size_t)p * 32 + i) * 2] = (float)std::cos(a);
      dst[((size_t)p * 32 + i) * 2 + 1] = (float)std::sin(a);
    }
}

// Allocate caches and scratch.  init(s, o) builds the reference model's state (attn.hpp:102); the three-argument form
// takes explicit shapes and roles.
inline void init(State& s, const Options& o, const Shape& sh, const Roles& roles) {
  s.opt = o; s.shape = sh; s.roles = roles;
  Device& dev = Device::get();
  const int L = sh.layers;
  {
    std::vector<float> tab((size_t)o.max_pos * 64);
    s.rope_plain = dev.alloc(tab.size() * 4, "rope_plain");
    s.rope_yarn = dev.alloc(tab.size() * 4, "rope_yarn");
    make_rope_table(tab.data(), o.max_pos, false);
    upload(s.rope_plain, tab.data(), tab.size() * 4);
    make_rope_table(tab.data(), o.max_pos, true);
    upload(s.rope_yarn, tab.data(), tab.size() * 4);
  }
  s.win.assign(L, Buffer{});
  s.slot_of_layer.assign(L, -1);
  s.topk_of_layer.assign(L, -1);
  int max_cap = 0;
  for (int l = 0; l < L; l++) {
    s.win[l] = dev.alloc((size_t)sh.window * sh.D * s.elem_bytes(), "win");
    if (s.is_kv_src(l)) {
      const int r = std::max(1, roles.ratio[l]), cap = o.max_pos / r;
      s.slot_of_layer[l] = (int)s.ckv.size();
      s.slot_layer.push_back(l);
      s.cap.push_back(cap);
      s.ckv.push_back(dev.alloc((size_t)(cap + kRowPad) * sh.D * s.elem_bytes(), "ckv"));
      s.ikey.push_back(dev.alloc((size_t)(cap + kRowPad) * sh.index_dim * s.key_bytes(), "ikey"));
      s.cst.push_back(dev.alloc((size_t)2 * r * sh.D * 4, "cst"));
      max_cap = std::max(max_cap, cap);
    }
    if (s.is_index_src(l)) {
      s.topk_of_layer[l] = (int)s.topk.size();
      s.topk.push_back(dev.alloc((size_t)std::max(1, o.max_chunk) * sh.topk * 4, "topk"));
    }
  }
  const int n_max = max_cap + kRowPad;
  s.dec_scores = dev.alloc((size_t)n_max * 4 + 64, "dec_scores");
  s.dec_bscores = dev.alloc((size_t)((n_max + sh.cand_bs - 1) / sh.cand_bs) * 4 + 64, "dec_bscores");
  s.q_prep = dev.alloc((size_t)sh.index_heads * sh.index_dim * 4, "q_prep");
  s.w_prep = dev.alloc((size_t)sh.index_heads * 4, "w_prep");
  s.topk_scratch = dev.alloc(msb_topk_scratch_bytes(n_max), "topk_scratch");
  s.sparse_scratch = dev.alloc(msb_sparse_scratch_bytes(sh.window + sh.topk, sh.heads, sh.D), "sparse_scratch");
  s.cand_list = dev.alloc((size_t)std::max(1, o.max_chunk) * sh.cand_blocks * 4, "cand_list");
}
inline void init(State& s, const Options& o) { init(s, o, Shape{}, Roles::reference()); }

// New sequence: compressor partial groups back to (0, -inf), top-k lists to "none" (attn.hpp:108).  The caches need no
// clearing: only rows below the current position are ever read.
inline void reset(State& s, void* stream = nullptr) {
  for (size_t i = 0; i < s.cst.size(); i++) {
    const size_t half = s.cst[i].size / 8;
    check(msb_fill_f32((float*)s.cst[i].ptr(), 0.f, half, stream), "reset");
    check(msb_fill_f32((float*)s.cst[i].ptr() + half, -INFINITY, half, stream), "reset");
  }
  std::vector<int> none((size_t)std::max(1, s.opt.max_chunk) * std::max(s.shape.topk, s.shape.cand_blocks), -1);
  for (auto& t : s.topk) upload(t, none.data(), t.size, stream);
  upload(s.cand_list, none.data(), s.cand_list.size, stream);
}

struct LayerIO {          // attn.hpp:112-127; all f32; n tokens: every per-token buffer is [n][...]
  int layer = 0;
  Buffer q, kv, kv_norm, sinks, out;
  Buffer c_kv, c_gate, c_norm, idx_wk, idx_knorm;    // kv source layers
  Buffer idx_q, idx_w;                               // index source layers
};
using StageHook = std::function<void(int stage)>;

// ---- building blocks.  n == 1 is the decode path.  n > 1 (a prefill chunk at positions start .. start + n - 1) runs
// the SAME kernels token by token in position order -- causal by construction and bit-identical to n decode calls, the
// first correct form of the reference's chunked prefill side (attn.mm:292-417,446-516: tiled indexer GEMM, running top-k
// merge, two-pass sparse attention), which is not built as batched kernels.  Because the window is a ring of `window`
// rows, a chunk must be processed through encode_layer (window row, compressor, index, attention per token in turn);
// the single building blocks accept n > 1 only where token order alone keeps them correct.
inline Buffer tok_row(const Buffer& b, int t, size_t row_floats) { return b.buf ? b.sub((size_t)t * row_floats * 4, row_floats * 4) : b; }
inline void encode_kv_window(Enc& e, State& s, int layer, const Buffer& kv, const Buffer& norm_w, int start, int n) {
  if (n > s.shape.window) check(MSB_E_ARG, "encode_kv_window: more tokens than window rows (use encode_layer for a chunk)");
  for (int t = 0; t < n; t++) {
    char* row = (char*)s.win[layer].ptr() + (size_t)((start + t) % s.shape.window) * s.shape.D * s.elem_bytes();
    check(msb_kv_window((const float*)tok_row(kv, t, s.shape.D).ptr(), (const float*)norm_w.ptr(), s.rope_row(layer, start + t),
                        s.opt.actq, s.shape.D, s.shape.elem_type, row, e.stream), "encode_kv_window");
  }
}
inline void encode_compress(Enc& e, State& s, int layer, const LayerIO& io, int start, int n, bool /*barrier_after*/ = true) {
  const int slot = s.slot_of_layer[layer];
  if (slot < 0) check(MSB_E_ARG, "encode_compress: not a KV source layer");
  const int r = std::max(1, s.roles.ratio[layer]);
  for (int t = 0; t < n; t++) {
    const int pos = start + t;
    check(msb_compress((const float*)tok_row(io.c_kv, t, s.shape.D).ptr(), (const float*)tok_row(io.c_gate, t, s.shape.D).ptr(),
                       (const float*)io.c_norm.ptr(), io.idx_wk.ptr(), (const float*)io.idx_knorm.ptr(),
                       s.rope_row(layer, (pos / r) * r), (float*)s.cst[slot].ptr(), r, pos, s.opt.actq, s.shape.D,
                       s.shape.index_dim, s.shape.elem_type, s.ckv[slot].ptr(), s.shape.key_type, s.ikey[slot].ptr(), e.stream),
          "encode_compress");
  }
}
// Index decode of an index source layer: scores of the source's keys below (pos + 1) / ratio, exact top-k into the
// layer's list; the candidate source also leaves its top candidate blocks in cand_list, and later index sources score
// only those blocks (attn.mm:222-290).
inline void encode_index_decode(Enc& e, State& s, int layer, const Buffer& iq, const Buffer& iw, int pos,
                                const StageHook& hook = {}, int row = 0) {
  const Shape& sh = s.shape;
  if (row < 0 || row >= std::max(1, s.opt.max_chunk)) check(MSB_E_ARG, "encode_index_decode: chunk row beyond Options::max_chunk");
  const int src = s.roles.kv_source[layer], slot = src >= 0 ? s.slot_of_layer[src] : -1, ti = s.topk_of_layer[layer];
  if (slot < 0 || ti < 0) check(MSB_E_ARG, "encode_index_decode: not an index source layer");
  const int r = std::max(1, s.roles.ratio[layer]), len = (pos + 1) / r;
  const float* cs = s.rope_row(layer, pos);
  if (s.uses_candidates(layer)) {
    const int nb = (len + sh.cand_bs - 1) / sh.cand_bs;
    check(msb_index_decode_list(sh.key_type, s.ikey[slot].ptr(), len, (const float*)iq.ptr(), (const float*)iw.ptr(), cs,
                                s.opt.actq, sh.index_heads, sh.topk, (const int*)s.cand_list.ptr() + (size_t)row * sh.cand_blocks,
                                std::min(nb, sh.cand_blocks), (float*)s.q_prep.ptr(), (float*)s.w_prep.ptr(),
                                (float*)s.dec_scores.ptr(), (int*)s.topk[ti].ptr() + (size_t)row * sh.topk, s.topk_scratch.ptr(),
                                s.topk_scratch.size, e.stream),
          "encode_index_decode (candidates)");
  } else {
    check(msb_index_decode(sh.key_type, s.ikey[slot].ptr(), len, (const float*)iq.ptr(), (const float*)iw.ptr(), cs,
                           s.opt.actq, sh.index_heads, sh.topk, (float*)s.q_prep.ptr(), (float*)s.w_prep.ptr(),
                           (float*)s.dec_scores.ptr(), (int*)s.topk[ti].ptr() + (size_t)row * sh.topk, s.topk_scratch.ptr(),
                           s.topk_scratch.size, 0, e.stream), "encode_index_decode");
    if (layer == s.roles.cand_source && len > 0) {
      const int nb = (len + sh.cand_bs - 1) / sh.cand_bs;
      check(msb_block_max((const float*)s.dec_scores.ptr(), len, sh.cand_bs, (float*)s.dec_bscores.ptr(), e.stream),
            "encode_index_decode (block maxima)");
      check(msb_topk((const float*)s.dec_bscores.ptr(), nb, sh.cand_blocks, (int*)s.cand_list.ptr() + (size_t)row * sh.cand_blocks,
                     s.topk_scratch.ptr(), s.topk_scratch.size, 0, e.stream), "encode_index_decode (candidate blocks)");
    }
  }
  if (hook) { hook(0); hook(1); }
}
// Sparse attention of the token at `start` over the layer's window ring and the rows its index source selected
// (attn.hpp:128-129).  fused_combine is accepted for source compatibility: the result is the same either way.
inline void encode_sparse(Enc& e, State& s, int layer, const Buffer& q, const Buffer& sinks, const Buffer& out, int start,
                          int n, bool /*fused_combine*/ = false, const StageHook& hook = {}, int row = 0) {
  if (n != 1) check(MSB_E_ARG, "encode_sparse: one token per call (a chunk goes through encode_layer: the selected rows are per token)");
  if (row < 0 || row >= std::max(1, s.opt.max_chunk)) check(MSB_E_ARG, "encode_sparse: chunk row beyond Options::max_chunk");
  const Shape& sh = s.shape;
  const int n_win = start + 1 < sh.window ? start + 1 : sh.window;
  const int src = s.roles.kv_source[layer], slot = src >= 0 ? s.slot_of_layer[src] : -1;
  const int isrc = s.roles.index_source[layer], ti = isrc >= 0 ? s.topk_of_layer[isrc] : -1;
  const bool sel = slot >= 0 && ti >= 0;
  check(msb_sparse_decode((const float*)q.ptr(), s.rope_row(layer, start), (const float*)sinks.ptr(), sh.elem_type,
                          s.win[layer].ptr(), n_win, sel ? s.ckv[slot].ptr() : nullptr,
                          sel ? (const int*)s.topk[ti].ptr() + (size_t)row * sh.topk : nullptr,
                          sel ? sh.topk : 0, sh.heads, sh.D, (float*)out.ptr(), s.sparse_scratch.ptr(), s.sparse_scratch.size,
                          e.stream), "encode_sparse");
  if (hook) { hook(2); hook(3); }
}
// encode_index_prefill (attn.hpp:122): the top-k list of every token of the chunk, row t of the source's list buffer.
inline void encode_index_prefill(Enc& e, State& s, int layer, const Buffer& iq, const Buffer& iw, int start, int n) {
  const Shape& sh = s.shape;
  for (int t = 0; t < n; t++)
    encode_index_decode(e, s, layer, tok_row(iq, t, (size_t)sh.index_heads * sh.index_dim), tok_row(iw, t, sh.index_heads), start + t, {}, t);
}
// The whole attention side of one layer for the tokens at start .. start + n - 1 (attn.hpp:113): per token, in position
// order, window row, compressor on KV source layers, index decode on index source layers, sparse attention.
inline void encode_layer(Enc& e, State& s, const LayerIO& io, int start, int n) {
  const Shape& sh = s.shape;
  if (n > std::max(1, s.opt.max_chunk)) check(MSB_E_ARG, "encode_layer: chunk longer than Options::max_chunk");
  for (int t = 0; t < n; t++) {
    LayerIO one = io;
    one.q = tok_row(io.q, t, (size_t)sh.heads * sh.D); one.kv = tok_row(io.kv, t, sh.D); one.out = tok_row(io.out, t, (size_t)sh.heads * sh.D);
    one.c_kv = tok_row(io.c_kv, t, sh.D); one.c_gate = tok_row(io.c_gate, t, sh.D);
    one.idx_q = tok_row(io.idx_q, t, (size_t)sh.index_heads * sh.index_dim); one.idx_w = tok_row(io.idx_w, t, sh.index_heads);
    encode_kv_window(e, s, io.layer, one.kv, io.kv_norm, start + t, 1);
    if (s.is_kv_src(io.layer)) encode_compress(e, s, io.layer, one, start + t, 1);
    if (s.is_index_src(io.layer)) encode_index_decode(e, s, io.layer, one.idx_q, one.idx_w, start + t, {}, t);
    encode_sparse(e, s, io.layer, one.q, io.sinks, one.out, start + t, 1, false, {}, t);
  }
}

}  // namespace attn
}  // namespace ms
