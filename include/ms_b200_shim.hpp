// C++ host shim: the reference's kernel-module call surface (namespaces ms::q, ms::arch, ms::attn of
// src/kernels/quant.hpp, arch.hpp, attn.hpp) re-expressed over libmacseek_b200's C ABI, so that the reference's
// layer-forward code (src/model/dec_layer.mm, ds41.mm) keeps calling the same functions with the same arguments.
//
//   reference                               here
//   ms::Buffer{buf, off, size}              ms::Buffer: buf is a DEVICE base pointer, ptr() = buf + off
//   ms::Enc (command buffer + encoder)      ms::Enc: a CUDA stream; barrier() is a no-op (streams are in order),
//                                            wait() synchronises and aborts on a device-side failure word
//   die() -> abort()                        check(): prints msb_last_error() and aborts
// Header-only; needs only <cuda_runtime_api.h>-free C: the stream is carried as void*.
#pragma once
#include <vector>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include "macseek_b200.h"

namespace ms {

struct Buffer {           // src/core/metal.hpp:11-18
  void* buf = nullptr;
  size_t off = 0;
  size_t size = 0;
  void* ptr() const { return buf ? static_cast<char*>(buf) + off : nullptr; }
  Buffer sub(size_t o, size_t s) const { return Buffer{buf, off + o, s}; }
};

struct Enc {              // src/core/metal.hpp:43-71
  void* stream = nullptr;                 // cudaStream_t
  explicit Enc(void* cuda_stream = nullptr) : stream(cuda_stream) {}
  void barrier() {}                       // dependent launches on one stream are already ordered
  void wait() {                           // Enc::wait aborts on a GPU error (src/core/metal.mm:160-162)
    const int st = msb_device_status();
    if (st != 0) { std::fprintf(stderr, "macseek_b200: device status %d (%s)\n", st, msb_last_error()); std::abort(); }
  }
};

inline void check(int rc, const char* what) {   // the reference's die() (src/kernels/quant.mm:34-37)
  if (rc != 0) { std::fprintf(stderr, "macseek_b200: %s failed: %s\n", what, msb_last_error()); std::abort(); }
}
[[noreturn]] inline void die(const char* msg) { std::fprintf(stderr, "macseek_b200: %s\n", msg); std::abort(); }

namespace q {             // src/kernels/quant.hpp
enum class QType : int { F32 = 0, F16 = 1, Q8_0 = 8, Q5_K = 13, Q6_K = 14, IQ2_XXS = 16, IQ1_S = 19, IQ4_NL = 20, BF16 = 30 };
inline size_t row_bytes(QType t, int64_t cols) { return msb_row_bytes((int)t, cols); }
inline bool matvec_supported(QType t) { return msb_block_bytes((int)t) != 0; }

inline void encode_matvec(Enc& e, QType t, const Buffer& W, int rows, int cols, const Buffer& x, const Buffer& y,
                          bool accumulate = false, int groups = 1) {
  check(msb_matvec((int)t, W.ptr(), rows, cols, (const float*)x.ptr(), (float*)y.ptr(), accumulate, groups, e.stream),
        "encode_matvec");
}
inline void encode_matvec_rmsnorm(Enc& e, QType t, const Buffer& W, int rows, int cols, const Buffer& x,
                                  const Buffer& norm_w, float eps, const Buffer& y, int /*tiles_per_tg*/ = 0) {
  check(msb_matvec_rmsnorm((int)t, W.ptr(), rows, cols, (const float*)x.ptr(), (const float*)norm_w.ptr(), eps,
                           (float*)y.ptr(), e.stream), "encode_matvec_rmsnorm");
}
// Not in the reference: the same as a launch of one small block per SM, for a second stream that runs beside another.
inline void encode_matvec_rmsnorm_shared(Enc& e, QType t, const Buffer& W, int rows, int cols, const Buffer& x,
                                         const Buffer& norm_w, float eps, const Buffer& y) {
  check(msb_matvec_rmsnorm_shared((int)t, W.ptr(), rows, cols, (const float*)x.ptr(), (const float*)norm_w.ptr(), eps,
                                  (float*)y.ptr(), e.stream), "encode_matvec_rmsnorm_shared");
}
inline void encode_matvec_n(Enc& e, QType t, const Buffer& W, int rows, int cols, const Buffer& X, const Buffer& Y, int n,
                            bool accumulate = false, int groups = 1) {
  check(msb_matvec_n((int)t, W.ptr(), rows, cols, (const float*)X.ptr(), (float*)Y.ptr(), n, accumulate, groups, e.stream),
        "encode_matvec_n");
}

constexpr int kMaxRouted = MSB_MAX_ROUTED;
// prefill projections (quant.hpp:37-46).  The reference's module-owned X16 / W16 scratch becomes an explicit Buffer.
inline size_t matmul_scratch_bytes(QType t, int rows, int cols, int n, bool with_x = true) {
  return msb_matmul_scratch_bytes((int)t, rows, cols, n, with_x ? 1 : 0);
}
inline void encode_f32_to_f16(Enc& e, const Buffer& X, const Buffer& X16, size_t count) {
  check(msb_f32_to_f16((const float*)X.ptr(), X16.ptr(), count, e.stream), "encode_f32_to_f16");
}
inline void encode_matmul_h(Enc& e, QType t, const Buffer& W, int rows, int cols, const Buffer& X16, const Buffer& Y, int n,
                            const Buffer& scratch, bool accumulate = false, int x_stride = 0) {
  check(msb_matmul_h((int)t, W.ptr(), rows, cols, X16.ptr(), x_stride, (float*)Y.ptr(), n, accumulate ? 1 : 0, scratch.ptr(),
                     scratch.size, e.stream), "encode_matmul_h");
}
inline void encode_matmul(Enc& e, QType t, const Buffer& W, int rows, int cols, const Buffer& X, const Buffer& Y, int n,
                          const Buffer& scratch, bool accumulate = false) {
  check(msb_matmul((int)t, W.ptr(), rows, cols, (const float*)X.ptr(), (float*)Y.ptr(), n, accumulate ? 1 : 0, scratch.ptr(),
                   scratch.size, e.stream), "encode_matmul");
}

struct ExpertSlot { Buffer gate, up, down; };
enum class MoePart { All, SharedGu, AfterSharedGu, Shared, Routed, SharedDown };
struct MoeDecodeArgs {     // quant.hpp:54-70, with dim / inter as fields (the reference: 5120 / 2304)
  int dim = 5120, inter = 2304;
  QType t_gate_up = QType::IQ1_S, t_down = QType::IQ1_S;
  int n_routed = 6;
  ExpertSlot slot[kMaxRouted];
  Buffer weights;
  bool has_shared = true;
  QType t_shared = QType::Q6_K;
  ExpertSlot shared;
  Buffer x, y, scratch;
};
inline size_t moe_decode_scratch_bytes(int inter = 2304, int max_routed = 6) { return msb_moe_decode_scratch_bytes(inter, max_routed); }
inline msb_moe_decode_args to_c(const MoeDecodeArgs& a) {
  msb_moe_decode_args c{};
  c.dim = a.dim; c.inter = a.inter;
  c.t_gate_up = (int)a.t_gate_up; c.t_down = (int)a.t_down; c.t_shared = (int)a.t_shared;
  c.n_routed = a.n_routed; c.has_shared = a.has_shared;
  for (int i = 0; i < a.n_routed && i < kMaxRouted; i++)
    c.slot[i] = msb_expert_slot{a.slot[i].gate.ptr(), a.slot[i].up.ptr(), a.slot[i].down.ptr()};
  c.shared = msb_expert_slot{a.shared.gate.ptr(), a.shared.up.ptr(), a.shared.down.ptr()};
  c.weights = (const float*)a.weights.ptr(); c.x = (const float*)a.x.ptr(); c.y = (float*)a.y.ptr();
  c.scratch = a.scratch.ptr(); c.scratch_bytes = a.scratch.size; c.swiglu_limit = 10.f;
  return c;
}
inline void encode_moe_decode(Enc& e, const MoeDecodeArgs& a) {
  const msb_moe_decode_args c = to_c(a);
  check(msb_moe_decode(&c, e.stream), "encode_moe_decode");
}
inline void encode_moe_decode_table_part(Enc& e, const MoeDecodeArgs& a, const Buffer& table, MoePart part) {
  const msb_moe_decode_args c = to_c(a);
  check(msb_moe_decode_table_part(&c, (const uint64_t*)table.ptr(), (int)part, e.stream), "encode_moe_decode_table_part");
}
inline void encode_moe_decode_table(Enc& e, const MoeDecodeArgs& a, const Buffer& table) {
  encode_moe_decode_table_part(e, a, table, MoePart::All);
}
// Not in the reference: routed experts resolved on the GPU from the router's ids (HBM-resident, expert-parallel).
inline void encode_moe_decode_ids(Enc& e, const MoeDecodeArgs& a, const Buffer& expert_table, const Buffer& ids,
                                  int expert_lo, int expert_hi, MoePart part = MoePart::All) {
  const msb_moe_decode_args c = to_c(a);
  check(msb_moe_decode_ids(&c, (const uint64_t*)expert_table.ptr(), (const int*)ids.ptr(), expert_lo, expert_hi,
                           (int)part, e.stream), "encode_moe_decode_ids");
}
// Not in the reference: the same on x = RMSNorm(norm_in) * norm_w built inside the gate/up launch (a.x ignored); the
// launch directly before in the stream must be encode_router_fused_rmsnorm over the same norm_in.
inline void encode_moe_decode_ids_normed(Enc& e, const MoeDecodeArgs& a, const Buffer& expert_table, const Buffer& ids,
                                         int expert_lo, int expert_hi, const Buffer& norm_in, const Buffer& norm_w,
                                         float norm_eps, MoePart part = MoePart::All) {
  const msb_moe_decode_args c = to_c(a);
  check(msb_moe_decode_ids_normed(&c, (const uint64_t*)expert_table.ptr(), (const int*)ids.ptr(), expert_lo, expert_hi,
                                  (int)part, (const float*)norm_in.ptr(), (const float*)norm_w.ptr(), norm_eps, e.stream),
        "encode_moe_decode_ids_normed");
}
// prefill MoE (quant.hpp:87-118), with dim / inter as fields
struct MoePrefillArgs {
  int dim = 5120, inter = 2304;
  QType t_gate_up = QType::IQ1_S, t_down = QType::IQ1_S;
  int n_tokens = 0, n_exp = 0;
  const ExpertSlot* slots = nullptr;   // host [n_exp]
  const int* offs = nullptr;           // host [n_exp + 1]
  Buffer tok, wt, slot_of;
  int k_per_token = 6;
  bool has_shared = true;
  QType t_shared = QType::Q6_K;
  ExpertSlot shared;
  Buffer X, Y, scratch;
};
inline size_t moe_prefill_scratch_bytes(int total_entries, int n_tokens, int n_exp = 384, int dim = 5120, int inter = 2304) {
  return msb_moe_prefill_scratch_bytes(total_entries, n_tokens, n_exp, dim, inter);
}
inline void encode_moe_prefill(Enc& e, const MoePrefillArgs& a) {
  std::vector<msb_expert_slot> slots((size_t)(a.n_exp > 0 ? a.n_exp : 1));
  for (int j = 0; j < a.n_exp; j++) slots[(size_t)j] = msb_expert_slot{a.slots[j].gate.ptr(), a.slots[j].up.ptr(), a.slots[j].down.ptr()};
  msb_moe_prefill_args c{};
  c.dim = a.dim; c.inter = a.inter;
  c.t_gate_up = (int)a.t_gate_up; c.t_down = (int)a.t_down; c.t_shared = (int)a.t_shared;
  c.n_tokens = a.n_tokens; c.n_exp = a.n_exp; c.slots = slots.data(); c.offs = a.offs;
  c.tok = (const int*)a.tok.ptr(); c.wt = (const float*)a.wt.ptr(); c.slot_of = (const int*)a.slot_of.ptr();
  c.k_per_token = a.k_per_token; c.has_shared = a.has_shared ? 1 : 0;
  c.shared = msb_expert_slot{a.shared.gate.ptr(), a.shared.up.ptr(), a.shared.down.ptr()};
  c.X = (const float*)a.X.ptr(); c.Y = (float*)a.Y.ptr(); c.scratch = a.scratch.ptr(); c.scratch_bytes = a.scratch.size;
  check(msb_moe_prefill(&c, e.stream), "encode_moe_prefill");
}
}  // namespace q

namespace arch {          // src/kernels/arch.hpp:79-130 (router, rmsnorm, argmax)
// router: msb_router_scratch_bytes(n_experts) bytes; sample (optional): msb_sample_scratch_bytes(max_rows) zeroed bytes
// for the sampling calls (the reference's Scratch::sample_part / counters, arch.hpp:30-33)
struct Scratch { Buffer router; int n_experts = 384; Buffer sample; int max_rows = 0; };
inline void encode_router_fused(Enc& e, Buffer x, Buffer W, Buffer bias, Buffer ids, Buffer w, const Scratch& s,
                                int dim = 5120, int k = 6, int score_fn = 0, float route_scale = 1.5f) {
  check(msb_router_fused((const float*)x.ptr(), (const float*)W.ptr(), (const float*)bias.ptr(), (int*)ids.ptr(),
                         (float*)w.ptr(), s.router.ptr(), s.router.size, s.n_experts, dim, k, score_fn, route_scale,
                         e.stream), "encode_router_fused");
}
// rmsnorm (arch.hpp:99-104) + router in one launch; x_out receives the normalised vector
inline void encode_router_fused_rmsnorm(Enc& e, Buffer h, Buffer norm_w, float eps, Buffer x_out, Buffer W, Buffer bias,
                                        Buffer ids, Buffer w, const Scratch& s, int dim = 5120, int k = 6,
                                        int score_fn = 0, float route_scale = 1.5f) {
  check(msb_router_fused_rmsnorm((const float*)h.ptr(), (const float*)norm_w.ptr(), eps, (float*)x_out.ptr(),
                                 (const float*)W.ptr(), (const float*)bias.ptr(), (int*)ids.ptr(), (float*)w.ptr(),
                                 s.router.ptr(), s.router.size, s.n_experts, dim, k, score_fn, route_scale, e.stream),
        "encode_router_fused_rmsnorm");
}
inline void encode_router_topk(Enc& e, Buffer logits, Buffer bias, Buffer ids, Buffer w, int n, int n_experts = 384,
                               int k = 6, int score_fn = 0, float route_scale = 1.5f) {
  check(msb_router_topk((const float*)logits.ptr(), (const float*)bias.ptr(), (int*)ids.ptr(), (float*)w.ptr(), n,
                        n_experts, k, score_fn, route_scale, e.stream), "encode_router_topk");
}
struct RouteLists { Buffer counts, offsets, entry, tok, w, slot_of; int max_tokens = 0; };
inline void encode_route_lists(Enc& e, Buffer ids, Buffer w, int n, const RouteLists& L, int k = 6, int n_experts = 384) {
  check(msb_route_lists((const int*)ids.ptr(), (const float*)w.ptr(), n, k, n_experts, (uint32_t*)L.counts.ptr(),
                        (uint32_t*)L.offsets.ptr(), (uint32_t*)L.entry.ptr(), (uint32_t*)L.tok.ptr(), (float*)L.w.ptr(),
                        (uint32_t*)L.slot_of.ptr(), e.stream), "encode_route_lists");
}
inline void encode_rmsnorm(Enc& e, Buffer x, Buffer w, Buffer y, int rows, int dim, float eps, int in_stride = 0,
                           int out_stride = 0) {
  check(msb_rmsnorm((const float*)x.ptr(), (const float*)w.ptr(), (float*)y.ptr(), rows, dim, eps, in_stride, out_stride,
                    e.stream), "encode_rmsnorm");
}
inline void encode_argmax(Enc& e, Buffer logits, int rows, int V, Buffer out_idx, Buffer out_val) {
  for (int r = 0; r < rows; r++)
    check(msb_argmax((const float*)logits.ptr() + (size_t)r * V, V, (int*)out_idx.ptr() + r,
                     out_val.buf ? (float*)out_val.ptr() + r : nullptr, e.stream), "encode_argmax");
}
// arch.hpp:111-115 with the reference's argument list: greedy, or Gumbel-max sampling when temperature > 0
inline void encode_argmax(Enc& e, Buffer logits, int rows, int V, Buffer out_idx, Buffer out_val, const Scratch& s,
                          float temperature = 0.0f, uint64_t seed = 0) {
  if (rows > s.max_rows) die("encode_argmax: rows beyond the scratch's max_rows");
  check(msb_argmax_rows((const float*)logits.ptr(), rows, V, (int*)out_idx.ptr(), out_val.buf ? (float*)out_val.ptr() : nullptr,
                        temperature, (unsigned long long)seed, s.sample.ptr(), s.sample.size, e.stream), "encode_argmax");
}
// arch.hpp:116-119
inline void encode_topk(Enc& e, Buffer logits, int rows, int V, int k, float temperature, Buffer out_v, Buffer out_i,
                        Buffer out_lse, const Scratch& s) {
  if (rows > s.max_rows) die("encode_topk: rows beyond the scratch's max_rows");
  check(msb_sample_topk((const float*)logits.ptr(), rows, V, k, temperature, (float*)out_v.ptr(), (int*)out_i.ptr(),
                        (float*)out_lse.ptr(), s.sample.ptr(), s.sample.size, e.stream), "encode_topk");
}
// arch.hpp:120-121
inline void encode_log_softmax(Enc& e, Buffer in, Buffer out, int rows, int V) {
  check(msb_log_softmax((const float*)in.ptr(), (float*)out.ptr(), rows, V, e.stream), "encode_log_softmax");
}
// arch.hpp:122-126 (host function; vals / ids are host copies of encode_topk's output)
inline uint32_t sample_top_p(const float* vals, const uint32_t* ids, int k, float lse, float temperature, float top_p,
                             double u) {
  return (uint32_t)msb_sample_top_p(vals, (const int*)ids, k, lse, temperature, top_p, u);
}
}  // namespace arch

namespace attn {          // src/kernels/attn.hpp:113-129, decode side
struct DecodeCaches {     // the decode-visible part of attn::State (attn.hpp:62-101) for one KV source
  int D = 512, heads = 64, window = 128, index_heads = 32, topk = 512;
  int key_type = MSB_F16, elem_type = MSB_F16;
  Buffer rope;            // float2 [max_pos][32]
  Buffer win, ckv, ikey;  // window ring, compressed KV rows, index keys
  Buffer topk_list, dec_scores, q_prep, w_prep, topk_scratch, sparse_scratch;
};
inline const float* rope_row(const DecodeCaches& s, int pos) { return (const float*)s.rope.ptr() + (size_t)pos * 64; }
inline void encode_kv_window(Enc& e, DecodeCaches& s, const Buffer& kv, const Buffer& norm_w, int pos, bool actq) {
  char* row = (char*)s.win.ptr() + (size_t)(pos % s.window) * s.D * 2;
  check(msb_kv_window((const float*)kv.ptr(), (const float*)norm_w.ptr(), rope_row(s, pos), actq, s.D, s.elem_type, row,
                      e.stream), "encode_kv_window");
}
inline void encode_index_decode(Enc& e, DecodeCaches& s, const Buffer& iq, const Buffer& iw, int pos, int length,
                                bool actq = true, bool exact_query = false) {
  check(msb_index_decode(s.key_type, s.ikey.ptr(), length, (const float*)iq.ptr(), (const float*)iw.ptr(), rope_row(s, pos),
                         actq, s.index_heads, s.topk, (float*)s.q_prep.ptr(), (float*)s.w_prep.ptr(),
                         (float*)s.dec_scores.ptr(), (int*)s.topk_list.ptr(), s.topk_scratch.ptr(), s.topk_scratch.size,
                         exact_query, e.stream), "encode_index_decode");
}
inline void encode_sparse(Enc& e, DecodeCaches& s, const Buffer& q, const Buffer& sinks, const Buffer& out, int pos) {
  const int n_win = pos + 1 < s.window ? pos + 1 : s.window;
  check(msb_sparse_decode((const float*)q.ptr(), rope_row(s, pos), (const float*)sinks.ptr(), s.elem_type, s.win.ptr(),
                          n_win, s.ckv.ptr(), (const int*)s.topk_list.ptr(), s.topk, s.heads, s.D, (float*)out.ptr(),
                          s.sparse_scratch.ptr(), s.sparse_scratch.size, e.stream), "encode_sparse");
}
}  // namespace attn

}  // namespace ms
