// ms::ds41 decode layer-forward surface over libmacseek_b200 (the reference's src/model/dec_layer.hpp:18-118 and the
// sequence of dec_layer.mm:138-313): W / LayerW / DecBufs / DecOptions / DecCtx, encode_dec_prologue,
// encode_dec_attn_side, encode_dec_moe_table, plus ms::arch::HcStep / encode_hc_step (arch.hpp:44-77).
//
// What is the same: the per-layer order of calls, the buffers they read and write, the hyper-connection boundaries with
// their lagged mixes, the KV-source / index-source roles, the router stage, the table MoE accumulating into `sub`.
// What is not carried over (each is a separate subsystem outside the per-token kernel path): the engram branch, the
// next-layer expert prediction, the CPU<->GPU router handshake (DecSync: with HBM-resident experts there is nothing to
// wait for -- encode_dec_moe_ids resolves the router's ids on the device), background chunks and profiling skips.
// Shapes the reference fixes (5120 / 1280 / 8192 x 4096 / 384 experts top-6) come from ds41::Config here.
#pragma once
#include "ms_b200_attn_state.hpp"

namespace ms {

namespace arch {
// One sublayer boundary of the 4-stream residual (arch.hpp:44-77).  Empty buffers switch parts off as in the reference.
struct HcStep {
  Buffer h_in, h_out;          // [n][4][dim]; h_out may equal h_in
  Buffer x_sub;                // [n][dim] sublayer output (empty: no hc_post)
  Buffer mix_prev;             // [n][24]
  Buffer fn, scale, base;      // hc_*_fn [24][4 dim], hc_*_scale [3], hc_*_base [24] (fn empty: no mixes)
  Buffer mix_out;              // [n][24], must not alias mix_prev
  Buffer norm_w;               // [dim]
  Buffer x_out;                // [n][dim] (empty: no hc_pre / RMSNorm)
  int n = 1;
  int row_splits = 0;          // accepted for source compatibility (the launch shape is chosen by the library)
};
struct DecScratch {            // the parts of arch::Scratch (arch.hpp:20-38) the decode path uses
  Scratch router;
  Buffer hc;                   // msb_hc_scratch_bytes(max_tokens), zero-filled
  int dim = 5120, max_tokens = 1;
  static DecScratch create(int dim, int n_experts, int max_tokens = 1) {
    DecScratch s;
    s.dim = dim; s.max_tokens = max_tokens;
    s.router.n_experts = n_experts;
    s.router.router = Device::get().alloc(msb_router_scratch_bytes(n_experts), "router scratch");
    s.hc = Device::get().alloc(msb_hc_scratch_bytes(max_tokens), "hc scratch");
    return s;
  }
};
inline void encode_hc_step(Enc& e, const HcStep& a, const DecScratch& s) {
  check(msb_hc_step((const float*)a.h_in.ptr(), (float*)a.h_out.ptr(), (const float*)a.x_sub.ptr(),
                    (const float*)a.mix_prev.ptr(), (const float*)a.fn.ptr(), (const float*)a.scale.ptr(),
                    (const float*)a.base.ptr(), (float*)a.mix_out.ptr(), (const float*)a.norm_w.ptr(), (float*)a.x_out.ptr(),
                    s.dim, a.n, s.hc.ptr(), s.hc.size, e.stream), "encode_hc_step");
}
inline void fill_identity_mix(float* mix24) {          // pre = [1,0,0,0], post = 0, comb = 0 (arch.hpp:78)
  for (int i = 0; i < 24; i++) mix24[i] = 0.f;
  mix24[0] = 1.f;
}
}  // namespace arch

namespace ds41 {

struct Config {            // the fields of src/model/config.hpp the decode layer reads
  int n_layers = 40, dim = 5120, q_lora = 1280, n_heads = 64, head_dim = 512, o_groups = 8, o_a_rows = 8192;
  int n_experts = 384, top_k = 6, inter = 2304;
  int score_fn = 0;        // 0 sqrt(softplus), 1 sigmoid
  float route_scale = 1.5f, norm_eps = 1e-20f;
};

struct W {                 // one weight: buffer + kernel type + shape (dec_layer.hpp:18-21)
  Buffer b; q::QType t = q::QType::F32; int rows = 0, cols = 0;
  explicit operator bool() const { return b.buf != nullptr; }
};
struct LayerW {            // dec_layer.hpp:22-30 without the engram weights
  W attn_norm, ffn_norm, q_a, q_a_norm, q_b, kv, kv_norm, o_a, o_b, sinks;
  W c_kv, c_gate, c_norm, idx_qb, idx_proj, idx_k, idx_knorm;
  W gate_inp, bias;
  W sh_gate, sh_up, sh_down;
  W hc_attn_fn, hc_attn_scale, hc_attn_base, hc_ffn_fn, hc_ffn_scale, hc_ffn_base;
};
struct DecBufs {           // activations of one decode token, all F32 (dec_layer.hpp:33-47)
  Buffer h, h2;            // [4][dim] hyper-connection state (h2: optional ping-pong partner)
  Buffer x, sub;           // [dim]
  Buffer mixA, mixF;       // [24]
  Buffer mix_ident;        // optional [24] identity mix read by layer 0 instead of mixF
  Buffer qa, qrn, q, kv, ckv, cgate, iq, iw, aout, oa;
  Buffer rids, rw;         // router ids int32[top_k], weights [top_k]
  Buffer moe_scratch;      // >= q::moe_decode_scratch_bytes()
};
struct DecOptions {        // the switches of dec_layer.hpp:52-84 that change the sequence encoded here
  bool reorder = false;    // kv window / compressor in the q_a-norm stage, fill(sub) in the router stage
  bool norm_qb = false;    // q_a_norm fused into the q_b / indexer q_b activation loads
  bool attn_comb = false;  // accepted; the split-K combine gives the same bits either way
  int hc_splits = 1;       // > 1: h ping-pongs between B.h and B.h2
};
struct DecCtx {            // dec_layer.hpp:96-107
  const Config* cfg = nullptr;
  const std::vector<LayerW>* L = nullptr;
  DecBufs B;
  attn::State* ast = nullptr;
  const arch::DecScratch* asc = nullptr;
  DecOptions o;
  int hcur = 0;
};
inline Buffer dec_cur_h(const DecCtx& c) { return c.hcur ? c.B.h2 : c.B.h; }

inline void matvec(Enc& e, const W& w, const Buffer& x, const Buffer& y) {
  q::encode_matvec(e, w.t, w.b, w.rows, w.cols, x, y);
}
inline void fill0(Enc& e, const Buffer& b, size_t n) { check(msb_fill_f32((float*)b.ptr(), 0.f, n, e.stream), "fill0"); }

// Token prologue after the embedding (dec_layer.mm:111-136): the embedding wrote B.h; the engram rows are not part of
// this path.
inline void encode_dec_prologue(Enc&, DecCtx& c, const Buffer& /*erow*/) { c.hcur = 0; }

// Attention side of layer l for the token at position pos: hc boundary into attention, projections, kv window (+
// compressor), indexer, sparse attention, o-projections, hc boundary into the FFN, router; `sub` is left zeroed for the
// MoE (dec_layer.mm:138-255).
inline void encode_dec_attn_side(Enc& e, DecCtx& c, int l, int pos) {
  const Config& cfg = *c.cfg;
  const LayerW& L = (*c.L)[l];
  const DecBufs& B = c.B;
  const arch::DecScratch& asc = *c.asc;
  const DecOptions& o = c.o;
  attn::State& S = *c.ast;
  const bool kvsrc = S.is_kv_src(l), idxsrc = S.is_index_src(l);
  const bool pp = o.hc_splits > 1 && B.h2.buf != nullptr;
  auto post_io = [&](arch::HcStep& a) {
    a.h_in = dec_cur_h(c);
    if (pp) { c.hcur ^= 1; a.h_out = dec_cur_h(c); a.row_splits = o.hc_splits; }
    else a.h_out = a.h_in;
  };
  // ---- hyper-connection boundary into attention ----
  {
    arch::HcStep a;
    if (l > 0) { post_io(a); a.x_sub = B.sub; }
    else { a.h_in = dec_cur_h(c); a.h_out = a.h_in; }
    a.mix_prev = (l == 0 && B.mix_ident.buf) ? B.mix_ident : B.mixF;
    a.fn = L.hc_attn_fn.b; a.scale = L.hc_attn_scale.b; a.base = L.hc_attn_base.b; a.mix_out = B.mixA;
    a.norm_w = L.attn_norm.b; a.x_out = B.x; a.n = 1;
    arch::encode_hc_step(e, a, asc);
    e.barrier();
  }
  // ---- attention projections ----
  matvec(e, L.q_a, B.x, B.qa);
  matvec(e, L.kv, B.x, B.kv);
  if (kvsrc) { matvec(e, L.c_kv, B.x, B.ckv); if (L.c_gate) matvec(e, L.c_gate, B.x, B.cgate); }
  if (idxsrc) matvec(e, L.idx_proj, B.x, B.iw);
  e.barrier();
  attn::LayerIO io;
  io.layer = l; io.q = B.q; io.kv = B.kv; io.kv_norm = L.kv_norm.b; io.sinks = L.sinks.b; io.out = B.aout;
  if (kvsrc) { io.c_kv = B.ckv; io.c_gate = L.c_gate ? B.cgate : Buffer{}; io.c_norm = L.c_norm.b; io.idx_wk = L.idx_k.b; io.idx_knorm = L.idx_knorm.b; }
  if (idxsrc) { io.idx_q = B.iq; io.idx_w = B.iw; }
  auto kv_stage = [&]() {
    attn::encode_kv_window(e, S, l, io.kv, io.kv_norm, pos, 1);
    if (kvsrc) attn::encode_compress(e, S, l, io, pos, 1, false);
  };
  if (o.norm_qb) {
    q::encode_matvec_rmsnorm(e, L.q_b.t, L.q_b.b, L.q_b.rows, L.q_b.cols, B.qa, L.q_a_norm.b, cfg.norm_eps, B.q);
    if (idxsrc) q::encode_matvec_rmsnorm(e, L.idx_qb.t, L.idx_qb.b, L.idx_qb.rows, L.idx_qb.cols, B.qa, L.q_a_norm.b, cfg.norm_eps, B.iq);
    if (o.reorder) kv_stage();
    e.barrier();
  } else {
    arch::encode_rmsnorm(e, B.qa, L.q_a_norm.b, B.qrn, 1, cfg.q_lora, cfg.norm_eps);
    if (o.reorder) kv_stage();
    e.barrier();
    matvec(e, L.q_b, B.qrn, B.q);
    if (idxsrc) matvec(e, L.idx_qb, B.qrn, B.iq);
    e.barrier();
  }
  if (!o.reorder) { kv_stage(); e.barrier(); }
  // ---- attention: indexer (index source layers) + sparse attention ----
  if (idxsrc) attn::encode_index_decode(e, S, l, io.idx_q, io.idx_w, pos);
  attn::encode_sparse(e, S, l, io.q, io.sinks, io.out, pos, 1, o.attn_comb);
  // ---- wo_a (block-diagonal) then wo_b ----
  q::encode_matvec(e, L.o_a.t, L.o_a.b, L.o_a.rows, L.o_a.cols, B.aout, B.oa, false, cfg.o_groups);
  e.barrier();
  matvec(e, L.o_b, B.oa, B.sub);
  e.barrier();
  // ---- hyper-connection boundary into the FFN ----
  {
    arch::HcStep a; post_io(a); a.x_sub = B.sub; a.mix_prev = B.mixA;
    a.fn = L.hc_ffn_fn.b; a.scale = L.hc_ffn_scale.b; a.base = L.hc_ffn_base.b; a.mix_out = B.mixF;
    a.norm_w = L.ffn_norm.b; a.x_out = B.x; a.n = 1;
    arch::encode_hc_step(e, a, asc);
    e.barrier();
  }
  // ---- router; the MoE accumulates into sub (consumed by the next hc step): zero it ----
  arch::encode_router_fused(e, B.x, L.gate_inp.b, L.bias.b, B.rids, B.rw, asc.router, cfg.dim, cfg.top_k, cfg.score_fn,
                            cfg.route_scale);
  fill0(e, B.sub, (size_t)cfg.dim);
  e.barrier();
}

inline q::MoeDecodeArgs dec_moe_args(const DecCtx& c, int l, q::QType t_gate_up, q::QType t_down) {
  const LayerW& L = (*c.L)[l];
  q::MoeDecodeArgs m;
  m.dim = c.cfg->dim; m.inter = c.cfg->inter;
  m.t_gate_up = t_gate_up; m.t_down = t_down;
  m.n_routed = c.cfg->top_k; m.weights = c.B.rw; m.has_shared = true; m.t_shared = L.sh_gate.t;
  m.shared = q::ExpertSlot{L.sh_gate.b, L.sh_up.b, L.sh_down.b};
  m.x = c.B.x; m.y = c.B.sub; m.scratch = c.B.moe_scratch;
  return m;
}
// MoE of layer l, table variant (dec_layer.mm:257-313 without the handshake): routed experts read from `table`
// ([top_k][3] device addresses, valid when this is encoded).
inline void encode_dec_moe_table(Enc& e, DecCtx& c, int l, q::QType t_gate_up, q::QType t_down, const Buffer& table) {
  q::encode_moe_decode_table_part(e, dec_moe_args(c, l, t_gate_up, t_down), table, q::MoePart::All);
  e.barrier();
}
// The same with HBM-resident experts: expert_table [n_experts][3] device addresses, the router's ids (B.rids) are
// resolved on the device, so no CPU round trip separates the router from the experts.
inline void encode_dec_moe_ids(Enc& e, DecCtx& c, int l, q::QType t_gate_up, q::QType t_down, const Buffer& expert_table,
                               int expert_lo, int expert_hi) {
  q::encode_moe_decode_ids(e, dec_moe_args(c, l, t_gate_up, t_down), expert_table, c.B.rids, expert_lo, expert_hi);
  e.barrier();
}
// After the last layer: the final hc step folds the last FFN output and produces the head's input (ds41.mm:491-499).
inline void encode_dec_final(Enc& e, DecCtx& c, const Buffer& out_norm_w, const Buffer& x_out) {
  arch::HcStep a;
  a.h_in = dec_cur_h(c); a.h_out = a.h_in; a.x_sub = c.B.sub; a.mix_prev = c.B.mixF; a.norm_w = out_norm_w; a.x_out = x_out; a.n = 1;
  arch::encode_hc_step(e, a, *c.asc);
  e.barrier();
}

}  // namespace ds41
}  // namespace ms
