// TEST INFRASTRUCTURE ONLY.  extern "C" doorway into the reference project's own scalar CPU routines
// (tests/ref/dequant.cpp, tests/ref/arch_ref.cpp, tests/ref/attn_ref.cpp and tests/quant_test_util.hpp of
// arnavprabhu/MacSeek), compiled straight from the reference checkout by oracle/Makefile into oracle/_ref/.
// Nothing here restates an algorithm: every function forwards to the reference symbol named in its comment.
// Used to pin oracle/msb_oracle.c, to generate tests/golden/, and as the timed CPU baseline ("kind": "reference").
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>
#include "ref/dequant.hpp"
#include "ref/arch_ref.hpp"
#include "ref/attn_ref.hpp"

extern "C" {

// ref::dequant_row (tests/ref/dequant.cpp:34)
void msref_dequant_row(int t, const void* src, float* dst, int64_t n) { ref::dequant_row((ref::QType)t, src, dst, n); }

// ms::q::row_bytes (src/kernels/quant_types.hpp:34)
uint64_t msref_row_bytes(int t, int64_t cols) { return ms::q::row_bytes((ref::QType)t, cols); }

// ref::random_blocks (tests/ref/dequant.cpp:133); out must hold row_bytes(t, n) bytes
void msref_random_blocks(int t, int64_t n, uint32_t seed, float scale, uint8_t* out) {
  auto v = ref::random_blocks((ref::QType)t, n, seed, scale);
  memcpy(out, v.data(), v.size());
}

// ref::matvec_ref (tests/ref/dequant.cpp:122)
void msref_matvec_ref(int t, const void* W, int rows, int cols, const float* x, float* y) {
  ref::matvec_ref((ref::QType)t, W, rows, cols, x, y);
}

// The loop of qt::ref_matvec (tests/quant_test_util.hpp:29-42) over rows [r0, r1): ref::dequant_row + double dot with
// the per-row magnitude sum.  The header itself cannot be included here (it pulls in the Metal device layer), so the
// loop body is spelled out around the reference's dequant_row.
static void ref_matvec_rows(int t, const uint8_t* W, int rows, int cols, const float* x, double* y, double* mag,
                            int groups, int r0, int r1) {
  std::vector<float> w(cols);
  const size_t rb = ms::q::row_bytes((ref::QType)t, cols);
  const int rpg = rows / groups;
  for (int r = r0; r < r1; r++) {
    ref::dequant_row((ref::QType)t, W + rb * r, w.data(), cols);
    const float* xg = x + (size_t)(r / rpg) * cols;
    double s = 0, m = 0;
    for (int c = 0; c < cols; c++) { double p = (double)w[c] * xg[c]; s += p; m += p < 0 ? -p : p; }
    y[r] = s;
    if (mag) mag[r] = m;
  }
}
// threads <= 1: the scalar loop as written; threads > 1: rows split over std::thread workers (the reference's own
// multi-threaded CPU references split rows the same way, tests/test_quant_moe_prefill.mm:30-46).
void msref_ref_matvec(int t, const void* W, int rows, int cols, const float* x, double* y, double* mag, int groups,
                      int threads) {
  if (threads <= 1) { ref_matvec_rows(t, (const uint8_t*)W, rows, cols, x, y, mag, groups, 0, rows); return; }
  std::vector<std::thread> th;
  for (int i = 0; i < threads; i++) {
    int r0 = (int)((int64_t)rows * i / threads), r1 = (int)((int64_t)rows * (i + 1) / threads);
    th.emplace_back(ref_matvec_rows, t, (const uint8_t*)W, rows, cols, x, y, mag, groups, r0, r1);
  }
  for (auto& q : th) q.join();
}

// ref_arch::router (tests/ref/arch_ref.cpp:97): 384 logits -> 6 ids, 6 weights
void msref_router(const float* logits, const float* bias, int* ids, float* w, float route_scale) {
  ref_arch::router(logits, bias, ids, w, route_scale);
}

// ref_arch::route_lists (tests/ref/arch_ref.cpp:114): n tokens x 6 -> per-expert lists
void msref_route_lists(const int* ids, const float* w, int n, uint32_t* counts, uint32_t* offsets, uint32_t* entry,
                       uint32_t* tok, float* lw, uint32_t* slot_of) {
  std::vector<uint32_t> c, o, e, t, s;
  std::vector<float> l;
  ref_arch::route_lists(ids, w, n, c, o, e, t, l, s);
  memcpy(counts, c.data(), c.size() * 4); memcpy(offsets, o.data(), o.size() * 4);
  memcpy(entry, e.data(), e.size() * 4); memcpy(tok, t.data(), t.size() * 4);
  memcpy(lw, l.data(), l.size() * 4); memcpy(slot_of, s.data(), s.size() * 4);
}

// ref_arch::argmax / rmsnorm (tests/ref/arch_ref.cpp)
int msref_argmax(const float* x, int n) { return ref_arch::argmax(x, n); }
// ref_arch::topk / logsumexp / log_softmax (tests/ref/arch_ref.cpp:199-219)
void msref_topk(const float* x, int n, int k, float* v, uint32_t* idx) { ref_arch::topk(x, n, k, v, idx); }
double msref_logsumexp(const float* x, int n, double scale) { return ref_arch::logsumexp(x, n, scale); }
void msref_log_softmax(const float* x, float* y, int n) { ref_arch::log_softmax(x, y, n); }
void msref_rmsnorm(const float* x, const float* w, float* y, int dim, double eps) { ref_arch::rmsnorm(x, w, y, dim, eps); }

// attnref::rope_table (tests/ref/attn_ref.cpp:34): [max_pos][32][2]
void msref_rope_table(int max_pos, int yarn, float* out) {
  auto t = attnref::rope_table(max_pos, yarn != 0);
  memcpy(out, t.data(), t.size() * 4);
}
// attnref::round_e4m3 / round_e2m1 / fp8_sim / fp4_sim_* (tests/ref/attn_ref.cpp:68-107)
float msref_round_e4m3(float x) { return attnref::round_e4m3(x); }
float msref_round_e2m1(float x) { return attnref::round_e2m1(x); }
void msref_fp8_sim(float* x, int n) { attnref::fp8_sim(x, n); }
void msref_fp4_sim_e8m0(float* x, int n) { attnref::fp4_sim_e8m0(x, n); }
void msref_fp4_sim_e4m3(float* x, int n) { attnref::fp4_sim_e4m3(x, n); }

// attnref::index_q (tests/ref/attn_ref.cpp:163): 32 heads x 128
void msref_index_q(const float* q_raw, const float* w_raw, const float* cs, int actq, float* q, float* w) {
  attnref::index_q(q_raw, w_raw, cs, actq != 0, q, w);
}
// attnref::index_scores (tests/ref/attn_ref.cpp:172): 32 heads, f32 keys [len][128]
void msref_index_scores(const float* q, const float* w, const float* keys, int len, float* sc) {
  std::vector<float> v;
  attnref::index_scores(q, w, keys, len, v);
  memcpy(sc, v.data(), (size_t)len * 4);
}
// attnref::topk_sorted (tests/ref/attn_ref.cpp:194); out[k], -1 padded; returns the count selected
int msref_topk_sorted(const float* sc, int n, int k, int* out) {
  std::vector<float> v(sc, sc + n);
  auto r = attnref::topk_sorted(v, k);
  for (int i = 0; i < k; i++) out[i] = i < (int)r.size() ? r[i] : -1;
  return (int)r.size();
}
// attnref::candidate_blocks (tests/ref/attn_ref.cpp:196); out[2048], -1 padded
int msref_candidate_blocks(const float* sc, int len, int* out) {
  std::vector<float> v(sc, sc + len);
  auto r = attnref::candidate_blocks(v, len);
  for (int i = 0; i < attnref::CB; i++) out[i] = i < (int)r.size() ? r[i] : -1;
  return (int)r.size();
}
// attnref::sparse_attn (tests/ref/attn_ref.cpp:204): rows given as one dense [n_rows][512] f32 array
void msref_sparse_attn(const float* q_raw, const float* cs, const float* rows, int n_rows, const float* sinks,
                       float* out) {
  std::vector<const float*> p(n_rows);
  for (int i = 0; i < n_rows; i++) p[i] = rows + (size_t)i * attnref::D;
  attnref::sparse_attn(q_raw, cs, p, sinks, out);
}
// attnref::window_row (tests/ref/attn_ref.cpp:109)
void msref_window_row(const float* kv_raw, const float* norm_w, const float* cs, int actq, float* out) {
  attnref::window_row(kv_raw, norm_w, cs, actq != 0, out);
}

// hyper-connection step and compressor of the reference (fixed shapes: 4 x 5120 streams; 512-wide latent, 128-wide keys)
void msref_hc_step(const float* h_in, const float* x_sub, const float* mix_prev, const float* fn, const float* scale,
                   const float* base, const float* norm_w, float* h_out, float* mix_out, float* x_out) {
  ref_arch::hc_step(h_in, x_sub, mix_prev, fn, scale, base, norm_w, h_out, mix_out, x_out);
}
// feeds tokens 0 .. n-1 to a fresh source; returns the number of rows emitted into ckv [rows][512] / ikey [rows][128]
int msref_compress_tokens(int ratio, int n, const float* ckv_in, const float* cgate_in, const float* cnorm_w,
                          const uint16_t* wk, const float* knorm_w, int actq, float* ckv, float* ikey) {
  attnref::Source s;
  attnref::source_init(s, ratio);
  std::vector<float> tab = attnref::rope_table(n + 1, true);
  for (int p = 0; p < n; p++)
    attnref::compress_token(s, p, ckv_in + (size_t)p * 512, cgate_in ? cgate_in + (size_t)p * 512 : nullptr, cnorm_w, wk,
                            knorm_w, tab, actq != 0);
  std::copy(s.ckv.begin(), s.ckv.end(), ckv);
  std::copy(s.ikey.begin(), s.ikey.end(), ikey);
  return s.rows();
}
int msref_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

}  // extern "C"
