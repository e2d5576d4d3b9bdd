/* TEST INFRASTRUCTURE ONLY -- CPU oracle for the MacSeek per-token hot path.
 *
 * A plain-C restatement of the reference project's scalar CPU routines (arnavprabhu/MacSeek, tests/ref/*.cpp,
 * tests/quant_test_util.hpp and the reference loops inside tests/test_quant_moe.mm), parameterised so that the same
 * code covers the reference's compile-time shapes (384 experts top-6, 32 index heads, k=512, 512-wide KV rows) and
 * the synthetic benchmark shapes (top-8 sigmoid router, 64 index heads, k=2048, 576-wide rows).
 *
 * Parity pinned: tests/test_oracle_pin.py compares every function below with the reference's own code compiled from
 * its sources (oracle/_ref/libmsref.so) and with the committed vectors under tests/golden/.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may load this library.  The shipped CUDA path
 * never calls it.
 */
#ifndef MSB_ORACLE_H
#define MSB_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids, src/kernels/quant_types.hpp:10-12 */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_Q8_0 = 8, ORC_Q5_K = 13, ORC_Q6_K = 14, ORC_IQ2_XXS = 16, ORC_IQ1_S = 19,
       ORC_IQ4_NL = 20, ORC_BF16 = 30, ORC_MXFP4 = 39 };

int orc_block_elems(int t);                 /* quant_types.hpp:15-21 */
size_t orc_block_bytes(int t);              /* quant_types.hpp:22-35 */
size_t orc_row_bytes(int t, int64_t cols);  /* quant_types.hpp:36 */

float orc_fp16_to_f32(uint16_t h);
uint16_t orc_f32_to_fp16(float f);
float orc_bf16_to_f32(uint16_t h);
uint16_t orc_f32_to_bf16(float f);          /* round to nearest even */
float orc_e4m3_to_f32(uint8_t v);           /* OCP FP8 E4M3 (finite-only variant, max 448) */
uint8_t orc_f32_to_e4m3(float f);           /* saturating round to nearest even */

/* tests/ref/dequant.cpp:34-120.  n = element count, a multiple of the block size. */
void orc_dequant_row(int t, const void* src, float* dst, int64_t n);

/* tests/quant_test_util.hpp:29-42 (double dot of dequantised rows, with sum |w x| per row); block-diagonal groups as
 * there.  n_cols activation columns: x[c] starts at x + c*x_stride, y/mag [c][rows].  threads > 1 splits rows. */
void orc_matvec(int t, const void* W, int rows, int cols, const float* x, int n_cols, int64_t x_stride, int groups,
                double* y, double* mag, int threads);

/* tests/quant_test_util.hpp:44-52 */
double orc_max_norm_err(const float* got, const double* ref, const double* mag, int n, int* worst);

/* MoE decode reference: the loop of tests/test_quant_moe.mm:70-91 with silu_clamped (:14-18).
 * Experts 0..n_routed-1 use t_gate_up/t_down and weight w[e]; expert n_routed (if has_shared) uses t_shared, weight 1.
 * gate/up [inter x dim], down [dim x inter].  h_out: float [n_exp][inter]; y (in: initial y as double, out: y + sum),
 * ymag (in: |y0|, out: + magnitudes).  limit = the swiglu clamp (10). */
typedef struct {
  int dim, inter, n_routed, has_shared;
  int t_gate_up, t_down, t_shared;
  const void* gate[16];
  const void* up[16];
  const void* down[16];   /* index n_routed = shared expert */
  const float* w;         /* [n_routed] */
  const float* x;         /* [dim] */
  float limit;
  int threads;
} orc_moe_decode_args;
void orc_moe_decode(const orc_moe_decode_args* a, float* h_out, double* y, double* ymag, double* hmag);

/* Router, tests/ref/arch_ref.cpp:97-112 generalised: E experts, top-k, score = sqrt(softplus) (score_fn 0) or
 * sigmoid (score_fn 1, reference/inference/model.py:816-817); key = (float)score + bias; ties -> lowest id;
 * w = score / (sum + 1e-20) * route_scale. */
void orc_router(const float* logits, const float* bias, int E, int k, int score_fn, float route_scale, int* ids,
                float* w);
/* tests/ref/arch_ref.cpp:114-131 with k entries per token and E experts. */
void orc_route_lists(const int* ids, const float* w, int n, int k, int E, uint32_t* counts, uint32_t* offsets,
                     uint32_t* entry, uint32_t* tok, float* lw, uint32_t* slot_of);
int orc_argmax(const float* x, int n);      /* ties -> lowest index, tests/ref/arch_ref.hpp:44 */
void orc_topk_desc(const float* x, int n, int k, float* v, uint32_t* idx);      /* arch_ref.cpp:199-206 */
double orc_logsumexp(const float* x, int n, double scale);                      /* arch_ref.cpp:208-214 */
void orc_log_softmax(const float* x, float* y, int n);                          /* arch_ref.cpp:216-219 */
double orc_gumbel(uint32_t i, uint64_t seed, uint32_t row);                     /* arch_sample.metal:15-26,68 */
uint32_t orc_sample_top_p(const float* vals, const uint32_t* ids, int k, float lse, float temperature, float top_p,
                          double u);                                            /* arch.mm:322-342 */
/* tests/ref/arch_ref.cpp:77-82 */
void orc_rmsnorm(const float* x, const float* w, float* y, int dim, double eps);

/* rope, tests/ref/attn_ref.cpp:15-56 */
void orc_rope_table(int max_pos, int yarn, float* out /* [max_pos][32][2] */);
void orc_rope(float* x64, const float* cs, int inverse);
/* quant-dequant simulations, tests/ref/attn_ref.cpp:58-107 */
float orc_round_e4m3(float x);
float orc_round_e2m1(float x);
void orc_fp8_sim(float* x, int n);
void orc_fp4_sim_e8m0(float* x, int n);
void orc_fp4_sim_e4m3(float* x, int n);

/* Indexer, tests/ref/attn_ref.cpp:163-184 with `heads` heads of `dim` (rope on the last 64 of each head). */
void orc_index_q(const float* q_raw, const float* w_raw, const float* cs, int actq, int heads, int dim, float* q,
                 float* w);
void orc_index_scores(const float* q, const float* w, const float* keys, int heads, int dim, int len, float* sc,
                      int threads);
/* tests/ref/attn_ref.cpp:186-194: top-k among finite scores, ties -> lower index, sorted ascending, -1 padded.
 * Returns the number selected. */
int orc_topk_sorted(const float* sc, int n, int k, int* out);
/* tests/ref/attn_ref.cpp:196-202 with block size bs and cap blocks. */
int orc_candidate_blocks(const float* sc, int len, int bs, int cap, int* out);
/* tests/ref/attn_ref.cpp:204-230 with H heads, row width D, rope on the last RD (=64) dims of q / inverse on out.
 * rows: dense [n_rows][D] f32. */
void orc_sparse_attn(const float* q_raw, const float* cs, const float* rows, int n_rows, const float* sinks, int H,
                     int D, float* out, int threads);
/* tests/ref/attn_ref.cpp:109-114 */
void orc_window_row(const float* kv_raw, const float* norm_w, const float* cs, int actq, int D, float* out);

/* hyper-connections: tests/ref/arch_ref.cpp:22-95 with the stream width D as a parameter (the reference: 5120) */
void orc_hc_split(const double* m, const float* scale, const float* base, float* mix, int iters, double eps);
void orc_hc_mixes(const float* h, const float* fn, const float* scale, const float* base, int D, float* mix, int iters,
                  double norm_eps, double hc_eps);
void orc_hc_step(const float* h_in, const float* x_sub, const float* mix_prev, const float* fn, const float* scale,
                 const float* base, const float* norm_w, int D, float* h_out, float* mix_out, float* x_out);
/* compressor + index key of one token: tests/ref/attn_ref.cpp:116-161 with the state passed explicitly */
int orc_compress_token(int ratio, int p, const float* ckv_in, const float* cgate_in, const float* cnorm_w,
                       const uint16_t* wk_bf16, const float* knorm_w, const float* cs_tab, int actq, int D, int ID,
                       float* st_kv, float* st_sc, float* ckv_row, float* ikey_row);

int orc_hardware_threads(void);

#ifdef __cplusplus
}
#endif
#endif
