/* TEST INFRASTRUCTURE ONLY -- see msb_oracle.h.  CPU restatement of the reference's scalar routines; each function
 * names the reference file:line it follows.  Never linked into, or called by, the shipped CUDA path. */
#include "msb_oracle.h"
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
#include "iq_grids_packed.h"

/* ------------------------------------------------------------------ geometry (src/kernels/quant_types.hpp:15-36) */
int orc_block_elems(int t) {
  if (t == ORC_F32 || t == ORC_F16 || t == ORC_BF16) return 1;
  if (t == ORC_Q8_0 || t == ORC_IQ4_NL || t == ORC_MXFP4) return 32;
  return 256;
}
size_t orc_block_bytes(int t) {
  switch (t) {
    case ORC_F32: return 4;
    case ORC_F16: case ORC_BF16: return 2;
    case ORC_Q8_0: return 34;
    case ORC_Q5_K: return 176;
    case ORC_Q6_K: return 210;
    case ORC_IQ2_XXS: return 66;
    case ORC_IQ1_S: return 50;
    case ORC_IQ4_NL: return 18;
    case ORC_MXFP4: return 17;
  }
  return 0;
}
size_t orc_row_bytes(int t, int64_t cols) { return (size_t)(cols / orc_block_elems(t)) * orc_block_bytes(t); }

/* ------------------------------------------------------------------ scalar conversions (tests/ref/dequant.cpp:17-19) */
float orc_fp16_to_f32(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
uint16_t orc_f32_to_fp16(float f) { _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h; }
float orc_bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
uint16_t orc_f32_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1);
  return (uint16_t)(u >> 16);
}
float orc_e4m3_to_f32(uint8_t v) {
  int s = v >> 7, e = (v >> 3) & 15, m = v & 7;
  float r;
  if (e == 0) r = ldexpf((float)m, -9);
  else if (e == 15 && m == 7) r = NAN;
  else r = ldexpf((float)(8 + m), e - 10);
  return s ? -r : r;
}
uint8_t orc_f32_to_e4m3(float f) {
  uint8_t s = signbit(f) ? 0x80 : 0;
  float a = fabsf(f);
  if (isnan(a)) return s | 0x7f;
  if (a >= 448.f) return s | 0x7e;
  /* nearest-even on the e4m3 lattice: same rounding as orc_round_e4m3 below */
  float r = orc_round_e4m3(a);
  if (r == 0) return s;
  int e; float m = frexpf(r, &e);          /* r = m * 2^e, m in [0.5,1) */
  int E = e - 1 + 7;                        /* biased exponent of 1.xxx * 2^(e-1) */
  if (E <= 0) return s | (uint8_t)lrintf(ldexpf(r, 9));
  return s | (uint8_t)(E << 3) | (uint8_t)(lrintf(ldexpf(m, 4)) - 8);
}

static inline uint16_t rd16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
static inline uint32_t rd32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }

/* codebook accessors over the packed tables */
static inline int iq1s_val(int idx, int j) { return (int)((kMsbIq1sPacked[idx] >> (2 * j)) & 3) - 1; }
static inline int iq2xxs_val(int idx, int j) {
  static const int lut[4] = {8, 25, 43, 0};
  return lut[(kMsbIq2xxsPacked[idx] >> (2 * j)) & 3];
}
static inline int ksign_bits(int i7) { return i7 | ((__builtin_popcount((unsigned)i7) & 1) << 7); }

static const int8_t kIq4nlValues[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static const int8_t kE2m1Doubled[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

/* tests/ref/dequant.cpp:29-32 */
static void k4_scale_min(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
  else { *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

/* ------------------------------------------------------------------ dequant (tests/ref/dequant.cpp:34-120)
 * The float expressions keep the reference's association: that is what makes the output bit-identical. */
void orc_dequant_row(int t, const void* srcv, float* y, int64_t n) {
  const uint8_t* s = (const uint8_t*)srcv;
  int64_t b, i;
  switch (t) {
    case ORC_F32: memcpy(y, s, (size_t)n * 4); return;                                          /* :37 */
    case ORC_F16: for (i = 0; i < n; i++) y[i] = orc_fp16_to_f32(rd16(s + 2 * i)); return;      /* :38 */
    case ORC_BF16: for (i = 0; i < n; i++) y[i] = orc_bf16_to_f32(rd16(s + 2 * i)); return;     /* :39 */
    case ORC_Q8_0:                                                                              /* :40-45 */
      for (b = 0; b < n / 32; b++, s += 34, y += 32) {
        const float d = orc_fp16_to_f32(rd16(s));
        for (int j = 0; j < 32; j++) y[j] = (float)(int8_t)s[2 + j] * d;
      }
      return;
    case ORC_Q5_K:                                                                              /* :46-60 */
      for (b = 0; b < n / 256; b++, s += 176, y += 256) {
        const float d = orc_fp16_to_f32(rd16(s)), dmin = orc_fp16_to_f32(rd16(s + 2));
        const uint8_t *sc = s + 4, *qh = s + 16, *ql = s + 48;
        for (int g = 0; g < 4; g++) {            /* 64 elements per step: two 32-element sub-blocks */
          uint8_t a, m;
          k4_scale_min(2 * g, sc, &a, &m);
          const float d1 = d * a, m1 = dmin * m;
          k4_scale_min(2 * g + 1, sc, &a, &m);
          const float d2 = d * a, m2 = dmin * m;
          const uint8_t* q = ql + 32 * g;
          for (int l = 0; l < 32; l++) y[64 * g + l] = d1 * (float)((q[l] & 0xF) + ((qh[l] >> (2 * g)) & 1) * 16) - m1;
          for (int l = 0; l < 32; l++) y[64 * g + 32 + l] = d2 * (float)((q[l] >> 4) + ((qh[l] >> (2 * g + 1)) & 1) * 16) - m2;
        }
      }
      return;
    case ORC_Q6_K:                                                                              /* :61-77 */
      for (b = 0; b < n / 256; b++, s += 210, y += 256) {
        const float d = orc_fp16_to_f32(rd16(s + 208));
        for (int half = 0; half < 2; half++) {
          const uint8_t *ql = s + 64 * half, *qh = s + 128 + 32 * half;
          const int8_t* sc = (const int8_t*)(s + 192 + 8 * half);
          float* o = y + 128 * half;
          for (int l = 0; l < 32; l++) {
            const int is = l / 16;
            const int8_t q1 = (int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
            const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            o[l] = d * sc[is] * q1;
            o[l + 32] = d * sc[is + 2] * q2;
            o[l + 64] = d * sc[is + 4] * q3;
            o[l + 96] = d * sc[is + 6] * q4;
          }
        }
      }
      return;
    case ORC_IQ1_S:                                                                             /* :78-92 */
      for (b = 0; b < n / 256; b++, s += 50) {
        const float d = orc_fp16_to_f32(rd16(s));
        for (int ib = 0; ib < 8; ib++) {
          const uint8_t* qs = s + 2 + 4 * ib;
          const uint16_t qh = rd16(s + 34 + 2 * ib);
          const float dl = d * (float)(2 * ((qh >> 12) & 7) + 1);
          const float delta = (qh & 0x8000) ? -0.125f : 0.125f;
          for (int l = 0; l < 4; l++, y += 8) {
            const int idx = qs[l] | (((qh >> (3 * l)) & 7) << 8);
            for (int j = 0; j < 8; j++) y[j] = dl * ((float)iq1s_val(idx, j) + delta);
          }
        }
      }
      return;
    case ORC_IQ2_XXS:                                                                           /* :93-106 */
      for (b = 0; b < n / 256; b++, s += 66) {
        const float d = orc_fp16_to_f32(rd16(s));
        for (int ib = 0; ib < 8; ib++) {
          const uint8_t* a8 = s + 2 + 8 * ib;
          const uint32_t a1 = rd32(a8 + 4);
          const float db = d * (0.5f + (float)(a1 >> 28)) * 0.25f;
          for (int l = 0; l < 4; l++, y += 8) {
            const int sg = ksign_bits((int)((a1 >> (7 * l)) & 127));
            for (int j = 0; j < 8; j++) y[j] = db * (float)iq2xxs_val(a8[l], j) * ((sg >> j) & 1 ? -1.f : 1.f);
          }
        }
      }
      return;
    case ORC_IQ4_NL:                                                                            /* :107-112 */
      for (b = 0; b < n / 32; b++, s += 18, y += 32) {
        const float d = orc_fp16_to_f32(rd16(s));
        for (int j = 0; j < 16; j++) {
          y[j] = d * (float)kIq4nlValues[s[2 + j] & 0xF];
          y[j + 16] = d * (float)kIq4nlValues[s[2 + j] >> 4];
        }
      }
      return;
    case ORC_MXFP4:                                                                             /* :24-27,113-118 */
      for (b = 0; b < n / 32; b++, s += 17, y += 32) {
        const uint32_t bits = s[0] < 2 ? (0x00200000u << s[0]) : ((uint32_t)(s[0] - 1) << 23);
        float d; memcpy(&d, &bits, 4);
        for (int j = 0; j < 16; j++) {
          y[j] = (float)kE2m1Doubled[s[1 + j] & 0xF] * d;
          y[j + 16] = (float)kE2m1Doubled[s[1 + j] >> 4] * d;
        }
      }
      return;
  }
}

/* ------------------------------------------------------------------ tiny thread pool helper */
typedef void (*orc_range_fn)(void* ctx, int lo, int hi);
typedef struct { orc_range_fn fn; void* ctx; int lo, hi; } orc_job;
static void* orc_job_main(void* p) { orc_job* j = (orc_job*)p; j->fn(j->ctx, j->lo, j->hi); return NULL; }
static void orc_parallel(orc_range_fn fn, void* ctx, int n, int threads) {
  if (threads <= 1 || n <= 1) { fn(ctx, 0, n); return; }
  if (threads > n) threads = n;
  if (threads > 256) threads = 256;
  pthread_t th[256]; orc_job jobs[256];
  for (int i = 0; i < threads; i++) {
    jobs[i].fn = fn; jobs[i].ctx = ctx;
    jobs[i].lo = (int)((int64_t)n * i / threads); jobs[i].hi = (int)((int64_t)n * (i + 1) / threads);
    pthread_create(&th[i], NULL, orc_job_main, &jobs[i]);
  }
  for (int i = 0; i < threads; i++) pthread_join(th[i], NULL);
}
int orc_hardware_threads(void) { long n = sysconf(_SC_NPROCESSORS_ONLN); return n > 0 ? (int)n : 1; }

/* ------------------------------------------------------------------ matvec (tests/quant_test_util.hpp:29-42) */
typedef struct {
  int t, rows, cols, n_cols, groups; int64_t x_stride;
  const uint8_t* W; const float* x; double* y; double* mag;
} mv_ctx;
static void mv_rows(void* p, int r0, int r1) {
  mv_ctx* c = (mv_ctx*)p;
  float* w = (float*)malloc(sizeof(float) * (size_t)c->cols);
  const size_t rb = orc_row_bytes(c->t, c->cols);
  const int rpg = c->rows / c->groups;
  for (int r = r0; r < r1; r++) {
    orc_dequant_row(c->t, c->W + rb * (size_t)r, w, c->cols);
    for (int col = 0; col < c->n_cols; col++) {
      const float* xg = c->x + col * c->x_stride + (size_t)(r / rpg) * c->cols;
      double s = 0, m = 0;
      for (int k = 0; k < c->cols; k++) { double pr = (double)w[k] * xg[k]; s += pr; m += fabs(pr); }
      c->y[(size_t)col * c->rows + r] = s;
      if (c->mag) c->mag[(size_t)col * c->rows + r] = m;
    }
  }
  free(w);
}
void orc_matvec(int t, const void* W, int rows, int cols, const float* x, int n_cols, int64_t x_stride, int groups,
                double* y, double* mag, int threads) {
  mv_ctx c = {t, rows, cols, n_cols, groups, x_stride, (const uint8_t*)W, x, y, mag};
  orc_parallel(mv_rows, &c, rows, threads);
}

/* tests/quant_test_util.hpp:44-52 */
double orc_max_norm_err(const float* got, const double* ref, const double* mag, int n, int* worst) {
  double e = 0;
  for (int i = 0; i < n; i++) {
    double d = fabs((double)got[i] - ref[i]) / (mag[i] + 1e-12);
    if (!(d <= e)) { e = d; if (worst) *worst = i; }
  }
  return e;
}

/* ------------------------------------------------------------------ MoE decode (tests/test_quant_moe.mm:14-18,70-91) */
static double silu_clamped(double g, double u, double w, double limit) {
  if (g > limit) g = limit;
  if (u > limit) u = limit;
  if (u < -limit) u = -limit;
  return g / (1.0 + exp(-g)) * u * w;
}
void orc_moe_decode(const orc_moe_decode_args* a, float* h_out, double* y, double* ymag, double* hmag) {
  const int D = a->dim, I = a->inter;
  const int n_exp = a->n_routed + (a->has_shared ? 1 : 0);
  double* g = (double*)malloc(sizeof(double) * (size_t)I * 4);
  double *gm = g + I, *u = g + 2 * I, *um = g + 3 * I;
  double* yd = (double*)malloc(sizeof(double) * (size_t)D * 2);
  double* ydm = yd + D;
  for (int e = 0; e < n_exp; e++) {
    const int shared = e == a->n_routed;
    const int tgu = shared ? a->t_shared : a->t_gate_up, td = shared ? a->t_shared : a->t_down;
    orc_matvec(tgu, a->gate[e], I, D, a->x, 1, 0, 1, g, gm, a->threads);
    orc_matvec(tgu, a->up[e], I, D, a->x, 1, 0, 1, u, um, a->threads);
    const double we = shared ? 1.0 : (double)a->w[e];
    float* h = h_out + (size_t)e * I;
    for (int r = 0; r < I; r++) {
      h[r] = (float)silu_clamped(g[r], u[r], we, a->limit);
      if (hmag) hmag[(size_t)e * I + r] = fabs(we) * (gm[r] + um[r]) * 12 + 1e-6;   /* error scale of :82 */
    }
    orc_matvec(td, a->down[e], D, I, h, 1, 0, 1, yd, ydm, a->threads);
    for (int i = 0; i < D; i++) { y[i] += yd[i]; ymag[i] += ydm[i]; }
  }
  free(g); free(yd);
}

/* ------------------------------------------------------------------ router (tests/ref/arch_ref.cpp:97-131) */
void orc_router(const float* logits, const float* bias, int E, int k, int score_fn, float route_scale, int* ids,
                float* w) {
  double* sc = (double*)malloc(sizeof(double) * (size_t)E * 2);
  double* key = sc + E;
  char* used = (char*)calloc((size_t)E, 1);
  for (int e = 0; e < E; e++) {
    const double x = logits[e];
    if (score_fn == 1) sc[e] = 1.0 / (1.0 + exp(-x));
    else { const double sp = x > 20 ? x : log1p(exp(x)); sc[e] = sqrt(sp); }
    key[e] = (double)(float)((float)sc[e] + (bias ? bias[e] : 0.f));
  }
  /* descending key, stable (ties -> lowest id): k rounds of arg-max with strict > */
  double s = 0;
  for (int j = 0; j < k; j++) {
    int best = -1;
    for (int e = 0; e < E; e++) if (!used[e] && (best < 0 || key[e] > key[best])) best = e;
    used[best] = 1; ids[j] = best; s += sc[best];
  }
  for (int j = 0; j < k; j++) w[j] = (float)(sc[ids[j]] / (s + 1e-20) * route_scale);
  free(sc); free(used);
}
void orc_route_lists(const int* ids, const float* w, int n, int k, int E, uint32_t* counts, uint32_t* offsets,
                     uint32_t* entry, uint32_t* tok, float* lw, uint32_t* slot_of) {
  const int N = n * k;
  memset(counts, 0, sizeof(uint32_t) * (size_t)E);
  for (int i = 0; i < N; i++) counts[ids[i]]++;
  offsets[0] = 0;
  for (int e = 0; e < E; e++) offsets[e + 1] = offsets[e] + counts[e];
  uint32_t* fill = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)E);
  memcpy(fill, offsets, sizeof(uint32_t) * (size_t)E);
  for (int i = 0; i < N; i++) {
    const uint32_t p = fill[ids[i]]++;
    entry[p] = (uint32_t)i; tok[p] = (uint32_t)(i / k); lw[p] = w[i]; slot_of[i] = p;
  }
  free(fill);
}
int orc_argmax(const float* x, int n) {
  int b = 0;
  for (int i = 1; i < n; i++) if (x[i] > x[b]) b = i;
  return b;
}
/* top-k descending, ties -> lower index (tests/ref/arch_ref.cpp:199-206: a partial sort under that order; here k
 * selection passes over the row, the same result) */
void orc_topk_desc(const float* x, int n, int k, float* v, uint32_t* idx) {
  unsigned char* used = (unsigned char*)calloc((size_t)n, 1);
  for (int r = 0; r < k; r++) {
    int b = -1;
    for (int i = 0; i < n; i++)
      if (!used[i] && (b < 0 || x[i] > x[b])) b = i;
    used[b] = 1; idx[r] = (uint32_t)b; v[r] = x[b];
  }
  free(used);
}
/* log(sum exp(scale x)) in double, max subtracted (tests/ref/arch_ref.cpp:208-214) */
double orc_logsumexp(const float* x, int n, double scale) {
  double m = -INFINITY;
  for (int i = 0; i < n; i++) if (x[i] * scale > m) m = x[i] * scale;
  double s = 0;
  for (int i = 0; i < n; i++) s += exp(x[i] * scale - m);
  return m + log(s);
}
/* y = x - logsumexp(x) (tests/ref/arch_ref.cpp:216-219) */
void orc_log_softmax(const float* x, float* y, int n) {
  const double l = orc_logsumexp(x, n, 1.0);
  for (int i = 0; i < n; i++) y[i] = (float)(x[i] - l);
}
/* Gumbel(0,1) noise of element i under the 64-bit seed and the row (src/kernels/arch_sample.metal:15-26,68): two rounds
 * of a 32-bit mixer, 24 bits -> u in (0,1), -log(-log u).  The reference has this on the GPU only; it is restated here
 * so that a test can reproduce WHICH element wins, not only the distribution. */
static uint32_t orc_hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
double orc_gumbel(uint32_t i, uint64_t seed, uint32_t row) {
  const uint32_t s0 = (uint32_t)seed + row * 0x2545F491u, s1 = (uint32_t)(seed >> 32);
  uint32_t x = orc_hash32(i * 0x9E3779B9u ^ s0);
  x = orc_hash32(x ^ (s1 * 0x85EBCA6Bu + 0x632BE5ABu));
  const double u = ((double)(x >> 8) + 0.5) * (1.0 / 16777216.0);
  return -log(-log(u));
}
/* CPU top-p sampler over a top-k list (src/kernels/arch.mm:322-342) */
uint32_t orc_sample_top_p(const float* vals, const uint32_t* ids, int k, float lse, float temperature, float top_p, double u) {
  if (temperature <= 0.0f || k <= 1) return ids[0];
  double pr[64], cum = 0.0, tot = 0.0, acc = 0.0;
  int keep = k;
  for (int i = 0; i < k; i++) {
    pr[i] = exp((double)vals[i] / temperature - (double)lse);
    cum += pr[i];
    if (cum >= top_p) { keep = i + 1; break; }
  }
  for (int i = 0; i < keep; i++) tot += pr[i];
  for (int i = 0; i < keep; i++) {
    acc += pr[i];
    if (u * tot < acc) return ids[i];
  }
  return ids[keep - 1];
}
void orc_rmsnorm(const float* x, const float* w, float* y, int dim, double eps) {
  double ss = 0;
  for (int i = 0; i < dim; i++) ss += (double)x[i] * x[i];
  const double r = 1.0 / sqrt(ss / dim + eps);
  for (int i = 0; i < dim; i++) y[i] = (float)(x[i] * r * (w ? w[i] : 1.0f));
}

/* ------------------------------------------------------------------ rope (tests/ref/attn_ref.cpp:15-56) */
static void rope_freqs(int yarn, float* f /* 32 */) {
  const int dim = 64;
  const double base = yarn ? 160000.0 : 10000.0;
  for (int i = 0; i < dim / 2; i++) f[i] = (float)(1.0 / pow(base, (double)(float)(2 * i) / dim));
  if (yarn) {
    const double factor = 16, orig = 65536, beta_fast = 32, beta_slow = 1;
    const double two_ln_base = 2 * log(base);
    double low = floor(dim * log(orig / (beta_fast * 2 * M_PI)) / two_ln_base);
    double high = ceil(dim * log(orig / (beta_slow * 2 * M_PI)) / two_ln_base);
    if (low < 0) low = 0;
    if (high > dim - 1) high = dim - 1;
    double span = high - low; if (span < 1e-3) span = 1e-3;
    for (int i = 0; i < dim / 2; i++) {
      float ramp = (float)((i - low) / span);
      ramp = ramp < 0.f ? 0.f : (ramp > 1.f ? 1.f : ramp);
      const float smooth = 1.0f - ramp;
      f[i] = f[i] / (float)factor * (1.0f - smooth) + f[i] * smooth;
    }
  }
}
void orc_rope_table(int max_pos, int yarn, float* out) {
  float f[32];
  rope_freqs(yarn, f);
  for (int p = 0; p < max_pos; p++)
    for (int i = 0; i < 32; i++) {
      const float a = (float)p * f[i];
      out[(size_t)p * 64 + 2 * i] = (float)cos((double)a);
      out[(size_t)p * 64 + 2 * i + 1] = (float)sin((double)a);
    }
}
void orc_rope(float* x, const float* cs, int inverse) {
  for (int i = 0; i < 32; i++) {
    const float c = cs[2 * i], s = inverse ? -cs[2 * i + 1] : cs[2 * i + 1];
    const float a = x[2 * i], b = x[2 * i + 1];
    x[2 * i] = a * c - b * s;
    x[2 * i + 1] = a * s + b * c;
  }
}
static void rmsnorm_f(float* x, const float* w, int n, float eps) {           /* attn_ref.cpp:58-63 */
  double ss = 0;
  for (int i = 0; i < n; i++) ss += (double)x[i] * x[i];
  const float r = 1.0f / sqrtf((float)(ss / n) + eps);
  for (int i = 0; i < n; i++) x[i] = w[i] * (x[i] * r);
}

/* ------------------------------------------------------------------ quant sims (tests/ref/attn_ref.cpp:65-107) */
static inline uint32_t fbits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bitsf(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline int floor_log2f(float a) { return (int)((fbits(a) >> 23) & 0xFF) - 127; }
static inline int ceil_log2f(float x) { uint32_t b = fbits(x); return (int)((b >> 23) & 0xFF) - 127 + ((b & 0x7FFFFF) ? 1 : 0); }
static inline float pow2i(int e) { return bitsf((uint32_t)(e + 127) << 23); }
static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }
float orc_round_e4m3(float x) {
  const float a = fabsf(x);
  int e = floor_log2f(a); if (e < -6) e = -6;
  return copysignf(nearbyintf(a * pow2i(3 - e)) * pow2i(e - 3), x);
}
float orc_round_e2m1(float x) {
  const float a = fabsf(x);
  int e = floor_log2f(a); if (e < 0) e = 0;
  return copysignf(nearbyintf(a * pow2i(1 - e)) * pow2i(e - 1), x);
}
void orc_fp8_sim(float* x, int n) {
  for (int b = 0; b < n; b += 32) {
    float amax = 0;
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[b + i]));
    amax = fmaxf(amax, 1e-4f);
    const int e = ceil_log2f(amax * (1.0f / 448.0f));
    const float s = pow2i(e), inv = pow2i(-e);
    for (int i = 0; i < 32; i++) x[b + i] = orc_round_e4m3(clampf(x[b + i] * inv, -448.0f, 448.0f)) * s;
  }
}
void orc_fp4_sim_e8m0(float* x, int n) {
  for (int b = 0; b < n; b += 32) {
    float amax = 0;
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[b + i]));
    amax = fmaxf(amax, 6.0f * 0x1p-126f);
    const int e = ceil_log2f(amax * (1.0f / 6.0f));
    const float s = pow2i(e), inv = pow2i(-e);
    for (int i = 0; i < 32; i++) x[b + i] = orc_round_e2m1(clampf(x[b + i] * inv, -6.0f, 6.0f)) * s;
  }
}
void orc_fp4_sim_e4m3(float* x, int n) {
  for (int b = 0; b < n; b += 16) {
    float amax = 0;
    for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(x[b + i]));
    amax = fmaxf(amax, 6.0f * 0x1p-9f);
    const float s = orc_round_e4m3(fminf(amax / 6.0f, 448.0f));
    for (int i = 0; i < 16; i++) x[b + i] = orc_round_e2m1(clampf(x[b + i] / s, -6.0f, 6.0f)) * s;
  }
}
void orc_window_row(const float* kv_raw, const float* norm_w, const float* cs, int actq, int D, float* out) {
  memcpy(out, kv_raw, sizeof(float) * (size_t)D);
  rmsnorm_f(out, norm_w, D, 1e-20f);
  orc_rope(out + D - 64, cs, 0);
  if (actq) orc_fp8_sim(out, D);
}

/* ------------------------------------------------------------------ indexer (tests/ref/attn_ref.cpp:163-202) */
void orc_index_q(const float* q_raw, const float* w_raw, const float* cs, int actq, int heads, int dim, float* q,
                 float* w) {
  memcpy(q, q_raw, sizeof(float) * (size_t)heads * dim);
  for (int h = 0; h < heads; h++) {
    orc_rope(q + h * dim + dim - 64, cs, 0);
    if (actq) orc_fp4_sim_e8m0(q + h * dim, dim);
  }
  for (int h = 0; h < heads; h++) w[h] = w_raw[h] * (float)(pow((double)dim, -0.5) * pow((double)heads, -0.5));
}
typedef struct { const float *q, *w, *keys; int heads, dim; float* sc; } is_ctx;
static void is_range(void* p, int t0, int t1) {
  is_ctx* c = (is_ctx*)p;
  for (int t = t0; t < t1; t++) {
    const float* k = c->keys + (size_t)t * c->dim;
    double s = 0;
    for (int h = 0; h < c->heads; h++) {
      double d = 0;
      for (int i = 0; i < c->dim; i++) d += (double)c->q[h * c->dim + i] * k[i];
      if (d > 0) s += d * c->w[h];
    }
    c->sc[t] = (float)s;
  }
}
void orc_index_scores(const float* q, const float* w, const float* keys, int heads, int dim, int len, float* sc,
                      int threads) {
  is_ctx c = {q, w, keys, heads, dim, sc};
  orc_parallel(is_range, &c, len, threads);
}

/* top-k: order = (score descending, index ascending) among finite (> -inf) scores; output ascending by index */
typedef struct { float s; int i; } sc_idx;
static int cmp_score_desc(const void* a, const void* b) {
  const sc_idx *x = (const sc_idx*)a, *y = (const sc_idx*)b;
  if (x->s != y->s) return x->s > y->s ? -1 : 1;
  return x->i < y->i ? -1 : (x->i > y->i ? 1 : 0);
}
static int cmp_int(const void* a, const void* b) { int x = *(const int*)a, y = *(const int*)b; return x < y ? -1 : x > y; }
int orc_topk_sorted(const float* sc, int n, int k, int* out) {
  sc_idx* v = (sc_idx*)malloc(sizeof(sc_idx) * (size_t)(n > 0 ? n : 1));
  int m = 0;
  for (int i = 0; i < n; i++) if (sc[i] > -INFINITY) { v[m].s = sc[i]; v[m].i = i; m++; }
  if (m > k) { qsort(v, (size_t)m, sizeof(sc_idx), cmp_score_desc); m = k; }
  for (int i = 0; i < m; i++) out[i] = v[i].i;
  qsort(out, (size_t)m, sizeof(int), cmp_int);
  for (int i = m; i < k; i++) out[i] = -1;
  free(v);
  return m;
}
int orc_candidate_blocks(const float* sc, int len, int bs, int cap, int* out) {
  const int nb = (len + bs - 1) / bs;
  float* b = (float*)malloc(sizeof(float) * (size_t)(nb > 0 ? nb : 1));
  for (int i = 0; i < nb; i++) b[i] = -INFINITY;
  for (int t = 0; t < len; t++) if (sc[t] > b[t / bs]) b[t / bs] = sc[t];
  if (len > 0) b[(len - 1) / bs] = INFINITY;
  const int m = orc_topk_sorted(b, nb, cap, out);
  free(b);
  return m;
}

/* ------------------------------------------------------------------ sparse attention (tests/ref/attn_ref.cpp:204-230) */
typedef struct { const float *q_raw, *cs, *rows, *sinks; int n_rows, D; float* out; } sa_ctx;
static void sa_heads(void* p, int h0, int h1) {
  sa_ctx* c = (sa_ctx*)p;
  const int D = c->D, R = c->n_rows;
  const double scale = 1.0 / sqrt((double)D);
  double* s = (double*)malloc(sizeof(double) * (size_t)(R + D + 1));
  double* o = s + R;
  float* q = (float*)malloc(sizeof(float) * (size_t)D);
  for (int h = h0; h < h1; h++) {
    memcpy(q, c->q_raw + (size_t)h * D, sizeof(float) * (size_t)D);
    orc_rope(q + D - 64, c->cs, 0);
    double m = c->sinks[h];
    for (int r = 0; r < R; r++) {
      const float* row = c->rows + (size_t)r * D;
      double d = 0;
      for (int i = 0; i < D; i++) d += (double)q[i] * row[i];
      s[r] = d * scale;
      if (s[r] > m) m = s[r];
    }
    double den = exp((double)c->sinks[h] - m);
    for (int i = 0; i < D; i++) o[i] = 0;
    for (int r = 0; r < R; r++) {
      const float* row = c->rows + (size_t)r * D;
      const double pr = exp(s[r] - m);
      den += pr;
      for (int i = 0; i < D; i++) o[i] += pr * row[i];
    }
    float* y = c->out + (size_t)h * D;
    for (int i = 0; i < D; i++) y[i] = (float)(o[i] / den);
    orc_rope(y + D - 64, c->cs, 1);
  }
  free(s); free(q);
}
void orc_sparse_attn(const float* q_raw, const float* cs, const float* rows, int n_rows, const float* sinks, int H,
                     int D, float* out, int threads) {
  sa_ctx c = {q_raw, cs, rows, sinks, n_rows, D, out};
  orc_parallel(sa_heads, &c, H, threads);
}

/* ---------------------------------------------------------------- hyper-connections (tests/ref/arch_ref.cpp:22-95)
 * D = width of one residual stream, 4 streams; mix[24] = pre[4], post[4], comb[4][4] (comb[j][k] at 8 + 4 j + k). */
static double sigmoid_d(double x) { return 1.0 / (1.0 + exp(-x)); }

void orc_hc_split(const double* m, const float* scale, const float* base, float* mix, int iters, double eps) { /* :22-50 */
  double c[4][4];
  for (int j = 0; j < 4; j++) mix[j] = (float)(sigmoid_d(m[j] * scale[0] + base[j]) + eps);
  for (int j = 0; j < 4; j++) mix[4 + j] = (float)(2.0 * sigmoid_d(m[4 + j] * scale[1] + base[4 + j]));
  for (int j = 0; j < 4; j++)
    for (int k = 0; k < 4; k++) c[j][k] = m[8 + 4 * j + k] * scale[2] + base[8 + 4 * j + k];
  for (int j = 0; j < 4; j++) { /* row softmax + eps */
    double mx = c[j][0], s = 0;
    for (int k = 1; k < 4; k++) if (c[j][k] > mx) mx = c[j][k];
    for (int k = 0; k < 4; k++) { c[j][k] = exp(c[j][k] - mx); s += c[j][k]; }
    for (int k = 0; k < 4; k++) c[j][k] = c[j][k] / s + eps;
  }
  for (int it = 0; it < iters; it++) {
    if (it > 0)
      for (int j = 0; j < 4; j++) { /* row normalisation */
        double s = c[j][0] + c[j][1] + c[j][2] + c[j][3];
        for (int k = 0; k < 4; k++) c[j][k] /= (s + eps);
      }
    for (int k = 0; k < 4; k++) { /* column normalisation */
      double s = c[0][k] + c[1][k] + c[2][k] + c[3][k];
      for (int j = 0; j < 4; j++) c[j][k] /= (s + eps);
    }
  }
  for (int j = 0; j < 4; j++)
    for (int k = 0; k < 4; k++) mix[8 + 4 * j + k] = (float)c[j][k];
}

void orc_hc_mixes(const float* h, const float* fn, const float* scale, const float* base, int D, float* mix, int iters,
                  double norm_eps, double hc_eps) { /* :52-66 */
  const int HCD = 4 * D;
  double ss = 0, m[24];
  for (int i = 0; i < HCD; i++) ss += (double)h[i] * h[i];
  const double rstd = 1.0 / sqrt(ss / HCD + norm_eps);
  for (int r = 0; r < 24; r++) {
    double a = 0;
    const float* f = fn + (size_t)r * HCD;
    for (int i = 0; i < HCD; i++) a += (double)f[i] * h[i];
    m[r] = a * rstd;
  }
  orc_hc_split(m, scale, base, mix, iters, hc_eps);
}

/* One sublayer boundary (:75-95).  x_sub / fn / x_out may be NULL as in the reference; h_out is written only with x_sub. */
void orc_hc_step(const float* h_in, const float* x_sub, const float* mix_prev, const float* fn, const float* scale,
                 const float* base, const float* norm_w, int D, float* h_out, float* mix_out, float* x_out) {
  const int HCD = 4 * D;
  float* hn = (float*)malloc(sizeof(float) * HCD);
  memcpy(hn, h_in, sizeof(float) * HCD);
  if (x_sub) {
    for (int d = 0; d < D; d++)
      for (int i = 0; i < 4; i++) {
        double a = (double)mix_prev[4 + i] * x_sub[d];
        for (int j = 0; j < 4; j++) a += (double)mix_prev[8 + 4 * j + i] * h_in[j * D + d];
        hn[i * D + d] = (float)a;
      }
    memcpy(h_out, hn, sizeof(float) * HCD);
  }
  if (fn) orc_hc_mixes(hn, fn, scale, base, D, mix_out, 20, 1e-20, 1e-6);
  if (x_out) {
    float* xp = (float*)malloc(sizeof(float) * D);
    for (int d = 0; d < D; d++) {
      double a = 0;
      for (int j = 0; j < 4; j++) a += (double)mix_prev[j] * hn[j * D + d];
      xp[d] = (float)a;
    }
    orc_rmsnorm(xp, norm_w, x_out, D, 1e-20);
    free(xp);
  }
  free(hn);
}

/* ---------------------------------------------------------------- compressor + index key (tests/ref/attn_ref.cpp:116-161)
 * One token at position p for a KV source of ratio r (1 or 2): st_kv / st_sc are the source's partial group
 * [r][D] (st_sc starts at -inf).  Returns 1 when a row was emitted: ckv_row[D] (roped, fp4 e4m3/16 when actq) and
 * ikey_row[ID] (roped, fp4 e8m0/32 when actq); cs_tab is the YaRN rope table [max_pos][32][2].  The rope dims are the
 * last 64 of each vector. */
int orc_compress_token(int ratio, int p, const float* ckv_in, const float* cgate_in, const float* cnorm_w,
                       const uint16_t* wk_bf16, const float* knorm_w, const float* cs_tab, int actq, int D, int ID,
                       float* st_kv, float* st_sc, float* ckv_row, float* ikey_row) {
  const int r = ratio;
  float* lat = ckv_row;
  if (r == 1) {
    memcpy(lat, ckv_in, sizeof(float) * D);
  } else {
    const int slot = p % r;
    memcpy(st_kv + (size_t)slot * D, ckv_in, sizeof(float) * D);
    memcpy(st_sc + (size_t)slot * D, cgate_in, sizeof(float) * D);
    if ((p + 1) % r != 0) return 0;
    for (int c = 0; c < D; c++) {
      float m = -INFINITY, e[8], sum = 0, v = 0;
      for (int j = 0; j < r; j++) m = fmaxf(m, st_sc[(size_t)j * D + c]);
      for (int j = 0; j < r; j++) { e[j] = expf(st_sc[(size_t)j * D + c] - m); sum += e[j]; }
      for (int j = 0; j < r; j++) v += st_kv[(size_t)j * D + c] * (e[j] / sum);
      lat[c] = v;
    }
  }
  rmsnorm_f(lat, cnorm_w, D, 1e-20f);
  const int row = p / r;
  const float* cs = cs_tab + (size_t)row * r * 64;
  for (int o = 0; o < ID; o++) { /* index key from the pre-rope latent */
    double acc = 0;
    for (int d = 0; d < D; d++) acc += (double)orc_bf16_to_f32(wk_bf16[(size_t)o * D + d]) * lat[d];
    ikey_row[o] = (float)acc;
  }
  rmsnorm_f(ikey_row, knorm_w, ID, 1e-20f);
  orc_rope(ikey_row + ID - 64, cs, 0);
  if (actq) orc_fp4_sim_e8m0(ikey_row, ID);
  orc_rope(lat + D - 64, cs, 0);
  if (actq) orc_fp4_sim_e4m3(lat, D);
  return 1;
}
