// extern "C" surface of libmacseek_b200 (declared in include/macseek_b200.h).
#include <vector>
#include <algorithm>
#include "msb_common.cuh"
#include "../../include/macseek_b200.h"

namespace msb {
const char* last_error_text();
int dequant(int t, const void* src, int64_t n, float* out, cudaStream_t st);
int matvec_n(int t, const void* W, int rows, int cols, const float* X, int64_t x_stride, float* Y, int64_t y_stride,
             int n, int accumulate, int groups, const float* norm_w, float norm_eps, cudaStream_t st, bool share = false);
int index_scores_tc(const void* keys, int len, const float* q, const float* w, int heads, float* scores, unsigned* hist,
                    int prep, const float* cs, int actq, float* q_out, float* w_out, const int* cand, int n_cand,
                    cudaStream_t st);
int f32_to_f16(const float* x, void* x16, size_t count, cudaStream_t st);
size_t matmul_scratch_bytes(int t, int rows, int cols, int n, bool with_x);
int matmul_h(int t, const void* W, int rows, int cols, const void* X16, int x_stride, float* Y, int n, bool accumulate,
             void* scratch, size_t scratch_bytes, cudaStream_t st);
int matmul(int t, const void* W, int rows, int cols, const float* X, float* Y, int n, bool accumulate, void* scratch,
           size_t scratch_bytes, cudaStream_t st);
struct MoePrefillArgs {
  int dim, inter, t_gate_up, t_down, t_shared, n_tokens, n_exp;
  const uint64_t* slot_ptrs;
  const int* offs;
  const int* tok;
  const float* wt;
  const int* slot_of;
  int k_per_token, has_shared;
  uint64_t shared_ptrs[3];
  const float* X;
  float* Y;
  void* scratch;
  size_t scratch_bytes;
  float limit;
};
size_t moe_prefill_scratch_bytes(int total, int n_tokens, int n_exp, int dim, int inter);
int moe_prefill(const MoePrefillArgs& a, cudaStream_t st);
size_t router_scratch_bytes(int E);
int router_fused(const float* x, const float* norm_w, float norm_eps, float* x_out, const float* W, const float* bias,
                 int* ids, float* wts, void* scratch, size_t scratch_bytes, int E, int dim, int k, int score_fn,
                 float route_scale, cudaStream_t st);
int router_topk(const float* logits, const float* bias, int* ids, float* wts, int n, int E, int k, int score_fn,
                float route_scale, cudaStream_t st);
int route_lists(const int* ids, const float* w, int n, int k, int E, unsigned* counts, unsigned* offsets,
                unsigned* entry, unsigned* tok, float* lw, unsigned* slot_of, cudaStream_t st);
size_t topk_scratch_bytes(int n_max);
int topk(const float* sc, int n, int k, int* out, void* scratch, size_t scratch_bytes, bool hist_ready, const int* pos_map,
         cudaStream_t st);
int index_prep(const float* q_raw, const float* w_raw, const float* cs, int actq, int heads, float* q, float* w,
               cudaStream_t st);
int index_scores(int key_type, const void* keys, int len, const float* q, const float* w, int heads, float* scores,
                 unsigned* hist, int exact_query, cudaStream_t st);
int block_max(const float* sc, int len, int bs, float* out, cudaStream_t st);
int index_scores_list_f16(const void* keys, int len, const float* q, const float* w, int heads, const int* cand, int n_cand,
                          float* scores, cudaStream_t st);
int device_alloc(size_t bytes, void** out);
int device_free(void* p);
int copy_to_device(void* dst, const void* src, size_t bytes, cudaStream_t st);
int copy_to_host(void* dst, const void* src, size_t bytes, cudaStream_t st);
int fill_f32(float* p, float v, size_t n, cudaStream_t st);
int copy_device(void* dst, const void* src, size_t bytes, cudaStream_t st);
size_t sample_scratch_bytes(int rows);
int argmax_rows(const float* logits, int rows, int V, int* out_idx, float* out_val, float temperature, uint64_t seed,
                void* scratch, size_t scratch_bytes, cudaStream_t st);
int sample_topk(const float* logits, int rows, int V, int k, float temperature, float* out_v, int* out_i, float* out_lse,
                void* scratch, size_t scratch_bytes, cudaStream_t st);
int log_softmax(const float* in, float* out, int rows, int V, cudaStream_t st);
int sample_top_p(const float* vals, const int* ids, int k, float lse, float temperature, float top_p, double u);
size_t hc_scratch_bytes(int n);
int hc_step(const float* h_in, float* h_out, const float* x_sub, const float* mix_prev, const float* fn, const float* scale,
            const float* base, float* mix_out, const float* norm_w, float* x_out, int D, int n, void* scratch,
            size_t scratch_bytes, cudaStream_t st);
int compress_token(const float* c_kv, const float* c_gate, const float* c_norm, const void* wk_bf16, const float* k_norm,
                   const float* cs, float* state, int ratio, int pos, int actq, int D, int ID, int elem_type, void* ckv_rows,
                   int key_type, void* ikey_rows, cudaStream_t st);
size_t sparse_scratch_bytes(int total_rows_max, int H, int D);
int sparse_decode(const float* q, const float* cs, const float* sinks, int elem_type, const void* win, int n_win,
                  const void* cache, const int* topk, int k, int H, int D, float* out, void* scratch,
                  size_t scratch_bytes, cudaStream_t st);
int rmsnorm(const float* x, const float* w, float* y, int rows, int dim, float eps, int in_stride, int out_stride,
            cudaStream_t st);
int kv_window(const float* kv, const float* norm_w, const float* cs, int actq, int D, int elem_type, void* out_row,
              cudaStream_t st);
int argmax(const float* x, int n, int* out_idx, float* out_val, cudaStream_t st);
int vec_add(float* y, const float* a, int n, cudaStream_t st);
int ep_combine(uint8_t* const* base, int world, int rank, float* h, int dim, cudaStream_t st);
void set_peer_wait_cycles(long long c);
int ep_alloc(size_t bytes, void** out);
int ep_free(void* p);
int ipc_export(void* p, unsigned char* handle64);
int ipc_import(const unsigned char* handle64, void** out);
int ipc_release(void* p);
}  // namespace msb
#include "moe_decode_params.cuh"

using namespace msb;

extern "C" {

const char* msb_last_error(void) { return last_error_text(); }
const char* msb_version(void) { return "macseek_b200 sm_100a"; }

int msb_init(void) {
  Tables t;
  return get_tables(&t);
}

int msb_device_status(void) {
  Tables t;
  int rc = get_tables(&t);
  if (rc) return rc;
  MSB_CUDA(cudaDeviceSynchronize());
  int v = 0;
  MSB_CUDA(cudaMemcpy(&v, t.status, sizeof v, cudaMemcpyDeviceToHost));
  // A kernel that gave up a wait returned early: the library's scheduling counters and tickets that follow the status
  // word may be left non-zero.  Nothing is in flight after the synchronise above, so the whole buffer is reset.
  if (v) MSB_CUDA(cudaMemset(t.status, 0, 2048));
  return v;
}

int msb_block_elems(int qtype) { return type_known(qtype) ? block_elems(qtype) : 0; }
size_t msb_block_bytes(int qtype) { return (size_t)block_bytes(qtype); }
size_t msb_row_bytes(int qtype, int64_t cols) { return type_known(qtype) ? row_bytes(qtype, cols) : 0; }

int msb_dequant(int qtype, const void* blocks, int64_t n, float* out, void* stream) {
  return dequant(qtype, blocks, n, out, (cudaStream_t)stream);
}

int msb_matvec(int qtype, const void* W, int rows, int cols, const float* x, float* y, int accumulate, int groups,
               void* stream) {
  return matvec_n(qtype, W, rows, cols, x, (int64_t)cols * groups, y, rows, 1, accumulate, groups, nullptr, 0.f,
                  (cudaStream_t)stream);
}

int msb_matvec_rmsnorm(int qtype, const void* W, int rows, int cols, const float* x, const float* norm_w, float eps,
                       float* y, void* stream) {
  if (!norm_w) return fail(kErrArg, "matvec_rmsnorm: null norm_w");
  return matvec_n(qtype, W, rows, cols, x, cols, y, rows, 1, 0, 1, norm_w, eps, (cudaStream_t)stream);
}

int msb_matvec_rmsnorm_shared(int qtype, const void* W, int rows, int cols, const float* x, const float* norm_w, float eps,
                              float* y, void* stream) {
  if (!norm_w) return fail(kErrArg, "matvec_rmsnorm_shared: null norm_w");
  return matvec_n(qtype, W, rows, cols, x, cols, y, rows, 1, 0, 1, norm_w, eps, (cudaStream_t)stream, true);
}

int msb_matvec_n(int qtype, const void* W, int rows, int cols, const float* X, float* Y, int n, int accumulate,
                 int groups, void* stream) {
  if (n < 1 || n > 16) return fail(kErrArg, "matvec_n: n = %d outside 1..16", n);
  return matvec_n(qtype, W, rows, cols, X, (int64_t)cols * groups, Y, rows, n, accumulate, groups, nullptr, 0.f,
                  (cudaStream_t)stream);
}

static int moe_fill(const msb_moe_decode_args* a, MoeParams* p) {
  if (!a) return fail(kErrArg, "moe_decode: null args");
  if (a->n_routed < 0 || a->n_routed > kMaxRouted) return fail(kErrArg, "moe_decode: n_routed %d outside 0..%d", a->n_routed, kMaxRouted);
  *p = MoeParams{};
  p->dim = a->dim; p->inter = a->inter; p->n_routed = a->n_routed; p->has_shared = a->has_shared;
  for (int i = 0; i < a->n_routed; i++) {
    p->gate[i] = (const uint8_t*)a->slot[i].gate; p->up[i] = (const uint8_t*)a->slot[i].up;
    p->down[i] = (const uint8_t*)a->slot[i].down;
  }
  p->sgate = (const uint8_t*)a->shared.gate; p->sup = (const uint8_t*)a->shared.up; p->sdown = (const uint8_t*)a->shared.down;
  p->weights = a->weights; p->x = a->x; p->y = a->y; p->h = (float*)a->scratch;
  p->limit = a->swiglu_limit > 0.f ? a->swiglu_limit : 10.f;
  if (reinterpret_cast<uintptr_t>(a->scratch) & 15 || reinterpret_cast<uintptr_t>(a->x) & 15)
    return fail(kErrArg, "moe_decode: x and scratch must be 16-byte aligned");
  return kOk;
}

int msb_f32_to_f16(const float* x, void* x16, size_t count, void* stream) { return f32_to_f16(x, x16, count, (cudaStream_t)stream); }
size_t msb_matmul_scratch_bytes(int qtype, int rows, int cols, int n, int with_x) {
  return matmul_scratch_bytes(qtype, rows, cols, n, with_x != 0);
}
int msb_matmul_h(int qtype, const void* W, int rows, int cols, const void* X16, int x_stride, float* Y, int n, int accumulate,
                 void* scratch, size_t scratch_bytes, void* stream) {
  return matmul_h(qtype, W, rows, cols, X16, x_stride, Y, n, accumulate != 0, scratch, scratch_bytes, (cudaStream_t)stream);
}
int msb_matmul(int qtype, const void* W, int rows, int cols, const float* X, float* Y, int n, int accumulate, void* scratch,
               size_t scratch_bytes, void* stream) {
  return matmul(qtype, W, rows, cols, X, Y, n, accumulate != 0, scratch, scratch_bytes, (cudaStream_t)stream);
}

size_t msb_moe_decode_scratch_bytes(int inter, int max_routed) { return moe_decode_scratch_bytes(inter, max_routed); }

int msb_moe_decode(const msb_moe_decode_args* a, void* stream) {
  MoeParams p;
  int rc = moe_fill(a, &p);
  if (rc) return rc;
  for (int i = 0; i < a->n_routed; i++)
    if (!p.gate[i] || !p.up[i] || !p.down[i]) return fail(kErrArg, "moe_decode: null expert matrix in slot %d", i);
  return moe_decode(p, a->t_gate_up, a->t_down, a->t_shared, MSB_MOE_ALL, a->scratch_bytes, (cudaStream_t)stream);
}

int msb_moe_decode_table_part(const msb_moe_decode_args* a, const uint64_t* table, int part, void* stream) {
  MoeParams p;
  int rc = moe_fill(a, &p);
  if (rc) return rc;
  if (!table) return fail(kErrArg, "moe_decode_table: null table");
  p.table = table; p.ids = nullptr; p.expert_lo = 0; p.expert_hi = 0x7fffffff;
  return moe_decode(p, a->t_gate_up, a->t_down, a->t_shared, part, a->scratch_bytes, (cudaStream_t)stream);
}

int msb_moe_decode_ids(const msb_moe_decode_args* a, const uint64_t* expert_table, const int* ids, int expert_lo,
                       int expert_hi, int part, void* stream) {
  MoeParams p;
  int rc = moe_fill(a, &p);
  if (rc) return rc;
  if (!expert_table || !ids) return fail(kErrArg, "moe_decode_ids: null table or ids");
  p.table = expert_table; p.ids = ids; p.expert_lo = expert_lo; p.expert_hi = expert_hi;
  return moe_decode(p, a->t_gate_up, a->t_down, a->t_shared, part, a->scratch_bytes, (cudaStream_t)stream);
}

int msb_moe_decode_ids_normed(const msb_moe_decode_args* a, const uint64_t* expert_table, const int* ids, int expert_lo,
                              int expert_hi, int part, const float* norm_in, const float* norm_w, float norm_eps,
                              void* stream) {
  if (!a) return fail(kErrArg, "moe_decode_ids_normed: null args");
  msb_moe_decode_args b = *a;
  if (norm_in) b.x = norm_in;     // only for the shared argument checks: the launch reads norm_in, never a.x
  MoeParams p;
  int rc = moe_fill(&b, &p);
  if (rc) return rc;
  if (!expert_table || !ids) return fail(kErrArg, "moe_decode_ids_normed: null table or ids");
  p.table = expert_table; p.ids = ids; p.expert_lo = expert_lo; p.expert_hi = expert_hi;
  if (norm_in) { p.x = nullptr; p.norm_in = norm_in; p.norm_w = norm_w; p.norm_eps = norm_eps; }
  return moe_decode(p, a->t_gate_up, a->t_down, a->t_shared, part, a->scratch_bytes, (cudaStream_t)stream);
}

// ---- msb_moe_decode with library-resident scratch: no allocation of any kind on this path.
// The scratch (the h rows of every routed slot + the shared expert) lives in a file-scope device array; its address is
// looked up once per device with cudaGetSymbolAddress and handed to the kernels like a caller's buffer.
int msb_moe_decode_noalloc(const msb_moe_decode_args* a, void* stream) {
  if (!a) return fail(kErrArg, "moe_decode_noalloc: null args");
  static_assert(kNoAllocFloats == (kMaxRouted + 1) * kNoAllocMaxInter, "scratch sized for kMaxRouted routed + the shared expert");
  if (a->inter > kNoAllocMaxInter || a->n_routed > kMaxRouted)
    return fail(kErrLimit, "moe_decode_noalloc: inter %d / n_routed %d beyond the built-in scratch (inter <= %d, n_routed <= %d)",
                a->inter, a->n_routed, kNoAllocMaxInter, kMaxRouted);
  size_t bytes = 0;
  float* scratch = noalloc_scratch(&bytes);      // cached by msb_init(); nothing is looked up or created here
  if (!scratch)
    return fail(kErrDevice, "moe_decode_noalloc: msb_init() has not run on this device (this entry point creates nothing)");
  msb_moe_decode_args b = *a;
  b.scratch = scratch;
  b.scratch_bytes = bytes;
  return msb_moe_decode(&b, stream);
}

static int ep_fill(const msb_ep_comm* comm, MoeParams* p) {
  if (!comm) return kOk;
  if (comm->world < 1 || comm->world > kMaxEpWorld || comm->rank < 0 || comm->rank >= comm->world)
    return fail(kErrArg, "moe_decode_ep: bad world %d / rank %d", comm->world, comm->rank);
  p->ep_world = comm->world; p->ep_rank = comm->rank;
  for (int r = 0; r < comm->world; r++) p->ep_base[r] = (uint8_t*)comm->base[r];
  return kOk;
}

int msb_moe_decode_ep(const msb_moe_decode_args* a, const uint64_t* expert_table, const int* ids, int expert_lo,
                      int expert_hi, const float* norm_in, const float* norm_w, float norm_eps, int shared_lo,
                      int shared_hi, const msb_ep_comm* comm, void* stream) {
  if (!a) return fail(kErrArg, "moe_decode_ep: null args");
  msb_moe_decode_args b = *a;
  if (norm_in) b.x = norm_in;
  MoeParams p;
  int rc = moe_fill(&b, &p);
  if (rc) return rc;
  if (!expert_table || !ids) return fail(kErrArg, "moe_decode_ep: null table or ids");
  p.table = expert_table; p.ids = ids; p.expert_lo = expert_lo; p.expert_hi = expert_hi;
  if (norm_in) { p.x = nullptr; p.norm_in = norm_in; p.norm_w = norm_w; p.norm_eps = norm_eps; }
  p.s_lo = shared_lo; p.s_hi = shared_hi;
  if (a->has_shared && shared_lo == shared_hi) p.has_shared = 0;      // an empty slice
  rc = ep_fill(comm, &p);
  if (rc) return rc;
  return moe_decode(p, a->t_gate_up, a->t_down, a->t_shared, MSB_MOE_ALL, a->scratch_bytes, (cudaStream_t)stream);
}

size_t msb_ep_exchange_bytes(int dim, int world) { return ep_exchange_bytes(dim, world); }
int msb_ep_combine(const msb_ep_comm* comm, float* h, int dim, void* stream) {
  if (!comm) return fail(kErrArg, "ep_combine: null comm");
  return ep_combine((uint8_t* const*)comm->base, comm->world, comm->rank, h, dim, (cudaStream_t)stream);
}
void msb_set_peer_wait_cycles(long long cycles) { set_peer_wait_cycles(cycles); }
int msb_ep_alloc(size_t bytes, void** out) { return ep_alloc(bytes, out); }
int msb_ep_free(void* p) { return ep_free(p); }
int msb_ipc_export(void* p, unsigned char* handle64) { return ipc_export(p, handle64); }
int msb_ipc_import(const unsigned char* handle64, void** out) { return ipc_import(handle64, out); }
int msb_ipc_release(void* p) { return ipc_release(p); }

size_t msb_moe_prefill_scratch_bytes(int total_entries, int n_tokens, int n_exp, int dim, int inter) {
  return moe_prefill_scratch_bytes(total_entries, n_tokens, n_exp, dim, inter);
}
int msb_moe_prefill(const msb_moe_prefill_args* a, void* stream) {
  if (!a) return fail(kErrArg, "moe_prefill: null args");
  if (a->n_exp < 0 || (a->n_exp > 0 && !a->slots)) return fail(kErrArg, "moe_prefill: bad expert list");
  std::vector<uint64_t> ptrs((size_t)std::max(a->n_exp, 1) * 3, 0);
  for (int j = 0; j < a->n_exp; j++) {
    ptrs[(size_t)j * 3] = (uint64_t)(uintptr_t)a->slots[j].gate;
    ptrs[(size_t)j * 3 + 1] = (uint64_t)(uintptr_t)a->slots[j].up;
    ptrs[(size_t)j * 3 + 2] = (uint64_t)(uintptr_t)a->slots[j].down;
  }
  MoePrefillArgs m;
  m.dim = a->dim; m.inter = a->inter; m.t_gate_up = a->t_gate_up; m.t_down = a->t_down; m.t_shared = a->t_shared;
  m.n_tokens = a->n_tokens; m.n_exp = a->n_exp; m.slot_ptrs = ptrs.data(); m.offs = a->offs; m.tok = a->tok; m.wt = a->wt;
  m.slot_of = a->slot_of; m.k_per_token = a->k_per_token; m.has_shared = a->has_shared;
  m.shared_ptrs[0] = (uint64_t)(uintptr_t)a->shared.gate; m.shared_ptrs[1] = (uint64_t)(uintptr_t)a->shared.up;
  m.shared_ptrs[2] = (uint64_t)(uintptr_t)a->shared.down;
  m.X = a->X; m.Y = a->Y; m.scratch = a->scratch; m.scratch_bytes = a->scratch_bytes; m.limit = a->swiglu_limit;
  return moe_prefill(m, (cudaStream_t)stream);
}

size_t msb_router_scratch_bytes(int n_experts) { return router_scratch_bytes(n_experts); }
int msb_router_fused(const float* x, const float* W, const float* bias, int* ids, float* w, void* scratch,
                     size_t scratch_bytes, int n_experts, int dim, int k, int score_fn, float route_scale, void* stream) {
  return router_fused(x, nullptr, 0.f, nullptr, W, bias, ids, w, scratch, scratch_bytes, n_experts, dim, k, score_fn,
                      route_scale, (cudaStream_t)stream);
}
int msb_router_fused_rmsnorm(const float* h, const float* norm_w, float eps, float* x_out, const float* W, const float* bias,
                             int* ids, float* w, void* scratch, size_t scratch_bytes, int n_experts, int dim, int k,
                             int score_fn, float route_scale, void* stream) {
  if (!norm_w) return fail(kErrArg, "router_fused_rmsnorm: null norm weights");
  return router_fused(h, norm_w, eps, x_out, W, bias, ids, w, scratch, scratch_bytes, n_experts, dim, k, score_fn,
                      route_scale, (cudaStream_t)stream);
}
int msb_router_topk(const float* logits, const float* bias, int* ids, float* w, int n_tokens, int n_experts, int k,
                    int score_fn, float route_scale, void* stream) {
  return router_topk(logits, bias, ids, w, n_tokens, n_experts, k, score_fn, route_scale, (cudaStream_t)stream);
}
int msb_route_lists(const int* ids, const float* w, int n_tokens, int k, int n_experts, uint32_t* counts,
                    uint32_t* offsets, uint32_t* entry, uint32_t* tok, float* lw, uint32_t* slot_of, void* stream) {
  return route_lists(ids, w, n_tokens, k, n_experts, counts, offsets, entry, tok, lw, slot_of, (cudaStream_t)stream);
}

int msb_index_prep(const float* q_raw, const float* w_raw, const float* cs, int actq, int heads, float* q, float* w,
                   void* stream) {
  return index_prep(q_raw, w_raw, cs, actq, heads, q, w, (cudaStream_t)stream);
}
int msb_index_scores(int key_type, const void* keys, int len, const float* q, const float* w, int heads, float* scores,
                     void* topk_scratch, int exact_query, void* stream) {
  return index_scores(key_type, keys, len, q, w, heads, scores, (unsigned*)topk_scratch, exact_query, (cudaStream_t)stream);
}
size_t msb_topk_scratch_bytes(int n_max) { return topk_scratch_bytes(n_max); }
int msb_topk(const float* scores, int n, int k, int* out, void* scratch, size_t scratch_bytes, int hist_ready,
             void* stream) {
  return topk(scores, n, k, out, scratch, scratch_bytes, hist_ready != 0, nullptr, (cudaStream_t)stream);
}
int msb_block_max(const float* scores, int len, int bs, float* out, void* stream) {
  return block_max(scores, len, bs, out, (cudaStream_t)stream);
}
int msb_index_decode(int key_type, const void* keys, int len, const float* q_raw, const float* w_raw, const float* cs,
                     int actq, int heads, int k, float* q_prep, float* w_prep, float* scores, int* topk_out,
                     void* topk_scratch, size_t topk_scratch_bytes_, int exact_query, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  // the fused histogram exists on the direct FP8 path only
  const bool fused = key_type == MSB_KEY_FP8_E4M3 && !exact_query && len > 0;
  static const bool legacy = getenv("MSB_IDX_LEGACY") && atoi(getenv("MSB_IDX_LEGACY")) != 0;
  int rc;
  if (fused && !legacy && (heads == 32 || heads == 64)) {
    // tcgen05 path: the query preparation runs inside the scoring kernel (q_prep / w_prep are still written)
    if (!keys || !q_raw || !w_raw || !cs || !q_prep || !w_prep || !scores || (reinterpret_cast<uintptr_t>(keys) & 15))
      return fail(kErrArg, "index_decode: null or misaligned pointer");
    rc = index_scores_tc(keys, len, q_raw, w_raw, heads, scores, (unsigned*)topk_scratch, 1, cs, actq, q_prep, w_prep, nullptr, 0, st);
  } else {
    rc = index_prep(q_raw, w_raw, cs, actq, heads, q_prep, w_prep, st);
    if (rc) return rc;
    rc = index_scores(key_type, keys, len, q_prep, w_prep, heads, scores, fused ? (unsigned*)topk_scratch : nullptr,
                      exact_query, st);
  }
  if (rc) return rc;
  return topk(scores, len, k, topk_out, topk_scratch, topk_scratch_bytes_, fused, nullptr, st);
}
int msb_index_decode_list(int key_type, const void* keys, int len, const float* q_raw, const float* w_raw, const float* cs,
                          int actq, int heads, int k, const int* cand_list, int n_cand, float* q_prep, float* w_prep,
                          float* scores, int* topk_out, void* topk_scratch, size_t topk_scratch_bytes_, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (key_type != MSB_KEY_FP8_E4M3 && key_type != MSB_F16) return fail(kErrType, "index_decode_list: F16 or FP8 keys (key type %d)", key_type);
  if (heads != 32 && heads != 64) return fail(kErrArg, "index_decode_list: heads must be 32 or 64 (got %d)", heads);
  if (len < 0 || n_cand < 0) return fail(kErrArg, "index_decode_list: bad sizes");
  if (!keys || !q_raw || !w_raw || !cs || !q_prep || !w_prep || !scores || !topk_out || !topk_scratch ||
      (n_cand > 0 && !cand_list) || (reinterpret_cast<uintptr_t>(keys) & 15))
    return fail(kErrArg, "index_decode_list: null or misaligned pointer");
  const int nvirt = n_cand * 8;
  if (nvirt > 0 && len > 0 && key_type == MSB_F16) {
    // F16 keys (the reference's cache layout): prepared query, one warp per candidate key, then the exact top-k
    int rc = index_prep(q_raw, w_raw, cs, actq, heads, q_prep, w_prep, st);
    if (rc) return rc;
    rc = index_scores_list_f16(keys, len, q_prep, w_prep, heads, cand_list, n_cand, scores, st);
    if (rc) return rc;
    return topk(scores, nvirt, k, topk_out, topk_scratch, topk_scratch_bytes_, false, cand_list, st);
  }
  if (nvirt > 0 && len > 0) {
    int rc = index_scores_tc(keys, len, q_raw, w_raw, heads, scores, (unsigned*)topk_scratch, 1, cs, actq, q_prep, w_prep,
                             cand_list, n_cand, st);
    if (rc) return rc;
    return topk(scores, nvirt, k, topk_out, topk_scratch, topk_scratch_bytes_, true, cand_list, st);
  }
  return topk(scores, 0, k, topk_out, topk_scratch, topk_scratch_bytes_, false, nullptr, st);
}
size_t msb_sparse_scratch_bytes(int total_rows_max, int heads, int D) { return sparse_scratch_bytes(total_rows_max, heads, D); }
int msb_sparse_decode(const float* q, const float* cs, const float* sinks, int elem_type, const void* win, int n_win,
                      const void* cache, const int* topk_list, int k, int heads, int D, float* out, void* scratch,
                      size_t scratch_bytes, void* stream) {
  return sparse_decode(q, cs, sinks, elem_type, win, n_win, cache, topk_list, k, heads, D, out, scratch, scratch_bytes,
                       (cudaStream_t)stream);
}

int msb_rmsnorm(const float* x, const float* w, float* y, int rows, int dim, float eps, int in_stride, int out_stride,
                void* stream) {
  return rmsnorm(x, w, y, rows, dim, eps, in_stride, out_stride, (cudaStream_t)stream);
}
int msb_kv_window(const float* kv, const float* norm_w, const float* cs, int actq, int D, int elem_type, void* out_row,
                  void* stream) {
  return kv_window(kv, norm_w, cs, actq, D, elem_type, out_row, (cudaStream_t)stream);
}
int msb_argmax(const float* x, int n, int* out_idx, float* out_val, void* stream) {
  return argmax(x, n, out_idx, out_val, (cudaStream_t)stream);
}
int msb_add(float* y, const float* a, int n, void* stream) { return vec_add(y, a, n, (cudaStream_t)stream); }

int msb_device_alloc(size_t bytes, void** out) { return device_alloc(bytes, out); }
int msb_device_free(void* p) { return device_free(p); }
int msb_copy_to_device(void* dst, const void* src, size_t bytes, void* stream) { return copy_to_device(dst, src, bytes, (cudaStream_t)stream); }
int msb_copy_to_host(void* dst, const void* src, size_t bytes, void* stream) { return copy_to_host(dst, src, bytes, (cudaStream_t)stream); }
int msb_fill_f32(float* p, float value, size_t n, void* stream) { return fill_f32(p, value, n, (cudaStream_t)stream); }
int msb_copy_device(void* dst, const void* src, size_t bytes, void* stream) { return copy_device(dst, src, bytes, (cudaStream_t)stream); }
size_t msb_sample_scratch_bytes(int rows) { return sample_scratch_bytes(rows); }
int msb_argmax_rows(const float* logits, int rows, int V, int* out_idx, float* out_val, float temperature,
                    unsigned long long seed, void* scratch, size_t scratch_bytes, void* stream) {
  return argmax_rows(logits, rows, V, out_idx, out_val, temperature, (uint64_t)seed, scratch, scratch_bytes, (cudaStream_t)stream);
}
int msb_sample_topk(const float* logits, int rows, int V, int k, float temperature, float* out_v, int* out_i,
                    float* out_lse, void* scratch, size_t scratch_bytes, void* stream) {
  return sample_topk(logits, rows, V, k, temperature, out_v, out_i, out_lse, scratch, scratch_bytes, (cudaStream_t)stream);
}
int msb_log_softmax(const float* in, float* out, int rows, int V, void* stream) {
  return log_softmax(in, out, rows, V, (cudaStream_t)stream);
}
int msb_sample_top_p(const float* vals, const int* ids, int k, float lse, float temperature, float top_p, double u) {
  if (!vals || !ids || k < 1) return -1;
  return sample_top_p(vals, ids, k, lse, temperature, top_p, u);
}

size_t msb_hc_scratch_bytes(int n_tokens) { return hc_scratch_bytes(n_tokens); }
int msb_hc_step(const float* h_in, float* h_out, const float* x_sub, const float* mix_prev, const float* fn,
                const float* scale, const float* base, float* mix_out, const float* norm_w, float* x_out, int dim,
                int n_tokens, void* scratch, size_t scratch_bytes, void* stream) {
  return hc_step(h_in, h_out, x_sub, mix_prev, fn, scale, base, mix_out, norm_w, x_out, dim, n_tokens, scratch, scratch_bytes,
                 (cudaStream_t)stream);
}
int msb_compress(const float* c_kv, const float* c_gate, const float* c_norm, const void* wk_bf16, const float* k_norm,
                 const float* cs, float* state, int ratio, int pos, int actq, int D, int index_dim, int elem_type,
                 void* ckv_rows, int key_type, void* ikey_rows, void* stream) {
  return compress_token(c_kv, c_gate, c_norm, wk_bf16, k_norm, cs, state, ratio, pos, actq, D, index_dim, elem_type, ckv_rows,
                        key_type, ikey_rows, (cudaStream_t)stream);
}

}  // extern "C"
