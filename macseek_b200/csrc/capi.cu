// extern "C" surface of libmacseek_b200 (declared in include/macseek_b200.h).
#include "msb_common.cuh"
#include "../../include/macseek_b200.h"

namespace msb {
const char* last_error_text();
int dequant(int t, const void* src, int64_t n, float* out, cudaStream_t st);
int matvec_n(int t, const void* W, int rows, int cols, const float* X, int64_t x_stride, float* Y, int64_t y_stride,
             int n, int accumulate, int groups, cudaStream_t st);
size_t router_scratch_bytes(int E);
int router_fused(const float* x, const float* W, const float* bias, int* ids, float* wts, void* scratch,
                 size_t scratch_bytes, int E, int dim, int k, int score_fn, float route_scale, cudaStream_t st);
int router_topk(const float* logits, const float* bias, int* ids, float* wts, int n, int E, int k, int score_fn,
                float route_scale, cudaStream_t st);
int route_lists(const int* ids, const float* w, int n, int k, int E, unsigned* counts, unsigned* offsets,
                unsigned* entry, unsigned* tok, float* lw, unsigned* slot_of, cudaStream_t st);
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
  if (v) MSB_CUDA(cudaMemset(t.status, 0, sizeof v));
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
  return matvec_n(qtype, W, rows, cols, x, (int64_t)cols * groups, y, rows, 1, accumulate, groups, (cudaStream_t)stream);
}

int msb_matvec_n(int qtype, const void* W, int rows, int cols, const float* X, float* Y, int n, int accumulate,
                 int groups, void* stream) {
  if (n < 1 || n > 16) return fail(kErrArg, "matvec_n: n = %d outside 1..16", n);
  return matvec_n(qtype, W, rows, cols, X, (int64_t)cols * groups, Y, rows, n, accumulate, groups, (cudaStream_t)stream);
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

size_t msb_router_scratch_bytes(int n_experts) { return router_scratch_bytes(n_experts); }
int msb_router_fused(const float* x, const float* W, const float* bias, int* ids, float* w, void* scratch,
                     size_t scratch_bytes, int n_experts, int dim, int k, int score_fn, float route_scale, void* stream) {
  return router_fused(x, W, bias, ids, w, scratch, scratch_bytes, n_experts, dim, k, score_fn, route_scale,
                      (cudaStream_t)stream);
}
int msb_router_topk(const float* logits, const float* bias, int* ids, float* w, int n_tokens, int n_experts, int k,
                    int score_fn, float route_scale, void* stream) {
  return router_topk(logits, bias, ids, w, n_tokens, n_experts, k, score_fn, route_scale, (cudaStream_t)stream);
}
int msb_route_lists(const int* ids, const float* w, int n_tokens, int k, int n_experts, uint32_t* counts,
                    uint32_t* offsets, uint32_t* entry, uint32_t* tok, float* lw, uint32_t* slot_of, void* stream) {
  return route_lists(ids, w, n_tokens, k, n_experts, counts, offsets, entry, tok, lw, slot_of, (cudaStream_t)stream);
}

}  // extern "C"
