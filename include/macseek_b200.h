/* libmacseek_b200 -- C ABI of the B200 (sm_100a) implementation of MacSeek's per-token hot path.
 *
 * Every function only ENQUEUES work on the given CUDA stream (a cudaStream_t passed as void*; NULL = the default
 * stream) and returns 0, or a negative MSB_E_* code with a message available from msb_last_error().  This is the
 * convention of the reference's host layer, whose encode_* functions "only encode into the given Enc (never
 * commit/wait)" (src/kernels/quant.hpp:3, arch.hpp:4-5, attn.hpp:3-4); a reference Buffer{buf, off} becomes the
 * device pointer buf + off, an Enc becomes the stream, and die()/abort() becomes a status code.
 * All pointers are device pointers unless a parameter is documented as host memory.  There is no CPU fallback.
 *
 * Weight matrices (W, expert matrices, expert tables) are treated as CONSTANTS: a kernel may start copying weight rows
 * before earlier work on the stream has finished (launches use programmatic stream serialization), so weights must be
 * in place and synchronised before the first call that reads them.  Activations, ids, scratch and outputs are ordered
 * on the stream as usual.
 */
#ifndef MACSEEK_B200_H
#define MACSEEK_B200_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { MSB_OK = 0, MSB_E_ARG = -1, MSB_E_TYPE = -2, MSB_E_CUDA = -3, MSB_E_SCRATCH = -4, MSB_E_DEVICE = -5,
       MSB_E_LIMIT = -6 };

/* Weight types: ggml type ids, as ms::q::QType (src/kernels/quant_types.hpp:10-12). */
enum { MSB_F32 = 0, MSB_F16 = 1, MSB_Q8_0 = 8, MSB_Q5_K = 13, MSB_Q6_K = 14, MSB_IQ2_XXS = 16, MSB_IQ1_S = 19,
       MSB_IQ4_NL = 20, MSB_BF16 = 30 };

const char* msb_last_error(void);
/* Library build tag, e.g. "macseek_b200 sm_100a". */
const char* msb_version(void);
/* Prepares the current device (codebook tables, status word).  Optional: every entry point does it on first use. */
int msb_init(void);
/* Synchronises the current device and returns the device-side failure word: 0, or 1/2 when a kernel abandoned a
 * bounded wait on its shared-memory ring, 3 for an abandoned peer wait.  A non-zero word means the launch that set it
 * (and anything queued behind it) returned early with incomplete outputs; the call then also resets the library's
 * device-side scheduling counters, so that later launches start from a clean state.  The word is cleared by the call. */
int msb_device_status(void);

/* Block geometry: ms::q::block_elems / block_bytes / row_bytes (src/kernels/quant_types.hpp:15-36). */
int msb_block_elems(int qtype);
size_t msb_block_bytes(int qtype);
size_t msb_row_bytes(int qtype, int64_t cols);

/* out[0..n) = dequantised blocks, bit-identical with the reference's CPU ref::dequant_row
 * (tests/ref/dequant.cpp:34-120; the GPU counterpart in the reference is q_deq_f16, src/kernels/quant_mm.metal:143-154).
 * n must be a whole number of blocks; out 16-byte aligned. */
int msb_dequant(int qtype, const void* blocks, int64_t n, float* out, void* stream);

/* y[rows] (+)= W[rows x cols] . x   -- ms::q::encode_matvec (src/kernels/quant.hpp:27-30, quant.mm:70-95).
 * W: raw GGUF block rows (2-byte aligned).  groups > 1: block-diagonal, row group g reads x[g*cols .. g*cols+cols).
 * Preconditions as the reference (quant.mm:73): cols a multiple of the block size, rows % groups == 0. */
int msb_matvec(int qtype, const void* W, int rows, int cols, const float* x, float* y, int accumulate, int groups,
               void* stream);
/* y = W . (x * rsqrt(mean(x^2) + eps) * norm_w): the input RMSNorm fused into the activation load --
 * ms::q::encode_matvec_rmsnorm (quant.hpp:19-26, quant.mm:107-127).  Every type is supported here (the reference
 * excludes the IQ types). */
int msb_matvec_rmsnorm(int qtype, const void* W, int rows, int cols, const float* x, const float* norm_w, float eps,
                       float* y, void* stream);
/* NO COUNTERPART IN THE REFERENCE.  msb_matvec_rmsnorm as a launch that shares the GPU: one small block per SM (96 KB of
 * shared memory, 288 threads) instead of filling every SM, so that kernels of ANOTHER stream (or graph branch) that
 * do not depend on it run beside it.  Slower alone, meant to hide under a latency-bound chain.  Same result as
 * msb_matvec_rmsnorm up to the fp32 summation order.  Types with a shared-memory codebook (IQ1_S, IQ2_XXS, IQ4_NL) and
 * rows too long for the small block fall back to the ordinary launch. */
int msb_matvec_rmsnorm_shared(int qtype, const void* W, int rows, int cols, const float* x, const float* norm_w, float eps,
                              float* y, void* stream);
/* Y[n x rows] (+)= X[n x cols*groups] . W^T, 1 <= n <= 16 -- ms::q::encode_matvec_n (quant.hpp:32-35, quant.mm:129-156).
 * Row stride of X = cols*groups, of Y = rows. */
int msb_matvec_n(int qtype, const void* W, int rows, int cols, const float* X, float* Y, int n, int accumulate,
                 int groups, void* stream);

/* ---- prefill projections: ms::q::encode_matmul / encode_f32_to_f16 / encode_matmul_h (src/kernels/quant.hpp:37-46).
 * Y[n x rows] (+)= X[n x cols] . W^T with half operands and fp32 accumulation on the tensor cores (tcgen05), as the
 * reference's Metal tensor path does.  The reference keeps module-owned scratch for the half copies of X and W
 * (quant.mm:175-184); here the caller passes it: msb_matmul_scratch_bytes(..., with_x) bytes (with_x = 1 for msb_matmul,
 * which converts X itself; 0 for msb_matmul_h, whose X16 is already half with row stride x_stride, 0 = cols). */
int msb_f32_to_f16(const float* x, void* x16, size_t count, void* stream);   /* count % 4 == 0 */
size_t msb_matmul_scratch_bytes(int qtype, int rows, int cols, int n, int with_x);
int msb_matmul_h(int qtype, const void* W, int rows, int cols, const void* X16, int x_stride, float* Y, int n, int accumulate,
                 void* scratch, size_t scratch_bytes, void* stream);
int msb_matmul(int qtype, const void* W, int rows, int cols, const float* X, float* Y, int n, int accumulate, void* scratch,
               size_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------- MoE decode (one token)
 * ms::q::MoeDecodeArgs / ExpertSlot / moe_decode_scratch_bytes / encode_moe_decode[_table[_part]] / MoePart
 * (src/kernels/quant.hpp:49-85, quant.mm:264-369).  dim and inter are run-time here (the reference fixes 5120 / 2304).
 *   h[e][r] = silu(min(gate_e[r].x, L)) * clamp(up_e[r].x, -L, L) * w_e     (shared expert: w = 1, stored last)
 *   y[r]   += sum_e down_e[r] . h[e]                                        (y is ACCUMULATED, quant.hpp:65)
 * gate/up: [inter x dim] rows, down: [dim x inter] rows, raw GGUF blocks at 2-byte aligned addresses.
 * Types: gate/up and down IQ1_S or IQ2_XXS; shared expert Q6_K or Q8_0 (quant.mm:255-261).
 * scratch: at least msb_moe_decode_scratch_bytes(inter, n_routed), 16-byte aligned; holds h as f32 [n_routed+1][inter]
 * afterwards.  Not thread-safe per device: the two kernels share library-owned scheduling counters (one MoE call in
 * flight per device at a time, as the reference's module-owned scratch, docs/modules/quant.md:265-268). */
#define MSB_MAX_ROUTED 16
typedef struct { const void* gate; const void* up; const void* down; } msb_expert_slot;
typedef struct {
  int dim, inter;
  int t_gate_up, t_down, t_shared;
  int n_routed;                       /* 0 .. MSB_MAX_ROUTED */
  int has_shared;
  msb_expert_slot slot[MSB_MAX_ROUTED];
  msb_expert_slot shared;
  const float* weights;               /* device F32[n_routed] routing weights (may be GPU-written) */
  const float* x;                     /* F32[dim] */
  float* y;                           /* F32[dim], accumulated */
  void* scratch;
  size_t scratch_bytes;
  float swiglu_limit;                 /* clamp L; 0 selects the reference's 10 */
} msb_moe_decode_args;
enum { MSB_MOE_ALL = 0, MSB_MOE_SHARED_GU = 1, MSB_MOE_AFTER_SHARED_GU = 2, MSB_MOE_SHARED = 3, MSB_MOE_ROUTED = 4,
       MSB_MOE_SHARED_DOWN = 5,
       /* not in the reference: the two launches of MSB_MOE_ALL one at a time (GU_ALL then DOWN_ALL == ALL, bit-identical) */
       MSB_MOE_GU_ALL = 6, MSB_MOE_DOWN_ALL = 7 };
size_t msb_moe_decode_scratch_bytes(int inter, int max_routed);
int msb_moe_decode(const msb_moe_decode_args* a, void* stream);
/* NO COUNTERPART IN THE REFERENCE.  msb_moe_decode for callers that cannot allocate device memory: a.scratch and
 * a.scratch_bytes are ignored, the h rows go to an array inside the library (static device memory, one instance per
 * device).  Nothing is allocated or looked up on this path: msb_init() must have run on the device before (else
 * MSB_E_DEVICE) -- it is msb_init() that resolves the array's address (cudaGetSymbolAddress, which loads the module
 * that holds it) and caches it under the library's lock; this call only reads that, so it is safe inside a stream
 * capture and from several host threads.  Limits: inter <= 4096 and n_routed <= 16 for the scratch, AND what
 * msb_moe_decode itself can stage -- the down launch keeps the quantised h of all n_routed + 1 experts (2.5 bytes per
 * element), its code tables and two ring slots in 227 KB of shared memory, so inter x (n_routed + 1) is bounded: e.g.
 * inter 2048 with 8 routed fits, inter 4096 with 8 routed does not.  Beyond either limit: MSB_E_LIMIT, nothing
 * enqueued, y untouched.  Nothing in the array has to start at zero (the gate/up launch writes every h row the down
 * launch reads).  Calls that overlap in time on one device (two streams) share the array and race: serialise them. */
int msb_moe_decode_noalloc(const msb_moe_decode_args* a, void* stream);
/* Routed matrices come from `table`: n_routed entries of 3 device addresses {gate, up, down} (uint64), a.slot[] is
 * ignored -- encode_moe_decode_table_part (quant.hpp:75-85). */
int msb_moe_decode_table_part(const msb_moe_decode_args* a, const uint64_t* table, int part, void* stream);
/* HBM-resident experts resolved on the GPU (what replaces the reference's CPU<->GPU handshake per layer,
 * src/model/ds41.mm:596-611): expert_table = [n_experts][3] device addresses, ids = device int32[n_routed] as written
 * by msb_router_*; only experts with expert_lo <= id < expert_hi (the ones resident on this GPU under expert
 * parallelism) are computed, the others contribute nothing to y. */
int msb_moe_decode_ids(const msb_moe_decode_args* a, const uint64_t* expert_table, const int* ids, int expert_lo,
                       int expert_hi, int part, void* stream);
/* NO COUNTERPART IN THE REFERENCE.  msb_moe_decode_ids whose activation is RMSNorm(norm_in) * norm_w, computed inside
 * the gate/up launch (a.x is ignored; same association as msb_router_fused_rmsnorm, so both see identical bits).  The
 * launch builds the activation and runs the shared expert's gate/up rows BEFORE the previous kernel of the stream has
 * finished, and waits for it only when it needs ids / weights.  Contract: the previous kernel of the stream is
 * msb_router_fused_rmsnorm over the same norm_in (it releases its dependents only after everything before it has
 * completed), and nothing between that launch and this one writes norm_in.  norm_in == NULL: plain msb_moe_decode_ids. */
int msb_moe_decode_ids_normed(const msb_moe_decode_args* a, const uint64_t* expert_table, const int* ids, int expert_lo,
                              int expert_hi, int part, const float* norm_in, const float* norm_w, float norm_eps,
                              void* stream);

/* ---------------------------------------------------------------- expert-parallel MoE decode over NVLink peer memory
 * NO COUNTERPART IN THE REFERENCE (one GPU, experts streamed from SSD).  The semantics follow the reference model's
 * expert-parallel MoE (reference/inference/model.py:869-904): contiguous expert ranges per rank, replicated router, the
 * ranks' outputs summed.  One process per GPU; rank r holds experts [r E/N, (r+1) E/N) and computes rows
 * [shared_lo, shared_hi) of the shared expert's gate/up and the same K range of its down matrix (multiples of 256).
 *
 * msb_moe_decode_ep = msb_moe_decode_ids_normed (norm_in may be NULL) restricted to that shared-expert slice.  With
 * comm == NULL the partial output is accumulated into a.y as usual (combine it yourself, e.g. ncclAllReduce).  With a
 * comm, a.y is ignored: the down launch stores its partial into slot `rank` of every rank's exchange buffer (plain
 * stores to peer-mapped memory) and every block of the launch counts itself, with a system-scope release, on this
 * rank's arrival counter there.  msb_ep_combine then waits -- bounded, about one second of SM clock, after which device
 * status 3 is recorded and h is left unchanged -- until the blocks of all `world` ranks have arrived (all ranks must be
 * identical GPUs: a launch's block count is part of the protocol) and adds the partials to h in rank order
 * (bit-identical on every rank).  Every rank must issue the same sequence of
 * msb_moe_decode_ep / msb_ep_combine pairs; the buffers are double-buffered by a device-side epoch, so the pair can be
 * captured in a CUDA graph and replayed.
 * Exchange buffers: msb_ep_exchange_bytes(dim, world) bytes from msb_ep_alloc (cudaMalloc + zero fill; not for use
 * inside a stream capture), exported with msb_ipc_export and mapped by the peers with msb_ipc_import (CUDA IPC, peer
 * access enabled on first use); base[r] is rank r's buffer as seen from this process (base[rank] = the local one). */
#define MSB_MAX_EP_WORLD 8
typedef struct { int world, rank; void* base[MSB_MAX_EP_WORLD]; } msb_ep_comm;
int msb_moe_decode_ep(const msb_moe_decode_args* a, const uint64_t* expert_table, const int* ids, int expert_lo,
                      int expert_hi, const float* norm_in, const float* norm_w, float norm_eps, int shared_lo,
                      int shared_hi, const msb_ep_comm* comm, void* stream);
size_t msb_ep_exchange_bytes(int dim, int world);
int msb_ep_combine(const msb_ep_comm* comm, float* h, int dim, void* stream);
/* Limit of msb_ep_combine's arrival wait in SM clock cycles (default 2e9; <= 0 restores it).  Host-side setting, read at
 * launch. */
void msb_set_peer_wait_cycles(long long cycles);
int msb_ep_alloc(size_t bytes, void** out);
int msb_ep_free(void* p);
int msb_ipc_export(void* p, unsigned char* handle64);           /* handle64: 64 bytes of host memory */
int msb_ipc_import(const unsigned char* handle64, void** out);
int msb_ipc_release(void* p);

/* ---------------------------------------------------------------- router
 * ms::arch::encode_router_fused / encode_router_topk / RouteLists / encode_route_lists (src/kernels/arch.hpp:79-97,
 * arch.mm:173-239).  E experts (<= 512), top-k (<= 16); score_fn 0 = sqrt(softplus(logit)) (arch_router.metal:16-24),
 * 1 = sigmoid (reference/inference/model.py:816-817); key = score + bias (bias may be NULL); ties -> lowest id;
 * w = score / (sum + 1e-20) * route_scale; ids / w in descending key order.  scratch (fused forms): at least
 * msb_router_scratch_bytes(E) bytes, 16-byte aligned; afterwards its first E floats are the logits. */
/* ---- MoE prefill: ms::q::MoePrefillArgs / moe_prefill_scratch_bytes / encode_moe_prefill (src/kernels/quant.hpp:87-118).
 * Grouped expert GEMMs on the tensor cores (tcgen05) with half operands and fp32 accumulation, as the reference's tensor
 * path.  Routing is expert-sorted: routed expert j owns entries [offs[j], offs[j+1]) of tok[] (token row in X) and wt[];
 * slot_of[t * k_per_token + k] = entry of token t's k-th expert (-1 = none);
 *   Y[t] += shared(t) + sum_k Z[slot_of[t][k]]   in that fixed order (run-to-run bit-identical).
 * slots and offs are HOST arrays (as in the reference, whose host side writes the tile tables at encode time); they are
 * read before the call returns.  Do not capture this call into a CUDA graph (the tables are copied from host memory). */
typedef struct {
  int dim, inter;                     /* the reference: 5120, 2304 */
  int t_gate_up, t_down, t_shared;
  int n_tokens, n_exp;
  const msb_expert_slot* slots;       /* host [n_exp], device addresses inside */
  const int* offs;                    /* host [n_exp + 1], offs[0] = 0, offs[n_exp] = total */
  const int* tok;                     /* device int32[total] */
  const float* wt;                    /* device F32[total] */
  const int* slot_of;                 /* device int32[n_tokens * k_per_token] */
  int k_per_token, has_shared;
  msb_expert_slot shared;
  const float* X;                     /* F32[n_tokens x dim] */
  float* Y;                           /* F32[n_tokens x dim], accumulated */
  void* scratch;
  size_t scratch_bytes;               /* >= msb_moe_prefill_scratch_bytes(total, n_tokens, n_exp, dim, inter) */
  float swiglu_limit;                 /* 0 selects the reference's 10 */
} msb_moe_prefill_args;
size_t msb_moe_prefill_scratch_bytes(int total_entries, int n_tokens, int n_exp, int dim, int inter);
/* Unlike the decode entry points this one is NOT enqueue-only: it reads offs[] and slots[] on the host, builds its tile
 * tables there and uploads them with stream-ordered copies from pageable host memory, which block the calling thread
 * until the copy engine has taken them.  It therefore cannot be captured into a CUDA graph, and a caller that overlaps
 * it with other host work should give it a thread of its own.  (The reference's encode_moe_prefill builds the same
 * per-expert dispatch list on the CPU, quant.mm:385-487.)  Like every entry point it creates the library's tables on
 * first use on a device: call msb_init() before any stream capture. */
int msb_moe_prefill(const msb_moe_prefill_args* a, void* stream);

size_t msb_router_scratch_bytes(int n_experts);
int msb_router_fused(const float* x, const float* W, const float* bias, int* ids, float* w, void* scratch,
                     size_t scratch_bytes, int n_experts, int dim, int k, int score_fn, float route_scale, void* stream);
/* The same with the RMSNorm that precedes the router fused in (the reference runs arch::encode_rmsnorm,
 * src/kernels/arch.hpp:99-104, as its own dispatch): logits = W . (h * rsqrt(mean(h^2) + eps) * norm_w); the normalised
 * vector is also written to x_out (may be NULL) for the MoE kernels that read it next. */
int msb_router_fused_rmsnorm(const float* h, const float* norm_w, float eps, float* x_out, const float* W,
                             const float* bias, int* ids, float* w, void* scratch, size_t scratch_bytes, int n_experts,
                             int dim, int k, int score_fn, float route_scale, void* stream);
int msb_router_topk(const float* logits, const float* bias, int* ids, float* w, int n_tokens, int n_experts, int k,
                    int score_fn, float route_scale, void* stream);
/* counts u32[E], offsets u32[E+1], entry/tok/slot_of u32[n*k], lw f32[n*k]; entries t*k+j ordered by (expert, entry). */
int msb_route_lists(const int* ids, const float* w, int n_tokens, int k, int n_experts, uint32_t* counts,
                    uint32_t* offsets, uint32_t* entry, uint32_t* tok, float* lw, uint32_t* slot_of, void* stream);

/* ---------------------------------------------------------------- lightning indexer (decode) and exact top-k
 * ms::attn::encode_index_decode (src/kernels/attn.hpp:121-122, attn.mm:222-290); math spec tests/ref/attn_ref.cpp:163-202.
 * Index keys: [len][128] rows, MSB_F16 (the reference's ikey cache, attn.hpp:69) or MSB_KEY_FP8_E4M3.
 * heads = 32 (reference) or 64. */
#define MSB_KEY_FP8_E4M3 101
/* Query preparation (index_q): rope on the last 64 dims of each head with cs = (cos, sin)[32] of the query position,
 * optional fp4 quant-dequant simulation (actq), head weights scaled by 128^-0.5 * heads^-0.5.  q: [heads][128]. */
int msb_index_prep(const float* q_raw, const float* w_raw, const float* cs, int actq, int heads, float* q, float* w,
                   void* stream);
/* scores[t] = sum_h relu(q_h . key_t) * w_h for t < len.  FP8 keys: the query is rounded to e4m3 for the tensor cores
 * unless exact_query != 0 (then the keys are widened to f16 and the fp32 query is used as two f16 terms).
 * topk_scratch (optional): when given, the histogram used by msb_topk(..., hist_ready = 1) is built on the fly. */
int msb_index_scores(int key_type, const void* keys, int len, const float* q, const float* w, int heads, float* scores,
                     void* topk_scratch, int exact_query, void* stream);
/* Exact top-k (k <= 2048) among the finite entries of scores[0..n): ties -> lower index; out[k] sorted ascending by
 * index, -1 padded (attn_ref.cpp:186-194).  scratch: msb_topk_scratch_bytes(n) bytes, ZERO-FILLED before its first
 * use; every call leaves it zeroed again. */
size_t msb_topk_scratch_bytes(int n_max);
int msb_topk(const float* scores, int n, int k, int* out, void* scratch, size_t scratch_bytes, int hist_ready,
             void* stream);
/* Block maxima over bs consecutive scores, the newest block pinned to +inf: the input of the candidate-block top-k
 * (attn_ref.cpp:196-202).  out[(len + bs - 1) / bs]. */
int msb_block_max(const float* scores, int len, int bs, float* out, void* stream);
/* prep + scores + top-k in one call (the sequence of encode_index_decode).  q_prep [heads][128] and w_prep [heads] are
 * caller-owned work buffers. */
int msb_index_decode(int key_type, const void* keys, int len, const float* q_raw, const float* w_raw, const float* cs,
                     int actq, int heads, int k, float* q_prep, float* w_prep, float* scores, int* topk_out,
                     void* topk_scratch, size_t topk_scratch_bytes, int exact_query, void* stream);
/* The candidate-restricted form of encode_index_decode (layers that "use candidates", src/kernels/attn.mm:226-229, kernel
 * attn_idx_score_dec2_list, attn_index.metal:1056-1112): only the keys of the key blocks in cand_list (8 keys per block,
 * ascending block indices as msb_topk over the block maxima returns them, -1 = none) are scored; every other key counts as
 * -inf.  scores[8 i + j] receives the score of key cand_list[i] * 8 + j; topk_out lists key indices, ascending, -1 padded.
 * F16 keys (the reference's layout: one warp per candidate key) or FP8 keys (tcgen05 kernel). */
int msb_index_decode_list(int key_type, const void* keys, int len, const float* q_raw, const float* w_raw, const float* cs,
                          int actq, int heads, int k, const int* cand_list, int n_cand, float* q_prep, float* w_prep,
                          float* scores, int* topk_out, void* topk_scratch, size_t topk_scratch_bytes, void* stream);

/* ---------------------------------------------------------------- sparse attention (decode)
 * ms::attn::encode_sparse (src/kernels/attn.hpp:128-129, attn.mm:419-445); math spec tests/ref/attn_ref.cpp:204-230.
 * q: F32 [heads][D] pre-rope; rows are K == V vectors of D elements (MSB_F16 or MSB_BF16), D = 512 or 576, rope on
 * the last 64 dims; the attended set is win[0..n_win) followed by cache[topk[i]] for every topk[i] >= 0.
 * out: F32 [heads][D] after the inverse rope.  scratch: msb_sparse_scratch_bytes(n_win + k, heads, D). */
size_t msb_sparse_scratch_bytes(int total_rows_max, int heads, int D);
int msb_sparse_decode(const float* q, const float* cs, const float* sinks, int elem_type, const void* win, int n_win,
                      const void* cache, const int* topk, int k, int heads, int D, float* out, void* scratch,
                      size_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------- small per-token kernels between the hot-path calls
 * y = x * rsqrt(mean(x^2) + eps) * w per row (w may be NULL); strides in floats, 0 = dim -- ms::arch::encode_rmsnorm
 * (src/kernels/arch.hpp:128-130). */
int msb_rmsnorm(const float* x, const float* w, float* y, int rows, int dim, float eps, int in_stride, int out_stride,
                void* stream);
/* Window KV row of one token: rmsnorm(kv) * norm_w -> rope on the last 64 dims -> optional fp8 quant-dequant
 * simulation -> stored as D elements of elem_type (MSB_F16 / MSB_BF16) at out_row -- the n == 1 path of
 * ms::attn::encode_kv_window (src/kernels/attn.hpp:113, attn.mm:186-193; math tests/ref/attn_ref.cpp:109-114). */
int msb_kv_window(const float* kv, const float* norm_w, const float* cs, int actq, int D, int elem_type, void* out_row,
                  void* stream);
/* Greedy argmax, ties -> lowest index -- the temperature 0 case of ms::arch::encode_argmax (arch.hpp:107-112).
 * out_val may be NULL. */
int msb_argmax(const float* x, int n, int* out_idx, float* out_val, void* stream);
/* y[i] += a[i] */
int msb_add(float* y, const float* a, int n, void* stream);

/* ---------------------------------------------------------------- sampling head (src/kernels/arch.hpp:109-126)
 * Scratch for the three calls below: msb_sample_scratch_bytes(rows) bytes, 16-byte aligned, zeroed once after
 * allocation (the kernels leave it ready for the next call).  One scratch serves one stream at a time. */
size_t msb_sample_scratch_bytes(int rows);
/* Argmax of each of `rows` rows of V logits, ties -> lowest index, one launch -- ms::arch::encode_argmax
 * (arch.hpp:111-115, arch_sample.metal:46-83).  temperature > 0: Gumbel-max sampling of softmax(logits / temperature)
 * (exact multinomial sampling over the whole row; counter-based noise keyed by (seed, row, index), the reference's
 * mixer arch_sample.metal:15-26); out_val (may be NULL) receives the winning (noisy) value. */
int msb_argmax_rows(const float* logits, int rows, int V, int* out_idx, float* out_val, float temperature,
                    unsigned long long seed, void* scratch, size_t scratch_bytes, void* stream);
/* Top-k (1 <= k <= 64) of each row: raw logits descending (ties -> lower index) in out_v [rows][64] and their ids in
 * out_i [rows][64], plus out_lse[row] = logsumexp(logits / temperature) over the WHOLE row (temperature <= 0 counts as
 * 1) -- ms::arch::encode_topk (arch.hpp:116-119, arch_sample.metal:124-181).  V <= 262144. */
int msb_sample_topk(const float* logits, int rows, int V, int k, float temperature, float* out_v, int* out_i,
                    float* out_lse, void* scratch, size_t scratch_bytes, void* stream);
/* out = in - logsumexp(in) per row; out may alias in -- ms::arch::encode_log_softmax (arch.hpp:120-121). */
int msb_log_softmax(const float* in, float* out, int rows, int V, void* stream);
/* HOST function, as in the reference (arch.hpp:122-126, arch.mm:322-342): temperature + top-p sampling from
 * msb_sample_topk's output copied to the host.  p_i = exp(v_i / T - lse); keeps the smallest prefix whose cumulative
 * mass reaches top_p, renormalised; u in [0, 1).  Returns the token id (ids[0] when temperature <= 0 or k <= 1). */
int msb_sample_top_p(const float* vals, const int* ids, int k, float lse, float temperature, float top_p, double u);

/* ---------------------------------------------------------------- device memory for hosts without CUDA headers
 * What the reference's Device::alloc (zero-filled) and Buffer::cpu() (shared storage) become with separate device memory
 * (src/core/metal.hpp:11-40): allocation, blocking copies on a stream, and the fill dispatch of the layer code
 * (src/model/dec_layer.mm, fill0).  Not for use inside a stream capture (except msb_fill_f32). */
int msb_device_alloc(size_t bytes, void** out);
int msb_device_free(void* p);
int msb_copy_to_device(void* dst, const void* src, size_t bytes, void* stream);
int msb_copy_to_host(void* dst, const void* src, size_t bytes, void* stream);
int msb_fill_f32(float* p, float value, size_t n, void* stream);
/* device -> device copy ordered on the stream (enqueue-only, capturable) */
int msb_copy_device(void* dst, const void* src, size_t bytes, void* stream);

/* ---------------------------------------------------------------- hyper-connection step and KV compressor
 * One sublayer boundary of the 4-stream residual -- ms::arch::encode_hc_step / HcStep (src/kernels/arch.hpp:44-77);
 * math tests/ref/arch_ref.cpp:22-95.  All F32; h [n][4][dim]; mix [n][24] = pre[4], post[4], comb[4][4].
 *   h_new  = x_sub ? post[i] * x_sub + sum_j comb[j][i] * h_in[j] : h_in     (h_out written only with x_sub; may alias h_in)
 *   mix_out = fn ? Sinkhorn split of fn . h_new * rsqrt(mean(h_new^2) + 1e-20) : -    (fn [24][4 dim], scale[3], base[24])
 *   x_out  = rmsnorm(sum_j mix_prev.pre[j] * h_new[j]) * norm_w                       (x_out NULL: skipped)
 * x_sub, fn, x_out may be NULL as in the reference; mix_out must not alias mix_prev.  scratch: msb_hc_scratch_bytes(n)
 * bytes, ZERO-FILLED before its first use (every call leaves its counters zeroed again). */
size_t msb_hc_scratch_bytes(int n_tokens);
int msb_hc_step(const float* h_in, float* h_out, const float* x_sub, const float* mix_prev, const float* fn,
                const float* scale, const float* base, float* mix_out, const float* norm_w, float* x_out, int dim,
                int n_tokens, void* scratch, size_t scratch_bytes, void* stream);
/* Compressor + index key of ONE decode token at position pos for a KV source of compression ratio `ratio` -- the n == 1
 * case of ms::attn::encode_compress (src/kernels/attn.hpp:118); math tests/ref/attn_ref.cpp:116-161.  c_kv / c_gate: the
 * layer's compressor projections F32[D] (c_gate only for ratio > 1); state: F32 [2][ratio][D] partial group of the source
 * (kv values, then gate scores; start it at 0 / -inf).  When position pos completes a group a row is written at index
 * pos / ratio: ckv_rows (D elements of elem_type MSB_F16 / MSB_BF16) and ikey_rows (index_dim elements, MSB_F16 or
 * MSB_KEY_FP8_E4M3); otherwise only the state is updated.  cs = (cos, sin)[32] of position (pos / ratio) * ratio; rope on
 * the last 64 dims of both vectors; actq: the fp4 quant-dequant simulations of the reference. */
int msb_compress(const float* c_kv, const float* c_gate, const float* c_norm, const void* wk_bf16, const float* k_norm,
                 const float* cs, float* state, int ratio, int pos, int actq, int D, int index_dim, int elem_type,
                 void* ckv_rows, int key_type, void* ikey_rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif
