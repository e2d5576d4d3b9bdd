// MoE router: logits = W[E x dim] . x (fp32), score = sqrt(softplus) or sigmoid, top-k of score + bias (ties -> lowest
// expert id), weights = score / (sum + 1e-20) * route_scale; plus the per-expert routing lists for the prefill grouped
// GEMM.  Replaces the reference's arch_router_fused / arch_router_topk / arch_route_count / arch_route_scatter Metal
// kernels (src/kernels/arch_router.metal:16-160) behind ms::arch::encode_router_fused / encode_router_topk /
// encode_route_lists (src/kernels/arch.hpp:79-97, arch.mm:173-239).
#include <algorithm>
#include "msb_common.cuh"

namespace msb {

constexpr int kRouterMaxE = 512;   // experts per token handled by the one-warp selection (16 per lane)
constexpr int kRouterMaxK = 16;
constexpr int kRouterKSplit = 4;   // K slices per expert row in the fused kernel

struct RouterParams {
  const float* x;
  const float* norm_w;   // not null: x is RMS-normalised with this gain before use (fused RMSNorm)
  float* x_out;          // with norm_w: the normalised x is also written here (may be null)
  float norm_eps;
  const float* W;
  const float* bias;     // may be null
  float* logits;         // [E] (written by the fused kernel; diagnostic, as the reference's Scratch::router_logits)
  float* partial;        // [E][kRouterKSplit]
  int* ids;
  float* wts;
  unsigned* ticket;      // zero between launches
  int E, dim, k, score_fn;
  float route_scale;
};

__device__ __forceinline__ float router_score(float x, int score_fn) {
  if (score_fn == 1) return 1.f / (1.f + expf(-x));
  const float sp = x > 20.f ? x : log1pf(expf(x));   // softplus, threshold 20 (arch_router.metal:20-24)
  return sqrtf(sp);
}

// One warp selects the top-k experts of one token (descending key; ties -> lowest id) and writes ids / weights.
// The bias values of the lane's experts (e = lane + 32 i) are passed in registers so that a caller can request them
// ahead of the logits.
constexpr int kRouterEPL = kRouterMaxE / 32;
__device__ __forceinline__ void router_load_bias(const float* bias, int E, int lane, float (&bz)[kRouterEPL]) {
#pragma unroll
  for (int i = 0; i < kRouterEPL; i++) {
    const int e = lane + 32 * i;
    bz[i] = (bias && e < E) ? __ldg(bias + e) : 0.f;
  }
}
// order-preserving map of a float onto an unsigned (NaN -> 0, below everything)
__device__ __forceinline__ unsigned router_ord(float f) {
  const unsigned u = __float_as_uint(f);
  return f == f ? (u ^ ((unsigned)((int)u >> 31) | 0x80000000u)) : 0u;
}
__device__ __forceinline__ void router_topk_warp(const float* logits, const float (&bz)[kRouterEPL], int E, int k,
                                                 int score_fn, float route_scale, int lane, int* ids, float* wts) {
  constexpr int EPL = kRouterEPL;
  float sc[EPL], key[EPL];
#pragma unroll
  for (int i = 0; i < EPL; i++) {
    const int e = lane + 32 * i;
    if (e < E) {
      sc[i] = router_score(logits[e], score_fn);
      key[i] = sc[i] + bz[i];
    } else {
      sc[i] = 0.f;
      key[i] = -INFINITY;
    }
  }
  float sum = 0.f, my_w = 0.f;
  int my_e = 0;
  unsigned taken = 0;
  bool rescan = true;
  float bk = -INFINITY, bs = 0.f;
  int be = 0x7fffffff;
  for (int j = 0; j < k; j++) {
    // this lane's best remaining candidate: ascending expert id with a strict compare keeps the lowest id on ties;
    // only the lane that lost its candidate in the previous round looks again
    if (rescan) {
      bk = -INFINITY; bs = 0.f; be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < EPL; i++) {
        const int e = lane + 32 * i;
        if (e < E && !((taken >> i) & 1u) && (be == 0x7fffffff || key[i] > bk)) { bk = key[i]; bs = sc[i]; be = e; }
      }
      rescan = false;
    }
    // warp-wide: the largest key, then the lowest expert id that holds it (one reduction instruction each)
    const unsigned uk = be == 0x7fffffff ? 0u : router_ord(bk);
    const unsigned m = __reduce_max_sync(0xffffffffu, uk);
    const int win = (int)__reduce_min_sync(0xffffffffu, (uk == m) ? (unsigned)be : 0x7fffffffu);
    const float wscore = __shfl_sync(0xffffffffu, bs, win & 31);   // the owner's best candidate is the winner
    if (lane == (win & 31)) { taken |= 1u << (win >> 5); rescan = true; }
    sum += wscore;
    if (lane == j) { my_e = win; my_w = wscore; }
  }
  const float inv = route_scale / (sum + 1e-20f);
  if (lane < k) { ids[lane] = my_e; wts[lane] = my_w * inv; }
}

// Fused decode router: every warp computes one (expert, K-slice) partial dot; the block that finishes last sums the
// slices in a fixed order, writes the logits and selects.
__global__ void __launch_bounds__(256) router_fused_kernel(const RouterParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit = blockIdx.x * 8 + warp;
  const int slice = p.dim / kRouterKSplit;   // floats per slice, a multiple of 4
  const bool live = unit < p.E * kRouterKSplit;
  const int e = unit / kRouterKSplit, ks = unit % kRouterKSplit;
  const float4* w = reinterpret_cast<const float4*>(p.W + (size_t)(live ? e : 0) * p.dim + (size_t)ks * slice);
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  // the router matrix is constant: its first 8 x 16 bytes per lane are requested before the grid dependency resolves
  float4 a[8];
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const int c = lane + 32 * k;
    a[k] = (live && c < slice / 4) ? __ldg(w + c) : zero4;
  }
  pdl_wait();
  // Dependents are released only now: a dependent that starts may rely on everything before this launch being complete
  // (the MoE gate/up launch reads the un-normalised vector before its own dependency resolves).
  pdl_launch_dependents();
  // this unit's slice of x (and of the norm gain) is requested before the norm's reduction, not after it
  const float4* xv = reinterpret_cast<const float4*>(p.x + (size_t)ks * slice);
  const float4* gv = reinterpret_cast<const float4*>(p.norm_w ? p.norm_w + (size_t)ks * slice : p.x);
  float4 b[8], g8[8];
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const int c = lane + 32 * k;
    b[k] = (live && c < slice / 4) ? xv[c] : zero4;
    g8[k] = (live && p.norm_w && c < slice / 4) ? __ldg(gv + c) : zero4;
  }
  float mul = 1.f;
  if (p.norm_w) {   // every block needs 1/rms of the whole vector: dim floats from L2, summed in a fixed order
    __shared__ float red[8];
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.dim / 4; i += 256) {
      const float4 v = reinterpret_cast<const float4*>(p.x)[i];
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    mul = rsqrtf(tot / (float)p.dim + p.norm_eps);
  }
  if (live) {
    float acc = 0.f;
    for (int c0 = lane; c0 < slice / 4; c0 += 32 * 8) {   // 8 independent 16-byte loads in flight per lane
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int c = c0 + 32 * k;
        if (c0 != lane) {
          a[k] = c < slice / 4 ? __ldg(w + c) : zero4;
          b[k] = c < slice / 4 ? xv[c] : zero4;
          g8[k] = (p.norm_w && c < slice / 4) ? __ldg(gv + c) : zero4;
        }
        if (p.norm_w && c < slice / 4) {
          b[k].x = b[k].x * mul * g8[k].x; b[k].y = b[k].y * mul * g8[k].y;
          b[k].z = b[k].z * mul * g8[k].z; b[k].w = b[k].w * mul * g8[k].w;
          if (e == 0 && p.x_out) reinterpret_cast<float4*>(p.x_out + (size_t)ks * slice)[c] = b[k];
        }
      }
#pragma unroll
      for (int k = 0; k < 8; k++) {
        acc = fmaf(a[k].x, b[k].x, acc); acc = fmaf(a[k].y, b[k].y, acc);
        acc = fmaf(a[k].z, b[k].z, acc); acc = fmaf(a[k].w, b[k].w, acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) p.partial[unit] = acc;
  }
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned t = atomicAdd(p.ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // the finishing block: the serial tail of the launch.  Bias (constant) and partial sums are requested together; the
  // logits reach the selecting warp through shared memory (the copy in global memory is a diagnostic).
  __shared__ float s_logits[kRouterMaxE];
  float bz[kRouterEPL];
  if (warp == 0) router_load_bias(p.bias, p.E, lane, bz);
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    const float4 q = __ldcg(reinterpret_cast<const float4*>(p.partial) + e);
    const float s = ((q.x + q.y) + q.z) + q.w;
    p.logits[e] = s;
    s_logits[e] = s;
  }
  __syncthreads();
  if (warp == 0) router_topk_warp(s_logits, bz, p.E, p.k, p.score_fn, p.route_scale, lane, p.ids, p.wts);
  if (threadIdx.x == 0) *p.ticket = 0;
}

// logits [n][E] -> ids [n][k], weights [n][k]; one warp per token.
__global__ void __launch_bounds__(128) router_topk_kernel(const float* logits, const float* bias, int* ids, float* wts,
                                                          int n, int E, int k, int score_fn, float route_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= n) return;
  float bz[kRouterEPL];
  router_load_bias(bias, E, threadIdx.x & 31, bz);
  router_topk_warp(logits + (size_t)t * E, bz, E, k, score_fn, route_scale, threadIdx.x & 31, ids + (size_t)t * k,
                   wts + (size_t)t * k);
}

// ---- routing lists: entries i = t*k + j sorted by (expert, i).  No atomics: a warp owns an expert and scans all
// entries in order with ballots, so the lists are identical from run to run.
__global__ void __launch_bounds__(256) route_count_kernel(const int* ids, unsigned* counts, int N, int E) {
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= E) return;
  unsigned c = 0;
  for (int i0 = 0; i0 < N; i0 += 32) {
    const int i = i0 + lane;
    c += __popc(__ballot_sync(0xffffffffu, i < N && ids[i] == e));
  }
  if (lane == 0) counts[e] = c;
}
__global__ void __launch_bounds__(1024) route_scan_kernel(const unsigned* counts, unsigned* offsets, int E) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ unsigned buf[1024];
  const int tid = threadIdx.x;
  // E <= 1024 per pass; serial carry over passes
  unsigned carry = 0;
  for (int base = 0; base < E; base += 1024) {
    const unsigned v = base + tid < E ? counts[base + tid] : 0;
    buf[tid] = v;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const unsigned a = tid >= o ? buf[tid - o] : 0;
      __syncthreads();
      buf[tid] += a;
      __syncthreads();
    }
    if (base + tid < E) offsets[base + tid] = carry + buf[tid] - v;
    carry += buf[1023];
    __syncthreads();
  }
  if (tid == 0) offsets[E] = carry;
}
__global__ void __launch_bounds__(256) route_scatter_kernel(const int* ids, const float* w, const unsigned* offsets,
                                                            unsigned* entry, unsigned* tok, float* lw, unsigned* slot_of,
                                                            int N, int E, int k) {
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= E) return;
  unsigned pos = offsets[e];
  for (int i0 = 0; i0 < N; i0 += 32) {
    const int i = i0 + lane;
    const bool hit = i < N && ids[i] == e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (hit) {
      const unsigned q = pos + __popc(m & ((1u << lane) - 1u));
      entry[q] = (unsigned)i; tok[q] = (unsigned)(i / k); lw[q] = w[i]; slot_of[i] = q;
    }
    pos += __popc(m);
  }
}

// ---------------------------------------------------------------- host side
// logits [E], padded to a multiple of 4 floats so that the partials [E][4] behind them are 16-byte aligned
size_t router_scratch_bytes(int E) { return sizeof(float) * ((size_t)((E + 3) & ~3) + (size_t)E * kRouterKSplit); }

int router_fused(const float* x, const float* norm_w, float norm_eps, float* x_out, const float* W, const float* bias,
                 int* ids, float* wts, void* scratch, size_t scratch_bytes, int E, int dim, int k, int score_fn,
                 float route_scale, cudaStream_t st) {
  if (E <= 0 || E > kRouterMaxE || k <= 0 || k > kRouterMaxK || k > E || dim <= 0 || dim % (4 * kRouterKSplit))
    return fail(kErrArg, "router: bad shape (E %d dim %d k %d)", E, dim, k);
  if (!x || !W || !ids || !wts || !scratch) return fail(kErrArg, "router: null pointer");
  if (scratch_bytes < router_scratch_bytes(E)) return fail(kErrScratch, "router: scratch too small");
  if (reinterpret_cast<uintptr_t>(scratch) & 15) return fail(kErrArg, "router: scratch must be 16-byte aligned");
  static_assert(kRouterKSplit == 4, "the finishing block reads one float4 of partials per expert");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return fail(kErrArg, "router: x and W must be 16-byte aligned");
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  RouterParams p;
  if ((norm_w && (reinterpret_cast<uintptr_t>(norm_w) & 15)) || (x_out && (reinterpret_cast<uintptr_t>(x_out) & 15)))
    return fail(kErrArg, "router: norm_w and x_out must be 16-byte aligned");
  p.x = x; p.norm_w = norm_w; p.norm_eps = norm_eps; p.x_out = norm_w ? x_out : nullptr;
  p.W = W; p.bias = bias; p.ids = ids; p.wts = wts;
  p.logits = reinterpret_cast<float*>(scratch);
  p.partial = p.logits + ((E + 3) & ~3);
  p.ticket = reinterpret_cast<unsigned*>(tb.status) + 16;
  p.E = E; p.dim = dim; p.k = k; p.score_fn = score_fn; p.route_scale = route_scale;
  const int units = E * kRouterKSplit;
  MSB_CUDA(launch_pdl(router_fused_kernel, dim3((units + 7) / 8), dim3(256), 0, st, p));
  MSB_LAUNCH_CHECK("router_fused_kernel");
  return kOk;
}

int router_topk(const float* logits, const float* bias, int* ids, float* wts, int n, int E, int k, int score_fn,
                float route_scale, cudaStream_t st) {
  if (E <= 0 || E > kRouterMaxE || k <= 0 || k > kRouterMaxK || k > E || n < 0)
    return fail(kErrArg, "router_topk: bad shape (n %d E %d k %d)", n, E, k);
  if (n == 0) return kOk;
  if (!logits || !ids || !wts) return fail(kErrArg, "router_topk: null pointer");
  MSB_CUDA(launch_pdl(router_topk_kernel, dim3((n + 3) / 4), dim3(128), 0, st, logits, bias, ids, wts, n, E, k, score_fn, route_scale));
  MSB_LAUNCH_CHECK("router_topk_kernel");
  return kOk;
}

int route_lists(const int* ids, const float* w, int n, int k, int E, unsigned* counts, unsigned* offsets,
                unsigned* entry, unsigned* tok, float* lw, unsigned* slot_of, cudaStream_t st) {
  if (n < 0 || k <= 0 || E <= 0) return fail(kErrArg, "route_lists: bad shape");
  if (!ids || !w || !counts || !offsets || !entry || !tok || !lw || !slot_of) return fail(kErrArg, "route_lists: null pointer");
  const int N = n * k;
  MSB_CUDA(launch_pdl(route_count_kernel, dim3((E + 7) / 8), dim3(256), 0, st, ids, counts, N, E));
  MSB_CUDA(launch_pdl(route_scan_kernel, dim3(1), dim3(1024), 0, st, counts, offsets, E));
  MSB_CUDA(launch_pdl(route_scatter_kernel, dim3((E + 7) / 8), dim3(256), 0, st, ids, w, offsets, entry, tok, lw, slot_of, N, E, k));
  MSB_LAUNCH_CHECK("route_lists");
  return kOk;
}

}  // namespace msb
