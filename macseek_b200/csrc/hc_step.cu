// Hyper-connection step of one sublayer boundary -- ms::arch::encode_hc_step (src/kernels/arch.hpp:44-77, kernels
// src/kernels/arch_hc.metal:49-323); math as tests/ref/arch_ref.cpp:22-95:
//   h_new[i]  = x_sub ? post[i] * x_sub + sum_j comb[j][i] * h_in[j] : h_in          (4 residual streams of width D)
//   mix_out   = fn ? split + Sinkhorn( fn . h_new * rsqrt(mean(h_new^2) + 1e-20), scale, base ) : -
//   x_out     = rmsnorm( sum_j pre[j] * h_new[j] ) * norm_w                          (pre / post / comb from mix_prev)
// One launch per call, all tokens: grid (blocks over D, tokens).  A block owns 32 consecutive columns d of the four
// streams; its 8 warps share the 24 rows of fn (3 rows each), so that the 96 fn values a column needs are fetched by 8
// threads at once instead of one after the other, and D / 32 blocks (128 at D = 4096) spread the 1.6 MB of fn over the
// machine.  Every thread reads its column of h_in (and x_sub) BEFORE the block's barrier and only warp 0 writes h_out
// afterwards, so h_out may alias h_in.  Each warp's shuffle sum is the block's partial of its rows; the block that
// finishes last (a ticket per token) adds the partials in block order, runs the 4 x 4 Sinkhorn on 16 lanes and scales
// x_out.  Bound by the latency of one pass over fn (24 x 4 D floats, read exactly once), not by its bytes.
#include <algorithm>
#include "msb_common.cuh"

namespace msb {

constexpr int kHcThreads = 256;
constexpr int kHcCols = 32;       // columns per block (one per lane); warp w takes fn rows [3 w, 3 w + 3)
constexpr int kHcMaxBlocks = 512; // D <= 16384
constexpr int kHcPart = 26;       // 24 fn rows, sum h_new^2, sum x^2

struct HcParams {
  const float* h_in;      // [n][4][D]
  float* h_out;           // [n][4][D] (written only with x_sub; may alias h_in)
  const float* x_sub;     // [n][D] or null
  const float* mix_prev;  // [n][24]
  const float* fn;        // [24][4 D] or null
  const float* scale;     // [3]
  const float* base;      // [24]
  float* mix_out;         // [n][24]
  const float* norm_w;    // [D]
  float* x_out;           // [n][D] or null
  float* part;            // [n][blocks][26] partial sums
  unsigned* ticket;       // [n], zero between launches
  int D, n, iters;
  float hc_eps;
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

__global__ void __launch_bounds__(kHcThreads) hc_step_kernel(const HcParams p) {
  pdl_launch_dependents();
  __shared__ float tot[kHcPart];
  __shared__ int is_last;
  const int tok = blockIdx.y, D = p.D, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* hin = p.h_in + (size_t)tok * 4 * D;
  float* hout = p.h_out + (size_t)tok * 4 * D;
  float* xo = p.x_out ? p.x_out + (size_t)tok * D : nullptr;
  const int d = blockIdx.x * kHcCols + lane;
  const bool live = d < D;
  float h[4] = {0.f, 0.f, 0.f, 0.f}, hn[4], xs = 0.f, f[3][4];
  // fn is a weight: requested before the dependency wait, it arrives while the previous kernel finishes
  if (live && p.fn) {
#pragma unroll
    for (int r = 0; r < 3; r++)
#pragma unroll
      for (int i = 0; i < 4; i++) f[r][i] = __ldg(p.fn + ((size_t)(3 * warp + r) * 4 + i) * D + d);
  }
  pdl_wait();
  float mp[24];
#pragma unroll
  for (int i = 0; i < 24; i++) mp[i] = p.mix_prev[(size_t)tok * 24 + i];
  if (live) {
#pragma unroll
    for (int j = 0; j < 4; j++) h[j] = hin[(size_t)j * D + d];
    if (p.x_sub) xs = p.x_sub[(size_t)tok * D + d];
  }
  if (p.x_sub) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float a = mp[4 + i] * xs;
#pragma unroll
      for (int j = 0; j < 4; j++) a = fmaf(mp[8 + 4 * j + i], h[j], a);
      hn[i] = a;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; i++) hn[i] = h[i];
  }
  float* part = p.part + ((size_t)tok * gridDim.x + blockIdx.x) * kHcPart;
  if (p.fn) {
#pragma unroll
    for (int r = 0; r < 3; r++) {
      float a = 0.f;
      if (live) {
#pragma unroll
        for (int i = 0; i < 4; i++) a = fmaf(f[r][i], hn[i], a);
      }
      a = warp_sum(a);
      if (lane == 0) part[3 * warp + r] = a;
    }
  }
  __syncthreads();                      // every warp has read its column of h_in: warp 0 may now overwrite it
  if (warp == 0) {
    float sq = 0.f, xq = 0.f;
    if (live) {
      if (p.x_sub) {
#pragma unroll
        for (int i = 0; i < 4; i++) hout[(size_t)i * D + d] = hn[i];
      }
      sq = hn[0] * hn[0] + hn[1] * hn[1] + hn[2] * hn[2] + hn[3] * hn[3];
      if (xo) {
        const float x = mp[0] * hn[0] + mp[1] * hn[1] + mp[2] * hn[2] + mp[3] * hn[3];
        xo[d] = x;                      // scaled by the finishing block
        xq = x * x;
      }
    }
    sq = warp_sum(sq); xq = warp_sum(xq);
    if (lane == 0) { part[24] = sq; part[25] = xq; }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = atomicAdd(&p.ticket[tok], 1u) == gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // entry e = warp, warp + 8, ...: its lanes take the blocks' partials 32 at a time (loads in flight together), the
  // shuffle tree then adds them in a fixed order
  for (int e = warp; e < kHcPart; e += kHcThreads / 32) {
    double v = 0.0;
    for (unsigned b = lane; b < gridDim.x; b += 32) v += (double)__ldcg(p.part + ((size_t)tok * gridDim.x + b) * kHcPart + e);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) tot[e] = (float)v;
  }
  if (tid == 0) p.ticket[tok] = 0;
  __syncthreads();
  if (p.fn && warp == 0) {
    const float rstd = rsqrtf(tot[24] / (float)(4 * D) + 1e-20f);
    float* mo = p.mix_out + (size_t)tok * 24;
    if (lane < 4) mo[lane] = sigmoidf_(tot[lane] * rstd * p.scale[0] + p.base[lane]) + p.hc_eps;
    else if (lane < 8) mo[lane] = 2.f * sigmoidf_(tot[lane] * rstd * p.scale[1] + p.base[lane]);
    // comb: lane = 4 j + k of the 4 x 4 matrix; row sums over k (xor 1, 2), column sums over j (xor 4, 8)
    const int e = lane & 15;
    float c = tot[8 + e] * rstd * p.scale[2] + p.base[8 + e];
    float mx = fmaxf(c, __shfl_xor_sync(0xffffffffu, c, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    c = expf(c - mx);
    float s = c + __shfl_xor_sync(0xffffffffu, c, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    c = c / s + p.hc_eps;
    for (int it = 0; it < p.iters; it++) {
      if (it > 0) {
        float rs = c + __shfl_xor_sync(0xffffffffu, c, 1);
        rs += __shfl_xor_sync(0xffffffffu, rs, 2);
        c = c / (rs + p.hc_eps);
      }
      float cs = c + __shfl_xor_sync(0xffffffffu, c, 4);
      cs += __shfl_xor_sync(0xffffffffu, cs, 8);
      c = c / (cs + p.hc_eps);
    }
    if (lane < 16) mo[8 + lane] = c;
  }
  if (xo) {
    const float r = rsqrtf(tot[25] / (float)D + 1e-20f);
    for (int d = tid; d < D; d += kHcThreads) xo[d] = __ldcg(xo + d) * r * p.norm_w[d];
  }
}

size_t hc_scratch_bytes(int n) { return ((size_t)n * kHcMaxBlocks * kHcPart + (size_t)n) * 4 + 64; }

int hc_step(const float* h_in, float* h_out, const float* x_sub, const float* mix_prev, const float* fn, const float* scale,
            const float* base, float* mix_out, const float* norm_w, float* x_out, int D, int n, void* scratch,
            size_t scratch_bytes, cudaStream_t st) {
  if (D <= 0 || n <= 0 || !h_in || !mix_prev) return fail(kErrArg, "hc_step: bad arguments");
  if (x_sub && !h_out) return fail(kErrArg, "hc_step: h_out missing");
  if (fn && (!scale || !base || !mix_out)) return fail(kErrArg, "hc_step: fn needs scale, base and mix_out");
  if (x_out && !norm_w) return fail(kErrArg, "hc_step: x_out needs norm_w");
  if (mix_out == mix_prev) return fail(kErrArg, "hc_step: mix_out must not alias mix_prev");
  if (!scratch || scratch_bytes < hc_scratch_bytes(n)) return fail(kErrScratch, "hc_step: scratch too small");
  HcParams p;
  p.h_in = h_in; p.h_out = h_out ? h_out : const_cast<float*>(h_in); p.x_sub = x_sub; p.mix_prev = mix_prev; p.fn = fn;
  p.scale = scale; p.base = base; p.mix_out = mix_out; p.norm_w = norm_w; p.x_out = x_out;
  p.ticket = reinterpret_cast<unsigned*>(scratch);            // first n words: zero-filled by the caller once
  p.part = reinterpret_cast<float*>(scratch) + ((n + 15) & ~15);
  p.D = D; p.n = n; p.iters = 20; p.hc_eps = 1e-6f;
  if (D > kHcMaxBlocks * kHcCols) return fail(kErrLimit, "hc_step: D %d beyond %d", D, kHcMaxBlocks * kHcCols);
  const int blocks = (D + kHcCols - 1) / kHcCols;
  MSB_CUDA(launch_pdl(hc_step_kernel, dim3(blocks, n), dim3(kHcThreads), 0, st, p));
  MSB_LAUNCH_CHECK("hc_step_kernel");
  return kOk;
}

}  // namespace msb
