// Small per-token kernels that sit between the hot-path calls of a decode layer: RMSNorm, the window KV row
// (RMSNorm + rope + optional fp8 quant-dequant simulation + store), greedy argmax and vector add.
// Counterparts in the reference: arch_rmsnorm / arch_argmax (src/kernels/arch.hpp:99-130, arch_sample.metal),
// attn_kv_window (src/kernels/attn_kv.metal:19-60) with the math of tests/ref/attn_ref.cpp:58-63,79-89,109-114.
#include <algorithm>
#include "msb_common.cuh"

namespace msb {

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; i++) t += sh[i];     // same order in every thread
  __syncthreads();
  return t;
}

// y[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * w   (w may be null); one block per row.  Rows of up to 8192 elements
// (16-byte aligned, dim % 4 == 0) are held in registers: every load is issued before the first use, so the row costs
// one memory latency instead of one per loop trip.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* x, const float* w, float* y, int dim, float eps,
                                                      int in_stride, int out_stride) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[32];
  const float* xr = x + (size_t)blockIdx.x * in_stride;
  float* yr = y + (size_t)blockIdx.x * out_stride;
  const bool vec = (dim & 3) == 0 && dim <= 8192 && ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(yr) |
                                                      reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  if (vec) {
    const int n4 = dim >> 2;
    float4 v[8], g[8];
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const int i = threadIdx.x + 256 * k;
      v[k] = i < n4 ? reinterpret_cast<const float4*>(xr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      g[k] = (w && i < n4) ? reinterpret_cast<const float4*>(w)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    ss = block_sum(ss, sh);
    const float r = rsqrtf(ss / (float)dim + eps);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      const int i = threadIdx.x + 256 * k;
      if (i < n4) reinterpret_cast<float4*>(yr)[i] = make_float4(v[k].x * r * g[k].x, v[k].y * r * g[k].y, v[k].z * r * g[k].z, v[k].w * r * g[k].w);
    }
    return;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) ss += xr[i] * xr[i];
  ss = block_sum(ss, sh);
  const float r = rsqrtf(ss / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) yr[i] = xr[i] * r * (w ? w[i] : 1.f);
}

__device__ __forceinline__ float pw2(int e) { return __uint_as_float((uint32_t)(e + 127) << 23); }
__device__ __forceinline__ float round_e4m3_dev(float x) {
  const float a = fabsf(x);
  int e = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;
  e = max(e, -6);
  return copysignf(nearbyintf(a * pw2(3 - e)) * pw2(e - 3), x);
}

// One token: out_row[D] = E( fp8sim( rope_last64( rmsnorm(kv) * norm_w ) ) ); D threads, D a multiple of 32.
template <bool BF>
__global__ void kv_window_kernel(const float* kv, const float* norm_w, const float* cs, int actq, int D, void* out_row) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[32];
  extern __shared__ float v[];
  const int d = threadIdx.x;
  const float x = kv[d];
  const float ss = block_sum(x * x, sh);
  const float r = 1.0f / sqrtf(ss / (float)D + 1e-20f);
  v[d] = norm_w[d] * (x * r);
  __syncthreads();
  float o = v[d];
  if (d >= D - 64) {
    const int i = (d - (D - 64)) >> 1;
    const float c = cs[2 * i], s = cs[2 * i + 1];
    const float a = v[d & ~1], b = v[d | 1];
    o = (d & 1) ? __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)) : __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
  }
  if (actq) {   // block of 32 = one warp: amax -> power-of-two scale -> e4m3 rounding
    float amax = fabsf(o);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    amax = fmaxf(amax, 1e-4f);
    const float q = __fmul_rn(amax, 1.0f / 448.0f);
    const uint32_t qb = __float_as_uint(q);
    const int e = (int)((qb >> 23) & 0xFF) - 127 + ((qb & 0x7FFFFF) ? 1 : 0);
    o = __fmul_rn(round_e4m3_dev(fminf(fmaxf(__fmul_rn(o, pw2(-e)), -448.f), 448.f)), pw2(e));
  }
  if (BF) reinterpret_cast<__nv_bfloat16*>(out_row)[d] = __float2bfloat16_rn(o);
  else reinterpret_cast<__half*>(out_row)[d] = __float2half_rn(o);
}

// greedy argmax, ties -> lowest index.  Each block scans a contiguous slice with 8 independent loads per thread in
// flight, writes its best (value, index), and the block that finishes last reduces the per-block results.
__device__ __forceinline__ bool better(float v, int i, float w, int j) { return v > w || (v == w && i < j); }
__global__ void __launch_bounds__(256) argmax_kernel(const float* x, int n, int* out_idx, float* out_val, float* pv, int* pi,
                                                     unsigned* ticket) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ int is_last;
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int i0 = blockIdx.x * per, i1 = min(n, i0 + per);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int base = i0 + threadIdx.x; base < i1; base += 256 * 8) {
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = base + 256 * k < i1 ? x[base + 256 * k] : -INFINITY;
#pragma unroll
    for (int k = 0; k < 8; k++)
      if (base + 256 * k < i1 && (v[k] > bv || bi == 0x7fffffff)) { bv = v[k]; bi = base + 256 * k; }
  }
  auto warp_best = [&]() {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
  };
  warp_best();
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; w++)
      if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
    pv[blockIdx.x] = bv; pi[blockIdx.x] = bi;
    __threadfence();
    is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  bv = -INFINITY; bi = 0x7fffffff;
  for (int b = threadIdx.x; b < (int)gridDim.x; b += 256) {
    const float v = reinterpret_cast<volatile float*>(pv)[b];
    const int i = reinterpret_cast<volatile int*>(pi)[b];
    if (better(v, i, bv, bi)) { bv = v; bi = i; }
  }
  warp_best();
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; w++)
      if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
    *out_idx = bi;
    if (out_val) *out_val = bv;
    *ticket = 0;
  }
}

__global__ void add_kernel(float* y, const float* a, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] += a[i];
}

int rmsnorm(const float* x, const float* w, float* y, int rows, int dim, float eps, int in_stride, int out_stride,
            cudaStream_t st) {
  if (rows <= 0 || dim <= 0 || !x || !y) return fail(kErrArg, "rmsnorm: bad arguments");
  MSB_CUDA(launch_pdl(rmsnorm_kernel, dim3(rows), dim3(256), 0, st, x, w, y, dim, eps, in_stride ? in_stride : dim, out_stride ? out_stride : dim));
  MSB_LAUNCH_CHECK("rmsnorm_kernel");
  return kOk;
}
int kv_window(const float* kv, const float* norm_w, const float* cs, int actq, int D, int elem_type, void* out_row,
              cudaStream_t st) {
  if (D <= 0 || D % 32 || D > 1024 || D < 64 || !kv || !norm_w || !cs || !out_row) return fail(kErrArg, "kv_window: bad arguments");
  if (elem_type == BF16) MSB_CUDA(launch_pdl(kv_window_kernel<true>, dim3(1), dim3(D), D * sizeof(float), st, kv, norm_w, cs, actq, D, out_row));
  else if (elem_type == F16) MSB_CUDA(launch_pdl(kv_window_kernel<false>, dim3(1), dim3(D), D * sizeof(float), st, kv, norm_w, cs, actq, D, out_row));
  else return fail(kErrType, "kv_window: rows must be F16 or BF16");
  MSB_LAUNCH_CHECK("kv_window_kernel");
  return kOk;
}
int argmax(const float* x, int n, int* out_idx, float* out_val, cudaStream_t st) {
  if (n <= 0 || !x || !out_idx) return fail(kErrArg, "argmax: bad arguments");
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  // library-owned partials (128 blocks) and ticket live behind the status word
  float* pv = reinterpret_cast<float*>(tb.status + 64);
  int* pi = tb.status + 64 + 128;
  unsigned* ticket = reinterpret_cast<unsigned*>(tb.status) + 20;
  const int blocks = std::max(1, std::min(128, (n + 2047) / 2048));
  MSB_CUDA(launch_pdl(argmax_kernel, dim3(blocks), dim3(256), 0, st, x, n, out_idx, out_val, pv, pi, ticket));
  MSB_LAUNCH_CHECK("argmax_kernel");
  return kOk;
}
int vec_add(float* y, const float* a, int n, cudaStream_t st) {
  if (n <= 0 || !y || !a) return fail(kErrArg, "add: bad arguments");
  MSB_CUDA(launch_pdl(add_kernel, dim3((n + 255) / 256), dim3(256), 0, st, y, a, n));
  MSB_LAUNCH_CHECK("add_kernel");
  return kOk;
}

}  // namespace msb
