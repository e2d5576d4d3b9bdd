// Small per-token kernels that sit between the hot-path calls of a decode layer: RMSNorm, the window KV row
// (RMSNorm + rope + optional fp8 quant-dequant simulation + store), greedy argmax and vector add.
// Counterparts in the reference: arch_rmsnorm / arch_argmax (src/kernels/arch.hpp:99-130, arch_sample.metal),
// attn_kv_window (src/kernels/attn_kv.metal:19-60) with the math of tests/ref/attn_ref.cpp:58-63,79-89,109-114.
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

// y[r] = x[r] * rsqrt(mean(x[r]^2) + eps) * w   (w may be null); one block per row
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* x, const float* w, float* y, int dim, float eps,
                                                      int in_stride, int out_stride) {
  __shared__ float sh[32];
  const float* xr = x + (size_t)blockIdx.x * in_stride;
  float* yr = y + (size_t)blockIdx.x * out_stride;
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

// greedy argmax, ties -> lowest index; single block
__global__ void __launch_bounds__(1024) argmax_kernel(const float* x, int n, int* out_idx, float* out_val) {
  __shared__ float sv[32];
  __shared__ int si[32];
  float bv = -INFINITY;
  int bi = 0x7fffffff;
#pragma unroll 8
  for (int i = threadIdx.x; i < n; i += blockDim.x) {   // ascending i per thread: a strict compare keeps the lowest index
    const float v = x[i];
    if (v > bv || bi == 0x7fffffff) { bv = v; bi = i; }
  }
  auto better = [](float v, int i, float w, int j) { return v > w || (v == w && i < j); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); w++)
      if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
    *out_idx = bi;
    if (out_val) *out_val = bv;
  }
}

__global__ void add_kernel(float* y, const float* a, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] += a[i];
}

int rmsnorm(const float* x, const float* w, float* y, int rows, int dim, float eps, int in_stride, int out_stride,
            cudaStream_t st) {
  if (rows <= 0 || dim <= 0 || !x || !y) return fail(kErrArg, "rmsnorm: bad arguments");
  rmsnorm_kernel<<<rows, 256, 0, st>>>(x, w, y, dim, eps, in_stride ? in_stride : dim, out_stride ? out_stride : dim);
  MSB_LAUNCH_CHECK("rmsnorm_kernel");
  return kOk;
}
int kv_window(const float* kv, const float* norm_w, const float* cs, int actq, int D, int elem_type, void* out_row,
              cudaStream_t st) {
  if (D <= 0 || D % 32 || D > 1024 || D < 64 || !kv || !norm_w || !cs || !out_row) return fail(kErrArg, "kv_window: bad arguments");
  if (elem_type == BF16) kv_window_kernel<true><<<1, D, D * sizeof(float), st>>>(kv, norm_w, cs, actq, D, out_row);
  else if (elem_type == F16) kv_window_kernel<false><<<1, D, D * sizeof(float), st>>>(kv, norm_w, cs, actq, D, out_row);
  else return fail(kErrType, "kv_window: rows must be F16 or BF16");
  MSB_LAUNCH_CHECK("kv_window_kernel");
  return kOk;
}
int argmax(const float* x, int n, int* out_idx, float* out_val, cudaStream_t st) {
  if (n <= 0 || !x || !out_idx) return fail(kErrArg, "argmax: bad arguments");
  argmax_kernel<<<1, 1024, 0, st>>>(x, n, out_idx, out_val);
  MSB_LAUNCH_CHECK("argmax_kernel");
  return kOk;
}
int vec_add(float* y, const float* a, int n, cudaStream_t st) {
  if (n <= 0 || !y || !a) return fail(kErrArg, "add: bad arguments");
  add_kernel<<<(n + 255) / 256, 256, 0, st>>>(y, a, n);
  MSB_LAUNCH_CHECK("add_kernel");
  return kOk;
}

}  // namespace msb
