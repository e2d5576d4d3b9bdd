// KV compressor + index key of one decode token -- ms::attn::encode_compress for n == 1 (src/kernels/attn.hpp:118,
// kernels src/kernels/attn_kv.metal:62-145); math as tests/ref/attn_ref.cpp:116-161:
//   ratio 1: latent = c_kv;  ratio r > 1: the token's (c_kv, c_gate) go to slot pos % r of the source's partial group and,
//   when the group is complete, latent[c] = sum_j kv[j][c] * softmax_j(gate[j][c])
//   latent = rmsnorm(latent) * c_norm
//   key    = rope(rmsnorm(Wk . latent) * k_norm)  -> fp4 (e2m1, ue8m0 scale per 32) simulation when actq -> ikey row
//   latent = rope(latent)                         -> fp4 (e2m1, e4m3 scale per 16) simulation when actq -> ckv row
// One block per call (the work is 128 x D MACs on a 128 KB bf16 matrix plus a few vector passes); rows land at index
// pos / r of the source's caches in the caches' element types.
#include <cuda_fp8.h>
#include "msb_common.cuh"

namespace msb {

constexpr int kCmpThreads = 512;
constexpr int kCmpMaxD = 1024;
constexpr int kKeyFp8 = 101;

struct CmpParams {
  const float* c_kv;      // [D]
  const float* c_gate;    // [D] (ratio > 1)
  const float* c_norm;    // [D]
  const uint16_t* wk;     // bf16 [ID][D]
  const float* k_norm;    // [ID]
  const float* cs;        // (cos, sin)[32] of position (pos / ratio) * ratio
  float* st;              // [2][ratio][D]: kv then gate scores of the partial group
  void* ckv_row;          // D elements of elem_type
  void* ikey_row;         // ID elements of key_type
  int D, ID, ratio, slot, emit, actq, elem_type, key_type;
};

__device__ __forceinline__ float bsum(float v, float* sh) {      // sum over the block, same order in every thread
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < kCmpThreads / 32; i++) t += sh[i];
  __syncthreads();
  return t;
}
__device__ __forceinline__ int floor_log2f_(float a) { return (int)((__float_as_uint(a) >> 23) & 0xFF) - 127; }
__device__ __forceinline__ int log2_ceilf_(float x) {
  const uint32_t b = __float_as_uint(x);
  return (int)((b >> 23) & 0xFF) - 127 + ((b & 0x7FFFFF) ? 1 : 0);
}
__device__ __forceinline__ float pow2f_(int e) { return __uint_as_float((uint32_t)(e + 127) << 23); }
__device__ __forceinline__ float round_e4m3_(float x) {          // attn_ref.cpp:69-74
  const float a = fabsf(x);
  const int e = max(floor_log2f_(a), -6);
  return copysignf(rintf(a * pow2f_(3 - e)) * pow2f_(e - 3), x);
}
__device__ __forceinline__ float round_e2m1_(float x) {          // attn_ref.cpp:75-80
  const float a = fabsf(x);
  const int e = max(floor_log2f_(a), 0);
  return copysignf(rintf(a * pow2f_(1 - e)) * pow2f_(e - 1), x);
}
__device__ __forceinline__ void store_elem(void* row, int i, float v, int type) {
  if (type == F16) reinterpret_cast<__half*>(row)[i] = __float2half_rn(v);
  else if (type == BF16) reinterpret_cast<__nv_bfloat16*>(row)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__nv_fp8_e4m3*>(row)[i] = __nv_fp8_e4m3(v);
}

__global__ void __launch_bounds__(kCmpThreads) compress_kernel(const CmpParams p) {
  pdl_launch_dependents();
  __shared__ float lat[kCmpMaxD];
  __shared__ float key[256];
  __shared__ float sh[kCmpThreads / 32];
  const int tid = threadIdx.x, D = p.D, ID = p.ID, r = p.ratio;
  pdl_wait();
  if (r > 1) {
    for (int c = tid; c < D; c += kCmpThreads) {
      p.st[(size_t)p.slot * D + c] = p.c_kv[c];
      p.st[(size_t)(r + p.slot) * D + c] = p.c_gate[c];
    }
    if (!p.emit) return;
    __syncthreads();
    for (int c = tid; c < D; c += kCmpThreads) {
      float m = -INFINITY, e[8], sum = 0.f, v = 0.f;
      for (int j = 0; j < r; j++) m = fmaxf(m, p.st[(size_t)(r + j) * D + c]);
      for (int j = 0; j < r; j++) { e[j] = expf(p.st[(size_t)(r + j) * D + c] - m); sum += e[j]; }
      for (int j = 0; j < r; j++) v += p.st[(size_t)j * D + c] * (e[j] / sum);
      lat[c] = v;
    }
  } else {
    for (int c = tid; c < D; c += kCmpThreads) lat[c] = p.c_kv[c];
  }
  __syncthreads();
  float ss = 0.f;
  for (int c = tid; c < D; c += kCmpThreads) ss += lat[c] * lat[c];
  ss = bsum(ss, sh);
  const float rl = 1.0f / sqrtf(ss / (float)D + 1e-20f);
  for (int c = tid; c < D; c += kCmpThreads) lat[c] = p.c_norm[c] * (lat[c] * rl);
  __syncthreads();
  // index key: one warp per output row, lanes over the latent (pre-rope)
  for (int o = tid >> 5; o < ID; o += kCmpThreads / 32) {
    const uint16_t* w = p.wk + (size_t)o * D;
    float a = 0.f;
    for (int d = (tid & 31) * 2; d < D; d += 64) {
      const uint32_t pr = *reinterpret_cast<const uint32_t*>(w + d);
      a = fmaf(__uint_as_float(pr << 16), lat[d], a);
      a = fmaf(__uint_as_float(pr & 0xFFFF0000u), lat[d + 1], a);
    }
    a = warp_sum(a);
    if ((tid & 31) == 0) key[o] = a;
  }
  __syncthreads();
  float ks = 0.f;
  for (int o = tid; o < ID; o += kCmpThreads) ks += key[o] * key[o];
  ks = bsum(ks, sh);
  const float rk = 1.0f / sqrtf(ks / (float)ID + 1e-20f);
  for (int o = tid; o < ID; o += kCmpThreads) key[o] = p.k_norm[o] * (key[o] * rk);
  __syncthreads();
  // rope on the last 64 dims of both vectors (pairs (2i, 2i+1), attn_ref.cpp:46-53)
  if (tid < 32) {
    const float c = p.cs[2 * tid], s = p.cs[2 * tid + 1];
    float* x = key + ID - 64;
    const float a = x[2 * tid], b = x[2 * tid + 1];
    x[2 * tid] = a * c - b * s; x[2 * tid + 1] = a * s + b * c;
  } else if (tid < 64) {
    const int i = tid - 32;
    const float c = p.cs[2 * i], s = p.cs[2 * i + 1];
    float* x = lat + D - 64;
    const float a = x[2 * i], b = x[2 * i + 1];
    x[2 * i] = a * c - b * s; x[2 * i + 1] = a * s + b * c;
  }
  __syncthreads();
  if (p.actq) {
    // key: fp4 e2m1 with a power-of-two scale per 32 elements (attn_ref.cpp:92-100): one warp per group
    for (int g = tid >> 5; g < ID / 32; g += kCmpThreads / 32) {
      const float v = key[32 * g + (tid & 31)];
      float amax = warp_max(fabsf(v));
      amax = fmaxf(amax, 6.0f * 1.17549435e-38f);
      const int e = log2_ceilf_(amax * (1.0f / 6.0f));
      const float s = pow2f_(e), inv = pow2f_(-e);
      key[32 * g + (tid & 31)] = round_e2m1_(fminf(fmaxf(v * inv, -6.0f), 6.0f)) * s;
    }
    // latent: fp4 e2m1 with an e4m3 scale per 16 elements (attn_ref.cpp:101-108): 16 lanes per group
    for (int c = tid; c < D; c += kCmpThreads) {
      const float v = lat[c];
      float amax = fabsf(v);
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      amax = fmaxf(amax, 6.0f * 0.001953125f);
      const float s = round_e4m3_(fminf(amax / 6.0f, 448.0f));
      lat[c] = round_e2m1_(fminf(fmaxf(v / s, -6.0f), 6.0f)) * s;
    }
    __syncthreads();
  }
  for (int o = tid; o < ID; o += kCmpThreads) store_elem(p.ikey_row, o, key[o], p.key_type == kKeyFp8 ? kKeyFp8 : F16);
  for (int c = tid; c < D; c += kCmpThreads) store_elem(p.ckv_row, c, lat[c], p.elem_type);
}

int compress_token(const float* c_kv, const float* c_gate, const float* c_norm, const void* wk_bf16, const float* k_norm,
                   const float* cs, float* state, int ratio, int pos, int actq, int D, int ID, int elem_type, void* ckv_rows,
                   int key_type, void* ikey_rows, cudaStream_t st) {
  if (ratio < 1 || ratio > 8 || D <= 0 || D > kCmpMaxD || (D % 64) || ID < 64 || ID > 256 || (ID % 32) || pos < 0)
    return fail(kErrArg, "compress: bad shape (ratio %d D %d ID %d)", ratio, D, ID);
  if (!c_kv || !c_norm || !wk_bf16 || !k_norm || !cs || !ckv_rows || !ikey_rows || (ratio > 1 && (!c_gate || !state)))
    return fail(kErrArg, "compress: null pointer");
  if (elem_type != F16 && elem_type != BF16) return fail(kErrType, "compress: rows must be F16 or BF16");
  if (key_type != F16 && key_type != kKeyFp8) return fail(kErrType, "compress: keys must be F16 or FP8 E4M3");
  CmpParams p;
  p.c_kv = c_kv; p.c_gate = c_gate; p.c_norm = c_norm; p.wk = (const uint16_t*)wk_bf16; p.k_norm = k_norm; p.cs = cs;
  p.st = state; p.D = D; p.ID = ID; p.ratio = ratio; p.slot = pos % ratio; p.emit = (pos + 1) % ratio == 0; p.actq = actq;
  p.elem_type = elem_type; p.key_type = key_type;
  const size_t row = (size_t)(pos / ratio);
  p.ckv_row = (char*)ckv_rows + row * D * 2;
  p.ikey_row = (char*)ikey_rows + row * ID * (key_type == kKeyFp8 ? 1 : 2);
  MSB_CUDA(launch_pdl(compress_kernel, dim3(1), dim3(kCmpThreads), 0, st, p));
  MSB_LAUNCH_CHECK("compress_kernel");
  return kOk;
}

}  // namespace msb
