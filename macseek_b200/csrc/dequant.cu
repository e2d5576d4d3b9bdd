// Exact dequantisation of raw GGUF blocks to fp32: out[i] is bit-identical with the reference's CPU routine
// ref::dequant_row (tests/ref/dequant.cpp:34-120).  One thread decodes 8 consecutive elements.
#include "quant_blocks.cuh"

namespace msb {

template <int T>
__global__ void dequant_kernel(const uint8_t* __restrict__ src, float* __restrict__ out, int64_t n8, Tables tb) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  constexpr int per_block = block_elems(T) / 8;
  const uint8_t* blk = src + (i / per_block) * block_bytes(T);
  float y[8];
  dequant8<T>(blk, (int)(i % per_block), tb, y);
  float4* o = reinterpret_cast<float4*>(out + 8 * i);
  o[0] = make_float4(y[0], y[1], y[2], y[3]);
  o[1] = make_float4(y[4], y[5], y[6], y[7]);
}

// dense types: plain widening copies
__global__ void widen_kernel(const uint8_t* __restrict__ src, float* __restrict__ out, int64_t n, int t) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (t == F32) out[i] = reinterpret_cast<const float*>(src)[i];
  else if (t == F16) out[i] = __half2float(reinterpret_cast<const __half*>(src)[i]);
  else out[i] = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(src)[i] << 16);
}

int dequant(int t, const void* src, int64_t n, float* out, cudaStream_t st) {
  if (!type_known(t)) return fail(kErrType, "dequant: unsupported type %d", t);
  if (n < 0 || n % block_elems(t) != 0 || (block_elems(t) == 1 ? 0 : n % 8) != 0)
    return fail(kErrArg, "dequant: %lld elements is not a whole number of %s blocks", (long long)n, type_name(t));
  if (n == 0) return kOk;
  if (!src || !out || (reinterpret_cast<uintptr_t>(out) & 15)) return fail(kErrArg, "dequant: bad pointer");
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  const int threads = 256;
  if (is_dense(t)) {
    MSB_CUDA(launch_pdl(widen_kernel, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, st, (const uint8_t*)src, out, n, t));
  } else {
    const int64_t n8 = n / 8;
    const unsigned grid = (unsigned)((n8 + threads - 1) / threads);
    const uint8_t* s = (const uint8_t*)src;
    switch (t) {
      case Q8_0: dequant_kernel<Q8_0><<<grid, threads, 0, st>>>(s, out, n8, tb); break;
      case Q5_K: dequant_kernel<Q5_K><<<grid, threads, 0, st>>>(s, out, n8, tb); break;
      case Q6_K: dequant_kernel<Q6_K><<<grid, threads, 0, st>>>(s, out, n8, tb); break;
      case IQ2_XXS: dequant_kernel<IQ2_XXS><<<grid, threads, 0, st>>>(s, out, n8, tb); break;
      case IQ1_S: dequant_kernel<IQ1_S><<<grid, threads, 0, st>>>(s, out, n8, tb); break;
      case IQ4_NL: dequant_kernel<IQ4_NL><<<grid, threads, 0, st>>>(s, out, n8, tb); break;
      default: return fail(kErrType, "dequant: unsupported type %d", t);
    }
  }
  MSB_LAUNCH_CHECK("dequant_kernel");
  return kOk;
}

}  // namespace msb
