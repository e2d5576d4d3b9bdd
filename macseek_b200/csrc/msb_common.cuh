// Shared device/host helpers of libmacseek_b200: status reporting, bounded mbarrier waits, 1-D TMA bulk copies,
// dp4a wrappers and the shared-memory codebook tables of the IQ formats.  sm_100a only.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>

namespace msb {

// ---------------------------------------------------------------- host-side status
// Every C entry point returns 0 on success or a negative MSB_E_* code; the text of the last failure of the calling
// thread is kept for msb_last_error().
enum : int { kOk = 0, kErrArg = -1, kErrType = -2, kErrCuda = -3, kErrScratch = -4, kErrDevice = -5, kErrLimit = -6 };
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
#define MSB_CUDA(expr)                                                    \
  do {                                                                    \
    cudaError_t _e = (expr);                                              \
    if (_e != cudaSuccess) return ::msb::cuda_fail(_e, #expr);            \
  } while (0)
#define MSB_LAUNCH_CHECK(name)                                            \
  do {                                                                    \
    cudaError_t _e = cudaGetLastError();                                  \
    if (_e != cudaSuccess) return ::msb::cuda_fail(_e, name);             \
  } while (0)

// Launch with programmatic dependent launch allowed: the grid may be scheduled while the previous kernel of the stream
// is still draining; every kernel of this library calls pdl_wait() before it touches anything a previous kernel wrote
// (and before it writes anything), so only set-up work overlaps.  MSB_PDL=0 turns the attribute off.
bool pdl_enabled();
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

// ggml type ids (the reference's ms::q::QType, src/kernels/quant_types.hpp:10-12)
enum QType : int { F32 = 0, F16 = 1, Q8_0 = 8, Q5_K = 13, Q6_K = 14, IQ2_XXS = 16, IQ1_S = 19, IQ4_NL = 20, BF16 = 30 };
__host__ __device__ constexpr int block_elems(int t) {
  return (t == F32 || t == F16 || t == BF16) ? 1 : (t == Q8_0 || t == IQ4_NL) ? 32 : 256;
}
__host__ __device__ constexpr int block_bytes(int t) {
  return t == F32 ? 4 : (t == F16 || t == BF16) ? 2 : t == Q8_0 ? 34 : t == Q5_K ? 176 : t == Q6_K ? 210
       : t == IQ2_XXS ? 66 : t == IQ1_S ? 50 : t == IQ4_NL ? 18 : 0;
}
inline bool type_known(int t) { return block_bytes(t) != 0; }
__host__ __device__ inline size_t row_bytes(int t, int64_t cols) { return (size_t)(cols / block_elems(t)) * block_bytes(t); }
const char* type_name(int t);

// device-side failure word (one int per device, Tables::status): set by a kernel whose bounded wait ran out; read by
// msb_device_status()
enum : int { kDevOk = 0, kDevWaitFull = 1, kDevWaitEmpty = 2, kDevPeerWait = 3 };

// ---------------------------------------------------------------- device primitives
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~1 s of SM clock, records `code` in the device status word and raises *abort so that
// every later wait of the block returns at once.  Returns false when the wait was abandoned.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;    // fast path: no flag read, no clock read
  if (*abort_flag) return false;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; i++)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > 2000000000LL) {
      *abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
}
// The same bounded wait for a warp whose wake-up is not urgent (an epilogue warp waiting for a whole tile, a copy thread
// waiting for a free slot): it sleeps `ns` between polls, so that its polling takes neither issue slots nor
// shared-memory cycles from the warps that do the work meanwhile.
__device__ __forceinline__ bool mbar_wait_sleep(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                int code, unsigned ns) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; i++) {
      if (mbar_try_wait(bar, parity)) return true;
      __nanosleep(ns);
    }
    if (*abort_flag) return false;
    if (clock64() - t0 > 2000000000LL) {
      *abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
}
// 1-D bulk copy global -> shared through the TMA engine; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void tma_load_1d(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
  int d; asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {   // a signed bytes, b unsigned bytes
  int d; asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {   // a unsigned bytes, b signed bytes
  int d; asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
  uint32_t d; asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"((uint32_t)c)); return (int)d;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Programmatic dependent launch: let the next kernel of the stream start its prologue / wait for the previous one.
// barrier over a subset of the block's warps (the producer warp of a streaming kernel never joins the consumers')
__device__ __forceinline__ void bar_sync_named(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif  // __CUDACC__

// ---------------------------------------------------------------- codebook tables (global memory, built at init)
// Plain tables (dequant kernels):
//   IQ2_XXS: 256 x uint2 (8 unsigned bytes 8/25/43);  signs: 128 x uint2 (byte 0xFF where the element is negative).
//   IQ4_NL : 256 x u16: low byte = value of the low nibble, high byte = value of the high nibble.
//   IQ1_S  : 2048 x 8 int8 values.
// Shared-memory images (dot kernels), already replicated per bank group so that one bulk copy fills the block's LUT
// (4-bit codes, eight per word; layouts in quant_blocks.cuh):
//   img_iq1s  [2048][8 copies] u32                                               (64 KB)
//   img_iq2g  [256][32 copies] u32, img_iq2s [128][32 copies] u32                (32 KB + 16 KB)
//   img_iq4   [256][8 copies]  u32 (byte pair in the low 16 bits)               (8 KB)
struct Tables {
  const uint2* iq2xxs_grid;    // [256]
  const uint2* iq2_signmask;   // [128]
  const uint16_t* iq4nl_pair;  // [256]
  const int8_t* iq1s_i8;       // [2048][8]
  const uint2* iq2_sel;        // [256] the same selectors for the IQ2_XXS grid (codes 0..2 = magnitudes 8, 25, 43)
  const uint4* iq2_sign16;     // [128] sign words for 8 halfs (0x8000 in the half of a negative element)
  const uint2* iq1s_sel;       // [2048] four 16-bit byte-permute selectors per entry: pair j of the entry's 8 codes picks
                               // two halfs out of the pool {h(code 0), h(code 1), h(code 2)} (MoE prefill weight producers)
  const uint8_t* img_iq1s;
  const uint8_t* img_iq2g;
  const uint8_t* img_iq2s;
  const uint8_t* img_iq4;
  int* status;                 // device failure word (kDev*) followed by library-owned scheduling counters
};
// Builds the tables on the current device the first time it is called for that device.
int get_tables(Tables* out);
bool tables_ready();
constexpr int kNoAllocMaxInter = 4096;                       // msb_moe_decode_noalloc: widest expert its scratch serves
constexpr int kNoAllocFloats = (16 + 1) * kNoAllocMaxInter;  // (max routed + shared) h rows
float* noalloc_scratch(size_t* bytes);

}  // namespace msb
