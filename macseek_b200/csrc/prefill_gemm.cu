// Prefill projection GEMM on the 5th-generation tensor cores:  Y[n x rows] (+)= X16[n x cols] . W^T
// Replaces the reference's q_mm / q_mm_dense / q_deq_f16 Metal kernels (src/kernels/quant_mm.metal:87-154) behind
// ms::q::encode_matmul / encode_matmul_h / encode_f32_to_f16 (src/kernels/quant.hpp:37-46, quant.mm:189-248).
// Same arithmetic as the reference: activations and weights as half operands, fp32 accumulation.
//
// The quantised weight matrix is first dequantised to half (exactly the reference's values, rounded to half once) into
// caller-provided scratch, as the reference does for n >= 512 (quant.mm:225-240); the contraction is then one
// persistent kernel: TMA tensor tiles (128-byte swizzle) of X16 [128 tokens x 64] and W16 [128 rows x 64] ->
// tcgen05.mma kind::f16 (M 128, N 128, K 16) -> 128 x 128 fp32 accumulators in TMEM (two, so the epilogue of one tile
// overlaps the main loop of the next) -> tcgen05.ld -> Y.  Warp roles: warps 0..3 epilogue, warp 4 one MMA-issuing
// thread, warp 5 one TMA-issuing thread.  Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>
#include <algorithm>
#include "quant_blocks.cuh"

namespace msb {

constexpr int kGmBM = 128, kGmBN = 256, kGmBK = 64;          // tile: tokens x weight rows x contraction (halfs)
constexpr int kGmABytes = kGmBM * kGmBK * 2, kGmBBytes = kGmBN * kGmBK * 2;
constexpr int kGmStages = 4;
constexpr int kGmThreads = 6 * 32;

struct GemmParams {
  CUtensorMap a_map;   // X16 [n][cols] half, box 64 x 128
  CUtensorMap b_map;   // W16 [rows][cols] half, box 64 x 128
  float* y;            // [n][rows]
  int* status;
  int n, rows, cols, accumulate;
};

struct GemmHead {
  uint64_t full[kGmStages], empty[kGmStages], accfull[2], accempty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint64_t gm_desc(uint32_t saddr) {   // K-major, 128-byte swizzle, 8-row groups 1024 B apart
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void gm_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void gm_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void gm_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void gm_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void gm_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void gm_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void gm_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(kGmThreads, 1) gemm_tc_kernel(const __grid_constant__ GemmParams p) {
  pdl_launch_dependents();
  extern __shared__ __align__(1024) uint8_t gm_smem_raw[];
  uint8_t* smem = gm_smem_raw + ((1024u - (smem_u32(gm_smem_raw) & 1023u)) & 1023u);   // swizzled tiles: 1024-byte aligned
  GemmHead* hd = reinterpret_cast<GemmHead*>(smem);
  uint8_t* stage0 = smem + 1024;                                   // per stage: A tile then B tile
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr uint32_t kCols = 2 * kGmBN;

  if (tid == 0) {
    for (int s = 0; s < kGmStages; s++) { mbar_init(&hd->full[s], 1); mbar_init(&hd->empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&hd->accfull[b], 1); mbar_init(&hd->accempty[b], 4); }
    hd->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&hd->tmem_base)), "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  gm_fence_before();
  __syncthreads();
  gm_fence_after();
  const uint32_t tmem = hd->tmem_base;
  volatile int* abort_flag = &hd->abort_flag;
  const int mt = (p.n + kGmBM - 1) / kGmBM, nt = (p.rows + kGmBN - 1) / kGmBN, kb = (p.cols + kGmBK - 1) / kGmBK;
  const int ntiles = mt * nt;
  const int my_tiles = ntiles > (int)blockIdx.x ? (ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  pdl_wait();   // X16 (and W16) come from kernels that ran before

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0) {
      uint32_t it = 0;
      for (int i = 0; i < my_tiles; i++) {
        const int tile = (int)blockIdx.x + i * (int)gridDim.x;
        const int m = tile % mt, nn = tile / mt;     // token tiles fastest: neighbouring CTAs share a weight tile
        bool ok = true;
        for (int k = 0; k < kb; k++, it++) {
          const int s = it % kGmStages;
          if (!mbar_wait(&hd->empty[s], ((it / kGmStages) & 1u) ^ 1u, abort_flag, p.status, kDevWaitEmpty)) { ok = false; break; }
          uint8_t* slot = stage0 + (size_t)s * (kGmABytes + kGmBBytes);
          mbar_arrive_expect_tx(&hd->full[s], kGmABytes + kGmBBytes);
          gm_tma_2d(slot, &p.a_map, k * kGmBK, m * kGmBM, &hd->full[s]);
          gm_tma_2d(slot + kGmABytes, &p.b_map, k * kGmBK, nn * kGmBN, &hd->full[s]);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      // instruction descriptor: D fp32, A and B f16, both K-major, N = 128, M = 128
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(kGmBN >> 3) << 17) | ((uint32_t)(kGmBM >> 4) << 24);
      uint32_t it = 0;
      for (int i = 0; i < my_tiles; i++) {
        const int buf = i & 1;
        if (!mbar_wait(&hd->accempty[buf], ((i >> 1) & 1u) ^ 1u, abort_flag, p.status, kDevWaitEmpty)) break;
        bool ok = true;
        for (int k = 0; k < kb; k++, it++) {
          const int s = it % kGmStages;
          if (!mbar_wait(&hd->full[s], (it / kGmStages) & 1u, abort_flag, p.status, kDevWaitFull)) { ok = false; break; }
          gm_fence_after();
          const uint32_t a_s = smem_u32(stage0 + (size_t)s * (kGmABytes + kGmBBytes)), b_s = a_s + kGmABytes;
#pragma unroll
          for (int ks = 0; ks < kGmBK / 16; ks++)     // K = 16 halfs = 32 bytes per instruction
            gm_mma_f16(tmem + (uint32_t)(buf * kGmBN), gm_desc(a_s + ks * 32), gm_desc(b_s + ks * 32), idesc,
                       (k > 0 || ks > 0) ? 1u : 0u);
          gm_commit(&hd->empty[s]);
        }
        if (!ok) break;
        gm_commit(&hd->accfull[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: TMEM lane = token
    const bool vec_ok = (p.rows % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0);
    for (int i = 0; i < my_tiles; i++) {
      const int buf = i & 1;
      const int tile = (int)blockIdx.x + i * (int)gridDim.x;
      const int m = tile % mt, nn = tile / mt;
      if (!__all_sync(0xffffffffu, mbar_wait(&hd->accfull[buf], (i >> 1) & 1u, abort_flag, p.status, kDevWaitFull))) break;
      gm_fence_after();
      const int token = m * kGmBM + 32 * warp + lane;
      const uint32_t taddr = tmem + ((uint32_t)(32 * warp) << 16) + (uint32_t)(buf * kGmBN);
#pragma unroll 1
      for (int c0 = 0; c0 < kGmBN; c0 += 32) {
        uint32_t r[32];
        gm_ld32(taddr + c0, r);
        gm_wait_ld();
        const int col0 = nn * kGmBN + c0;
        if (token < p.n && col0 < p.rows) {
          float* dst = p.y + (size_t)token * p.rows + col0;
          if (vec_ok && col0 + 32 <= p.rows) {
#pragma unroll
            for (int q = 0; q < 8; q++) {
              float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                                     __uint_as_float(r[4 * q + 3]));
              if (p.accumulate) {
                const float4 o = reinterpret_cast<const float4*>(dst)[q];
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              reinterpret_cast<float4*>(dst)[q] = v;
            }
          } else {
#pragma unroll
            for (int q = 0; q < 32; q++)
              if (col0 + q < p.rows) dst[q] = p.accumulate ? dst[q] + __uint_as_float(r[q]) : __uint_as_float(r[q]);
          }
        }
      }
      gm_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->accempty[buf]);
    }
  }
  // ------------------------------------------------------------------ teardown (every thread arrives here)
  gm_fence_before();
  __syncthreads();
  if (warp == 4) {
    gm_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kCols) : "memory");
  }
}

// ---------------------------------------------------------------- operand preparation
// weights -> half, the reference's dequantised value rounded to half once (q_deq_f16, quant_mm.metal:131-154)
template <int T>
__global__ void dequant_f16_kernel(const uint8_t* __restrict__ src, __half* __restrict__ out, int64_t n8, Tables tb) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  constexpr int per_block = block_elems(T) / 8;
  const uint8_t* blk = src + (i / per_block) * block_bytes(T);
  float y[8];
  dequant8<T>(blk, (int)(i % per_block), tb, y);
  __half2 h[4];
#pragma unroll
  for (int k = 0; k < 4; k++) h[k] = __floats2half2_rn(y[2 * k], y[2 * k + 1]);
  *reinterpret_cast<uint4*>(out + 8 * i) = *reinterpret_cast<uint4*>(h);
}
// the same for a group of equally sized matrices in one launch (blockIdx.y = matrix; srcs[g] = its device address, its
// half copy at out + g * count): a few-microsecond launch per 8 M-weight matrix never reaches the memory system's pace
template <int T>
__global__ void dequant_f16_group_kernel(const uint64_t* __restrict__ srcs, __half* __restrict__ out, int64_t n8, Tables tb) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint8_t* src = reinterpret_cast<const uint8_t*>(srcs[blockIdx.y]);
  constexpr int per_block = block_elems(T) / 8;
  const uint8_t* blk = src + (i / per_block) * block_bytes(T);
  float y[8];
  dequant8<T>(blk, (int)(i % per_block), tb, y);
  __half2 h[4];
#pragma unroll
  for (int k = 0; k < 4; k++) h[k] = __floats2half2_rn(y[2 * k], y[2 * k + 1]);
  *reinterpret_cast<uint4*>(out + ((int64_t)blockIdx.y * n8 + i) * 8) = *reinterpret_cast<uint4*>(h);
}
// dense sources: part 0 = half(w); part 1 (F32 only) = half(w - half(w)), the second term of a two-pass product
__global__ void dense_f16_kernel(const uint8_t* __restrict__ src, __half* __restrict__ out, int64_t n, int t, int part) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float w;
  if (t == F32) w = reinterpret_cast<const float*>(src)[i];
  else if (t == F16) w = __half2float(reinterpret_cast<const __half*>(src)[i]);
  else w = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(src)[i] << 16);
  const __half hi = __float2half_rn(w);
  out[i] = part == 0 ? hi : __float2half_rn(w - __half2float(hi));
}
// activations -> half (encode_f32_to_f16); count % 4 == 0
__global__ void f32_to_f16_kernel(const float* __restrict__ x, __half* __restrict__ out, size_t n4) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 v = reinterpret_cast<const float4*>(x)[i];
  __half2 h[2] = {__floats2half2_rn(v.x, v.y), __floats2half2_rn(v.z, v.w)};
  reinterpret_cast<uint2*>(out)[i] = *reinterpret_cast<uint2*>(h);
}

// ---------------------------------------------------------------- host side
namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn gm_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
// half matrix [rows][cols] with row stride `stride` halfs, tiles of box_rows x 64 halfs, 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, int rows, int cols, int64_t stride, int box_rows) {
  EncodeTiledFn encode = gm_encode_fn();
  if (!encode) return fail(kErrCuda, "matmul: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)stride * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kGmBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult cr = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(kErrCuda, "matmul: tensor map encode failed (%d)", (int)cr);
  return kOk;
}

// Y (+)= X16 . W16^T, both operands half in global memory
int gemm_f16(const void* x16, int64_t x_stride, const void* w16, float* y, int n, int rows, int cols, bool accumulate,
             cudaStream_t st) {
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  GemmParams p;
  rc = make_map(&p.a_map, x16, n, cols, x_stride, kGmBM);
  if (rc) return rc;
  rc = make_map(&p.b_map, w16, rows, cols, cols, kGmBN);
  if (rc) return rc;
  p.y = y; p.status = tb.status; p.n = n; p.rows = rows; p.cols = cols; p.accumulate = accumulate ? 1 : 0;
  const int tiles = ((n + kGmBM - 1) / kGmBM) * ((rows + kGmBN - 1) / kGmBN);
  const size_t smem = 1024 + 1024 + (size_t)kGmStages * (kGmABytes + kGmBBytes);
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    MSB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev & 63] = true;
  }
  MSB_CUDA(launch_pdl(gemm_tc_kernel, dim3(std::max(1, std::min(sms, tiles))), dim3(kGmThreads), smem, st, p));
  MSB_LAUNCH_CHECK("gemm_tc_kernel");
  return kOk;
}

}  // namespace

// W (type t) -> half [rows x cols]; part 1 = the F32 remainder term (also used by the MoE prefill for its dense experts)
int weights_to_f16(int t, const void* W, int64_t count, __half* out, int part, cudaStream_t st) {
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  const int threads = 256;
  if (is_dense(t)) {
    MSB_CUDA(launch_pdl(dense_f16_kernel, dim3((unsigned)((count + threads - 1) / threads)), dim3(threads), 0, st,
                        (const uint8_t*)W, out, count, t, part));
  } else {
    const int64_t n8 = count / 8;
    const dim3 grid((unsigned)((n8 + threads - 1) / threads));
    const uint8_t* s = (const uint8_t*)W;
    switch (t) {
      case Q8_0: MSB_CUDA(launch_pdl(dequant_f16_kernel<Q8_0>, grid, dim3(threads), 0, st, s, out, n8, tb)); break;
      case Q5_K: MSB_CUDA(launch_pdl(dequant_f16_kernel<Q5_K>, grid, dim3(threads), 0, st, s, out, n8, tb)); break;
      case Q6_K: MSB_CUDA(launch_pdl(dequant_f16_kernel<Q6_K>, grid, dim3(threads), 0, st, s, out, n8, tb)); break;
      case IQ2_XXS: MSB_CUDA(launch_pdl(dequant_f16_kernel<IQ2_XXS>, grid, dim3(threads), 0, st, s, out, n8, tb)); break;
      case IQ1_S: MSB_CUDA(launch_pdl(dequant_f16_kernel<IQ1_S>, grid, dim3(threads), 0, st, s, out, n8, tb)); break;
      case IQ4_NL: MSB_CUDA(launch_pdl(dequant_f16_kernel<IQ4_NL>, grid, dim3(threads), 0, st, s, out, n8, tb)); break;
      default: return fail(kErrType, "matmul: unsupported weight type %d", t);
    }
  }
  MSB_LAUNCH_CHECK("weights_to_f16");
  return kOk;
}

// n_mat block-quantised matrices of `count` weights each, addresses in the device array d_srcs, to half copies laid
// back to back at out
int weights_to_f16_group(int t, const uint64_t* d_srcs, int n_mat, int64_t count, __half* out, cudaStream_t st) {
  if (n_mat <= 0) return kOk;
  if (is_dense(t) || n_mat > 65535) return fail(kErrType, "matmul: grouped conversion needs a block-quantised type");
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  const int threads = 256;
  const int64_t n8 = count / 8;
  const dim3 grid((unsigned)((n8 + threads - 1) / threads), (unsigned)n_mat);
  switch (t) {
    case Q8_0: MSB_CUDA(launch_pdl(dequant_f16_group_kernel<Q8_0>, grid, dim3(threads), 0, st, d_srcs, out, n8, tb)); break;
    case Q5_K: MSB_CUDA(launch_pdl(dequant_f16_group_kernel<Q5_K>, grid, dim3(threads), 0, st, d_srcs, out, n8, tb)); break;
    case Q6_K: MSB_CUDA(launch_pdl(dequant_f16_group_kernel<Q6_K>, grid, dim3(threads), 0, st, d_srcs, out, n8, tb)); break;
    case IQ2_XXS: MSB_CUDA(launch_pdl(dequant_f16_group_kernel<IQ2_XXS>, grid, dim3(threads), 0, st, d_srcs, out, n8, tb)); break;
    case IQ1_S: MSB_CUDA(launch_pdl(dequant_f16_group_kernel<IQ1_S>, grid, dim3(threads), 0, st, d_srcs, out, n8, tb)); break;
    case IQ4_NL: MSB_CUDA(launch_pdl(dequant_f16_group_kernel<IQ4_NL>, grid, dim3(threads), 0, st, d_srcs, out, n8, tb)); break;
    default: return fail(kErrType, "matmul: unsupported weight type %d", t);
  }
  MSB_LAUNCH_CHECK("weights_to_f16_group");
  return kOk;
}

int f32_to_f16(const float* x, void* x16, size_t count, cudaStream_t st) {
  if (count % 4) return fail(kErrArg, "f32_to_f16: count %zu is not a multiple of 4", count);
  if (count == 0) return kOk;
  if (!x || !x16 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(x16) & 7))
    return fail(kErrArg, "f32_to_f16: null or misaligned pointer");
  const size_t n4 = count / 4;
  MSB_CUDA(launch_pdl(f32_to_f16_kernel, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, st, x, (__half*)x16, n4));
  MSB_LAUNCH_CHECK("f32_to_f16_kernel");
  return kOk;
}

// scratch of matmul_h: the half copy of W (nothing for F16 weights); matmul adds the half copy of X
size_t matmul_scratch_bytes(int t, int rows, int cols, int n, bool with_x) {
  size_t b = t == F16 ? 0 : (size_t)rows * cols * 2;
  b = (b + 255) & ~(size_t)255;
  if (with_x) b += ((size_t)n * cols * 2 + 255) & ~(size_t)255;
  return b ? b + 256 : 0;   // + room to align the base
}

int matmul_h(int t, const void* W, int rows, int cols, const void* X16, int x_stride, float* Y, int n, bool accumulate,
             void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (!type_known(t)) return fail(kErrType, "matmul: unsupported weight type %d", t);
  if (rows <= 0 || cols <= 0 || n < 0 || cols % block_elems(t) || cols % 8)
    return fail(kErrArg, "matmul: bad shape (rows %d cols %d n %d, type %s)", rows, cols, n, type_name(t));
  if (n == 0) return kOk;
  if (x_stride == 0) x_stride = cols;
  if (x_stride < cols || x_stride % 8) return fail(kErrArg, "matmul: x_stride %d must be >= cols and a multiple of 8", x_stride);
  if (!W || !X16 || !Y || (reinterpret_cast<uintptr_t>(X16) & 15)) return fail(kErrArg, "matmul: null or misaligned pointer");
  if (scratch_bytes < matmul_scratch_bytes(t, rows, cols, n, false) || (t != F16 && !scratch))
    return fail(kErrScratch, "matmul: scratch too small");
  const void* w16 = W;
  if (t == F16) {
    if (reinterpret_cast<uintptr_t>(W) & 15) return fail(kErrArg, "matmul: F16 weights must be 16-byte aligned");
  } else {
    __half* wbuf = reinterpret_cast<__half*>((reinterpret_cast<uintptr_t>(scratch) + 255) & ~(uintptr_t)255);
    int rc = weights_to_f16(t, W, (int64_t)rows * cols, wbuf, 0, st);
    if (rc) return rc;
    w16 = wbuf;
  }
  int rc = gemm_f16(X16, x_stride, w16, Y, n, rows, cols, accumulate, st);
  if (rc || t != F32) return rc;
  // F32 weights keep their precision: second pass with the remainder term w - half(w)
  __half* wbuf = reinterpret_cast<__half*>((reinterpret_cast<uintptr_t>(scratch) + 255) & ~(uintptr_t)255);
  rc = weights_to_f16(t, W, (int64_t)rows * cols, wbuf, 1, st);
  if (rc) return rc;
  return gemm_f16(X16, x_stride, wbuf, Y, n, rows, cols, true, st);
}

int matmul(int t, const void* W, int rows, int cols, const float* X, float* Y, int n, bool accumulate, void* scratch,
           size_t scratch_bytes, cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || n < 0) return fail(kErrArg, "matmul: bad shape");
  if (n == 0) return kOk;
  if (!scratch || scratch_bytes < matmul_scratch_bytes(t, rows, cols, n, true)) return fail(kErrScratch, "matmul: scratch too small");
  const size_t wpart = matmul_scratch_bytes(t, rows, cols, n, false);
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(scratch) + 255) & ~(uintptr_t)255);
  void* x16 = base + ((wpart + 255) & ~(size_t)255);
  int rc = f32_to_f16(X, x16, (size_t)n * cols, st);
  if (rc) return rc;
  return matmul_h(t, W, rows, cols, x16, cols, Y, n, accumulate, scratch, wpart, st);
}

}  // namespace msb
