// Lightning-indexer scoring on the 5th-generation tensor cores (tcgen05 + TMEM), FP8 keys.
//   score[t] = sum_h relu(q_h . k_t) * w_h          (tests/ref/attn_ref.cpp:172-184 is the math spec)
// Same contract as idx_score_fp8_kernel (index.cu), which replaces the reference's attn_idx_score_dec2 Metal kernel
// (src/kernels/attn_index.metal:616-677); this version feeds the [len x 128] x [128 x heads] contraction to
// tcgen05.mma instead of mma.sync, whose FP8 rate on this part is what bounded the older kernel.
//
// One persistent CTA per SM, 6 warps with fixed roles:
//   warp 5       one thread streams key tiles of 128 rows x 128 bytes with TMA tensor copies (cp.async.bulk.tensor.2d,
//                128-byte swizzle, rows past the end zero-filled) into an 8-slot shared-memory ring: 128 KB in flight
//                per SM without a single load instruction.
//   warp 4       one thread issues, per tile, 4 x tcgen05.mma (M = 128 keys, N = heads, K = 32, both operands K-major
//                with the 128-byte swizzle) into one of two TMEM accumulators (heads fp32 columns each) and commits to
//                the barriers that free the shared-memory slot and publish the accumulator.
//   warps 0..3   first stage the query as e4m3 in the swizzled operand layout; then epilogue: TMEM lane = key, so
//                each thread reads its key's `heads` dot products (tcgen05.ld), applies relu and the head weights in
//                head order, writes the score and feeds the selection histogram.
// Every mbarrier wait is bounded (mbar_wait): on expiry the block's abort flag makes every role leave its loop, the
// block still meets at the final barrier and the TMEM columns are released.
#include <cuda.h>
#include <cuda_fp8.h>
#include <algorithm>
#include <cmath>
#include "msb_common.cuh"

namespace msb {

constexpr int kTcDim = 128;               // key bytes = contraction length
constexpr int kTcTile = 128;              // keys per tile = MMA M
constexpr int kTcTileBytes = kTcTile * kTcDim;
constexpr int kTcStages = 6;
constexpr int kTcThreads = 6 * 32;
constexpr int kTcHistBins = 4096;
constexpr uint32_t kTcSbo = 1024;          // bytes between 8-row groups of the swizzled K-major layout (8 x 128)

struct IdxTcParams {
  CUtensorMap keys;    // [len][128] bytes, box 128 x 128, 128-byte swizzle
  CUtensorMap keys8;   // the same matrix with a box of 128 x 8 rows (candidate-list mode: one key block per copy)
  const int* cand;     // candidate-list mode: [n_cand] key-block indices (8 keys each), -1 = none; else null
  int n_cand;          // entries of cand; the kernel scores n_cand * 8 virtual positions
  const float* q;      // [H][128] query: prepared, or raw when prep != 0
  const float* w;      // [H] head weights: prepared, or raw when prep != 0
  const float* cs;     // prep: [32][2] (cos, sin) of the query position
  float* q_out;        // prep: the prepared query is also written here (block 0), as index_prep would
  float* w_out;        // prep: likewise the prepared head weights
  float wscale;        // prep: dim^-0.5 * heads^-0.5
  int prep, actq;      // prep: fold the query preparation (rope, optional fp4 simulation, weight scale) in
  float* scores;       // [len]
  unsigned* hist;      // [4096] or null
  int* status;         // device failure word
  int len;
};

struct IdxTcHead {
  uint64_t full[kTcStages], empty[kTcStages], accfull[2], accempty[2], qbar;
  uint32_t tmem_base;
  int abort_flag;
  unsigned hist[kTcHistBins];
};

__device__ __forceinline__ uint32_t tc_order_key(float f) {   // larger float <=> larger key (as index.cu)
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
// shared-memory matrix descriptor: K-major, 128-byte swizzle (layout type 2), descriptor version 1 (sm_100); the two
// 16-byte K-chunks of one instruction are adjacent (leading offset 1 unit), 8-row groups kTcSbo bytes apart
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(kTcSbo >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// 2-D TMA tile load into shared memory, completion on an mbarrier (x = byte column, y = row)
__device__ __forceinline__ void tc_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float tc_pow2i(int e) { return __uint_as_float((uint32_t)(e + 127) << 23); }
__device__ __forceinline__ float tc_round_e2m1(float x) {   // as round_e2m1 of index.cu (attn_ref.cpp:93-100)
  const float a = fabsf(x);
  int e = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;
  e = max(e, 0);
  return copysignf(nearbyintf(a * tc_pow2i(1 - e)) * tc_pow2i(e - 1), x);
}

template <int H>
__global__ void __launch_bounds__(kTcThreads, 1) idx_score_tc_kernel(const __grid_constant__ IdxTcParams p) {
  static_assert(H == 32 || H == 64, "heads = MMA N");
  pdl_launch_dependents();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the swizzled operand tiles need 1024-byte aligned shared addresses: align by hand (the launch adds the slack)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  IdxTcHead* hd = reinterpret_cast<IdxTcHead*>(smem);
  uint8_t* qs = smem + ((sizeof(IdxTcHead) + 1023) & ~(size_t)1023);      // [H x 128] e4m3, canonical layout
  uint8_t* stage0 = qs + H * kTcDim;                                      // kTcStages key tiles
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr uint32_t kCols = 2 * H;                                       // two accumulators of H fp32 columns

  if (tid == 0) {
    for (int s = 0; s < kTcStages; s++) { mbar_init(&hd->full[s], 1); mbar_init(&hd->empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&hd->accfull[b], 1); mbar_init(&hd->accempty[b], 4); }
    mbar_init(&hd->qbar, 4);
    hd->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&hd->tmem_base)), "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (p.hist)
    for (int b = tid; b < kTcHistBins; b += kTcThreads) hd->hist[b] = 0;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = hd->tmem_base;
  volatile int* abort_flag = &hd->abort_flag;
  // candidate-list mode: virtual position v = 8 * i + j is key cand[i] * 8 + j; scores[] is indexed by v
  const int ntiles = ((p.cand ? p.n_cand * 8 : p.len) + kTcTile - 1) / kTcTile;
  const int my_tiles = ntiles > (int)blockIdx.x ? (ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  pdl_wait();   // the query (and possibly the newest keys) come from kernels that ran before

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA producer
    if (p.cand) {
      // candidate-list mode, whole warp: lane i < 16 owns key block i of the tile (8 rows = one 1024-byte swizzle group)
      for (int i = 0; i < my_tiles; i++) {
        const int s = i % kTcStages;
        const int tile = (int)blockIdx.x + i * (int)gridDim.x;
        const int ci = tile * 16 + lane;
        int blk = -1;
        if (lane < 16 && ci < p.n_cand) blk = __ldg(p.cand + ci);
        const bool valid = blk >= 0 && (long long)blk * 8 < p.len;
        const unsigned m = __ballot_sync(0xffffffffu, valid);
        if (!__all_sync(0xffffffffu, mbar_wait(&hd->empty[s], ((i / kTcStages) & 1u) ^ 1u, abort_flag, p.status, kDevWaitEmpty))) break;
        if (lane == 0) mbar_arrive_expect_tx(&hd->full[s], 1024u * (unsigned)__popc(m));
        __syncwarp();
        if (valid) tc_tma_2d(stage0 + (size_t)s * kTcTileBytes + lane * 1024, &p.keys8, 0, blk * 8, &hd->full[s]);
      }
    } else if (lane == 0) {
      for (int i = 0; i < my_tiles; i++) {
        const int s = i % kTcStages;
        const int tile = (int)blockIdx.x + i * (int)gridDim.x;
        if (!mbar_wait(&hd->empty[s], ((i / kTcStages) & 1u) ^ 1u, abort_flag, p.status, kDevWaitEmpty)) break;
        mbar_arrive_expect_tx(&hd->full[s], kTcTileBytes);
        tc_tma_2d(stage0 + (size_t)s * kTcTileBytes, &p.keys, 0, tile * kTcTile, &hd->full[s]);
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(H >> 3) << 17) | ((uint32_t)(kTcTile >> 4) << 24);
      const uint32_t q_s = smem_u32(qs);
      bool ok = mbar_wait(&hd->qbar, 0, abort_flag, p.status, kDevWaitFull);
      for (int i = 0; ok && i < my_tiles; i++) {
        const int s = i % kTcStages, buf = i & 1;
        if (!mbar_wait(&hd->full[s], (i / kTcStages) & 1u, abort_flag, p.status, kDevWaitFull)) break;
        if (!mbar_wait(&hd->accempty[buf], ((i >> 1) & 1u) ^ 1u, abort_flag, p.status, kDevWaitEmpty)) break;
        tc_fence_after();
        const uint32_t a_s = smem_u32(stage0 + (size_t)s * kTcTileBytes);
#pragma unroll
        for (int ks = 0; ks < 4; ks++)      // K = 32 bytes per instruction: the start address moves along the row
          tc_mma_f8(tmem + (uint32_t)(buf * H), tc_desc(a_s + ks * 32), tc_desc(q_s + ks * 32), idesc, ks > 0 ? 1u : 0u);
        tc_commit(&hd->empty[s]);           // the slot is free once these MMAs have read it
        tc_commit(&hd->accfull[buf]);       // ... and the accumulator is complete
      }
    }
  } else {
    // ------------------------------------------------------------------ query staging, then epilogue
    // query -> e4m3 in the swizzled K-major layout (row = head, 16-byte chunk j of row n at chunk j ^ (n % 8));
    // chunk c = (head, K-chunk) = 16 consecutive floats; all loads of a thread are issued before the conversions
    {
      constexpr int kPer = H * 8 / 128;
      float4 f[kPer][4];
#pragma unroll
      for (int i = 0; i < kPer; i++) {
        const int c = tid + 128 * i, n = c >> 3, j = c & 7;
        const float4* src = reinterpret_cast<const float4*>(p.q + (size_t)n * kTcDim + j * 16);
        f[i][0] = src[0]; f[i][1] = src[1]; f[i][2] = src[2]; f[i][3] = src[3];
      }
      if (p.prep) {
        // query preparation of index_prep (attn_ref.cpp:163-170) on this thread's 16 dims: rope on dims 64..127
        // (interleaved pairs), then the optional e2m1 simulation with a power-of-two scale per 32 dims (= this
        // thread's chunk and its neighbour's)
#pragma unroll
        for (int i = 0; i < kPer; i++) {
          const int c = tid + 128 * i, n = c >> 3, j = c & 7;
          float* v = reinterpret_cast<float*>(&f[i][0]);
          if (j >= 4) {
#pragma unroll
            for (int e = 0; e < 8; e++) {
              const int pi = (16 * j - 64) / 2 + e;
              const float cc = p.cs[2 * pi], sn = p.cs[2 * pi + 1];
              const float a = v[2 * e], b = v[2 * e + 1];
              v[2 * e] = __fsub_rn(__fmul_rn(a, cc), __fmul_rn(b, sn));
              v[2 * e + 1] = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, cc));
            }
          }
          if (p.actq) {
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < 16; e++) amax = fmaxf(amax, fabsf(v[e]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, 6.0f * 1.17549435e-38f);
            const float r = __fmul_rn(amax, 1.0f / 6.0f);
            const uint32_t rb = __float_as_uint(r);
            const int ex = (int)((rb >> 23) & 0xFF) - 127 + ((rb & 0x7FFFFF) ? 1 : 0);
            const float sc = tc_pow2i(ex), inv = tc_pow2i(-ex);
#pragma unroll
            for (int e = 0; e < 16; e++)
              v[e] = __fmul_rn(tc_round_e2m1(fminf(fmaxf(__fmul_rn(v[e], inv), -6.0f), 6.0f)), sc);
          }
          if (blockIdx.x == 0 && p.q_out) {
            float4* dst = reinterpret_cast<float4*>(p.q_out + (size_t)n * kTcDim + j * 16);
            dst[0] = f[i][0]; dst[1] = f[i][1]; dst[2] = f[i][2]; dst[3] = f[i][3];
          }
        }
      }
      auto pack = [](const float4& v) {
        return (uint32_t)__nv_cvt_float_to_fp8(v.x, __NV_SATFINITE, __NV_E4M3) |
               ((uint32_t)__nv_cvt_float_to_fp8(v.y, __NV_SATFINITE, __NV_E4M3) << 8) |
               ((uint32_t)__nv_cvt_float_to_fp8(v.z, __NV_SATFINITE, __NV_E4M3) << 16) |
               ((uint32_t)__nv_cvt_float_to_fp8(v.w, __NV_SATFINITE, __NV_E4M3) << 24);
      };
#pragma unroll
      for (int i = 0; i < kPer; i++) {
        const int c = tid + 128 * i, n = c >> 3, j = c & 7;
        *reinterpret_cast<uint4*>(qs + n * kTcDim + ((j ^ (n & 7)) << 4)) =
            make_uint4(pack(f[i][0]), pack(f[i][1]), pack(f[i][2]), pack(f[i][3]));
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->qbar);
    }
    float wr[H];                                   // head weights in registers
#pragma unroll
    for (int h = 0; h < H; h += 4) {
      const float4 w4 = *reinterpret_cast<const float4*>(p.w + h);
      wr[h] = w4.x; wr[h + 1] = w4.y; wr[h + 2] = w4.z; wr[h + 3] = w4.w;
    }
    if (p.prep) {
#pragma unroll
      for (int h = 0; h < H; h++) wr[h] *= p.wscale;
      if (blockIdx.x == 0 && p.w_out && tid < H) p.w_out[tid] = p.w[tid] * p.wscale;
    }
    for (int i = 0; i < my_tiles; i++) {
      const int buf = i & 1;
      const int tile = (int)blockIdx.x + i * (int)gridDim.x;
      if (!__all_sync(0xffffffffu, mbar_wait(&hd->accfull[buf], (i >> 1) & 1u, abort_flag, p.status, kDevWaitFull))) break;
      tc_fence_after();
      const uint32_t taddr = tmem + ((uint32_t)(32 * warp) << 16) + (uint32_t)(buf * H);
      uint32_t r[H / 32][32];
#pragma unroll
      for (int c = 0; c < H / 32; c++) tc_ld32(taddr + 32 * c, r[c]);
      tc_wait_ld();
      // the accumulator is in registers: hand it back before the arithmetic
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->accempty[buf]);
      float sc = 0.f;
#pragma unroll
      for (int c = 0; c < H / 32; c++)
#pragma unroll
        for (int h = 0; h < 32; h++) sc = fmaf(fmaxf(__uint_as_float(r[c][h]), 0.f), wr[32 * c + h], sc);
      const long long key = (long long)tile * kTcTile + 32 * warp + lane;   // key index, or virtual position
      bool live = key < p.len;
      if (p.cand) {
        // rows of blocks that were not loaded hold stale bytes: their (meaningless) sums are masked here
        const int ci = (int)(key >> 3);
        const int blk = ci < p.n_cand ? __ldg(p.cand + ci) : -1;
        const bool valid = blk >= 0 && (long long)blk * 8 + (key & 7) < p.len;
        if (!valid) sc = -INFINITY;
        live = key < (long long)p.n_cand * 8;
      }
      if (live) p.scores[key] = sc;
      if (p.hist) {   // neighbouring scores mostly share a bin: one shared-memory atomic per distinct bin per warp
        const uint32_t bin = (live && sc > -INFINITY) ? tc_order_key(sc) >> 20 : 0xFFFFFFFFu;
        const unsigned m = __match_any_sync(0xffffffffu, bin);
        if (bin != 0xFFFFFFFFu && lane == __ffs(m) - 1) atomicAdd(&hd->hist[bin], (unsigned)__popc(m));
      }
    }
  }
  // ------------------------------------------------------------------ teardown (every thread arrives here)
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kCols) : "memory");
  }
  if (p.hist)
    for (int b = tid; b < kTcHistBins; b += kTcThreads) {
      const unsigned v = hd->hist[b];
      if (v) atomicAdd(&p.hist[b], v);
    }
}

size_t idx_score_tc_smem(int heads) {
  return ((sizeof(IdxTcHead) + 1023) & ~(size_t)1023) + (size_t)heads * kTcDim + (size_t)kTcStages * kTcTileBytes + 1024;
}

namespace {
// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on the driver library)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
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
}  // namespace

// FP8 keys, heads 32 or 64.  Returns kOk or an error code; the caller has validated the pointers (keys 16-byte aligned).
// prep != 0: q / w are the raw projections and the preparation of index_prep is folded in (cs, actq; the prepared
// values are also written to q_out / w_out when those are given).
// cand != null: candidate-list mode, scores[8 * i + j] = score of key cand[i] * 8 + j (-inf where there is no such key).
int index_scores_tc(const void* keys, int len, const float* q, const float* w, int heads, float* scores, unsigned* hist,
                    int prep, const float* cs, int actq, float* q_out, float* w_out, const int* cand, int n_cand,
                    cudaStream_t st) {
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return fail(kErrCuda, "index_scores: cuTensorMapEncodeTiled is not available from this driver");
  IdxTcParams p;
  const cuuint64_t gdim[2] = {(cuuint64_t)kTcDim, (cuuint64_t)len};       // innermost first, in bytes (uint8 elements)
  const cuuint64_t gstride[1] = {(cuuint64_t)kTcDim};                     // bytes between rows
  const cuuint32_t box[2] = {(cuuint32_t)kTcDim, (cuuint32_t)kTcTile};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult cr = encode(&p.keys, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(keys), gdim, gstride, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(kErrCuda, "index_scores: tensor map encode failed (%d)", (int)cr);
  const cuuint32_t box8[2] = {(cuuint32_t)kTcDim, 8};
  const CUresult cr8 = encode(&p.keys8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(keys), gdim, gstride, box8, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr8 != CUDA_SUCCESS) return fail(kErrCuda, "index_scores: tensor map encode failed (%d)", (int)cr8);
  p.cand = cand; p.n_cand = cand ? n_cand : 0;
  p.q = q; p.w = w; p.scores = scores; p.hist = hist; p.status = tb.status; p.len = len;
  p.prep = prep; p.cs = cs; p.actq = actq; p.q_out = q_out; p.w_out = w_out;
  p.wscale = (float)(pow((double)kTcDim, -0.5) * pow((double)heads, -0.5));
  const int ntiles = ((cand ? n_cand * 8 : len) + kTcTile - 1) / kTcTile;
  const int grid = std::max(1, std::min(sms, ntiles));
  const size_t smem = idx_score_tc_smem(heads);
  static bool configured[2][64] = {};
  if (heads == 64) {
    if (!configured[0][dev & 63]) {
      MSB_CUDA(cudaFuncSetAttribute(idx_score_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured[0][dev & 63] = true;
    }
    MSB_CUDA(launch_pdl(idx_score_tc_kernel<64>, dim3(grid), dim3(kTcThreads), smem, st, p));
  } else {
    if (!configured[1][dev & 63]) {
      MSB_CUDA(cudaFuncSetAttribute(idx_score_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured[1][dev & 63] = true;
    }
    MSB_CUDA(launch_pdl(idx_score_tc_kernel<32>, dim3(grid), dim3(kTcThreads), smem, st, p));
  }
  MSB_LAUNCH_CHECK("idx_score_tc_kernel");
  return kOk;
}

}  // namespace msb
