// Lightning indexer, decode side: query preparation, key scoring on the tensor cores, exact top-k.
//   score[t] = sum_h relu(q_h . k_t) * w_h   for t < len          (tests/ref/attn_ref.cpp:172-184 is the math spec)
//   top-k among finite scores, ties -> lower index, output sorted ascending by index, -1 padded (:186-194)
// Replaces the reference's attn_idx_prep_thread / attn_idx_score_dec2 / attn_topk_compact / attn_topk_final Metal
// kernels (src/kernels/attn_index.metal:129-145,616-677,703-797) behind ms::attn::encode_index_decode
// (src/kernels/attn.hpp:121-122, attn.mm:222-290).
//
// Scoring is a [len x 128] x [128 x heads] contraction: FP8 (e4m3) keys go straight into mma.sync m16n8k32 with the
// query held in registers as e4m3 B fragments; F16 keys use m16n8k16 with the fp32 query split into two f16 terms
// (hi + lo) so that no query precision is lost.  fp32 accumulation throughout; heads are summed in a fixed order.
// Selection: a 4096-bin histogram of the order-preserving key's top 12 bits (built by the scoring kernel) gives the
// threshold bin; a grid-wide compaction collects everything above it plus the threshold bin's members; one block
// finishes exactly (radix select on the remaining key bits, then on the index for ties) and sorts by index.
#include <cuda_fp8.h>
#include <algorithm>
#include "msb_common.cuh"

namespace msb {

constexpr int kIdxDim = 128;
constexpr int kKeyF16 = 1, kKeyFp8 = 101;
constexpr int kHistBins = 4096;

// tcgen05 scoring kernel for FP8 keys (index_tc.cu)
int index_scores_tc(const void* keys, int len, const float* q, const float* w, int heads, float* scores, unsigned* hist,
                    int prep, const float* cs, int actq, float* q_out, float* w_out, const int* cand, int n_cand,
                    cudaStream_t st);

__device__ __forceinline__ uint32_t order_key(float f) {   // larger float <=> larger key
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ bool selectable(float f) { return f > -INFINITY; }   // finite or +inf; NaN never

__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct IdxParams {
  const uint8_t* keys;
  const float* q;      // [H][128] prepared query
  const float* w;      // [H] prepared head weights
  float* scores;       // [len]
  unsigned* hist;      // [4096] or null
  int len;
};

__device__ __forceinline__ void hist_flush(unsigned* sh, unsigned* gh, int tid, int nthreads) {
  __syncthreads();
  for (int b = tid; b < kHistBins; b += nthreads) {
    const unsigned v = sh[b];
    if (v) atomicAdd(&gh[b], v);
  }
}

// ---------------------------------------------------------------- FP8 keys: direct e4m3 MMA, query in registers
// K permutation: lane (g, t) holds bytes 32t .. 32t+31 of key rows g and g+8; k-step s pairs words (2s, 2s+1) of the
// row with the same bytes of the query, so the contraction covers every dimension once.
template <int H>
__global__ void __launch_bounds__(384, 1) idx_score_fp8_kernel(const IdxParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NT = H / 8;
  __shared__ unsigned sh_hist[kHistBins];
  const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int ntiles = (p.len + 15) / 16;
  // software pipeline: the next tile's 64 bytes per lane are requested before the current tile is multiplied
  auto fetch = [&](int tile, uint4 (&r)[4]) {
    const int k0 = tile * 16 + g, k1 = k0 + 8;
    r[0] = r[1] = r[2] = r[3] = make_uint4(0, 0, 0, 0);
    if (tile < ntiles && k0 < p.len) {
      const uint4* src = reinterpret_cast<const uint4*>(p.keys + (size_t)k0 * kIdxDim + 32 * t);
      r[0] = __ldg(src); r[1] = __ldg(src + 1);
    }
    if (tile < ntiles && k1 < p.len) {
      const uint4* src = reinterpret_cast<const uint4*>(p.keys + (size_t)k1 * kIdxDim + 32 * t);
      r[2] = __ldg(src); r[3] = __ldg(src + 1);
    }
  };
  // three tiles of keys per warp in flight (48 registers): requested before the query is staged, so that the first
  // round trips to HBM overlap the prologue
  uint4 cur[4], nx1[4], nx2[4];
  int tile = blockIdx.x * (blockDim.x >> 5) + (tid >> 5);
  fetch(tile, cur);
  fetch(tile + warps, nx1);
  fetch(tile + 2 * warps, nx2);
  if (p.hist)
    for (int b = tid; b < kHistBins; b += blockDim.x) sh_hist[b] = 0;
  // the query goes through shared memory as e4m3 bytes: a coalesced, latency-parallel load instead of 256 dependent
  // global loads per thread
  __shared__ __align__(16) uint8_t q8[H * kIdxDim];
  __shared__ float wsh[H];
  {
    constexpr int kQ4 = (H * kIdxDim / 4 + 383) / 384;   // 16-byte pieces per thread (block of 384)
    float4 v[kQ4];
#pragma unroll
    for (int j = 0; j < kQ4; j++) {                      // all loads in flight before the first conversion
      const int i = tid + 384 * j;
      v[j] = i < H * kIdxDim / 4 ? reinterpret_cast<const float4*>(p.q)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kQ4; j++) {
      const int i = tid + 384 * j;
      const uint32_t b = (uint32_t)__nv_cvt_float_to_fp8(v[j].x, __NV_SATFINITE, __NV_E4M3) |
                         ((uint32_t)__nv_cvt_float_to_fp8(v[j].y, __NV_SATFINITE, __NV_E4M3) << 8) |
                         ((uint32_t)__nv_cvt_float_to_fp8(v[j].z, __NV_SATFINITE, __NV_E4M3) << 16) |
                         ((uint32_t)__nv_cvt_float_to_fp8(v[j].w, __NV_SATFINITE, __NV_E4M3) << 24);
      if (i < H * kIdxDim / 4) reinterpret_cast<uint32_t*>(q8)[i] = b;
    }
  }
  for (int i = tid; i < H; i += blockDim.x) wsh[i] = p.w[i];
  __syncthreads();
  uint32_t B[NT][4][2];
  float wr[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    const uint32_t* qr = reinterpret_cast<const uint32_t*>(q8 + (size_t)(nt * 8 + g) * kIdxDim + 32 * t);
#pragma unroll
    for (int s = 0; s < 4; s++) { B[nt][s][0] = qr[2 * s]; B[nt][s][1] = qr[2 * s + 1]; }
    wr[nt][0] = wsh[nt * 8 + 2 * t];
    wr[nt][1] = wsh[nt * 8 + 2 * t + 1];
  }
  if (p.hist) __syncthreads();
  for (; tile < ntiles; tile += warps) {
    uint4 nx3[4];
    fetch(tile + 3 * warps, nx3);
    const int k0 = tile * 16 + g, k1 = k0 + 8;
    const uint32_t A0[8] = {cur[0].x, cur[0].y, cur[0].z, cur[0].w, cur[1].x, cur[1].y, cur[1].z, cur[1].w};
    const uint32_t A1[8] = {cur[2].x, cur[2].y, cur[2].z, cur[2].w, cur[3].x, cur[3].y, cur[3].z, cur[3].w};
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < 4; s++) mma_e4m3(c, A0[2 * s], A1[2 * s], A0[2 * s + 1], A1[2 * s + 1], B[nt][s][0], B[nt][s][1]);
      s0 += fmaxf(c[0], 0.f) * wr[nt][0] + fmaxf(c[1], 0.f) * wr[nt][1];
      s1 += fmaxf(c[2], 0.f) * wr[nt][0] + fmaxf(c[3], 0.f) * wr[nt][1];
    }
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    if (t == 0) {   // lanes 0, 4, ..., 28 hold the 16 scores of the tile
      if (k0 < p.len) p.scores[k0] = s0;
      if (k1 < p.len) p.scores[k1] = s1;
      if (p.hist) {   // neighbouring scores mostly share a bin: one shared-memory atomic per distinct bin per warp
        const uint32_t b0 = (k0 < p.len && selectable(s0)) ? order_key(s0) >> 20 : 0xFFFFFFFFu;
        const uint32_t b1 = (k1 < p.len && selectable(s1)) ? order_key(s1) >> 20 : 0xFFFFFFFFu;
        const unsigned m0 = __match_any_sync(0x11111111u, b0), m1 = __match_any_sync(0x11111111u, b1);
        if (b0 != 0xFFFFFFFFu && lane == __ffs(m0) - 1) atomicAdd(&sh_hist[b0], (unsigned)__popc(m0));
        if (b1 != 0xFFFFFFFFu && lane == __ffs(m1) - 1) atomicAdd(&sh_hist[b1], (unsigned)__popc(m1));
      }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) { cur[i] = nx1[i]; nx1[i] = nx2[i]; nx2[i] = nx3[i]; }
  }
  if (p.hist) hist_flush(sh_hist, p.hist, tid, blockDim.x);
}

// ---------------------------------------------------------------- F16 keys (or FP8 widened to F16): m16n8k16
// Query columns: [0, H) = f16(q), and with SPLIT [H, 2H) = f16(q - f16(q)).  The B fragments live in shared memory as
// Bs[n-tile][k-step][lane] = {b0, b1}; a warp scores 32 keys (two m-tiles) per pass over them.  (No fused histogram
// here: the selection builds its own.)
// K permutation: lane (g, t) holds elements 32t .. 32t+31 of its rows; k-step s uses elements 32t+4s .. 32t+4s+3.
template <int H, bool FP8IN, bool SPLIT>
__global__ void __launch_bounds__(256, 1) idx_score_f16_kernel(const IdxParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NTH = H / 8;                 // n-tiles per term
  constexpr int NT = SPLIT ? 2 * NTH : NTH;
  __shared__ uint2 Bs[NT][8][32];
  const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t = lane & 3;
  for (int i = tid; i < NT * 8 * 32; i += blockDim.x) {
    const int ln = i & 31, s = (i >> 5) & 7, nt = i >> 8;
    const int gg = ln >> 2, tt = ln & 3;
    const bool lo = SPLIT && nt >= NTH;
    const float* qr = p.q + (size_t)((lo ? nt - NTH : nt) * 8 + gg) * kIdxDim + 32 * tt + 4 * s;
    __half h[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const __half hi = __float2half_rn(qr[j]);
      h[j] = lo ? __float2half_rn(qr[j] - __half2float(hi)) : hi;
    }
    uint2 v;
    v.x = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
    v.y = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
    Bs[nt][s][ln] = v;
  }
  float wr[NTH][2];
#pragma unroll
  for (int nt = 0; nt < NTH; nt++) { wr[nt][0] = p.w[nt * 8 + 2 * t]; wr[nt][1] = p.w[nt * 8 + 2 * t + 1]; }
  __syncthreads();
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int ntiles = (p.len + 31) / 32;
  for (int tile = blockIdx.x * (blockDim.x >> 5) + (tid >> 5); tile < ntiles; tile += warps) {
    uint32_t A[4][16];   // rows g, g+8, g+16, g+24 of the tile; 16 half2 each
#pragma unroll
    for (int r = 0; r < 4; r++) {
      const int k = tile * 32 + g + 8 * r;
      if (k < p.len) {
        if (FP8IN) {
          const uint4* src = reinterpret_cast<const uint4*>(p.keys + (size_t)k * kIdxDim + 32 * t);
          const uint4 a = __ldg(src), b = __ldg(src + 1);
          const uint32_t wds[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const __half2_raw lo2 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wds[i] & 0xFFFFu), __NV_E4M3);
            const __half2_raw hi2 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wds[i] >> 16), __NV_E4M3);
            A[r][2 * i] = (uint32_t)lo2.x | ((uint32_t)lo2.y << 16);
            A[r][2 * i + 1] = (uint32_t)hi2.x | ((uint32_t)hi2.y << 16);
          }
        } else {
          const uint4* src = reinterpret_cast<const uint4*>(p.keys + ((size_t)k * kIdxDim + 32 * t) * 2);
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const uint4 a = __ldg(src + i);
            A[r][4 * i] = a.x; A[r][4 * i + 1] = a.y; A[r][4 * i + 2] = a.z; A[r][4 * i + 3] = a.w;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; i++) A[r][i] = 0;
      }
    }
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NTH; nt++) {
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < 8; s++) {
        const uint2 b = Bs[nt][s][lane];
        mma_f16(c0, A[0][2 * s], A[1][2 * s], A[0][2 * s + 1], A[1][2 * s + 1], b.x, b.y);
        mma_f16(c1, A[2][2 * s], A[3][2 * s], A[2][2 * s + 1], A[3][2 * s + 1], b.x, b.y);
        if (SPLIT) {
          const uint2 bl = Bs[nt + NTH][s][lane];
          mma_f16(c0, A[0][2 * s], A[1][2 * s], A[0][2 * s + 1], A[1][2 * s + 1], bl.x, bl.y);
          mma_f16(c1, A[2][2 * s], A[3][2 * s], A[2][2 * s + 1], A[3][2 * s + 1], bl.x, bl.y);
        }
      }
      sc[0] += fmaxf(c0[0], 0.f) * wr[nt][0] + fmaxf(c0[1], 0.f) * wr[nt][1];
      sc[1] += fmaxf(c0[2], 0.f) * wr[nt][0] + fmaxf(c0[3], 0.f) * wr[nt][1];
      sc[2] += fmaxf(c1[0], 0.f) * wr[nt][0] + fmaxf(c1[1], 0.f) * wr[nt][1];
      sc[3] += fmaxf(c1[2], 0.f) * wr[nt][0] + fmaxf(c1[3], 0.f) * wr[nt][1];
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
      sc[r] += __shfl_xor_sync(0xffffffffu, sc[r], 1);
      sc[r] += __shfl_xor_sync(0xffffffffu, sc[r], 2);
      const int k = tile * 32 + g + 8 * r;
      if (t == 0 && k < p.len) p.scores[k] = sc[r];
    }
  }
}

// ---------------------------------------------------------------- query preparation (attn_ref.cpp:163-170)
// rope on the last 64 dims of each head (interleaved pairs), optional fp4 (e2m1, power-of-two block-32 scale)
// quant-dequant simulation, head weights scaled by dim^-0.5 * heads^-0.5.  One warp per head.
__device__ __forceinline__ float pow2i(int e) { return __uint_as_float((uint32_t)(e + 127) << 23); }
__device__ __forceinline__ float round_e2m1(float x) {
  const float a = fabsf(x);
  int e = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;
  e = max(e, 0);
  return copysignf(nearbyintf(a * pow2i(1 - e)) * pow2i(e - 1), x);
}
__global__ void idx_prep_kernel(const float* q_raw, const float* w_raw, const float* cs, int actq, int heads, float* q,
                                float* w) {
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= heads) return;
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; i++) v[i] = q_raw[(size_t)h * kIdxDim + 32 * i + lane];
  // dims 64..127 are roped: pair (64 + 2j, 64 + 2j + 1) with (cos, sin) j.  Lane holds dims 64+lane and 96+lane.
  {
    const float o2 = __shfl_xor_sync(0xffffffffu, v[2], 1), o3 = __shfl_xor_sync(0xffffffffu, v[3], 1);
    const int j2 = lane >> 1, j3 = 16 + (lane >> 1);
    const float c2 = cs[2 * j2], s2 = cs[2 * j2 + 1], c3 = cs[2 * j3], s3 = cs[2 * j3 + 1];
    // even element: a*c - b*s ; odd element: a*s + b*c  with (a, b) = (even, odd)
    v[2] = (lane & 1) ? __fadd_rn(__fmul_rn(o2, s2), __fmul_rn(v[2], c2)) : __fsub_rn(__fmul_rn(v[2], c2), __fmul_rn(o2, s2));
    v[3] = (lane & 1) ? __fadd_rn(__fmul_rn(o3, s3), __fmul_rn(v[3], c3)) : __fsub_rn(__fmul_rn(v[3], c3), __fmul_rn(o3, s3));
  }
  if (actq) {
#pragma unroll
    for (int i = 0; i < 4; i++) {   // block i = dims 32i .. 32i+31 = one value per lane
      float amax = fabsf(v[i]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      amax = fmaxf(amax, 6.0f * 1.17549435e-38f);
      const float r = __fmul_rn(amax, 1.0f / 6.0f);
      const uint32_t rb = __float_as_uint(r);
      const int e = (int)((rb >> 23) & 0xFF) - 127 + ((rb & 0x7FFFFF) ? 1 : 0);
      const float s = pow2i(e), inv = pow2i(-e);
      v[i] = __fmul_rn(round_e2m1(fminf(fmaxf(__fmul_rn(v[i], inv), -6.0f), 6.0f)), s);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++) q[(size_t)h * kIdxDim + 32 * i + lane] = v[i];
  if (lane == 0) w[h] = w_raw[h] * (float)(pow((double)kIdxDim, -0.5) * pow((double)heads, -0.5));
}

// ---------------------------------------------------------------- exact top-k
struct TopkCtl { unsigned n_sel, n_cand, ticket, pad1; };

__global__ void topk_hist_kernel(const float* sc, int n, unsigned* hist) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ unsigned sh[kHistBins];
  for (int b = threadIdx.x; b < kHistBins; b += blockDim.x) sh[b] = 0;
  __syncthreads();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const float f = sc[i];
    if (selectable(f)) atomicAdd(&sh[order_key(f) >> 20], 1u);
  }
  hist_flush(sh, hist, threadIdx.x, blockDim.x);
}

// threshold bin: the highest bin b with (count of bins > b) < k <= (count of bins >= b); -1 when fewer than k finite
// scores exist (everything is selected).  Computed by every block of the compaction and by the final block.
// Inclusive scan of one value per thread over the block (a multiple of 32 threads, at most 1024): warp shuffles, then
// the warp totals.  `wsum` is 32 words of shared memory; the caller synchronises before reusing it.
__device__ __forceinline__ unsigned block_scan_incl(unsigned v, unsigned* wsum, unsigned* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  unsigned x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) wsum[warp] = x;
  __syncthreads();
  if (warp == 0) {
    unsigned s = lane < nw ? wsum[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    wsum[lane] = s;
  }
  __syncthreads();
  *total = wsum[nw - 1];
  return x + (warp ? wsum[warp - 1] : 0u);
}

// The thread's run of bins, from the top (blocks of kTopkThreads): issued early, consumed by threshold_from().
constexpr int kTopkThreads = 1024;                 // block size of the selection kernels
constexpr int kBinsPerThread = kHistBins / kTopkThreads;
struct BinRun { unsigned c[kBinsPerThread]; };
__device__ __forceinline__ void threshold_load(const unsigned* hist, BinRun& r) {
#pragma unroll
  for (int j = 0; j < kBinsPerThread; j++) r.c[j] = __ldcg(hist + (kHistBins - 1 - (threadIdx.x * kBinsPerThread + j)));
}
// count_out (may be null): the population of the threshold bin itself
__device__ __forceinline__ int threshold_from(const BinRun& r, int k, unsigned* sh /* [1024] */, unsigned* above_out, unsigned* count_out) {
  const int tid = threadIdx.x;
  constexpr int per = kBinsPerThread;
  unsigned mine = 0;
#pragma unroll
  for (int j = 0; j < kBinsPerThread; j++) mine += r.c[j];
  unsigned total;
  const unsigned incl = block_scan_incl(mine, sh, &total), excl = incl - mine;
  __shared__ int res_bin;
  __shared__ unsigned res_above, res_count;
  if (tid == 0) { res_bin = -1; res_above = total; res_count = 0; }
  __syncthreads();
  if (excl < (unsigned)k && incl >= (unsigned)k) {   // the threshold lies in this thread's run
    unsigned run = excl;
#pragma unroll
    for (int j = 0; j < kBinsPerThread; j++) {
      if (run + r.c[j] >= (unsigned)k) { res_bin = kHistBins - 1 - (tid * per + j); res_above = run; res_count = r.c[j]; break; }
      run += r.c[j];
    }
  }
  __syncthreads();
  *above_out = res_above;
  if (count_out) *count_out = res_count;
  return res_bin;
}
__device__ int threshold_bin(const unsigned* hist, int k, unsigned* sh /* [1024] */, unsigned* above_out) {
  BinRun r;
  threshold_load(hist, r);
  return threshold_from(r, k, sh, above_out, nullptr);
}

// forward declaration: the last step, run by the compaction block that finishes last
__device__ void topk_final_block(const float* sc, int n, int k, unsigned* hist, unsigned* fine, TopkCtl* ctl,
                                 const int* sel, const uint2* cand, int* out, int bm_words, const int* pos_map,
                                 bool have_bin, int bin_known, unsigned above_known);

// Compaction over the whole grid (blocks of 1024 threads), then the exact finish in the block that takes the last
// ticket: one launch for the whole selection after the histogram.
__global__ void __launch_bounds__(kTopkThreads, 2) topk_select_kernel(const float* sc, int n, int k, unsigned* hist, unsigned* fine,
                                                           TopkCtl* ctl, int* sel, uint2* cand, int* out, int bm_words,
                                                           int fused, const int* pos_map) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ unsigned sh[1024];
  __shared__ unsigned sh_fine[kHistBins];
  __shared__ int is_last;
  const int lane = threadIdx.x & 31;
  const int per_block = (n + gridDim.x - 1) / gridDim.x;
  const int i0 = blockIdx.x * per_block, i1 = min(n, i0 + per_block);
  // the first trip's scores (usually the only trip) are requested together with the histogram, ahead of the scan
  float f0[4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int i = i0 + j * (int)blockDim.x + (int)threadIdx.x;
    f0[j] = i < i1 ? sc[i] : -INFINITY;
  }
  unsigned above;
  const int bstar = threshold_bin(hist, k, sh, &above);
  for (int b = threadIdx.x; b < kHistBins; b += blockDim.x) sh_fine[b] = 0;
  __syncthreads();
  // The block's picks are collected in shared memory first (dynamic region: per_block ints for the outright selections,
  // per_block (index, key) pairs for the threshold bin's members) and appended to the global lists with ONE atomic per
  // kind and block: thousands of same-address atomics from individual warps were the bulk of this kernel's time.
  extern __shared__ unsigned dyn_smem[];
  int* sel_buf = reinterpret_cast<int*>(dyn_smem);
  uint2* cand_buf = reinterpret_cast<uint2*>(dyn_smem + ((per_block + 1) & ~1));
  __shared__ unsigned s_n1, s_n2, s_g1, s_g2;
  if (threadIdx.x == 0) { s_n1 = 0; s_n2 = 0; }
  __syncthreads();
  // 4 independent loads per thread per trip
  for (int base = i0; base < i1; base += blockDim.x * 4) {
    float f[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int i = base + j * (int)blockDim.x + (int)threadIdx.x;
      f[j] = base == i0 ? f0[j] : (i < i1 ? sc[i] : -INFINITY);
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int i = base + j * (int)blockDim.x + (int)threadIdx.x;
      int kind = 0;   // 1 = selected outright, 2 = threshold-bin candidate
      uint32_t key = 0;
      if (i < i1 && selectable(f[j])) {
        key = order_key(f[j]);
        const int b = (int)(key >> 20);
        kind = b > bstar ? 1 : (b == bstar ? 2 : 0);
        if (kind == 2) atomicAdd(&sh_fine[(key >> 8) & 0xFFFu], 1u);   // next 12 key bits of the threshold bin's members
      }
      const unsigned m1 = __ballot_sync(0xffffffffu, kind == 1), m2 = __ballot_sync(0xffffffffu, kind == 2);
      unsigned b1 = 0, b2 = 0;
      if (lane == 0) {
        if (m1) b1 = atomicAdd(&s_n1, (unsigned)__popc(m1));
        if (m2) b2 = atomicAdd(&s_n2, (unsigned)__popc(m2));
      }
      b1 = __shfl_sync(0xffffffffu, b1, 0);
      b2 = __shfl_sync(0xffffffffu, b2, 0);
      const unsigned lt = (1u << lane) - 1u;
      if (kind == 1) sel_buf[b1 + __popc(m1 & lt)] = i;
      if (kind == 2) cand_buf[b2 + __popc(m2 & lt)] = make_uint2((unsigned)i, key);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    s_g1 = s_n1 ? atomicAdd(&ctl->n_sel, s_n1) : 0u;
    s_g2 = s_n2 ? atomicAdd(&ctl->n_cand, s_n2) : 0u;
  }
  __syncthreads();
  for (unsigned i = threadIdx.x; i < s_n1; i += blockDim.x) { const unsigned pos = s_g1 + i; if (pos < 2048u) sel[pos] = sel_buf[i]; }
  for (unsigned i = threadIdx.x; i < s_n2; i += blockDim.x) cand[s_g2 + i] = cand_buf[i];
  hist_flush(sh_fine, fine, threadIdx.x, blockDim.x);
  if (!fused) return;
  // the block that takes the last ticket sees every other block's lists and finishes the selection
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&ctl->ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  topk_final_block(sc, n, k, hist, fine, ctl, sel, cand, out, bm_words, pos_map, true, bstar, above);
}

// the last step as its own launch (one block)
__global__ void __launch_bounds__(kTopkThreads) topk_final_kernel(const float* sc, int n, int k, unsigned* hist, unsigned* fine,
                                                          TopkCtl* ctl, const int* sel, const uint2* cand, int* out, int bm_words,
                                                          const int* pos_map) {
  pdl_launch_dependents();
  pdl_wait();
  topk_final_block(sc, n, k, hist, fine, ctl, sel, cand, out, bm_words, pos_map, false, 0, 0u);
}

// The selection's last step, run by ONE block of 1024 threads (the compaction block that finishes last).
// out[k] ascending, -1 padded.  Resets the histograms and ctl for the next call.
// pos_map != null: the scores are indexed by virtual position 8 * i + j standing for key pos_map[i] * 8 + j (candidate
// list, ascending); the output lists key indices (still ascending, as the list is).
// have_bin: the caller already holds the coarse threshold bin and the count above it (the compaction computed them).
__device__ void topk_final_block(const float* sc, int n, int k, unsigned* hist, unsigned* fine, TopkCtl* ctl,
                                 const int* sel, const uint2* cand, int* out, int bm_words, const int* pos_map,
                                 bool have_bin, int bin_known, unsigned above_known) {
  __shared__ unsigned sh[1024];
  __shared__ int buf[2048];
  __shared__ unsigned long long c2[1024];
  __shared__ unsigned s_cnt, s_c2, s_need, s_digit;
  extern __shared__ unsigned bitmap[];          // bm_words words when the bitmap path is used (n <= 32 * bm_words)
  const int tid = threadIdx.x, NT = blockDim.x;   // kTopkThreads
  // chosen indices go into a bitmap of the n positions (read back in ascending order: no sort), or, for very long
  // inputs that do not fit shared memory, into buf[] which is then sorted
  auto emit = [&](unsigned idx) {
    if (bm_words) atomicOr(&bitmap[idx >> 5], 1u << (idx & 31));
    else { const unsigned pos = atomicAdd(&s_cnt, 1u); if (pos < 2048u) buf[pos] = (int)idx; }
  };
  // Every global read of the finish that does not depend on another one is requested here, together: the counters,
  // the fine histogram, the first 2 NT outright selections and the first NT threshold-bin candidates.  One memory
  // latency instead of four in a row on what is the serial tail of the selection.
  const unsigned n_sel = *reinterpret_cast<volatile unsigned*>(&ctl->n_sel);
  const unsigned n_cand = *reinterpret_cast<volatile unsigned*>(&ctl->n_cand);
  BinRun fr;
  threshold_load(fine, fr);
  const int sel0 = __ldcg(sel + min(tid, 2047)), sel1 = __ldcg(sel + min(tid + NT, 2047));
  const uint2 cand0 = __ldcg(cand + min(tid, max(n, 1) - 1));
  for (int i = tid; i < bm_words; i += NT) bitmap[i] = 0;
  unsigned above = above_known;
  const int bstar = have_bin ? bin_known : threshold_bin(hist, k, sh, &above);
  for (int i = tid; i < 2048; i += NT) buf[i] = 0x7fffffff;
  if (tid == 0) { s_cnt = 0; s_c2 = 0; }
  __syncthreads();
  for (unsigned i = tid, j = 0; i < n_sel && i < 2048u; i += NT, j++)
    emit((unsigned)(j == 0 ? sel0 : j == 1 ? sel1 : __ldcg(sel + i)));
  if (bstar >= 0 && n_cand > 0) {
    const unsigned need = (unsigned)k - above;   // how many of the threshold bin's members are taken
    unsigned above2, m2;
    const int fstar = threshold_from(fr, (int)need, sh, &above2, &m2);
    if (fstar >= 0 && m2 <= 1024u) {
      const unsigned need2 = need - above2;
#pragma unroll 4
      for (unsigned i = tid; i < n_cand; i += NT) {
        const uint2 cd = i == (unsigned)tid ? cand0 : __ldcg(cand + i);
        const unsigned idx = cd.x;
        const uint32_t key = cd.y;
        const int fb = (int)((key >> 8) & 0xFFFu);
        if (fb > fstar) {
          emit(idx);
        } else if (fb == fstar) {
          const unsigned pos = atomicAdd(&s_c2, 1u);
          if (pos < 1024u) c2[pos] = ((unsigned long long)(0xFFu - (key & 0xFFu)) << 32) | idx;   // ascending = better
        }
      }
      __syncthreads();
      const unsigned m = min(s_c2, 1024u);
      for (unsigned e2 = tid; e2 < m; e2 += NT) {
        const unsigned long long mine = c2[e2];
        unsigned rank = 0;
        for (unsigned j = 0; j < m; j++) rank += c2[j] < mine;
        if (rank < need2) emit((unsigned)(mine & 0xFFFFFFFFu));
      }
      __syncthreads();
    } else {
      // radix select (descending) on the low 20 bits of the key: find T = the need-th largest key among candidates
      unsigned prefix = 0, mask = 0, remaining = need;
      for (int shift = 12; shift >= -4; shift -= 8) {
        const int sft = shift < 0 ? 0 : shift;
        const unsigned dmask = shift < 0 ? 0xFu : 0xFFu;
        for (int b = tid; b < 256; b += NT) sh[b] = 0;
        __syncthreads();
        for (unsigned i = tid; i < n_cand; i += NT) {
          const unsigned key = __ldcg(cand + i).y & 0xFFFFFu;
          if ((key & mask) == prefix) atomicAdd(&sh[(key >> sft) & dmask], 1u);
        }
        __syncthreads();
        if (tid == 0) {
          unsigned run = 0;
          int d = (int)dmask;
          for (; d > 0; d--) {
            if (run + sh[d] >= remaining) break;
            run += sh[d];
          }
          s_digit = (unsigned)d; s_need = remaining - run;
        }
        __syncthreads();
        prefix |= s_digit << sft;
        mask |= dmask << sft;
        remaining = s_need;
        __syncthreads();
      }
      const unsigned T = prefix;         // exact threshold key (low 20 bits); `remaining` members equal to T are taken
      // ties at T: take the `remaining` lowest indices.  Radix select (ascending) on the index, 3 x 8 bits (n <= 2^24).
      unsigned ip = 0, im = 0, irem = remaining;
      for (int shift = 16; shift >= 0; shift -= 8) {
        for (int b = tid; b < 256; b += NT) sh[b] = 0;
        __syncthreads();
        for (unsigned i = tid; i < n_cand; i += NT) {
          const uint2 cd = __ldcg(cand + i);
          if ((cd.y & 0xFFFFFu) == T && (cd.x & im) == ip) atomicAdd(&sh[(cd.x >> shift) & 0xFFu], 1u);
        }
        __syncthreads();
        if (tid == 0) {
          unsigned run = 0;
          int d = 0;
          for (; d < 255; d++) {
            if (run + sh[d] >= irem) break;
            run += sh[d];
          }
          s_digit = (unsigned)d; s_need = irem - run;
        }
        __syncthreads();
        ip |= s_digit << shift;
        im |= 0xFFu << shift;
        irem = s_need;
        __syncthreads();
      }
      const unsigned idxT = ip;          // members equal to T with index <= idxT are taken
      for (unsigned i = tid; i < n_cand; i += NT) {
        const uint2 cd = __ldcg(cand + i);
        const unsigned idx = cd.x;
        const unsigned key = cd.y & 0xFFFFFu;
        if (key > T || (key == T && idx <= idxT)) emit(idx);
      }
      __syncthreads();
    }
  }
  __syncthreads();
  if (bm_words) {
    // ascending read-out: every thread owns a contiguous run of bitmap words; an exclusive scan of the run
    // populations gives each run its offset in the output
    const int per = (bm_words + NT - 1) / NT;
    const int w0 = min(bm_words, tid * per), w1 = min(bm_words, w0 + per);
    unsigned cnt = 0;
    for (int w = w0; w < w1; w++) cnt += __popc(bitmap[w]);
    unsigned total;
    unsigned pos = block_scan_incl(cnt, sh, &total) - cnt;
    for (int w = w0; w < w1; w++) {
      unsigned m = bitmap[w];
      while (m) {
        const int bit = __ffs(m) - 1;
        m &= m - 1;
        if (pos < (unsigned)k) { const int v = w * 32 + bit; out[pos] = pos_map ? pos_map[v >> 3] * 8 + (v & 7) : v; }
        pos++;
      }
    }
    for (int i = tid + (int)min(total, (unsigned)k); i < k; i += NT) out[i] = -1;
  } else {
    const unsigned filled = min(s_cnt, 2048u);
    // bitonic sort of the used power-of-two prefix, ascending (unused slots hold INT_MAX)
    int P = 32;
    while (P < (int)filled) P <<= 1;
    for (int size = 2; size <= P; size <<= 1)
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int i = tid; i < P / 2; i += NT) {
          const int lo = 2 * i - (i & (stride - 1));
          const int hi = lo + stride;
          const bool up = ((lo & size) == 0);
          const int a = buf[lo], b2 = buf[hi];
          if ((a > b2) == up) { buf[lo] = b2; buf[hi] = a; }
        }
        __syncthreads();
      }
    for (int i = tid; i < k; i += NT) {
      const bool ok = i < (int)filled && buf[i] != 0x7fffffff;
      out[i] = !ok ? -1 : (pos_map ? pos_map[buf[i] >> 3] * 8 + (buf[i] & 7) : buf[i]);
    }
  }
  for (int b = tid; b < kHistBins; b += NT) { hist[b] = 0; fine[b] = 0; }
  if (tid == 0) { ctl->n_sel = 0; ctl->n_cand = 0; ctl->ticket = 0; }
  (void)n;
}

// block maxima over `bs` consecutive scores; the newest (possibly partial) block is pinned to +inf
// (attn_ref.cpp:196-202)
__global__ void block_max_kernel(const float* sc, int len, int bs, float* out, int nb) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  float m = -INFINITY;
  for (int i = b * bs; i < min(len, (b + 1) * bs); i++) m = fmaxf(m, sc[i]);
  if (b == (len - 1) / bs) m = INFINITY;
  out[b] = m;
}

// ---------------------------------------------------------------- host side
size_t topk_scratch_bytes(int n_max) {
  return 2 * sizeof(unsigned) * kHistBins + 64 + sizeof(int) * 2048 + sizeof(uint2) * (size_t)std::max(n_max, 1);
}

// scratch layout: hist[4096] | fine[4096] | ctl (64 B) | sel[2048] | cand[n_max] as (index, key) pairs.  The histograms and ctl must be zero
// on entry; the final kernel leaves them zero again.
int topk(const float* sc, int n, int k, int* out, void* scratch, size_t scratch_bytes, bool hist_ready, const int* pos_map,
         cudaStream_t st) {
  if (n < 0 || k <= 0 || k > 2048) return fail(kErrArg, "topk: n %d k %d (k must be 1..2048)", n, k);
  if (!out || !scratch || (n > 0 && !sc)) return fail(kErrArg, "topk: null pointer");
  if (scratch_bytes < topk_scratch_bytes(n)) return fail(kErrScratch, "topk: scratch too small");
  unsigned* hist = reinterpret_cast<unsigned*>(scratch);
  unsigned* fine = hist + kHistBins;
  TopkCtl* ctl = reinterpret_cast<TopkCtl*>(fine + kHistBins);
  int* sel = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(ctl) + 64);
  uint2* cand = reinterpret_cast<uint2*>(sel + 2048);
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // positions bitmap in shared memory for n up to 1M (128 KB); longer inputs use the sorting read-out
  const int bm_words = n <= (1 << 20) ? std::max(1, (n + 31) / 32) : 0;
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    MSB_CUDA(cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
    MSB_CUDA(cudaFuncSetAttribute(topk_final_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
    configured[dev & 63] = true;
  }
  // MSB_TOPK_FUSED=0: selection and read-out as two launches (topk_select_kernel + topk_final_kernel) instead of one
  static const int fused = getenv("MSB_TOPK_FUSED") ? atoi(getenv("MSB_TOPK_FUSED")) : 1;
  const int nthreads = kTopkThreads;
  // one element per thread and up to two blocks per SM: the per-block fixed work (threshold, fine histogram) is small
  // next to the latency of a longer per-thread loop
  int blocks = std::max(1, std::min(2 * sms * (1024 / nthreads), (n + nthreads - 1) / nthreads));
  // staging of a block's picks: per_block ints + per_block (index, key) pairs; blocks are added until that fits
  auto stage_of = [&](int nb) { const size_t pb = ((size_t)n + nb - 1) / nb; return ((pb + 1) & ~(size_t)1) * 4 + pb * 8 + 16; };
  while (stage_of(blocks) > 100 * 1024) blocks *= 2;
  const size_t stage_bytes = stage_of(blocks);
  if (n > 0 && !hist_ready) MSB_CUDA(launch_pdl(topk_hist_kernel, dim3(std::max(1, std::min(sms * 2, (n + 1023) / 1024))), dim3(256), 0, st, sc, n, hist));
  if (fused) {
    MSB_CUDA(launch_pdl(topk_select_kernel, dim3(blocks), dim3(nthreads), std::max((size_t)bm_words * 4, stage_bytes), st, sc, n, k, hist,
                        fine, ctl, sel, cand, out, bm_words, 1, pos_map));
  } else {
    if (n > 0) MSB_CUDA(launch_pdl(topk_select_kernel, dim3(blocks), dim3(nthreads), stage_bytes, st, sc, n, k, hist, fine, ctl, sel, cand, out, bm_words, 0, pos_map));
    MSB_CUDA(launch_pdl(topk_final_kernel, dim3(1), dim3(kTopkThreads), (size_t)bm_words * 4, st, sc, n, k, hist, fine, ctl,
                        (const int*)sel, (const uint2*)cand, out, bm_words, pos_map));
  }
  MSB_LAUNCH_CHECK("topk");
  return kOk;
}

int index_prep(const float* q_raw, const float* w_raw, const float* cs, int actq, int heads, float* q, float* w,
               cudaStream_t st) {
  if (heads <= 0 || !q_raw || !w_raw || !cs || !q || !w) return fail(kErrArg, "index_prep: bad arguments");
  MSB_CUDA(launch_pdl(idx_prep_kernel, dim3((heads + 3) / 4), dim3(128), 0, st, q_raw, w_raw, cs, actq, heads, q, w));
  MSB_LAUNCH_CHECK("idx_prep_kernel");
  return kOk;
}

int index_scores(int key_type, const void* keys, int len, const float* q, const float* w, int heads, float* scores,
                 unsigned* hist, int exact_query, cudaStream_t st) {
  if (len < 0 || (heads != 32 && heads != 64)) return fail(kErrArg, "index_scores: heads must be 32 or 64 (got %d)", heads);
  if (key_type != kKeyF16 && key_type != kKeyFp8) return fail(kErrType, "index_scores: key type %d", key_type);
  if (len == 0) return kOk;
  if (!keys || !q || !w || !scores || (reinterpret_cast<uintptr_t>(keys) & 15))
    return fail(kErrArg, "index_scores: null or misaligned pointer");
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  IdxParams p{(const uint8_t*)keys, q, w, scores, hist, len};
  // MSB_IDX_LEGACY=1: FP8 scoring on mma.sync (idx_score_fp8_kernel) instead of the tcgen05 kernel
  static const bool legacy = getenv("MSB_IDX_LEGACY") && atoi(getenv("MSB_IDX_LEGACY")) != 0;
  if (key_type == kKeyFp8 && !exact_query && !legacy) return index_scores_tc(keys, len, q, w, heads, scores, hist, 0, nullptr, 0, nullptr, nullptr, nullptr, 0, st);
  if (key_type == kKeyFp8 && !exact_query) {
    const int grid = std::max(1, std::min(sms, (len + 16 * 12 - 1) / (16 * 12)));
    if (heads == 64) MSB_CUDA(launch_pdl(idx_score_fp8_kernel<64>, dim3(grid), dim3(384), 0, st, p));
    else MSB_CUDA(launch_pdl(idx_score_fp8_kernel<32>, dim3(grid), dim3(384), 0, st, p));
  } else {
    const int grid = std::max(1, std::min(sms, (len + 32 * 8 - 1) / (32 * 8)));
    if (key_type == kKeyFp8) {
      if (heads == 64) MSB_CUDA(launch_pdl(idx_score_f16_kernel<64, true, true>, dim3(grid), dim3(256), 0, st, p));
      else MSB_CUDA(launch_pdl(idx_score_f16_kernel<32, true, true>, dim3(grid), dim3(256), 0, st, p));
    } else {
      if (heads == 64) MSB_CUDA(launch_pdl(idx_score_f16_kernel<64, false, true>, dim3(grid), dim3(256), 0, st, p));
      else MSB_CUDA(launch_pdl(idx_score_f16_kernel<32, false, true>, dim3(grid), dim3(256), 0, st, p));
    }
  }
  MSB_LAUNCH_CHECK("idx_score_kernel");
  return kOk;
}

// Candidate-restricted scoring for F16 keys (the reference's attn_idx_score_dec2_list, attn_index.metal:1056-1112):
// scores[8 i + j] = score of key cand[i] * 8 + j, -inf when cand[i] < 0 or the key is beyond len.  One warp per key:
// the key's 128 values sit in shared memory, lane l accumulates heads l and l + 32 over all 128 dims against the
// prepared fp32 query held in shared memory with a padded row stride (conflict-free), then the warp adds
// relu(q_h . k) * w_h over the heads in a fixed order.
template <int H>
__global__ void __launch_bounds__(256) idx_score_list_f16_kernel(const __half* keys, int len, const float* q, const float* w,
                                                                 const int* cand, int n_cand, float* scores) {
  pdl_launch_dependents();
  extern __shared__ float sm[];
  float* qs = sm;                         // [H][129]
  float* ks = sm + H * 129;               // [8][128]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();
  for (int i = tid; i < H * 128; i += 256) qs[(i >> 7) * 129 + (i & 127)] = q[i];
  __syncthreads();
  for (int b = blockIdx.x; b < n_cand; b += gridDim.x) {
    const int blk = cand[b];
    const long key = (long)blk * 8 + warp;
    const bool live = blk >= 0 && key < len;
    float sc = -INFINITY;
    if (live) {
      const __half2* kp = reinterpret_cast<const __half2*>(keys + (size_t)key * 128);
      const float2 a = __half22float2(kp[lane * 2]), c = __half22float2(kp[lane * 2 + 1]);
      float* kr = ks + warp * 128 + lane * 4;
      kr[0] = a.x; kr[1] = a.y; kr[2] = c.x; kr[3] = c.y;
      __syncwarp();
      float acc[H / 32];
#pragma unroll
      for (int g = 0; g < H / 32; g++) acc[g] = 0.f;
      const float* kk = ks + warp * 128;
#pragma unroll 8
      for (int d = 0; d < 128; d++) {
        const float kv = kk[d];
#pragma unroll
        for (int g = 0; g < H / 32; g++) acc[g] = fmaf(qs[(lane + 32 * g) * 129 + d], kv, acc[g]);
      }
      float v = 0.f;
#pragma unroll
      for (int g = 0; g < H / 32; g++) v += fmaxf(acc[g], 0.f) * w[lane + 32 * g];
      sc = warp_sum(v);
      __syncwarp();
    }
    if (lane == 0) scores[(size_t)b * 8 + warp] = sc;
  }
}

int index_scores_list_f16(const void* keys, int len, const float* q, const float* w, int heads, const int* cand, int n_cand,
                          float* scores, cudaStream_t st) {
  if (heads != 32 && heads != 64) return fail(kErrArg, "index_scores_list: heads must be 32 or 64");
  if (!keys || !q || !w || !cand || !scores || n_cand <= 0) return fail(kErrArg, "index_scores_list: bad arguments");
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const size_t smem = ((size_t)heads * 129 + 8 * 128) * sizeof(float);
  const int grid = std::max(1, std::min(n_cand, sms * 4));
  if (heads == 64) MSB_CUDA(launch_pdl(idx_score_list_f16_kernel<64>, dim3(grid), dim3(256), smem, st, (const __half*)keys, len, q, w, cand, n_cand, scores));
  else MSB_CUDA(launch_pdl(idx_score_list_f16_kernel<32>, dim3(grid), dim3(256), smem, st, (const __half*)keys, len, q, w, cand, n_cand, scores));
  MSB_LAUNCH_CHECK("idx_score_list_f16_kernel");
  return kOk;
}

int block_max(const float* sc, int len, int bs, float* out, cudaStream_t st) {
  if (len <= 0 || bs <= 0 || !sc || !out) return fail(kErrArg, "block_max: bad arguments");
  const int nb = (len + bs - 1) / bs;
  MSB_CUDA(launch_pdl(block_max_kernel, dim3((nb + 255) / 256), dim3(256), 0, st, sc, len, bs, out, nb));
  MSB_LAUNCH_CHECK("block_max_kernel");
  return kOk;
}

}  // namespace msb
