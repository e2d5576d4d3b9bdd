// Weight-streaming pipeline shared by the decode kernels (matvec, MoE gate/up, MoE down).
//
// A block is (NW consumer warps + 1 producer warp).  The producer warp walks the block's list of "pieces" -- R rows x
// a contiguous run of 32-element units of one weight matrix -- and brings each piece into one slot of a shared-memory
// ring with 1-D TMA bulk copies (one per row; the source is rounded down to 16 bytes and the copy length up, so raw
// GGUF rows that are only 2-byte aligned still move as 16-byte bursts).  Consumer warps wait on the slot's "full"
// mbarrier, decode their rows straight out of shared memory, and release the slot through its "empty" mbarrier.
// Every wait is bounded (mbar_wait): a stuck barrier ends the kernel with a status code instead of hanging the GPU.
#pragma once
#include "quant_blocks.cuh"

namespace msb {

constexpr int kMaxStages = 4;
constexpr int kSmemLimit = 227 * 1024;

struct Ring {
  uint8_t* slot[kMaxStages];
  uint64_t* full;    // [stages]
  uint64_t* empty;   // [stages]
  volatile int* abort_flag;
  int* status;
  int stages;
};

struct Piece {
  const uint8_t* src;    // global address of the first row's first byte of the piece
  uint32_t row_stride;   // bytes between consecutive rows in global memory
  uint32_t bytes;        // bytes per row of the piece
  int nrows;             // rows present (1 .. R)
};

__host__ __device__ inline uint32_t piece_pitch(uint32_t max_piece_bytes) {
  // room for the source misalignment (<= 15), rounded to 16, plus 16 bytes that load_words may read past the end;
  // an odd multiple of 16 keeps consecutive rows on different bank groups
  uint32_t p = ((max_piece_bytes + 15 + 15) & ~15u) + 16;
  if ((p & 16u) == 0) p += 16;
  return p;
}

#ifdef __CUDACC__
__device__ __forceinline__ void ring_init(Ring& r, int tid, int consumer_warps) {
  if (tid == 0) {
    for (int s = 0; s < r.stages; s++) { mbar_init(&r.full[s], 1); mbar_init(&r.empty[s], consumer_warps); }
    *r.abort_flag = 0;
    mbar_fence_init();
  }
}

// Producer warp: fill the slot for use number n (n counts pieces handled by this block).  Returns false after an
// abandoned wait.
__device__ __forceinline__ bool produce_piece(const Ring& r, uint32_t n, const Piece& p, uint32_t pitch, int lane) {
  const int s = n % r.stages;
  const uint32_t ph = (n / r.stages) & 1u;
  if (!mbar_wait(&r.empty[s], ph ^ 1u, r.abort_flag, r.status, kDevWaitEmpty)) return false;
  uint32_t mine = 0;
  for (int row = lane; row < p.nrows; row += 32) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p.src) + (uintptr_t)row * p.row_stride;
    mine += (uint32_t)(((a & 15u) + p.bytes + 15u) & ~15u);
  }
  uint32_t total = mine;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  if (lane == 0) mbar_arrive_expect_tx(&r.full[s], total);
  __syncwarp();
  for (int row = lane; row < p.nrows; row += 32) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p.src) + (uintptr_t)row * p.row_stride;
    const uint32_t len = (uint32_t)(((a & 15u) + p.bytes + 15u) & ~15u);
    tma_load_1d(r.slot[s] + (size_t)row * pitch, reinterpret_cast<const void*>(a & ~(uintptr_t)15), len, &r.full[s]);
  }
  return true;
}

__device__ __forceinline__ bool consumer_wait(const Ring& r, uint32_t n) {
  return mbar_wait(&r.full[n % r.stages], (n / r.stages) & 1u, r.abort_flag, r.status, kDevWaitFull);
}
__device__ __forceinline__ void consumer_release(const Ring& r, uint32_t n, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(&r.empty[n % r.stages]);
}
// shared-memory address of local row `lr` of the piece held in the slot of use n
__device__ __forceinline__ const uint8_t* piece_row(const Ring& r, uint32_t n, const Piece& p, uint32_t pitch, int lr) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p.src) + (uintptr_t)lr * p.row_stride;
  return r.slot[n % r.stages] + (size_t)lr * pitch + (a & 15u);
}

// Copy the lookup tables a type needs into shared memory (replicated per bank group) and return the lane's view.
__device__ __forceinline__ void fill_luts(uint8_t* lut, bool iq1s, bool iq2, bool iq4, const Tables& tb, int tid, int nthreads,
                                          LaneLuts& L, int lane) {
  uint8_t* p = lut;
  L.iq1s = L.iq2g = L.iq2s = L.iq4 = lut;
  if (iq1s) {
    uint32_t* d = reinterpret_cast<uint32_t*>(p);
    for (int i = tid; i < 2048 * kIq1sCopies; i += nthreads) d[i] = __ldg(tb.iq1s_nib + i / kIq1sCopies);
    L.iq1s = p + 4 * (lane % kIq1sCopies);
    p += kIq1sLutBytes;
  }
  if (iq2) {
    uint2* d = reinterpret_cast<uint2*>(p);
    for (int i = tid; i < 256 * kIq2Copies; i += nthreads) d[i] = __ldg(tb.iq2xxs_grid + i / kIq2Copies);
    L.iq2g = p + 8 * (lane % kIq2Copies);
    p += kIq2GridLutBytes;
    d = reinterpret_cast<uint2*>(p);
    for (int i = tid; i < 128 * kIq2Copies; i += nthreads) d[i] = __ldg(tb.iq2_signmask + i / kIq2Copies);
    L.iq2s = p + 8 * (lane % kIq2Copies);
    p += kIq2SignLutBytes;
  }
  if (iq4) {
    uint32_t* d = reinterpret_cast<uint32_t*>(p);
    for (int i = tid; i < 256 * kIq4Copies; i += nthreads) d[i] = __ldg(tb.iq4nl_pair + i / kIq4Copies);
    L.iq4 = p + 4 * (lane % kIq4Copies);
    p += kIq4LutBytes;
  }
}

// Partial dot products of one staged piece for the rows of this lane group.
//   LPR lanes share a row; the warp covers G = 32 / LPR row groups x NR rows; NC activation columns.
//   acc[r][c] += sum over the piece's units handled by this lane.
template <int T, int LPR, int NR, int NC>
__device__ __forceinline__ void consume_piece(const Ring& r, uint32_t n, const Piece& p, uint32_t pitch, int warp_row0,
                                              int lane, const XqSmem (&xq)[NC], int unit0, int nunits,
                                              const LaneLuts& L, float (&acc)[NR][NC]) {
  constexpr int G = 32 / LPR;
  const int grp = lane / LPR, li = lane % LPR;
  const uint8_t* rowp[NR];
#pragma unroll
  for (int i = 0; i < NR; i++) rowp[i] = piece_row(r, n, p, pitch, warp_row0 + grp * NR + i);
  (void)G;
  for (int uu = li; uu < nunits; uu += LPR) {
    if constexpr (is_dense(T)) {
#pragma unroll
      for (int i = 0; i < NR; i++)
#pragma unroll
        for (int c = 0; c < NC; c++) acc[i][c] += unit_dot_dense<T>(rowp[i], uu, xq[c].xf + 32 * unit0);
    } else {
      XRegs xr[NC];
#pragma unroll
      for (int c = 0; c < NC; c++) load_xq(xq[c], unit0 + uu, xr[c]);
#pragma unroll
      for (int i = 0; i < NR; i++) {
        Dec<T> d;
        decode_unit<T>(rowp[i], uu, L, d);
#pragma unroll
        for (int c = 0; c < NC; c++) acc[i][c] += dot_unit<T>(d, xr[c]);
      }
    }
  }
}

template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
#endif

}  // namespace msb
