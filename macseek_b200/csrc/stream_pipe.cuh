// Weight-streaming pipeline shared by the decode kernels (matvec, MoE gate/up, MoE down).
//
// One bulk copy costs the SM's copy engine a fixed ~60 ns whatever its size (measured: 272-byte copies stream at
// 0.7 TB/s, 1 KB copies at 2.4 TB/s, 4 KB copies at 4.1 TB/s), so pieces are laid out as few, large, contiguous
// copies: a tile of consecutive full rows is ONE copy.
//
// A block is (NW consumer warps + 1 producer warp).  The producer warp walks the block's list of "pieces" -- R rows x
// a contiguous run of 32-element units of one or several weight matrices -- and brings each piece into one slot of a shared-memory
// ring with 1-D TMA bulk copies (one per row; the source is rounded down to 16 bytes and the copy length up, so raw
// GGUF rows that are only 2-byte aligned still move as 16-byte bursts).  Consumer warps wait on the slot's "full"
// mbarrier, decode their rows straight out of shared memory, and release the slot through its "empty" mbarrier.
// Every wait is bounded (mbar_wait): a stuck barrier ends the kernel with a status code instead of hanging the GPU.
#pragma once
#include "quant_blocks.cuh"

namespace msb {

constexpr int kMaxStages = 4;
constexpr int kSmemLimit = 227 * 1024;

// Scalar members only (no arrays): the struct must stay in registers, a dynamically indexed member would push it to
// local memory.
struct Ring {
  uint8_t* slot0;        // slot s = slot0 + s * slot_bytes
  uint32_t slot_bytes;
  uint64_t* full;        // [stages]
  uint64_t* empty;       // [stages]
  volatile int* abort_flag;
  int* status;
  int stages;
  __device__ __forceinline__ uint8_t* slot(uint32_t n) const { return slot0 + (size_t)(n % stages) * slot_bytes; }
};

struct Piece {
  const uint8_t* const* src;  // [nsrc] global address of each source's first row (array in shared or param memory)
  int nsrc;                   // sources staged side by side in one slot (e.g. gate and up rows, or one per expert)
  int rows_per_src;           // local rows reserved per source in the slot
  int nrows;                  // rows present per source (1 .. rows_per_src)
  uint32_t row_stride;        // bytes between consecutive rows in global memory
  uint32_t bytes;             // bytes per row of the piece
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

// Producer warp: fill the slot for use number n (n counts pieces handled by this block).  Local row
// lr = source * rows_per_src + row lands at slot + lr * pitch (+ the source address's low 4 bits).
// Returns false after an abandoned wait.
__device__ __forceinline__ bool produce_piece(const Ring& r, uint32_t n, const Piece& p, uint32_t pitch, int lane) {
  const int s = n % r.stages;
  const uint32_t ph = (n / r.stages) & 1u;
  if (!mbar_wait(&r.empty[s], ph ^ 1u, r.abort_flag, r.status, kDevWaitEmpty)) return false;
  const int total_rows = p.nsrc * p.rows_per_src;
  uint32_t mine = 0;
  for (int lr = lane; lr < total_rows; lr += 32) {
    const int si = lr / p.rows_per_src, row = lr - si * p.rows_per_src;
    if (row >= p.nrows) continue;
    const uintptr_t a = reinterpret_cast<uintptr_t>(p.src[si]) + (uintptr_t)row * p.row_stride;
    mine += (uint32_t)(((a & 15u) + p.bytes + 15u) & ~15u);
  }
  uint32_t total = mine;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  if (lane == 0) mbar_arrive_expect_tx(&r.full[s], total);
  __syncwarp();
  for (int lr = lane; lr < total_rows; lr += 32) {
    const int si = lr / p.rows_per_src, row = lr - si * p.rows_per_src;
    if (row >= p.nrows) continue;
    const uintptr_t a = reinterpret_cast<uintptr_t>(p.src[si]) + (uintptr_t)row * p.row_stride;
    const uint32_t len = (uint32_t)(((a & 15u) + p.bytes + 15u) & ~15u);
    uint8_t* dst = r.slot0 + (size_t)s * r.slot_bytes + (size_t)lr * pitch;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a & ~(uintptr_t)15);
    for (uint32_t o = 0; o < len; o += 32768u) tma_load_1d(dst + o, src + o, min(32768u, len - o), &r.full[s]);
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
// shared-memory address of row `row` of source `si` of the piece held in the slot of use n
__device__ __forceinline__ const uint8_t* piece_row(const Ring& r, uint32_t n, const Piece& p, uint32_t pitch, int si,
                                                    int row) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p.src[si]) + (uintptr_t)row * p.row_stride;
  return r.slot(n) + (size_t)(si * p.rows_per_src + row) * pitch + (a & 15u);
}

// Bring the lookup tables a type needs into shared memory with bulk copies of the pre-replicated images and return
// the lane's view.  `bar` is a dedicated mbarrier (initialised with count 1 by the caller before a __syncthreads);
// every thread waits for the bytes (bounded).  Returns false after an abandoned wait.
__device__ __forceinline__ bool load_luts(uint8_t* lut, bool iq1s, bool iq2, bool iq4, const Tables& tb, int tid,
                                          uint64_t* bar, volatile int* abort_flag, LaneLuts& L, int lane) {
  saddr_t p = smem_u32(lut);
  L.iq1s = L.iq2g = L.iq2s = L.iq4 = p;
  uint32_t total = 0;
  if (iq1s) { L.iq1s = p + 4 * (lane % kIq1sCopies); p += kIq1sLutBytes; total += kIq1sLutBytes; }
  if (iq2) {
    L.iq2g = p + 4 * (lane % kIq2Copies); p += kIq2GridLutBytes;
    L.iq2s = p + 4 * (lane % kIq2Copies); p += kIq2SignLutBytes;
    total += kIq2GridLutBytes + kIq2SignLutBytes;
  }
  if (iq4) { L.iq4 = p + 4 * (lane % kIq4Copies); p += kIq4LutBytes; total += kIq4LutBytes; }
  if (total == 0) return true;
  if (tid == 0) {
    mbar_arrive_expect_tx(bar, total);
    uint8_t* q = lut;
    auto copy = [&](const uint8_t* src, uint32_t bytes) {
      for (uint32_t o = 0; o < bytes; o += 16384) tma_load_1d(q + o, src + o, min(16384u, bytes - o), bar);
      q += bytes;
    };
    if (iq1s) copy(tb.img_iq1s, kIq1sLutBytes);
    if (iq2) { copy(tb.img_iq2g, kIq2GridLutBytes); copy(tb.img_iq2s, kIq2SignLutBytes); }
    if (iq4) copy(tb.img_iq4, kIq4LutBytes);
  }
  return mbar_wait(bar, 0, abort_flag, tb.status, kDevWaitFull);
}

// Partial dot products of `nunits` staged units for NRT rows of one lane group: LPR lanes split the units, the x
// registers of a unit are loaded once and shared by the NRT rows and NC activation columns.
//   acc[i][c] += sum over this lane's units of  row_i[unit] . x_c[unit0 + unit]
template <int T, int LPR, int NRT, int NC>
__device__ __forceinline__ void consume_rows(const saddr_t (&rowp)[NRT], int li, const XqSmem (&xq)[NC], int unit0,
                                             int nunits, const LaneLuts& L, float (&acc)[NRT][NC]) {
  if constexpr (T == Q6_K) {
    // lanes split the row's half super-blocks (the staged run starts on a super-block and holds whole ones)
    for (int it = li; it < nunits / 4; it += LPR) {
      saddr_t blk[NRT];
#pragma unroll
      for (int i = 0; i < NRT; i++) blk[i] = rowp[i] + (uint32_t)(it >> 1) * 210u;
      q6k_half_block<NRT, NC>(blk, it & 1, xq, unit0 + 4 * it, acc);
    }
    return;
  }
  if constexpr (T == IQ1_S) {
    // lanes split the row's half super-blocks, as above
    for (int it = li; it < nunits / 4; it += LPR) {
      saddr_t blk[NRT];
#pragma unroll
      for (int i = 0; i < NRT; i++) blk[i] = rowp[i] + (uint32_t)(it >> 1) * 50u;
      iq1s_half_block<NRT, NC>(blk, it & 1, xq, unit0 + 4 * it, L, acc);
    }
    return;
  }
  if constexpr (is_dense(T)) {
    // lanes split the run's 16-byte weight granules (4 fp32 or 8 16-bit elements), consecutive lanes on consecutive
    // granules; the activation is fp32 in shared memory (two planes for 16-bit weights, see the staging code)
    constexpr int kGran = T == F32 ? 8 : 4;            // granules per 32-element unit
    const int ng = nunits * kGran;
    for (int g = li; g < ng; g += LPR) {
      float xv[NC][8];
#pragma unroll
      for (int c = 0; c < NC; c++) {
        const saddr_t xa = xq[c].xf_s + 16u * (uint32_t)(unit0 * kGran + g);
        const float4 x0 = lds_f128(xa);
        xv[c][0] = x0.x; xv[c][1] = x0.y; xv[c][2] = x0.z; xv[c][3] = x0.w;
        if (T != F32) {
          const float4 x1 = lds_f128(xa + 64u * (uint32_t)xq[c].U);
          xv[c][4] = x1.x; xv[c][5] = x1.y; xv[c][6] = x1.z; xv[c][7] = x1.w;
        }
      }
#pragma unroll
      for (int i = 0; i < NRT; i++) {
        const saddr_t wp = rowp[i] + 16u * (uint32_t)g;
        uint32_t w[4];
        if ((wp & 15u) == 0) { const uint4 v = lds_u128(wp); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
        else load_words<4>(wp, w);
        float a[8];
        if (T == F32) {
#pragma unroll
          for (int k = 0; k < 4; k++) a[k] = __uint_as_float(w[k]);
        } else {
#pragma unroll
          for (int k = 0; k < 4; k++) {
            if (T == BF16) { a[2 * k] = __uint_as_float(w[k] << 16); a[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u); }
            else { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k])); a[2 * k] = f.x; a[2 * k + 1] = f.y; }
          }
        }
#pragma unroll
        for (int c = 0; c < NC; c++) {
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int k = 0; k < (T == F32 ? 4 : 8); k += 2) { s0 = fmaf(a[k], xv[c][k], s0); s1 = fmaf(a[k + 1], xv[c][k + 1], s1); }
          acc[i][c] += s0 + s1;
        }
      }
    }
    return;
  }
  if constexpr (T != IQ1_S && T != Q6_K && !is_dense(T))
  for (int uu = li; uu < nunits; uu += LPR) {
    XRegs xr[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) load_xq(xq[c], unit0 + uu, xr[c]);
#pragma unroll
    for (int i = 0; i < NRT; i++) {
      Dec<T> d;
      decode_unit<T>(rowp[i], uu, L, d);
#pragma unroll
      for (int c = 0; c < NC; c++) acc[i][c] += dot_unit<T>(d, xr[c]);
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

// Largest staged chunk (in 32-element units) of a type-t row such that `rows` row pieces fit in slot_bytes; a multiple
// of the lane stride and of a super-block where possible.  0 if nothing fits.
inline int chunk_units_for(int t, int units, int rows, int lpr, size_t slot_bytes) {
  const bool sb = block_elems(t) == 256;
  const int step = sb ? (lpr > 8 ? lpr : 8) : lpr;
  const long per_row = (long)(slot_bytes / rows) - 64;          // piece_pitch(b) <= b + 62
  if (per_row <= 0) return 0;
  const long by_bytes = sb ? per_row / block_bytes(t) * 8 : per_row / units_bytes(t, 1);
  long chunk = by_bytes < units ? by_bytes : units;
  if (chunk < units && chunk >= step) chunk = chunk / step * step;   // else: a short chunk, some lanes idle
  if (sb) chunk = chunk / 8 * 8;
  return (int)chunk;
}

}  // namespace msb
