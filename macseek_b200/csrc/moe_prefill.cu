// MoE prefill: grouped expert GEMMs on the 5th-generation tensor cores.
// Replaces the reference's prefill MoE kernels (src/kernels/quant_moe_prefill.metal:22-344) behind
// ms::q::encode_moe_prefill (src/kernels/quant.hpp:87-118, quant.mm:427-612).  Same arithmetic as the reference's
// tensor path: activations, expert weights and the intermediate H as half operands, fp32 accumulation;
//   H[e][r] = half( silu(min(g,10)) * clamp(u,-10,10) * wt[e] ),  Z[e] = H[e] . down^T,
//   Y[t] += Z[shared row of t] + sum_k Z[slot_of[t][k]]   in that fixed order.
//
// Routing arrives expert-sorted (entries [offs[j], offs[j+1]) of tok[] / wt[] belong to routed expert j).  Launches:
//   gather      Xg[entry] = half(X[tok[entry]]); the shared expert's rows (every token, weight 1) follow the routed ones
//   gate/up     one grouped GEMM per weight type (routed experts, shared expert): tile = 128 entries x (64 gate rows +
//               the same 64 up rows), SwiGLU in the epilogue, H stored as half
//   down        the same grouped GEMM with 128 down rows per tile, Z stored as fp32
//   combine     the fixed-order sum into Y
// Grouped GEMM kernel, one persistent CTA per SM, 14 warps: warps 0..3 epilogue (TMEM lane = entry), warp 4 one
// MMA-issuing thread (tcgen05.mma kind::f16, M 128, N 128, K 16), warp 5 one TMA thread for the activation tiles
// (128-byte swizzle), warps 6..13 dequantise the tile's weight rows from the raw GGUF blocks straight into the swizzled
// shared-memory operand layout (no half copy of the experts in HBM: every expert weight is used by one tile row block
// only).  Tiles come from a table the host builds from offs[].  Every mbarrier wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>
#include <algorithm>
#include <vector>
#include "quant_blocks.cuh"

namespace msb {

constexpr int kMpBM = 128, kMpBN = 128, kMpBK = 64;
constexpr int kMpABytes = kMpBM * kMpBK * 2, kMpBBytes = kMpBN * kMpBK * 2;
constexpr int kMpStages = 5;
constexpr int kMpBNDense = 256, kMpStagesDense = 4;   // the TMA-fed variant's N tile and ring depth (4 x 48 KB)
// selector tables of the in-kernel decode.  IQ1_S: 2048 x 8 bytes.  IQ2_XXS: the 256 x 8-byte magnitude selectors in
// 8 copies (copy = lane % 8; 16 KB) and the 128 sign patterns as one word each in 16 copies (copy = lane % 16; 8 KB),
// so that the lanes of one shared-memory wavefront mostly read different banks: with single copies of these small
// tables the look-ups' bank conflicts kept the LSU data pipe 82 % busy.
constexpr int kMpLutBytes = 24576;
constexpr int kMpIq2SelCopies = 8, kMpIq2SignCopies = 16, kMpIq2SignOff = 256 * 8 * kMpIq2SelCopies;
constexpr int kMpProducerWarps = 8;
constexpr int kMpBatch = 2;            // K blocks a producer thread decodes per hand-over to the MMA (1, 2 or 4)
// Raw-block staging of the in-kernel decode: per producer warp 16 tile rows x 8 units x 16 bytes {word a, word b, block
// scale}, rows 160 bytes apart (so that the four rows a quarter warp touches with one 16-byte access sit 32 bytes apart
// modulo 128: no bank conflicts on either side)
constexpr int kMpStgRow = 160, kMpStgWarp = 16 * kMpStgRow, kMpStgBytes = kMpProducerWarps * kMpStgWarp;
constexpr int kMpThreads = (4 + 1 + 1 + kMpProducerWarps) * 32;

struct MpTile { int slot, row0, rows, n0; };   // expert slot, first entry row, valid rows (<= 128), first weight row

struct MpGemmParams {
  CUtensorMap a_map;        // activations [rows_total][K] half, box 64 x 128
  CUtensorMap b_map;        // dense source: half weights of the dense experts stacked by rows, box 64 x (64 | 128)
  const MpTile* tiles;
  const uint64_t* wptr;     // [slots][3] device addresses {gate, up, down}
  const float* wt;          // [rows_total] routing weight per entry row (mode 0)
  __half* h;                // mode 0 output [rows_total][n_out]
  float* z;                 // mode 1 output [rows_total][n_out]
  int* status;
  int ntiles, K, n_out;     // K = contraction length (dim / inter), n_out = output row width (inter / dim)
                            // dense source: tile.slot = index of the expert in the stacked half matrix, whose rows
                            // are [slot * 2 n_out, +n_out) gate, [.. + n_out, +n_out) up (mode 0) or [slot * n_out, +n_out) down
  float limit;
  Tables tb;
};

struct MpHead {
  uint64_t full[kMpStages], empty[kMpStages], accfull[2], accempty[2];   // kMpStages >= kMpStagesDense
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint64_t mp_desc(uint32_t saddr) {   // K-major, 128-byte swizzle, 8-row groups 1024 B apart
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mp_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mp_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void mp_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mp_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mp_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mp_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void mp_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One 32-element unit of an IQ1_S / IQ2_XXS row -> 32 halfs (4 chunks of 8), each value the reference's dequantised
// float (the arithmetic of dequant8, tests/ref/dequant.cpp:72-120) rounded to half once.  The unit's raw bytes are
// fetched one K block ahead (they come from HBM: every expert weight is read once); the scalars (block scale, 3/4-bit
// sub-scale, delta / signs word) are combined once for the 32 elements.
struct MpRaw { uint32_t a, b; float d; };   // IQ1_S: qs word, qh;  IQ2_XXS: grid-index word, signs + scale word;  d = block scale

template <int T>
__device__ __forceinline__ MpRaw mp_fetch_unit(const uint8_t* blk, int ib) {
  MpRaw r;
  r.d = ldg_half(blk);
  if (T == IQ1_S) {
    r.a = ldg_u16(blk + 2 + 4 * ib) | (ldg_u16(blk + 4 + 4 * ib) << 16);
    r.b = ldg_u16(blk + 34 + 2 * ib);
  } else {
    const uint8_t* a8 = blk + 2 + 8 * ib;
    r.a = ldg_u16(a8) | (ldg_u16(a8 + 2) << 16);
    r.b = ldg_u16(a8 + 4) | (ldg_u16(a8 + 6) << 16);
  }
  return r;
}
// lut: the selector tables in shared memory (IQ1_S: uint2 [2048]; IQ2_XXS: see kMpLutBytes) -- the raw-byte
// fetches of 256 rows at a time sweep the L1, so tables left in global memory miss it on most look-ups
template <int T>
__device__ __forceinline__ void mp_decode_unit(const MpRaw& r, const uint8_t* lut, int lane, uint4 (&out)[4]) {
  if (T == IQ1_S) {
    const uint32_t qs = r.a, qh = r.b;
    const float dl = __fmul_rn(r.d, (float)(2 * ((qh >> 12) & 7u) + 1));
    const float delta = (qh & 0x8000u) ? -0.125f : 0.125f;
    // a unit has only three distinct values dl * (g + delta), g = -1, 0, 1: round them to half once (exactly what the
    // per-element arithmetic gives) and let a byte permute pick two of them per table selector
    const __half2 h01 = __floats2half2_rn(__fmul_rn(dl, __fadd_rn(-1.f, delta)), __fmul_rn(dl, __fadd_rn(0.f, delta)));
    const __half2 h2x = __floats2half2_rn(__fmul_rn(dl, __fadd_rn(1.f, delta)), 0.f);
    const uint32_t pool_lo = *reinterpret_cast<const uint32_t*>(&h01), pool_hi = *reinterpret_cast<const uint32_t*>(&h2x);
#pragma unroll
    for (int l = 0; l < 4; l++) {
      const uint32_t idx = ((qs >> (8 * l)) & 0xFFu) | (((qh >> (3 * l)) & 7u) << 8);
      const uint2 sel = reinterpret_cast<const uint2*>(lut)[idx];
      out[l] = make_uint4(__byte_perm(pool_lo, pool_hi, sel.x & 0xFFFFu), __byte_perm(pool_lo, pool_hi, sel.x >> 16),
                          __byte_perm(pool_lo, pool_hi, sel.y & 0xFFFFu), __byte_perm(pool_lo, pool_hi, sel.y >> 16));
    }
  } else {
    const uint32_t q = r.a, a1 = r.b;
    const float db = __fmul_rn(__fmul_rn(r.d, __fadd_rn(0.5f, (float)(a1 >> 28))), 0.25f);
    // three magnitudes per unit (db * 8, db * 25, db * 43), rounded to half once; the sign is the half's top bit
    const __half2 h01 = __floats2half2_rn(__fmul_rn(db, 8.f), __fmul_rn(db, 25.f));
    const __half2 h2x = __floats2half2_rn(__fmul_rn(db, 43.f), 0.f);
    const uint32_t pool_lo = *reinterpret_cast<const uint32_t*>(&h01), pool_hi = *reinterpret_cast<const uint32_t*>(&h2x);
#pragma unroll
    for (int l = 0; l < 4; l++) {
      const uint2 sel = reinterpret_cast<const uint2*>(lut)[((q >> (8 * l)) & 0xFFu) * kMpIq2SelCopies + (lane & (kMpIq2SelCopies - 1))];
      const uint32_t sg = reinterpret_cast<const uint32_t*>(lut + kMpIq2SignOff)[((a1 >> (7 * l)) & 127u) * kMpIq2SignCopies +
                                                                                 (lane & (kMpIq2SignCopies - 1))];
      constexpr uint32_t kS = 0x80008000u;
      out[l] = make_uint4(__byte_perm(pool_lo, pool_hi, sel.x & 0xFFFFu) ^ (sg & kS), __byte_perm(pool_lo, pool_hi, sel.x >> 16) ^ ((sg << 1) & kS),
                          __byte_perm(pool_lo, pool_hi, sel.y & 0xFFFFu) ^ ((sg << 2) & kS), __byte_perm(pool_lo, pool_hi, sel.y >> 16) ^ ((sg << 3) & kS));
    }
  }
}

// MODE 0: gate/up + SwiGLU -> H (half);  MODE 1: down -> Z (fp32).  T = weight type of every tile of the launch.
// DENSE: the weight tiles come by TMA from a half copy (experts with many entries are dequantised once instead of once
// per entry tile); the producer warps idle.
template <int T, int MODE, bool DENSE>
__global__ void __launch_bounds__(kMpThreads, 1) moep_gemm_kernel(const __grid_constant__ MpGemmParams p) {
  pdl_launch_dependents();
  extern __shared__ __align__(1024) uint8_t mp_smem_raw[];
  uint8_t* smem = mp_smem_raw + ((1024u - (smem_u32(mp_smem_raw) & 1023u)) & 1023u);
  MpHead* hd = reinterpret_cast<MpHead*>(smem);
  uint8_t* stage0 = smem + 1024;
  // The TMA-fed variant works on 128 x 256 tiles: a 128 x 128 x 64 step reads 32 KB of operands from shared memory for
  // 256 tensor-pipe cycles of work, exactly the shared-memory bandwidth, so any hiccup stalls the MMA; at N = 256 the
  // step reads 48 KB for 512 cycles.  The producer-fed variant stays at N = 128 (its pace is the producers').
  constexpr int BN = DENSE ? kMpBNDense : kMpBN, BBytes = BN * kMpBK * 2, STG = DENSE ? kMpStagesDense : kMpStages;
  uint8_t* lut = stage0 + (size_t)STG * (kMpABytes + BBytes);      // kMpLutBytes, producers of IQ types only
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr uint32_t kCols = 2 * BN;
  if constexpr (!DENSE && (T == IQ1_S || T == IQ2_XXS)) {
    // constant tables: copied before the dependency wait
    if (T == IQ1_S) {
      for (int i = tid; i < 2048; i += kMpThreads) reinterpret_cast<uint2*>(lut)[i] = __ldg(p.tb.iq1s_sel + i);
    } else {
      for (int i = tid; i < 256 * kMpIq2SelCopies; i += kMpThreads) reinterpret_cast<uint2*>(lut)[i] = __ldg(p.tb.iq2_sel + i / kMpIq2SelCopies);
      // sign pattern word: bit 15 - j = sign of element 2 j, bit 31 - j = sign of element 2 j + 1 (j = 0..3), so that
      // (word << j) & 0x80008000 is the XOR mask of the j-th pair of halfs
      for (int i = tid; i < 128 * kMpIq2SignCopies; i += kMpThreads) {
        const uint4 sg = __ldg(p.tb.iq2_sign16 + i / kMpIq2SignCopies);
        const uint32_t w[4] = {sg.x, sg.y, sg.z, sg.w};
        uint32_t e = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) e |= ((w[j] >> 15) & 1u) << (15 - j) | ((w[j] >> 31) & 1u) << (31 - j);
        reinterpret_cast<uint32_t*>(lut + kMpIq2SignOff)[i] = e;
      }
    }
  }

  if (tid == 0) {
    for (int s = 0; s < STG; s++) { mbar_init(&hd->full[s], DENSE ? 1 : 1 + kMpProducerWarps); mbar_init(&hd->empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&hd->accfull[b], 1); mbar_init(&hd->accempty[b], 4); }
    hd->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&hd->tmem_base)), "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  mp_fence_before();
  __syncthreads();
  mp_fence_after();
  const uint32_t tmem = hd->tmem_base;
  volatile int* abort_flag = &hd->abort_flag;
  const int kb = p.K / kMpBK;
  const int my_tiles = p.ntiles > (int)blockIdx.x ? (p.ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  pdl_wait();

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA thread: activation tiles
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int i = 0; ok && i < my_tiles; i++) {
        const MpTile tl = p.tiles[(int)blockIdx.x + i * (int)gridDim.x];
        for (int k = 0; k < kb; k++, it++) {
          const int s = it % STG;
          if (!mbar_wait_sleep(&hd->empty[s], ((it / STG) & 1u) ^ 1u, abort_flag, p.status, kDevWaitEmpty, 100)) { ok = false; break; }
          uint8_t* slot = stage0 + (size_t)s * (kMpABytes + BBytes);
          mbar_arrive_expect_tx(&hd->full[s], DENSE ? kMpABytes + BBytes : kMpABytes);
          mp_tma_2d(slot, &p.a_map, k * kMpBK, tl.row0, &hd->full[s]);
          if (DENSE) {
            if (MODE == 0) {   // BN / 2 gate rows, then the same up rows
              mp_tma_2d(slot + kMpABytes, &p.b_map, k * kMpBK, tl.slot * 2 * p.n_out + tl.n0, &hd->full[s]);
              mp_tma_2d(slot + kMpABytes + BBytes / 2, &p.b_map, k * kMpBK, tl.slot * 2 * p.n_out + p.n_out + tl.n0, &hd->full[s]);
            } else {
              mp_tma_2d(slot + kMpABytes, &p.b_map, k * kMpBK, tl.slot * p.n_out + tl.n0, &hd->full[s]);
            }
          }
        }
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kMpBM >> 4) << 24);
      uint32_t it = 0;
      bool ok = true;
      for (int i = 0; ok && i < my_tiles; i++) {
        const int buf = i & 1;
        if (!mbar_wait_sleep(&hd->accempty[buf], ((i >> 1) & 1u) ^ 1u, abort_flag, p.status, kDevWaitEmpty, 100)) break;
        for (int k = 0; k < kb; k++, it++) {
          const int s = it % STG;
          if (!mbar_wait_sleep(&hd->full[s], (it / STG) & 1u, abort_flag, p.status, kDevWaitFull, 40)) { ok = false; break; }
          mp_fence_after();
          const uint32_t a_s = smem_u32(stage0 + (size_t)s * (kMpABytes + BBytes)), b_s = a_s + kMpABytes;
#pragma unroll
          for (int ks = 0; ks < kMpBK / 16; ks++)
            mp_mma_f16(tmem + (uint32_t)(buf * BN), mp_desc(a_s + ks * 32), mp_desc(b_s + ks * 32), idesc,
                       (k > 0 || ks > 0) ? 1u : 0u);
          mp_commit(&hd->empty[s]);
        }
        if (ok) mp_commit(&hd->accfull[buf]);
      }
    }
  } else if (warp >= 6 && DENSE) {
    // dense source: nothing to produce
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ weight producers: raw blocks -> half operand tile
    // chunk c = (tile row r, 8-element group j of the 64-wide K block); 8 consecutive threads share a row (one block
    // of the raw matrix), a warp writes four whole 128-byte rows: conflict-free stores at the swizzled positions
    const int pt = tid - 6 * 32;
    const size_t rb = row_bytes(T, p.K);
    constexpr int per_block = block_elems(T) / 8;          // 8-element groups per raw block
    uint32_t it = 0;
    bool ok = true;
    for (int i = 0; ok && i < my_tiles; i++) {
      const MpTile tl = p.tiles[(int)blockIdx.x + i * (int)gridDim.x];
      const uint64_t* wp = p.wptr + (size_t)tl.slot * 3;
      const uint8_t* w0 = reinterpret_cast<const uint8_t*>(MODE == 0 ? wp[0] : wp[2]);   // gate | down
      const uint8_t* w1 = reinterpret_cast<const uint8_t*>(wp[1]);                        // up (mode 0)
      // unit path (IQ1_S / IQ2_XXS): thread (ur, un) decodes unit un of tile row ur in every 64-wide K block.  The raw
      // bytes are FETCHED in another arrangement, one 256-element block (four K blocks) at a time: lane (row 4 q + lane / 8
      // of the warp's 16, unit lane % 8), q = 0..3, so that one load instruction of the warp touches 4 rows' blocks
      // instead of 16 (a quarter of the L1 wavefronts, which together with the table look-ups and the tile stores
      // bound the producers).  The fetched {a, b, d} go through a per-warp staging array in shared memory, written
      // when the block's turn comes and read back by the decoding thread; the next block's loads are in flight
      // meanwhile (the rows' bytes come from HBM, every expert weight being read once).
      const int ur = pt >> 1, un = pt & 1, pw = pt >> 5;
      const bool ulive = tl.n0 + (MODE == 0 ? (ur & 63) : ur) < p.n_out;
      const int kg = kb / 4;                                 // K is a multiple of 256
      const uint8_t* frow[4];                                // the four rows this lane fetches for (null: past n_out)
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int trow = 16 * pw + 4 * q + (lane >> 3);      // mode 0: tile rows 0..63 = gate rows n0.., 64..127 = up
        const int wrow = tl.n0 + (MODE == 0 ? (trow & 63) : trow);
        const uint8_t* base = (MODE == 0 && trow >= 64) ? w1 : w0;
        frow[q] = wrow < p.n_out ? base + (size_t)wrow * rb : nullptr;
      }
      auto fetch_g = [&](int g, MpRaw (&r)[4]) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
          r[q] = MpRaw{0u, 0u, 0.f};
          if constexpr (T == IQ1_S || T == IQ2_XXS) {
            if (frow[q] && g < kg) r[q] = mp_fetch_unit<T>(frow[q] + (size_t)g * block_bytes(T), lane & 7);
          }
        }
      };
      // The rows' raw blocks are asked into L2 now, all of them (rb bytes per row, the eight lanes of a row taking
      // alternate 128-byte lines): the loads above then pay an L2 hit instead of an HBM miss.
      if constexpr (T == IQ1_S || T == IQ2_XXS) {
#pragma unroll
        for (int q = 0; q < 4; q++)
          if (frow[q])
            for (size_t off = (size_t)(lane & 7) * 128; off < rb; off += 1024) asm volatile("prefetch.global.L2 [%0];" ::"l"(frow[q] + off));
      }
      const saddr_t stg = smem_u32(lut + kMpLutBytes) + (uint32_t)(pw * kMpStgWarp);
      const saddr_t stg_w = stg + (uint32_t)((lane >> 3) * kMpStgRow + (lane & 7) * 16);      // + 4 q rows
      const saddr_t stg_r = stg + (uint32_t)((lane >> 1) * kMpStgRow + un * 16);               // + 2 kk units
      MpRaw ring[4];
      fetch_g(0, ring);
      for (int k0 = 0; ok && k0 < kb; k0 += 4) {
      if constexpr (T == IQ1_S || T == IQ2_XXS) {
        static_assert(kMpBN * 2 == kMpProducerWarps * 32, "one unit per producer thread");
        __syncwarp();                                        // the previous block's reads are done
#pragma unroll
        for (int q = 0; q < 4; q++)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg_w + (uint32_t)(4 * q * kMpStgRow)), "r"(ring[q].a),
                       "r"(ring[q].b), "r"(__float_as_uint(ring[q].d)), "r"(0u)
                       : "memory");
        __syncwarp();
        fetch_g(k0 / 4 + 1, ring);
        // kMpBatch K blocks per hand-over: their units are decoded into registers first (nothing there depends on a free
        // slot), then the slots are awaited, the tiles stored and ONE proxy fence + warp barrier covers them all
#pragma unroll
        for (int kk = 0; kk < 4; kk += kMpBatch) {
          if (!ok) break;
          uint4 o4[kMpBatch][4];
#pragma unroll
          for (int b = 0; b < kMpBatch; b++) {
            const uint4 v = lds_u128(stg_r + (uint32_t)(32 * (kk + b)));
            MpRaw cur;
            cur.a = v.x; cur.b = v.y; cur.d = __uint_as_float(v.z);
#pragma unroll
            for (int l = 0; l < 4; l++) o4[b][l] = make_uint4(0, 0, 0, 0);
            if (ulive) mp_decode_unit<T>(cur, lut, lane, o4[b]);
          }
#pragma unroll
          for (int b = 0; b < kMpBatch; b++) {
            const uint32_t itb = it + b;
            if (ok && !__all_sync(0xffffffffu, mbar_wait(&hd->empty[itb % STG], ((itb / STG) & 1u) ^ 1u, abort_flag,
                                                         p.status, kDevWaitEmpty)))
              ok = false;
          }
          if (!ok) break;
#pragma unroll
          for (int b = 0; b < kMpBatch; b++) {
            uint8_t* bt = stage0 + (size_t)((it + b) % STG) * (kMpABytes + BBytes) + kMpABytes;
#pragma unroll
            for (int l = 0; l < 4; l++) *reinterpret_cast<uint4*>(bt + ur * 128 + (((4 * un + l) ^ (ur & 7)) << 4)) = o4[b][l];
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
#pragma unroll
            for (int b = 0; b < kMpBatch; b++) mbar_arrive(&hd->full[(it + b) % STG]);
          }
          it += kMpBatch;
        }
      } else
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
        if (!ok) break;
        const int k = k0 + kk;
        const int s = it % STG;
        if (!__all_sync(0xffffffffu, mbar_wait(&hd->empty[s], ((it / STG) & 1u) ^ 1u, abort_flag, p.status, kDevWaitEmpty))) {
          ok = false;
          break;
        }
        uint8_t* bt = stage0 + (size_t)s * (kMpABytes + BBytes) + kMpABytes;
#pragma unroll
        for (int q = 0; q < kMpBN * 8 / (kMpProducerWarps * 32); q++) {
          const int c = pt + q * kMpProducerWarps * 32, r = c >> 3, j = c & 7;
          // mode 0: tile rows 0..63 = gate rows n0.., 64..127 = the same up rows; mode 1: down rows n0..n0+127
          const uint8_t* base = (MODE == 0 && r >= 64) ? w1 : w0;
          const int wrow = tl.n0 + (MODE == 0 ? (r & 63) : r);
          uint4 out = make_uint4(0, 0, 0, 0);
          if (wrow < p.n_out) {
            const int e8 = k * (kMpBK / 8) + j;            // 8-element group index inside the weight row
            float y[8];
            if constexpr (is_dense(T)) {
#pragma unroll
              for (int e = 0; e < 8; e++) y[e] = 0.f;      // dense expert weights are not a reference combination
            } else {
              dequant8<T>(base + (size_t)wrow * rb + (size_t)(e8 / per_block) * block_bytes(T), e8 % per_block, p.tb, y);
            }
            __half2 hh[4];
#pragma unroll
            for (int e = 0; e < 4; e++) hh[e] = __floats2half2_rn(y[2 * e], y[2 * e + 1]);
            out = *reinterpret_cast<uint4*>(hh);
          }
          *reinterpret_cast<uint4*>(bt + r * 128 + ((j ^ (r & 7)) << 4)) = out;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&hd->full[s]);
        it++;
      }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: TMEM lane = entry row
    for (int i = 0; i < my_tiles; i++) {
      const int buf = i & 1;
      const MpTile tl = p.tiles[(int)blockIdx.x + i * (int)gridDim.x];
      if (!__all_sync(0xffffffffu, mbar_wait_sleep(&hd->accfull[buf], (i >> 1) & 1u, abort_flag, p.status, kDevWaitFull, 400))) break;
      mp_fence_after();
      const int lrow = 32 * warp + lane;
      const bool live = lrow < tl.rows;
      const size_t grow = (size_t)tl.row0 + lrow;
      const uint32_t taddr = tmem + ((uint32_t)(32 * warp) << 16) + (uint32_t)(buf * BN);
      if (MODE == 0) {
        const float wt = live ? p.wt[grow] : 0.f;
#pragma unroll 1
        for (int c0 = 0; c0 < BN / 2; c0 += 32) {      // gate columns [0, BN / 2), the same rows' up columns behind them
          uint32_t g[32], u[32];
          mp_ld32(taddr + c0, g);
          mp_ld32(taddr + BN / 2 + c0, u);
          mp_wait_ld();
          if (live) {
            __half2 hh[16];
#pragma unroll
            for (int q = 0; q < 16; q++) {
              float hv[2];
#pragma unroll
              for (int e = 0; e < 2; e++) {
                const float gg = fminf(__uint_as_float(g[2 * q + e]), p.limit);
                const float uu = fminf(fmaxf(__uint_as_float(u[2 * q + e]), -p.limit), p.limit);
                hv[e] = gg / (1.f + expf(-gg)) * uu * wt;
              }
              hh[q] = __floats2half2_rn(hv[0], hv[1]);
            }
            const int col0 = tl.n0 + c0;
            __half* dst = p.h + grow * p.n_out + col0;
            if (col0 + 32 <= p.n_out) {
#pragma unroll
              for (int q = 0; q < 4; q++) reinterpret_cast<uint4*>(dst)[q] = reinterpret_cast<uint4*>(hh)[q];
            } else {
              for (int q = 0; q < 32; q++)
                if (col0 + q < p.n_out) dst[q] = reinterpret_cast<__half*>(hh)[q];
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          mp_ld32(taddr + c0, r);
          mp_wait_ld();
          const int col0 = tl.n0 + c0;
          if (live && col0 < p.n_out) {
            float* dst = p.z + grow * p.n_out + col0;
            if (col0 + 32 <= p.n_out) {
#pragma unroll
              for (int q = 0; q < 8; q++)
                reinterpret_cast<float4*>(dst)[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                                __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
            } else {
              for (int q = 0; q < 32; q++)
                if (col0 + q < p.n_out) dst[q] = __uint_as_float(r[q]);
            }
          }
        }
      }
      mp_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->accempty[buf]);
    }
  }
  mp_fence_before();
  __syncthreads();
  if (warp == 4) {
    mp_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kCols) : "memory");
  }
}

// Xg[row] = half(X[src token]); rows [0, total) follow tok[], rows [total, total + n_tokens) are the tokens in order
// (the shared expert's entries); their routing weight 1 is written to wt_all.
__global__ void __launch_bounds__(256) moep_gather_kernel(const float* __restrict__ X, const int* __restrict__ tok,
                                                          const float* __restrict__ wt, __half* __restrict__ xg,
                                                          float* __restrict__ wt_all, int total, int n_tokens, int dim) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int t = row < total ? tok[row] : row - total;
  if (threadIdx.x == 0) wt_all[row] = row < total ? wt[row] : 1.0f;
  const float4* src = reinterpret_cast<const float4*>(X + (size_t)t * dim);
  uint2* dst = reinterpret_cast<uint2*>(xg + (size_t)row * dim);
  for (int i = threadIdx.x; i < dim / 4; i += 256) {
    const float4 v = src[i];
    __half2 h[2] = {__floats2half2_rn(v.x, v.y), __floats2half2_rn(v.z, v.w)};
    dst[i] = *reinterpret_cast<uint2*>(h);
  }
}

// Y[t] += Z[total + t] (shared, if any) + sum over k of Z[slot_of[t * kpt + k]] (slots < 0 skipped), in that order
__global__ void __launch_bounds__(256) moep_combine_kernel(const float* __restrict__ z, const int* __restrict__ slot_of,
                                                           float* __restrict__ Y, int total, int n_tokens, int kpt, int dim,
                                                           int has_shared) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < dim / 4; i += 256) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (has_shared) acc = reinterpret_cast<const float4*>(z + (size_t)(total + t) * dim)[i];
    for (int k = 0; k < kpt; k++) {
      const int e = slot_of[(size_t)t * kpt + k];
      if (e < 0) continue;
      const float4 v = reinterpret_cast<const float4*>(z + (size_t)e * dim)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float4 y = reinterpret_cast<float4*>(Y + (size_t)t * dim)[i];
    y.x += acc.x; y.y += acc.y; y.z += acc.z; y.w += acc.w;
    reinterpret_cast<float4*>(Y + (size_t)t * dim)[i] = y;
  }
}

// ---------------------------------------------------------------- host side
namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn mp_encode_fn() {
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
int mp_make_map(CUtensorMap* map, const void* base, int64_t rows, int cols, int box_rows = kMpBM) {
  EncodeTiledFn encode = mp_encode_fn();
  if (!encode) return fail(kErrCuda, "moe_prefill: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kMpBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult cr = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(kErrCuda, "moe_prefill: tensor map encode failed (%d)", (int)cr);
  return kOk;
}

template <int T, int MODE, bool DENSE>
int mp_launch(MpGemmParams& p, int sms, int dev, cudaStream_t st) {
  if (p.ntiles <= 0) return kOk;
  static_assert((size_t)kMpStagesDense * (kMpABytes + kMpBNDense * kMpBK * 2) <= (size_t)kMpStages * (kMpABytes + kMpBBytes) + kMpLutBytes + kMpStgBytes,
                "the TMA-fed variant's ring fits in the same allocation");
  const size_t smem = 1024 + 1024 + (size_t)kMpStages * (kMpABytes + kMpBBytes) + kMpLutBytes + kMpStgBytes;
  auto kern = moep_gemm_kernel<T, MODE, DENSE>;
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    MSB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev & 63] = true;
  }
  MSB_CUDA(launch_pdl(kern, dim3(std::max(1, std::min(sms, p.ntiles))), dim3(kMpThreads), smem, st, p));
  MSB_LAUNCH_CHECK("moep_gemm_kernel");
  return kOk;
}
template <int MODE>
int mp_launch_type(int t, MpGemmParams& p, int sms, int dev, cudaStream_t st) {
  switch (t) {
    case IQ1_S: return mp_launch<IQ1_S, MODE, false>(p, sms, dev, st);
    case IQ2_XXS: return mp_launch<IQ2_XXS, MODE, false>(p, sms, dev, st);
    case Q6_K: return mp_launch<Q6_K, MODE, false>(p, sms, dev, st);
    case Q8_0: return mp_launch<Q8_0, MODE, false>(p, sms, dev, st);
  }
  return fail(kErrType, "moe_prefill: unsupported expert weight type %s", type_name(t));
}
size_t al256(size_t b) { return (b + 255) & ~(size_t)255; }
// Experts with at least kMpDenseMin entries (at most kMpDenseMax routed ones, the largest first, plus the shared expert)
// are dequantised to half once and read by TMA; the others are dequantised tile by tile inside the kernel.
constexpr int kMpDenseMin = 256, kMpDenseMax = 24;
// upper bounds of the tile counts
size_t mp_row_tiles(int total, int n_exp, int n_tokens) {
  return (size_t)(total + kMpBM - 1) / kMpBM + (size_t)n_exp + (size_t)(n_tokens + kMpBM - 1) / kMpBM + 1;
}
}  // namespace

struct MoePrefillArgs {
  int dim, inter, t_gate_up, t_down, t_shared, n_tokens, n_exp;
  const uint64_t* slot_ptrs;   // host [n_exp][3] device addresses {gate, up, down}
  const int* offs;             // host [n_exp + 1]
  const int* tok;              // device [total]
  const float* wt;             // device [total]
  const int* slot_of;          // device [n_tokens * k_per_token]
  int k_per_token, has_shared;
  uint64_t shared_ptrs[3];
  const float* X;
  float* Y;
  void* scratch;
  size_t scratch_bytes;
  float limit;
};

size_t moe_prefill_scratch_bytes(int total, int n_tokens, int n_exp, int dim, int inter) {
  const size_t rows = (size_t)total + n_tokens;
  const size_t rt = mp_row_tiles(total, n_exp, n_tokens);
  size_t b = 256;
  b += al256(rt * ((inter + 63) / 64) * sizeof(MpTile)) + al256(rt * ((dim + 127) / 128) * sizeof(MpTile));
  b += al256((size_t)(n_exp + 1) * 3 * sizeof(uint64_t)) + al256(rows * sizeof(float));
  b += al256(rows * dim * 2) + al256(rows * inter * 2) + al256(rows * dim * 4);
  b += al256((size_t)(kMpDenseMax + 1) * 3 * sizeof(uint64_t));   // addresses of the dense experts' matrices
  b += 2 * al256((size_t)(kMpDenseMax + 1) * 2 * inter * dim * 2) ;   // half copies of the dense experts: gate|up, down (+ slack)
  return b;
}

int weights_to_f16(int t, const void* W, int64_t count, __half* out, int part, cudaStream_t st);   // prefill_gemm.cu
int weights_to_f16_group(int t, const uint64_t* d_srcs, int n_mat, int64_t count, __half* out, cudaStream_t st);

int moe_prefill(const MoePrefillArgs& a, cudaStream_t st) {
  if (a.dim <= 0 || a.inter <= 0 || a.dim % 256 || a.inter % 256) return fail(kErrArg, "moe_prefill: dim/inter must be multiples of 256");
  if (a.n_tokens < 0 || a.n_exp < 0 || a.k_per_token <= 0) return fail(kErrArg, "moe_prefill: bad counts");
  if (a.n_tokens == 0) return kOk;
  if (a.n_exp > 0 && (!a.slot_ptrs || !a.offs || !a.tok || !a.wt)) return fail(kErrArg, "moe_prefill: null routing arrays");
  if (!a.slot_of || !a.X || !a.Y || !a.scratch) return fail(kErrArg, "moe_prefill: null pointer");
  const int total = a.n_exp > 0 ? a.offs[a.n_exp] : 0;
  if (a.n_exp > 0 && a.offs[0] != 0) return fail(kErrArg, "moe_prefill: offs[0] must be 0");
  for (int j = 0; j < a.n_exp; j++)
    if (a.offs[j + 1] < a.offs[j]) return fail(kErrArg, "moe_prefill: offs must not decrease");
  if (a.scratch_bytes < moe_prefill_scratch_bytes(total, a.n_tokens, a.n_exp, a.dim, a.inter))
    return fail(kErrScratch, "moe_prefill: scratch too small");
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int n_sh = a.has_shared ? a.n_tokens : 0;
  const size_t rows = (size_t)total + n_sh;
  // dense experts: the largest routed experts with many entries, and the shared expert when there are many tokens
  std::vector<int> dense_of(a.n_exp + 1, -1);
  std::vector<int> dense_slots;
  {
    std::vector<std::pair<int, int>> bym;
    for (int j = 0; j < a.n_exp; j++)
      if (a.offs[j + 1] - a.offs[j] >= kMpDenseMin) bym.push_back({a.offs[j + 1] - a.offs[j], j});
    std::sort(bym.begin(), bym.end(), [](const std::pair<int, int>& x, const std::pair<int, int>& y) {
      return x.first != y.first ? x.first > y.first : x.second < y.second;
    });
    for (size_t q = 0; q < bym.size() && (int)dense_slots.size() < kMpDenseMax; q++) {
      dense_of[bym[q].second] = (int)dense_slots.size();
      dense_slots.push_back(bym[q].second);
    }
    if (n_sh >= kMpDenseMin) { dense_of[a.n_exp] = (int)dense_slots.size(); dense_slots.push_back(a.n_exp); }
  }
  // tile tables: per expert, weight-row tiles outer, entry tiles inner (CTAs that run together share a weight tile);
  // t?r: routed experts decoded in the kernel, t?s: shared expert decoded in the kernel, t?d: dense (slot = dense index)
  std::vector<MpTile> t1r, t1s, t1d, t2r, t2s, t2d;
  auto add_tiles = [&](std::vector<MpTile>& v, int slot, int row0, int m, int n_out, int step) {
    for (int n0 = 0; n0 < n_out; n0 += step)
      for (int m0 = 0; m0 < m; m0 += kMpBM) v.push_back(MpTile{slot, row0 + m0, std::min(kMpBM, m - m0), n0});
  };
  for (int j = 0; j < a.n_exp; j++) {
    const int m = a.offs[j + 1] - a.offs[j];
    if (m <= 0) continue;
    if (dense_of[j] >= 0) {
      add_tiles(t1d, dense_of[j], a.offs[j], m, a.inter, kMpBNDense / 2);
      add_tiles(t2d, dense_of[j], a.offs[j], m, a.dim, kMpBNDense);
    } else {
      add_tiles(t1r, j, a.offs[j], m, a.inter, 64);
      add_tiles(t2r, j, a.offs[j], m, a.dim, kMpBN);
    }
  }
  if (n_sh) {
    if (dense_of[a.n_exp] >= 0) {
      add_tiles(t1d, dense_of[a.n_exp], total, n_sh, a.inter, kMpBNDense / 2);
      add_tiles(t2d, dense_of[a.n_exp], total, n_sh, a.dim, kMpBNDense);
    } else {
      add_tiles(t1s, a.n_exp, total, n_sh, a.inter, 64);
      add_tiles(t2s, a.n_exp, total, n_sh, a.dim, kMpBN);
    }
  }
  std::vector<uint64_t> wptr((size_t)(a.n_exp + 1) * 3, 0);
  for (int j = 0; j < a.n_exp; j++)
    for (int q = 0; q < 3; q++) {
      wptr[(size_t)j * 3 + q] = a.slot_ptrs[(size_t)j * 3 + q];
      if (!wptr[(size_t)j * 3 + q] && a.offs[j + 1] > a.offs[j]) return fail(kErrArg, "moe_prefill: null matrix of expert slot %d", j);
    }
  for (int q = 0; q < 3; q++) wptr[(size_t)a.n_exp * 3 + q] = a.shared_ptrs[q];
  if (n_sh && (!a.shared_ptrs[0] || !a.shared_ptrs[1] || !a.shared_ptrs[2])) return fail(kErrArg, "moe_prefill: null shared expert matrix");
  // scratch carve-up
  uint8_t* cur = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(a.scratch) + 255) & ~(uintptr_t)255);
  const size_t rt = mp_row_tiles(total, a.n_exp, a.n_tokens);
  MpTile* d_t1 = reinterpret_cast<MpTile*>(cur); cur += al256(rt * ((a.inter + 63) / 64) * sizeof(MpTile));
  MpTile* d_t2 = reinterpret_cast<MpTile*>(cur); cur += al256(rt * ((a.dim + 127) / 128) * sizeof(MpTile));
  uint64_t* d_wptr = reinterpret_cast<uint64_t*>(cur); cur += al256((size_t)(a.n_exp + 1) * 3 * sizeof(uint64_t));
  float* d_wt = reinterpret_cast<float*>(cur); cur += al256(rows * sizeof(float));
  __half* d_xg = reinterpret_cast<__half*>(cur); cur += al256(rows * a.dim * 2);
  __half* d_h = reinterpret_cast<__half*>(cur); cur += al256(rows * a.inter * 2);
  float* d_z = reinterpret_cast<float*>(cur); cur += al256(rows * a.dim * 4);
  uint64_t* d_dsrc = reinterpret_cast<uint64_t*>(cur); cur += al256((size_t)(kMpDenseMax + 1) * 3 * sizeof(uint64_t));
  __half* d_wgu = reinterpret_cast<__half*>(cur); cur += al256((size_t)(kMpDenseMax + 1) * 2 * a.inter * a.dim * 2);
  __half* d_wd = reinterpret_cast<__half*>(cur);
  // the tables go to the device (pageable source: the runtime stages them before returning)
  auto upload = [&](void* dst, const void* src, size_t bytes) -> cudaError_t {
    return bytes ? cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, st) : cudaSuccess;
  };
  MSB_CUDA(upload(d_t1, t1r.data(), t1r.size() * sizeof(MpTile)));
  MSB_CUDA(upload(d_t1 + t1r.size(), t1s.data(), t1s.size() * sizeof(MpTile)));
  MSB_CUDA(upload(d_t1 + t1r.size() + t1s.size(), t1d.data(), t1d.size() * sizeof(MpTile)));
  MSB_CUDA(upload(d_t2, t2r.data(), t2r.size() * sizeof(MpTile)));
  MSB_CUDA(upload(d_t2 + t2r.size(), t2s.data(), t2s.size() * sizeof(MpTile)));
  MSB_CUDA(upload(d_t2 + t2r.size() + t2s.size(), t2d.data(), t2d.size() * sizeof(MpTile)));
  MSB_CUDA(upload(d_wptr, wptr.data(), wptr.size() * sizeof(uint64_t)));
  if (rows == 0) return kOk;
  MSB_CUDA(launch_pdl(moep_gather_kernel, dim3((unsigned)rows), dim3(256), 0, st, a.X, a.tok, a.wt, d_xg, d_wt, total, n_sh,
                      a.dim));
  // half copies of the dense experts (gate rows then up rows per expert; down rows per expert).  The routed ones come
  // first in dense_slots and share their types: one grouped launch for all their gate / up matrices, one for the down
  // matrices; the shared expert, when it is dense, has its own type and three launches.
  {
    const size_t gu = (size_t)a.inter * a.dim;
    const size_t nd_r = dense_slots.size() - ((!dense_slots.empty() && dense_slots.back() == a.n_exp) ? 1 : 0);
    if (nd_r > 0 && !is_dense(a.t_gate_up) && !is_dense(a.t_down)) {
      std::vector<uint64_t> dsrc(3 * nd_r);
      for (size_t q = 0; q < nd_r; q++) {
        dsrc[2 * q] = wptr[(size_t)dense_slots[q] * 3];
        dsrc[2 * q + 1] = wptr[(size_t)dense_slots[q] * 3 + 1];
        dsrc[2 * nd_r + q] = wptr[(size_t)dense_slots[q] * 3 + 2];
      }
      MSB_CUDA(upload(d_dsrc, dsrc.data(), dsrc.size() * sizeof(uint64_t)));
      rc = weights_to_f16_group(a.t_gate_up, d_dsrc, (int)(2 * nd_r), (int64_t)gu, d_wgu, st);
      if (rc) return rc;
      rc = weights_to_f16_group(a.t_down, d_dsrc + 2 * nd_r, (int)nd_r, (int64_t)gu, d_wd, st);
      if (rc) return rc;
    }
    for (size_t q = 0; q < dense_slots.size(); q++) {
      const int j = dense_slots[q];
      if (j != a.n_exp && !is_dense(a.t_gate_up) && !is_dense(a.t_down)) continue;    // done above
      const int t_gu = j == a.n_exp ? a.t_shared : a.t_gate_up, t_d = j == a.n_exp ? a.t_shared : a.t_down;
      rc = weights_to_f16(t_gu, reinterpret_cast<const void*>(wptr[(size_t)j * 3]), (int64_t)gu, d_wgu + (2 * q) * gu, 0, st);
      if (rc) return rc;
      rc = weights_to_f16(t_gu, reinterpret_cast<const void*>(wptr[(size_t)j * 3 + 1]), (int64_t)gu, d_wgu + (2 * q + 1) * gu, 0, st);
      if (rc) return rc;
      rc = weights_to_f16(t_d, reinterpret_cast<const void*>(wptr[(size_t)j * 3 + 2]), (int64_t)gu, d_wd + q * gu, 0, st);
      if (rc) return rc;
    }
  }
  MpGemmParams p;
  p.wptr = d_wptr; p.wt = d_wt; p.h = d_h; p.z = d_z; p.status = tb.status; p.limit = a.limit > 0.f ? a.limit : 10.f; p.tb = tb;
  // gate/up + SwiGLU
  rc = mp_make_map(&p.a_map, d_xg, (int64_t)rows, a.dim);
  if (rc) return rc;
  p.K = a.dim; p.n_out = a.inter;
  p.tiles = d_t1; p.ntiles = (int)t1r.size();
  rc = mp_launch_type<0>(a.t_gate_up, p, sms, dev, st);
  if (rc) return rc;
  p.tiles = d_t1 + t1r.size(); p.ntiles = (int)t1s.size();
  rc = mp_launch_type<0>(a.t_shared, p, sms, dev, st);
  if (rc) return rc;
  if (!t1d.empty()) {
    rc = mp_make_map(&p.b_map, d_wgu, (int64_t)dense_slots.size() * 2 * a.inter, a.dim, kMpBNDense / 2);
    if (rc) return rc;
    p.tiles = d_t1 + t1r.size() + t1s.size(); p.ntiles = (int)t1d.size();
    rc = mp_launch<F16, 0, true>(p, sms, dev, st);
    if (rc) return rc;
  }
  // down
  rc = mp_make_map(&p.a_map, d_h, (int64_t)rows, a.inter);
  if (rc) return rc;
  p.K = a.inter; p.n_out = a.dim;
  p.tiles = d_t2; p.ntiles = (int)t2r.size();
  rc = mp_launch_type<1>(a.t_down, p, sms, dev, st);
  if (rc) return rc;
  p.tiles = d_t2 + t2r.size(); p.ntiles = (int)t2s.size();
  rc = mp_launch_type<1>(a.t_shared, p, sms, dev, st);
  if (rc) return rc;
  if (!t2d.empty()) {
    rc = mp_make_map(&p.b_map, d_wd, (int64_t)dense_slots.size() * a.dim, a.inter, kMpBNDense);
    if (rc) return rc;
    p.tiles = d_t2 + t2r.size() + t2s.size(); p.ntiles = (int)t2d.size();
    rc = mp_launch<F16, 1, true>(p, sms, dev, st);
    if (rc) return rc;
  }
  MSB_CUDA(launch_pdl(moep_combine_kernel, dim3((unsigned)a.n_tokens), dim3(256), 0, st, (const float*)d_z, a.slot_of, a.Y, total,
                      a.n_tokens, a.k_per_token, a.dim, a.has_shared ? 1 : 0));
  MSB_LAUNCH_CHECK("moe_prefill");
  return kOk;
}

}  // namespace msb
