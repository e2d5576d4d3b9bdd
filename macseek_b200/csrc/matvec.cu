// Decode matvec family: y[n][rows] (+)= X[n][cols (* groups)] . W^T with W as raw GGUF block rows.
// Replaces the reference's q_mv / q_mv_rn / q_mvn Metal kernels (src/kernels/quant_mv.metal:7-39,68-129,148-202)
// behind ms::q::encode_matvec / encode_matvec_rmsnorm / encode_matvec_n (src/kernels/quant.hpp:19-35,
// quant.mm:70-156).
//
// Layout of the work: persistent blocks (16 consumer warps + 1 TMA producer warp); block b of group g walks row tiles
// b, b + blocks_per_group, ... of that group.  A tile is R consecutive rows brought in as ONE contiguous bulk copy
// (rows too long for a ring slot are streamed in K chunks, one large copy per row).  Short rows: each warp owns
// G * NR whole rows (LPR lanes per row).  Long rows: KS warps share a row, each taking a contiguous run of units; their
// partial sums meet in shared memory and are added in warp order.  A row's result never depends on which block
// computed the other rows.
#include <algorithm>
#include <cstdlib>
#include "stream_pipe.cuh"

namespace msb {

constexpr int kMvNW = 16;
constexpr size_t kLightSmemLimit = 110 * 1024;   // a light block's shared memory: two fit one SM
constexpr size_t kShareSmemLimit = 96 * 1024;    // a sharing launch: ONE light block per SM, the rest of the SM left free
thread_local bool g_share_launch = false;        // set around a launch by matvec_n(..., share = true)

struct MvParams {
  const uint8_t* W;
  const float* x;
  float* y;
  const float* norm_w;          // fused input RMSNorm: x * rsqrt(mean(x^2) + eps) * norm_w (null = plain matvec)
  float norm_eps;
  int rows, cols, n;            // n activation columns
  int rows_per_group, groups;
  int64_t x_stride, y_stride;   // elements between activation columns / output columns
  uint32_t row_bytes;
  int accumulate;
  int units;                    // cols / 32
  int ks;                       // warps sharing one row (1 = each warp owns whole rows)
  int tile_rows;                // R
  int chunk_units;              // units per staged piece (== units: whole rows, the tile is one contiguous copy)
  int blocks_per_group;
  int tiles_per_group;
  int stages;
  uint32_t pitch;               // shared-memory distance between staged rows
  uint32_t stage_bytes;
  Tables tb;
};

struct MvSmemHead {
  uint64_t full[kMaxStages], empty[kMaxStages];
  uint64_t lutbar, tilebar;
  int abort_flag;
  float red[32];
  float part[2][kMvNW][4];
};

// NW consumer warps + 1 producer warp.  NW = 16: one block per SM with most of its shared memory (long streams).
// NW = 8: a light block (at most half an SM's shared memory and registers) so that two are resident per SM -- two of
// this launch, or the tail of this launch and the head of the next, whose producer warps then prefetch their first
// tiles while the previous kernel is still running (programmatic dependent launch).
template <int T, int LPR, int NR, int NC, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, NW == 8 ? 2 : 1) matvec_kernel(const MvParams p) {
  constexpr int G = 32 / LPR;
  pdl_launch_dependents();
  extern __shared__ __align__(128) uint8_t smem[];
  // [head][luts][xq columns][ring slots]
  MvSmemHead* hd = reinterpret_cast<MvSmemHead*>(smem);
  Ring ring;
  ring.full = hd->full; ring.empty = hd->empty;
  ring.abort_flag = &hd->abort_flag; ring.status = p.tb.status; ring.stages = p.stages;
  uint8_t* cur = smem + ((sizeof(MvSmemHead) + 127) & ~(size_t)127);
  uint8_t* lut = cur;
  cur += lut_bytes_for(T);
  XqSmem xq[NC];
  const int U = p.units;
#pragma unroll
  for (int c = 0; c < NC; c++) { xq_bind(xq[c], cur, U, is_dense(T), xq_padded(T)); cur += xq_bytes(U, is_dense(T), xq_padded(T)); }
  cur = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(cur) + 127) & ~(uintptr_t)127);
  ring.slot0 = cur; ring.slot_bytes = p.stage_bytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = blockIdx.x / p.blocks_per_group, slot = blockIdx.x % p.blocks_per_group;
  ring_init(ring, tid, NW);
  if (tid == 0) { mbar_init(&hd->lutbar, 1); mbar_init(&hd->tilebar, NW); mbar_fence_init(); }
  __syncthreads();
  const int R = p.tile_rows, KS = p.ks;
  const bool whole = p.chunk_units >= U;             // whole rows per piece: the tile is one contiguous copy
  const int nchunks = whole ? 1 : (U + p.chunk_units - 1) / p.chunk_units;
  const uint8_t* Wg = p.W + (size_t)group * p.rows_per_group * p.row_bytes;
  uint32_t n = 0;
  if (warp == NW) {
    // ---------------- producer warp
    const uint8_t* srcv[1];
    Piece pc;
    pc.src = srcv; pc.nsrc = 1; pc.row_stride = p.row_bytes;
    for (int t = slot; t < p.tiles_per_group; t += p.blocks_per_group) {
      const int r0 = t * R, nrows = min(R, p.rows_per_group - r0);
      for (int c = 0; c < nchunks; c++, n++) {
        if (whole) {
          srcv[0] = Wg + (size_t)r0 * p.row_bytes;
          pc.rows_per_src = 1; pc.nrows = 1; pc.bytes = (uint32_t)nrows * p.row_bytes;
        } else {
          const int u0 = c * p.chunk_units, nu = min(p.chunk_units, U - u0);
          srcv[0] = Wg + (size_t)r0 * p.row_bytes + units_bytes(T, u0);
          pc.rows_per_src = R; pc.nrows = nrows; pc.bytes = units_bytes(T, nu);
        }
        if (!produce_piece(ring, n, pc, p.pitch, lane)) return;
      }
    }
    return;
  }
  // ---------------- consumer warps
  LaneLuts L;
  const bool luts_ok = load_luts(lut, T == IQ1_S, T == IQ2_XXS, T == IQ4_NL, p.tb, tid, &hd->lutbar, &hd->abort_flag, L, lane);
  // Everything up to here, and the producer warp's weight copies, is independent of the previous kernel (weights are
  // constants); x (and y, when accumulating) are not.
  pdl_wait();
  // activation of this block's group -> shared (fixed point, or fp32 for dense weights), optionally RMS-normalised
#pragma unroll
  for (int c = 0; c < NC; c++) {
    const float* xg = p.x + (size_t)c * p.x_stride + (size_t)group * p.cols;
    float mul = 1.f;
    if (p.norm_w) {
      float ss = 0.f;
      for (int i = tid; i < p.cols / 4; i += NW * 32) {
        const float4 v = reinterpret_cast<const float4*>(xg)[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = warp_sum(ss);
      if (lane == 0) hd->red[warp] = ss;
      bar_sync_named(1, NW * 32);
      float tot = 0.f;
      for (int w = 0; w < NW; w++) tot += hd->red[w];
      bar_sync_named(1, NW * 32);
      mul = rsqrtf(tot / (float)p.cols + p.norm_eps);
    }
    if (is_dense(T)) {
      float4* d = reinterpret_cast<float4*>(const_cast<float*>(xq[c].xf));
      for (int i = tid; i < U * 8; i += NW * 32) {
        float4 v = reinterpret_cast<const float4*>(xg)[i];
        if (p.norm_w) {
          const float4 gw = reinterpret_cast<const float4*>(p.norm_w)[i];
          v.x = v.x * mul * gw.x; v.y = v.y * mul * gw.y; v.z = v.z * mul * gw.z; v.w = v.w * mul * gw.w;
        }
        // 16-bit weights: one 16-byte weight granule spans 8 activations, kept as two float4 planes (elements
        // 8g..8g+3 and 8g+4..8g+7 of granule g) so that lanes on consecutive granules read consecutive addresses
        d[T == F32 ? i : (i & 1) * (U * 4) + (i >> 1)] = v;
      }
    } else {
      quantize_x(xg, xq[c], tid, NW * 32, mul, p.norm_w);
    }
  }
  bar_sync_named(1, NW * 32);
  if (!luts_ok) return;

  const int grp = lane / LPR, li = lane % LPR;
  // rows of this lane group inside the tile, and (KS > 1) this warp's share of the row's units
  const int lr0 = KS > 1 ? warp / KS : (warp * G + grp) * NR;
  const int kpart = KS > 1 ? warp % KS : 0;
  const int step = block_elems(T) == 256 ? 8 : 1;
  uint32_t tile_count = 0;
  for (int t = slot; t < p.tiles_per_group; t += p.blocks_per_group) {
    const int r0 = t * R;
    float acc[NR][NC];
#pragma unroll
    for (int i = 0; i < NR; i++)
#pragma unroll
      for (int c = 0; c < NC; c++) acc[i][c] = 0.f;
    for (int c = 0; c < nchunks; c++, n++) {
      const int u0 = whole ? 0 : c * p.chunk_units, nu = whole ? U : min(p.chunk_units, U - u0);
      const uintptr_t a0 = reinterpret_cast<uintptr_t>(Wg) + (size_t)r0 * p.row_bytes + units_bytes(T, u0);
      const saddr_t slot_s = smem_u32(ring.slot(n));
      int ua = 0, ub = nu;                           // this warp's run of units inside the piece
      if (KS > 1) {
        const int per = ((nu + KS * step - 1) / (KS * step)) * step;
        ua = min(nu, kpart * per); ub = min(nu, ua + per);
      }
      saddr_t rowp[NR];
#pragma unroll
      for (int i = 0; i < NR; i++) {
        const uint32_t mis = whole ? (uint32_t)(a0 & 15u) : (uint32_t)((a0 + (uintptr_t)(lr0 + i) * p.row_bytes) & 15u);
        rowp[i] = slot_s + (uint32_t)(lr0 + i) * p.pitch + mis + (uint32_t)units_bytes(T, ua);
      }
      if (!consumer_wait(ring, n)) return;
      if (ub > ua) consume_rows<T, LPR, NR, NC>(rowp, li, xq, u0 + ua, ub - ua, L, acc);
      consumer_release(ring, n, lane);
    }
    if (KS > 1) {
      // NR == 1, LPR == 32: one partial per warp and column; the first warp of the row adds them in warp order
      const int pb = tile_count & 1;
#pragma unroll
      for (int c = 0; c < NC; c++) {
        const float v = group_sum<32>(acc[0][c]);
        if (lane == 0) hd->part[pb][warp][c] = v;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->tilebar);
      if (!mbar_wait(&hd->tilebar, tile_count & 1u, ring.abort_flag, ring.status, kDevWaitFull)) return;
      if (kpart == 0 && lane < NC && r0 + lr0 < p.rows_per_group) {
        float v = 0.f;
        for (int k = 0; k < KS; k++) v += hd->part[pb][warp + k][lane];
        float* yp = p.y + (size_t)lane * p.y_stride + (size_t)group * p.rows_per_group + r0 + lr0;
        *yp = p.accumulate ? *yp + v : v;
      }
      tile_count++;
    } else {
#pragma unroll
      for (int i = 0; i < NR; i++) {
#pragma unroll
        for (int c = 0; c < NC; c++) {
          const float v = group_sum<LPR>(acc[i][c]);
          if (li == 0 && r0 + lr0 + i < p.rows_per_group) {
            float* yp = p.y + (size_t)c * p.y_stride + (size_t)group * p.rows_per_group + r0 + lr0 + i;
            *yp = p.accumulate ? *yp + v : v;
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------- host side
namespace {

// lanes per row: of 32/16/8 the one that wastes the fewest lane iterations on `items` work items per row, among
// those whose smallest whole-row tile (16 warps x 32/lpr rows) fits `tile_cap` bytes; 32 when none does (long rows
// are then shared by several warps or streamed in chunks)
int pick_lpr(int items, size_t row_bytes, size_t tile_cap, int nw) {
  int best = 32;
  double best_eff = 0;
  for (int lpr : {32, 16, 8}) {
    if (lpr < 32 && (size_t)nw * (32 / lpr) * row_bytes + 192 > tile_cap) continue;
    const int iters = (items + lpr - 1) / lpr;
    const double eff = (double)items / (iters * lpr);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = lpr; }
  }
  return best;
}

template <int T, int LPR, int NR, int NC, int NW>
int launch_cfg(MvParams& p, size_t fixed, int stages, size_t slot_bytes, cudaStream_t st, int dev) {
  const size_t smem = fixed + (size_t)stages * slot_bytes;
  auto kern = matvec_kernel<T, LPR, NR, NC, NW>;
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    MSB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    configured[dev & 63] = true;
  }
  p.stages = stages;
  p.stage_bytes = (uint32_t)slot_bytes;
  MSB_CUDA(launch_pdl(kern, dim3(p.blocks_per_group * p.groups), dim3((NW + 1) * 32), smem, st, p));
  MSB_LAUNCH_CHECK("matvec_kernel");
  return kOk;
}

// Tile shape: as many consecutive whole rows as fit one ring slot (one contiguous copy), bounded by what the type's
// decode cost warrants and by the need to spread the matrix over every SM.
template <int T, int LPR, int NC, int NW>
int launch_rows(MvParams& p, cudaStream_t st, int dev, int sms_real) {
  // light blocks: two per SM, each within half of the SM's shared memory
  const bool share = NW == 8 && g_share_launch;
  const int sms = (NW == 8 && !share) ? 2 * sms_real : sms_real;
  const size_t smem_limit = share ? kShareSmemLimit : NW == 8 ? kLightSmemLimit : (size_t)kSmemLimit;
  constexpr int G = 32 / LPR;
  constexpr int kMaxNR = (T == IQ1_S || T == IQ2_XXS) ? 4 : 2;
  const size_t fixed = ((sizeof(MvSmemHead) + 127) & ~(size_t)127) + lut_bytes_for(T) +
                       (size_t)NC * xq_bytes(p.units, is_dense(T), xq_padded(T)) + 128;
  if (fixed + 2 * 8192 > smem_limit)
    return fail(kErrLimit, "matvec: cols %d x n %d does not fit in shared memory", p.cols, p.n);
  const size_t avail = smem_limit - fixed;
  // A tile may take up to half of the free shared memory (a two-slot ring): rows that share a lane's activation
  // registers cut the shared-memory traffic per weight, which matters more than ring depth once a slot holds tens of KB.
  size_t slot = (avail / 2) & ~(size_t)127;
  int stages = 2;
  const long rows_fit = ((long)slot - 64) / (long)p.row_bytes;
  const int want_tiles = std::max(1, sms / p.groups);
  auto tiles_of = [&](int r) { return (p.rows_per_group + r - 1) / r; };
  p.chunk_units = p.units;
  p.pitch = p.row_bytes;
  int nr = 1, ks = 1, R = 0;
  if (rows_fit >= 1) {
    // whole rows per warp (KS = 1, R = 16 * G * NR), largest first
    for (int cand : {4, 2, 1}) {
      if (cand > kMaxNR || (NC > 1 && cand > 2) || (T == Q6_K && NC > 2 && cand > 1)) continue;
      const int r = NW * G * cand;
      if (r <= rows_fit && (tiles_of(r) >= want_tiles || cand == 1)) { R = r; nr = cand; break; }
    }
    // several warps per row when whole-row tiles do not fit or leave SMs idle
    if (LPR == 32 && (R == 0 || tiles_of(R) < want_tiles)) {
      for (int cand : {2, 4, 8, 16}) {
        if (cand > NW) break;
        const int r = NW / cand;
        if (r > rows_fit) continue;
        R = r; ks = cand; nr = 1;
        if (tiles_of(r) >= want_tiles) break;
      }
    }
    if (R == 0) {   // LPR < 32 and the smallest whole-row tile does not fit: per-row chunks instead
      nr = 1; ks = 1;
      R = NW * G;
      stages = 3;
      slot = std::min(slot, (avail / 3) & ~(size_t)127);
      const int chunk = chunk_units_for(T, p.units, R, LPR, slot);
      if (chunk <= 0) return fail(kErrLimit, "matvec: no staging shape fits (type %s cols %d)", type_name(T), p.cols);
      p.chunk_units = chunk;
      p.pitch = piece_pitch(units_bytes(T, chunk));
    }
  } else {
    // one row does not fit a slot: all 16 warps share a row, K streamed in chunks (one large copy each)
    if (LPR != 32) return fail(kErrLimit, "matvec: row of %u bytes does not fit (type %s)", p.row_bytes, type_name(T));
    ks = NW; nr = 1; R = 1;
    stages = 3;
    slot = std::min(slot, (avail / 3) & ~(size_t)127);
    const int chunk = chunk_units_for(T, p.units, 1, 32 * NW, slot);
    if (chunk <= 0) return fail(kErrLimit, "matvec: no staging shape fits (type %s cols %d)", type_name(T), p.cols);
    p.chunk_units = chunk;
    p.pitch = piece_pitch(units_bytes(T, chunk));
  }
  if (p.chunk_units >= p.units) {
    // whole-row tiles: the slot is exactly one tile (plus the source's misalignment), the ring as deep as then fits
    slot = ((size_t)R * p.row_bytes + 64 + 127) & ~(size_t)127;
    stages = (int)std::min<size_t>(kMaxStages, avail / slot);
  }
  p.tile_rows = R;
  p.ks = ks;
  p.tiles_per_group = tiles_of(R);
  p.blocks_per_group = std::max(1, std::min(p.tiles_per_group, sms / p.groups));
  if (nr >= 4) {
    if constexpr (kMaxNR >= 4 && NC == 1) return launch_cfg<T, LPR, 4, NC, NW>(p, fixed, stages, slot, st, dev);
  }
  if (nr >= 2) return launch_cfg<T, LPR, 2, NC, NW>(p, fixed, stages, slot, st, dev);
  return launch_cfg<T, LPR, 1, NC, NW>(p, fixed, stages, slot, st, dev);
}

template <int T, int NC>
int launch_type(MvParams& p, cudaStream_t st, int dev, int sms) {
  // Light blocks for matrices whose per-SM share is small next to the fixed cost of a launch (the layer's projections;
  // not the output head): only for the table-free types and a single activation column.
  bool light = false;
  if constexpr (NC == 1 && lut_bytes_for(T) == 0) {
    const size_t total = (size_t)p.rows_per_group * p.groups * p.row_bytes;
    light = total <= (size_t)96 << 20;
    const size_t fixed_l = (size_t)NC * xq_bytes(p.units, is_dense(T), xq_padded(T)) + 1024;
    if (fixed_l + 2 * 16384 > kLightSmemLimit) light = false;
    const size_t light_limit = (g_share_launch && fixed_l + 2 * 16384 <= kShareSmemLimit) ? kShareSmemLimit : kLightSmemLimit;
    if (light_limit == kLightSmemLimit) g_share_launch = false;    // does not fit the sharing form: an ordinary launch
    else light = true;
    if (light) {
      const size_t cap = (light_limit - fixed_l) / 2;
      // Q6_K and IQ1_S rows are split by half super-block (4 units), the other types by unit
      switch (pick_lpr((T == Q6_K || T == IQ1_S) ? p.units / 4 : p.units, p.row_bytes, cap, 8)) {
        case 32: return launch_rows<T, 32, NC, 8>(p, st, dev, sms);
        case 16: return launch_rows<T, 16, NC, 8>(p, st, dev, sms);
        default: return launch_rows<T, 8, NC, 8>(p, st, dev, sms);
      }
    }
  }
  const size_t fixed = lut_bytes_for(T) + (size_t)NC * xq_bytes(p.units, is_dense(T), xq_padded(T)) + 1024;
  const size_t tile_cap = fixed < (size_t)kSmemLimit ? ((size_t)kSmemLimit - fixed) / 2 : 0;
  switch (pick_lpr((T == Q6_K || T == IQ1_S) ? p.units / 4 : p.units, p.row_bytes, tile_cap, kMvNW)) {
    case 32: return launch_rows<T, 32, NC, kMvNW>(p, st, dev, sms);
    case 16: return launch_rows<T, 16, NC, kMvNW>(p, st, dev, sms);
    default: return launch_rows<T, 8, NC, kMvNW>(p, st, dev, sms);
  }
}

template <int NC>
int launch_cols(int t, MvParams& p, cudaStream_t st, int dev, int sms) {
  switch (t) {
    case F32: return launch_type<F32, NC>(p, st, dev, sms);
    case F16: return launch_type<F16, NC>(p, st, dev, sms);
    case BF16: return launch_type<BF16, NC>(p, st, dev, sms);
    case Q8_0: return launch_type<Q8_0, NC>(p, st, dev, sms);
    case Q5_K: return launch_type<Q5_K, NC>(p, st, dev, sms);
    case Q6_K: return launch_type<Q6_K, NC>(p, st, dev, sms);
    case IQ2_XXS: return launch_type<IQ2_XXS, NC>(p, st, dev, sms);
    case IQ1_S: return launch_type<IQ1_S, NC>(p, st, dev, sms);
    case IQ4_NL: return launch_type<IQ4_NL, NC>(p, st, dev, sms);
  }
  return fail(kErrType, "matvec: unsupported weight type %d", t);
}
}  // namespace

// Y[n x rows] (+)= X[n x cols*groups] . W^T.  n columns are processed four (then two, then one) at a time; each pass
// streams W once.  norm_w != null fuses the input RMSNorm (groups must be 1).
int matvec_n(int t, const void* W, int rows, int cols, const float* X, int64_t x_stride, float* Y, int64_t y_stride,
             int n, int accumulate, int groups, const float* norm_w, float norm_eps, cudaStream_t st, bool share) {
  struct ShareScope { ShareScope(bool s) { g_share_launch = s; } ~ShareScope() { g_share_launch = false; } } scope(share);
  if (!type_known(t)) return fail(kErrType, "matvec: unsupported weight type %d", t);
  const int qk = block_elems(t) == 1 ? 32 : block_elems(t);
  if (rows <= 0 || cols <= 0 || n <= 0 || groups < 1 || rows % groups != 0 || cols % qk != 0 || cols % 32 != 0)
    return fail(kErrArg, "matvec: bad shape (type %s rows %d cols %d n %d groups %d)", type_name(t), rows, cols, n, groups);
  if (!W || !X || !Y) return fail(kErrArg, "matvec: null pointer");
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 1) || ((x_stride * 4) & 15))
    return fail(kErrArg, "matvec: activations must be 16-byte aligned, weights 2-byte aligned");
  if (norm_w && (groups != 1 || (reinterpret_cast<uintptr_t>(norm_w) & 15)))
    return fail(kErrArg, "matvec_rmsnorm: groups must be 1 and norm_w 16-byte aligned");
  MvParams p{};
  int rc = get_tables(&p.tb);
  if (rc) return rc;
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  p.W = (const uint8_t*)W;
  p.norm_w = norm_w; p.norm_eps = norm_eps;
  p.rows = rows; p.cols = cols;
  p.rows_per_group = rows / groups; p.groups = groups;
  p.x_stride = x_stride; p.y_stride = y_stride;
  p.row_bytes = (uint32_t)row_bytes(t, cols);
  p.accumulate = accumulate;
  p.units = cols / 32;
  // activation columns per pass: as many as leave at least half of the shared memory to the weight ring
  int max_nc = 4;
  while (max_nc > 1 && lut_bytes_for(t) + (size_t)max_nc * xq_bytes(p.units, is_dense(t), xq_padded(t)) > (size_t)kSmemLimit / 2) max_nc >>= 1;
  for (int c0 = 0; c0 < n;) {
    const int left = n - c0;
    p.x = X + (size_t)c0 * x_stride;
    p.y = Y + (size_t)c0 * y_stride;
    if (left >= 4 && max_nc >= 4) { p.n = 4; rc = launch_cols<4>(t, p, st, dev, sms); c0 += 4; }
    else if (left >= 2 && max_nc >= 2) { p.n = 2; rc = launch_cols<2>(t, p, st, dev, sms); c0 += 2; }
    else { p.n = 1; rc = launch_cols<1>(t, p, st, dev, sms); c0 += 1; }
    if (rc) return rc;
  }
  return kOk;
}

}  // namespace msb
