// Fused MoE decode for one token: routed experts (IQ1_S / IQ2_XXS) + one shared expert (Q6_K / Q8_0).
//   moe_gu_kernel  : h[e][r] = silu(min(gate_e[r].x, L)) * clamp(up_e[r].x, -L, L) * w_e   (all experts, one launch)
//   moe_down_kernel: y[r] += sum_e down_e[r] . h[e]                                        (all experts, one launch)
// Replaces the reference's q_moe_gu[_t] / q_moe_down[_t] Metal kernels (src/kernels/quant_moe.metal:50-147,175-259)
// behind ms::q::encode_moe_decode / encode_moe_decode_table[_part] (src/kernels/quant.hpp:49-85, quant.mm:264-369).
//
// Work distribution: persistent blocks walk the launch's row tiles with a fixed stride (big shared-expert tiles first);
// the tile list is formed on the device from the experts resident on this GPU (expert parallelism), so the split adapts
// without a host round trip.  A row's partial sums are always formed in the same order, whichever block computes it.
#include <algorithm>
#include <cstdlib>
#include "stream_pipe.cuh"
#include "moe_decode_params.cuh"

namespace msb {

struct MoeSmemHead {
  uint64_t full[kMaxStages], empty[kMaxStages];
  uint64_t lutbar, tilebar;
  int abort_flag;
  int n_local;
  int meta[kMaxStages];
  int local_slot[kMaxRouted];
  const uint8_t* p0[kMaxRouted];   // gate (gu kernel) or down (down kernel) of local routed slot i
  const uint8_t* p1[kMaxRouted];   // up
  const uint8_t* srcs[kMaxStages][kMaxRouted];   // per ring slot: source addresses of the staged piece
  float part[2][kMoeNW][2];        // per-warp partial sums of a tile (double-buffered): down: [0]; gate/up: (g, u)
  float rpart[2][kMoeNW][kMoeNW / 2];   // down: per-warp partial sums of the routed experts for the tile's rows
};

__device__ __forceinline__ float swiglu(float g, float u, float w, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-g)) * u * w;
}

// Resolve which routed slots are handled by this GPU and their matrix addresses.  Called by ONE WHOLE WARP: lane k looks
// slot k up (its id, then its table row: two dependent reads, all slots at once rather than one after the other) and
// the resident ones are compacted in slot order.
__device__ __forceinline__ void resolve_local(const MoeParams& p, MoeSmemHead* hd, bool want_routed, bool down, int lane) {
  static_assert(kMaxRouted <= 32, "one lane per routed slot");
  bool mine = want_routed && lane < p.n_routed;
  const uint8_t* a0 = nullptr;
  const uint8_t* a1 = nullptr;
  if (mine) {
    if (p.table) {
      const int id = p.ids ? p.ids[lane] : lane;       // no ids: the table holds one entry per routed slot
      if (p.ids && (id < p.expert_lo || id >= p.expert_hi)) mine = false;
      if (mine) {
        const uint64_t* row = p.table + (size_t)id * 3;
        a0 = reinterpret_cast<const uint8_t*>(down ? row[2] : row[0]);
        a1 = reinterpret_cast<const uint8_t*>(row[1]);
      }
    } else {
      a0 = down ? p.down[lane] : p.gate[lane];
      a1 = p.up[lane];
    }
  }
  const unsigned m = __ballot_sync(0xffffffffu, mine);
  if (mine) {
    const int pos = __popc(m & ((1u << lane) - 1u));
    hd->p0[pos] = a0; hd->p1[pos] = a1; hd->local_slot[pos] = lane;
  }
  if (lane == 0) hd->n_local = __popc(m);
  __syncwarp();
}

// Producer side of "first piece of a tile": wait for the slot, publish the tile id, then the piece.
__device__ __forceinline__ bool announce_tile(const Ring& ring, uint32_t n, MoeSmemHead* hd, int tile, int lane) {
  const int s = n % ring.stages;
  if (!mbar_wait(&ring.empty[s], ((n / ring.stages) & 1u) ^ 1u, ring.abort_flag, ring.status, kDevWaitEmpty)) return false;
  if (lane == 0) *reinterpret_cast<volatile int*>(&hd->meta[s]) = tile;
  __syncwarp();
  return true;
}
__device__ __forceinline__ void end_of_tiles(const Ring& ring, uint32_t n, MoeSmemHead* hd, int lane) {
  const int s = n % ring.stages;
  if (!mbar_wait(&ring.empty[s], ((n / ring.stages) & 1u) ^ 1u, ring.abort_flag, ring.status, kDevWaitEmpty)) return;
  if (lane == 0) {
    *reinterpret_cast<volatile int*>(&hd->meta[s]) = -1;
    mbar_arrive(&ring.full[s]);
  }
}

// ---------------------------------------------------------------------------------------------------- gate/up
// A tile is R rows of one expert's gate matrix and the same R rows of its up matrix, staged side by side in one ring
// slot (two contiguous copies, one barrier): a lane decodes the gate and the up rows it owns against activation
// registers loaded once.  Routed experts (cheap bytes, expensive decode): each warp owns NR whole row pairs.  Shared
// expert (long rows): KS warps share a row pair, each a contiguous run of units; the (gate, up) partial sums meet in
// shared memory.
struct GuTile { const uint8_t* G; const uint8_t* U; int r0, R, KS, rlim; uint32_t rb, pitch; float* hrow; float w; };

__device__ __forceinline__ bool gu_tile_produce(const MoeParams& p, const Ring& ring, uint32_t& n, const GuTile& tl,
                                                int lane, int tile, MoeSmemHead* hd) {
  const int s = n % ring.stages;
  if (!announce_tile(ring, n, hd, tile, lane)) return false;
  if (lane == 0) {
    hd->srcs[s][0] = tl.G + (size_t)tl.r0 * tl.rb;
    hd->srcs[s][1] = tl.U + (size_t)tl.r0 * tl.rb;
  }
  __syncwarp();
  Piece pc;
  pc.src = hd->srcs[s]; pc.nsrc = 2; pc.rows_per_src = 1; pc.nrows = 1; pc.row_stride = tl.rb;
  pc.bytes = (uint32_t)min(tl.R, tl.rlim - tl.r0) * tl.rb;
  if (!produce_piece(ring, n, pc, tl.pitch, lane)) return false;
  n++;
  return true;
}

template <int T, int LPR, int NR>
__device__ __forceinline__ bool gu_tile_consume(const MoeParams& p, const Ring& ring, uint32_t& n, const GuTile& tl, int U,
                                                int warp, int lane, const XqSmem (&xq)[1], const LaneLuts& L,
                                                MoeSmemHead* hd, uint32_t& tile_count) {
  constexpr int Gn = 32 / LPR;
  const int grp = lane / LPR, li = lane % LPR;
  const int KS = tl.KS;
  const int lr0 = KS > 1 ? warp / KS : (warp * Gn + grp) * NR;
  const int kpart = KS > 1 ? warp % KS : 0;
  constexpr int step = block_elems(T) == 256 ? 8 : 1;
  int ua = 0, ub = U;
  if (KS > 1) {
    const int per = ((U + KS * step - 1) / (KS * step)) * step;
    ua = min(U, kpart * per); ub = min(U, ua + per);
  }
  float acc[2 * NR][1];    // [0 .. NR): gate rows, [NR .. 2 NR): up rows
#pragma unroll
  for (int i = 0; i < 2 * NR; i++) acc[i][0] = 0.f;
  {
    const uintptr_t ag = reinterpret_cast<uintptr_t>(tl.G) + (size_t)tl.r0 * tl.rb;
    const uintptr_t au = reinterpret_cast<uintptr_t>(tl.U) + (size_t)tl.r0 * tl.rb;
    const saddr_t slot = smem_u32(ring.slot(n)) + (uint32_t)units_bytes(T, ua);
    saddr_t rowp[2 * NR];
#pragma unroll
    for (int i = 0; i < NR; i++) {
      rowp[i] = slot + (uint32_t)(ag & 15u) + (uint32_t)(lr0 + i) * tl.rb;
      rowp[NR + i] = slot + tl.pitch + (uint32_t)(au & 15u) + (uint32_t)(lr0 + i) * tl.rb;
    }
    if (!consumer_wait(ring, n)) return false;
    if (ub > ua) consume_rows<T, LPR, 2 * NR, 1>(rowp, li, xq, ua, ub - ua, L, acc);
    consumer_release(ring, n, lane);
    n++;
  }
  if (KS > 1) {
    const int pb = tile_count & 1;
    const float g = group_sum<32>(acc[0][0]), u = group_sum<32>(acc[NR][0]);
    if (lane == 0) { hd->part[pb][warp][0] = g; hd->part[pb][warp][1] = u; }
    __syncwarp();
    if (lane == 0) mbar_arrive(&hd->tilebar);
    if (!mbar_wait(&hd->tilebar, tile_count & 1u, ring.abort_flag, ring.status, kDevWaitFull)) return false;
    if (kpart == 0 && lane == 0 && tl.r0 + lr0 < tl.rlim) {
      float gs = 0.f, us = 0.f;
      for (int k = 0; k < KS; k++) { gs += hd->part[pb][warp + k][0]; us += hd->part[pb][warp + k][1]; }
      tl.hrow[tl.r0 + lr0] = swiglu(gs, us, tl.w, p.limit);
    }
    tile_count++;
  } else {
#pragma unroll
    for (int i = 0; i < NR; i++) {
      const float g = group_sum<LPR>(acc[i][0]), u = group_sum<LPR>(acc[NR + i][0]);
      if (li == 0 && tl.r0 + lr0 + i < tl.rlim) tl.hrow[tl.r0 + lr0 + i] = swiglu(g, u, tl.w, p.limit);
    }
  }
  return true;
}

// Tile order: block b takes tiles b, b + grid, b + 2 grid, ... (tiles of one kind cost the same, so a fixed stride
// balances as well as a shared counter would, without a global atomic round trip per tile).  The producer warp stages
// its first tile before the grid dependency is resolved when it is a shared-expert tile (constant data); everything
// that depends on the router's output waits for the consumers, which resolve the dependency, the resident experts and
// the activation, at the block barrier.
__device__ __forceinline__ int next_tile(int t) { return t + (int)gridDim.x; }

template <int TR, int TS, int LPR>
__global__ void __launch_bounds__((kMoeNW + 1) * 32, 1) moe_gu_kernel(const MoeParams p) {
  pdl_launch_dependents();
  extern __shared__ __align__(128) uint8_t smem[];
  MoeSmemHead* hd = reinterpret_cast<MoeSmemHead*>(smem);
  Ring ring;
  ring.full = hd->full; ring.empty = hd->empty;
  ring.abort_flag = &hd->abort_flag; ring.status = p.tb.status; ring.stages = p.stages;
  uint8_t* cur = smem + ((sizeof(MoeSmemHead) + 127) & ~(size_t)127);
  uint8_t* lut = cur;
  cur += lut_bytes_for(TR);
  const int U = p.dim / 32;
  XqSmem xq[1];
  xq_bind(xq[0], cur, U, false, xq_padded(TR) || xq_padded(TS));
  cur += xq_bytes(U, false, xq_padded(TR) || xq_padded(TS));
  cur = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(cur) + 127) & ~(uintptr_t)127);
  ring.slot0 = cur; ring.slot_bytes = p.stage_bytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  ring_init(ring, tid, kMoeNW);
  if (tid == 0) { mbar_init(&hd->lutbar, 1); mbar_init(&hd->tilebar, kMoeNW); mbar_fence_init(); }
  __syncthreads();

  const int R_R = p.gu_r_rows, R_S = p.gu_s_rows;
  const int tiles_s = p.gu_s ? (p.s_hi - p.s_lo + R_S - 1) / R_S : 0;
  const int tiles_r1 = (p.inter + R_R - 1) / R_R;
  const uint32_t rb_r = (uint32_t)row_bytes(TR, p.dim), rb_s = (uint32_t)row_bytes(TS, p.dim);
  // tile id -> what to stream: shared-expert tiles first (they are the largest), then the resident routed experts
  auto tile_of = [&](int t) {
    GuTile tl;
    if (t < tiles_s) {
      tl.G = p.sgate; tl.U = p.sup; tl.r0 = p.s_lo + t * R_S; tl.R = R_S; tl.KS = p.gu_s_ks; tl.rb = rb_s; tl.pitch = p.gu_s_pitch;
      tl.rlim = p.s_hi;
      tl.hrow = p.h + (size_t)p.n_routed * p.inter; tl.w = 1.0f;
    } else {
      const int i = (t - tiles_s) / tiles_r1, rt = (t - tiles_s) % tiles_r1;
      const int k = hd->local_slot[i];
      tl.G = hd->p0[i]; tl.U = hd->p1[i]; tl.r0 = rt * R_R; tl.R = R_R; tl.KS = 1; tl.rb = rb_r; tl.pitch = p.gu_r_pitch;
      tl.rlim = p.inter;
      tl.hrow = p.h + (size_t)k * p.inter; tl.w = __ldcg(p.weights + k);
    }
    return tl;
  };
  uint32_t n = 0;
  if (warp == kMoeNW) {
    int t = blockIdx.x;
    if (p.norm_in) {
      // every shared-expert tile is constant data and the consumers build the activation themselves: stream them
      // all before the router's result is needed
      while (t < tiles_s) {
        if (!gu_tile_produce(p, ring, n, tile_of(t), lane, t, hd)) return;
        t = next_tile(t);
      }
      pdl_wait();
      resolve_local(p, hd, p.gu_r != 0, false, lane);   // published to the consumers by the tiles' barriers
    } else {
      const bool early = t < tiles_s;
      if (early && !gu_tile_produce(p, ring, n, tile_of(t), lane, t, hd)) return;
      __syncthreads();
      pdl_wait();
      if (early) t = next_tile(t);
    }
    const int ntiles = tiles_s + hd->n_local * tiles_r1;
    while (t < ntiles) {
      if (!gu_tile_produce(p, ring, n, tile_of(t), lane, t, hd)) return;
      t = next_tile(t);
    }
    end_of_tiles(ring, n, hd, lane);
    return;
  }
  LaneLuts L;
  const bool luts_ok = load_luts(lut, TR == IQ1_S, TR == IQ2_XXS, false, p.tb, tid, &hd->lutbar, &hd->abort_flag, L, lane);
  bool resolved = true;
  if (p.norm_in) {
    // 1 / rms in the association of the router's fused norm (256 threads strided over the vector, eight warp sums
    // added in order), so that both kernels see bit-identical activations
    if (tid < 256) {
      float ss = 0.f;
      for (int i = tid; i < p.dim / 4; i += 256) {
        const float4 v = reinterpret_cast<const float4*>(p.norm_in)[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = warp_sum(ss);
      if (lane == 0) hd->part[0][warp][0] = ss;   // free until the first tile
    }
    bar_sync_named(1, kMoeNW * 32);
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += hd->part[0][i][0];
    const float mul = rsqrtf(tot / (float)p.dim + p.norm_eps);
    quantize_x(p.norm_in, xq[0], tid, kMoeNW * 32, mul, p.norm_w);
    bar_sync_named(1, kMoeNW * 32);
    resolved = false;
  } else {
    pdl_wait();     // the router's ids / weights and x come from the previous kernels
    if (warp == 0) resolve_local(p, hd, p.gu_r != 0, false, lane);
    quantize_x(p.x, xq[0], tid, kMoeNW * 32);
    __syncthreads();
  }
  if (!luts_ok) return;
  const bool two_pairs = R_R == kMoeNW * (32 / LPR) * 2;   // row pairs per lane group of a routed tile: 2 or 1
  uint32_t tile_count = 0;
  for (;;) {
    if (!consumer_wait(ring, n)) return;
    const int t = *reinterpret_cast<volatile int*>(&hd->meta[n % ring.stages]);
    if (t < 0) return;
    if (!resolved && t >= tiles_s) { pdl_wait(); resolved = true; }   // first routed tile: the router has finished
    const GuTile tl = tile_of(t);
    bool ok;
    if (t < tiles_s) ok = gu_tile_consume<TS, LPR, 1>(p, ring, n, tl, U, warp, lane, xq, L, hd, tile_count);
    else if (two_pairs) ok = gu_tile_consume<TR, LPR, 2>(p, ring, n, tl, U, warp, lane, xq, L, hd, tile_count);
    else ok = gu_tile_consume<TR, LPR, 1>(p, ring, n, tl, U, warp, lane, xq, L, hd, tile_count);
    if (!ok) return;
  }
}

// ---------------------------------------------------------------------------------------------------- down
// Routed part of a down tile.  A work item is (resident expert, run of PU consecutive units of its rows); warps take
// items round robin.  Inside an item LP lanes split the run and each lane applies the activation registers it loaded
// to NRT of the tile's 8 rows (32 / LP row groups x NRT rows = 8), so the expert's h is read from shared memory once
// per 8 rows instead of once per row.  Every warp leaves its 8 row sums (zero without items) in rpart.
template <int TR, int LP, int NRT>
__device__ __forceinline__ void down_routed(const MoeParams& p, MoeSmemHead* hd, saddr_t slot, uint32_t rb_r, int r0, int Ui,
                                            int n_local, int warp, int lane, const XqSmem (&xq)[1], const LaneLuts& L,
                                            int pb) {
  static_assert(NRT * (32 / LP) == kMoeNW / 2, "row groups x rows per lane = rows of a tile");
  constexpr int PU = TR == IQ1_S ? 4 * LP : LP;      // IQ1_S lanes work on half super-blocks (4 units)
  const int rg = lane / LP, li = lane % LP;
  const int parts = (Ui + PU - 1) / PU;
  float acc[NRT][1];
#pragma unroll
  for (int i = 0; i < NRT; i++) acc[i][0] = 0.f;
  for (int it = warp; it < n_local * parts; it += kMoeNW) {
    const int e = it / parts, ua = (it - e * parts) * PU, nu = min(PU, Ui - ua);
    const uintptr_t a = reinterpret_cast<uintptr_t>(hd->p0[e]) + (size_t)r0 * rb_r;
    saddr_t rowp[NRT];
#pragma unroll
    for (int i = 0; i < NRT; i++)
      rowp[i] = slot + (uint32_t)e * p.d_src_pitch + (uint32_t)(a & 15u) + (uint32_t)(rg * NRT + i) * rb_r +
                (uint32_t)units_bytes(TR, ua);
    consume_rows<TR, LP, NRT, 1>(rowp, li, xq, hd->local_slot[e] * Ui + ua, nu, L, acc);
  }
#pragma unroll
  for (int i = 0; i < NRT; i++) {
    const float v = group_sum<LP>(acc[i][0]);
    if (li == 0) hd->rpart[pb][warp][rg * NRT + i] = v;
  }
}

// Tile = 8 output rows.  The first piece stages those 8 rows of every resident routed expert's down matrix (one
// contiguous copy per expert, side by side), the second the shared expert's rows.  Two warps share a row: the even
// warp takes the even sources (and the first half of the shared expert's units), the odd warp the rest; the two
// partial sums meet in shared memory and are added in a fixed order.
template <int TR, int TS, int LPR>
__global__ void __launch_bounds__((kMoeNW + 1) * 32, 1) moe_down_kernel(const MoeParams p) {
  constexpr int R = kMoeNW / 2;
  constexpr int Gn = 32 / LPR;
  pdl_launch_dependents();
  extern __shared__ __align__(128) uint8_t smem[];
  MoeSmemHead* hd = reinterpret_cast<MoeSmemHead*>(smem);
  Ring ring;
  ring.full = hd->full; ring.empty = hd->empty;
  ring.abort_flag = &hd->abort_flag; ring.status = p.tb.status; ring.stages = p.stages;
  uint8_t* cur = smem + ((sizeof(MoeSmemHead) + 127) & ~(size_t)127);
  uint8_t* lut = cur;
  cur += lut_bytes_for(TR);
  const int Ui = p.inter / 32;
  const int U = (p.n_routed + 1) * Ui;          // h rows of every slot, shared expert last
  XqSmem xq[1];
  xq_bind(xq[0], cur, U, false, xq_padded(TR) || xq_padded(TS));
  cur += xq_bytes(U, false, xq_padded(TR) || xq_padded(TS));
  cur = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(cur) + 127) & ~(uintptr_t)127);
  ring.slot0 = cur; ring.slot_bytes = p.stage_bytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  ring_init(ring, tid, kMoeNW);
  if (tid == 0) { mbar_init(&hd->lutbar, 1); mbar_init(&hd->tilebar, kMoeNW); mbar_fence_init(); }
  __syncthreads();
  const int ntiles = (p.dim + R - 1) / R;
  const uint32_t rb_r = (uint32_t)row_bytes(TR, p.inter), rb_s = (uint32_t)row_bytes(TS, p.inter);
  // the shared expert's K range handled here: units [s_u0, s_u0 + Us) of each of its rows
  const int s_u0 = p.s_lo / 32, Us = (p.s_hi - p.s_lo) / 32;
  const bool s_whole = Us == Ui;
  const uint32_t s_off = (uint32_t)units_bytes(TS, s_u0), s_bytes = (uint32_t)units_bytes(TS, Us);
  uint32_t n = 0;
  if (warp == kMoeNW) {
    // Per tile: the shared expert's rows first (constant data: the first tile's are staged before the grid
    // dependency is resolved), then the rows of every resident routed expert.
    int t = blockIdx.x;                      // the grid has at most ntiles blocks
    bool first_done = false;
    Piece pc;
    pc.rows_per_src = 1; pc.nrows = 1;
    auto shared_piece = [&](bool announce) {
      const int s = n % ring.stages;
      const int r0 = t * R, nrows = min(R, p.dim - r0);
      if (announce ? !announce_tile(ring, n, hd, t, lane)
                   : !mbar_wait(&ring.empty[s], ((n / ring.stages) & 1u) ^ 1u, ring.abort_flag, ring.status, kDevWaitEmpty))
        return false;
      if (lane == 0) hd->srcs[s][0] = p.sdown + (size_t)r0 * rb_s + s_off;
      __syncwarp();
      pc.src = hd->srcs[s]; pc.nsrc = 1; pc.row_stride = rb_s;
      if (s_whole) { pc.rows_per_src = 1; pc.nrows = 1; pc.bytes = (uint32_t)nrows * rb_s; }      // one contiguous copy
      else { pc.rows_per_src = R; pc.nrows = nrows; pc.bytes = s_bytes; }                        // a K range of each row
      if (!produce_piece(ring, n, pc, s_whole ? 0 : p.d_s_pitch, lane)) return false;
      pc.rows_per_src = 1; pc.nrows = 1;
      n++;
      return true;
    };
    if (p.d_s) { if (!shared_piece(true)) return; first_done = true; }
    __syncthreads();
    pdl_wait();
    const int n_local = hd->n_local;
    while (t < ntiles) {
      const int r0 = t * R, nrows = min(R, p.dim - r0);
      bool announced = first_done;
      if (p.d_s && !first_done) { if (!shared_piece(true)) return; announced = true; }
      first_done = false;
      if (n_local > 0) {
        const int s = n % ring.stages;
        if (!announced ? !announce_tile(ring, n, hd, t, lane)
                       : !mbar_wait(&ring.empty[s], ((n / ring.stages) & 1u) ^ 1u, ring.abort_flag, ring.status, kDevWaitEmpty))
          return;
        for (int e = lane; e < n_local; e += 32) hd->srcs[s][e] = hd->p0[e] + (size_t)r0 * rb_r;
        __syncwarp();
        pc.src = hd->srcs[s]; pc.nsrc = n_local; pc.row_stride = rb_r; pc.bytes = (uint32_t)nrows * rb_r;
        if (!produce_piece(ring, n, pc, p.d_src_pitch, lane)) return;
        n++;
      }
      t = next_tile(t);
    }
    end_of_tiles(ring, n, hd, lane);
    return;
  }
  LaneLuts L;
  const bool luts_ok = load_luts(lut, TR == IQ1_S, TR == IQ2_XXS, false, p.tb, tid, &hd->lutbar, &hd->abort_flag, L, lane);
  pdl_wait();     // h comes from the gate/up kernel
  // expert-parallel exchange: the epoch (completed combines on this rank) picks the slot / counter parity
  unsigned ep_epoch = 0;
  if (p.ep_world > 0) ep_epoch = *reinterpret_cast<volatile unsigned*>(p.ep_base[p.ep_rank]);
  const int ep_par = (int)(ep_epoch & 1u);
  if (warp == 0) resolve_local(p, hd, p.d_r != 0, true, lane);
  if (p.ep_world > 0) {
    // expert parallel: only the h rows this rank will read (its resident experts' and its slice of the shared expert's)
    // are quantised -- a fraction of the (n_routed + 1) x inter values, and this runs on every block before its first tile
    bar_sync_named(1, kMoeNW * 32);
    const int nl = hd->n_local, nu = nl * Ui + (p.d_s ? Us : 0), nr = p.n_routed;
    const int* slot = hd->local_slot;
    quantize_units(p.h, xq[0], tid, kMoeNW * 32, 1.f, nullptr, nu, [=](int v) {
      const int j = v / Ui;
      return j < nl ? slot[j] * Ui + (v - j * Ui) : nr * Ui + s_u0 + (v - nl * Ui);
    });
  } else {
    quantize_x(p.h, xq[0], tid, kMoeNW * 32);
  }
  __syncthreads();
  if (!luts_ok) return;
  const int n_local = hd->n_local;
  const int row = warp >> 1, half = warp & 1;
  const int grp = lane / LPR, li = lane % LPR;   // LPR < 32: lane groups take alternate sources / unit runs
  uint32_t tile_count = 0;
  if (p.ep_world > 0 && n_local == 0 && !p.d_s && warp == 0 && lane < p.ep_world) {
    // nothing of this token's MoE lives here: the exchange still needs this rank's (zero) partial
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
      float* dst = reinterpret_cast<float*>(p.ep_base[lane] + kEpSlotsOff) + ((size_t)(ep_par * p.ep_world + p.ep_rank)) * p.dim + (size_t)t * R;
      reinterpret_cast<float4*>(dst)[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      reinterpret_cast<float4*>(dst)[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  for (;;) {
    if (!consumer_wait(ring, n)) return;
    const int t = *reinterpret_cast<volatile int*>(&hd->meta[n % ring.stages]);
    if (t < 0) break;
    const int r0 = t * R;
    float acc[1][1] = {{0.f}};
    if (p.d_s) {
      if (!consumer_wait(ring, n)) return;
      const saddr_t slot = smem_u32(ring.slot(n));
      // staged: the tile's rows back to back (whole rows), or one K range per row at pitch d_s_pitch
      const uintptr_t a = reinterpret_cast<uintptr_t>(p.sdown) + (size_t)r0 * rb_s + s_off + (s_whole ? 0 : (size_t)row * rb_s);
      const saddr_t row_s = slot + (uint32_t)(a & 15u) + (uint32_t)row * (s_whole ? rb_s : p.d_s_pitch);
      // the 2 * Gn lane groups that share this row split its units into equal runs of whole super-blocks
      const int parts = 2 * Gn, me = half * Gn + grp;
      constexpr int step = block_elems(TS) == 256 ? 8 : 1;
      const int per = ((Us + parts * step - 1) / (parts * step)) * step;
      const int ua = min(Us, me * per), ub = min(Us, ua + per);
      if (ub > ua) {
        const saddr_t rowp[1] = {row_s + (uint32_t)units_bytes(TS, ua)};
        consume_rows<TS, LPR, 1, 1>(rowp, li, xq, p.n_routed * Ui + s_u0 + ua, ub - ua, L, acc);
      }
      consumer_release(ring, n, lane);
      n++;
    }
    const int pb = tile_count & 1;
    if (n_local > 0) {
      if (!consumer_wait(ring, n)) return;
      const saddr_t slot = smem_u32(ring.slot(n));
      if constexpr (TR == IQ1_S) down_routed<TR, 8, 2>(p, hd, slot, rb_r, r0, Ui, n_local, warp, lane, xq, L, pb);
      else if (n_local >= 5) down_routed<TR, 32, 8>(p, hd, slot, rb_r, r0, Ui, n_local, warp, lane, xq, L, pb);
      else if (n_local >= 3) down_routed<TR, 16, 4>(p, hd, slot, rb_r, r0, Ui, n_local, warp, lane, xq, L, pb);
      else down_routed<TR, 8, 2>(p, hd, slot, rb_r, r0, Ui, n_local, warp, lane, xq, L, pb);
      consumer_release(ring, n, lane);
      n++;
    }
    // combine: the shared expert's lane groups inside the warp (fixed order); then, per row, the two warps that split the
    // shared expert's units and every warp's routed sum, in warp order
    float v = group_sum<LPR>(acc[0][0]);
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) hd->part[pb][warp][0] = v;
    __syncwarp();
    if (lane == 0) mbar_arrive(&hd->tilebar);
    if (!mbar_wait(&hd->tilebar, tile_count & 1u, ring.abort_flag, ring.status, kDevWaitFull)) return;
    if (warp == 0) {
      float s = 0.f;
      if (lane < R && r0 + lane < p.dim) {
        s = hd->part[pb][2 * lane][0] + hd->part[pb][2 * lane + 1][0];
        if (n_local > 0)
          for (int w = 0; w < kMoeNW; w++) s += hd->rpart[pb][w][lane];
      }
      if (p.ep_world > 0) {
        // this rank's partial sums of the tile's 8 rows go to every rank's exchange buffer: lane r gathers the eight
        // values and writes them to rank r as two 16-byte peer stores (dim is a multiple of 256: tiles are whole)
        float v[R];
#pragma unroll
        for (int k = 0; k < R; k++) v[k] = __shfl_sync(0xffffffffu, s, k);
        if (lane < p.ep_world) {
          float* dst = reinterpret_cast<float*>(p.ep_base[lane] + kEpSlotsOff) + ((size_t)(ep_par * p.ep_world + p.ep_rank)) * p.dim + r0;
          reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
          reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
      } else if (lane < R && r0 + lane < p.dim) {
        p.y[r0 + lane] += s;
      }
    }
    tile_count++;
  }
  if (p.ep_world > 0 && warp == 0) {
    // Every row of this block is stored (by lanes of this warp).  One release per block: after the warp barrier lane r
    // adds 1 to the arrival counter of this exchange in rank r's buffer with release semantics at system scope, which
    // orders the block's partial rows before it; every rank's counters live on cache lines of their own (one per source
    // rank), so a counter sees gridDim.x additions however many ranks there are.  No block waits for another.
    __syncwarp();
    if (lane < p.ep_world) {
      unsigned* cnt = ep_arrivals(p.ep_base[lane], ep_par, p.ep_rank);
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(cnt), "r"(1u) : "memory");
    }
  }
}

// ---------------------------------------------------------------------------------------------------- host side
namespace {

bool routed_type_ok(int t) { return t == IQ1_S || t == IQ2_XXS; }
bool shared_type_ok(int t) { return t == Q6_K || t == Q8_0; }

int lpr_for(int units) {
  for (int lpr : {32, 16, 8})
    if (units % lpr == 0) return lpr;
  return 0;
}

template <typename K>
int set_smem(K kern, int dev, bool* done) {
  if (!done[dev & 63]) {
    MSB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    done[dev & 63] = true;
  }
  return kOk;
}

template <int TR, int TS, int LPR>
int launch_gu(MoeParams& p, int sms, int dev, cudaStream_t st) {
  constexpr int Gn = 32 / LPR;
  const int U = p.dim / 32;
  const size_t fixed = ((sizeof(MoeSmemHead) + 127) & ~(size_t)127) + lut_bytes_for(TR) + xq_bytes(U, false, xq_padded(TR) || xq_padded(TS)) + 128;
  if (fixed + 3 * 8192 > (size_t)kSmemLimit) return fail(kErrLimit, "moe_decode: dim %d does not fit in shared memory", p.dim);
  const size_t avail = (size_t)kSmemLimit - fixed;
  const size_t rb_r = row_bytes(TR, p.dim), rb_s = row_bytes(TS, p.dim);
  // room for R rows of one matrix in a slot: the source's misalignment, rounded to 16, plus the word the decoders may
  // read past the end
  auto pitch_of = [](size_t bytes) { return (uint32_t)((bytes + 15 + 16 + 15) & ~(size_t)15); };
  // routed tiles: every warp owns 2 whole row pairs (gate + up) per lane group, 1 when a two-deep ring of those does
  // not fit
  int stages = 0;
  for (int pairs : {2, 1}) {
    p.gu_r_rows = kMoeNW * Gn * pairs;
    p.gu_r_pitch = pitch_of((size_t)p.gu_r_rows * rb_r);
    stages = (int)std::min<size_t>(kMaxStages, avail / (2 * (size_t)p.gu_r_pitch + 128));
    if (stages >= 2) break;
  }
  if (stages < 2) return fail(kErrLimit, "moe_decode: routed gate/up tile does not fit (dim %d)", p.dim);
  const size_t slot = (avail / stages) & ~(size_t)127;
  // shared tiles: as many whole row pairs as fit, several warps per row when the rows are long
  p.gu_s_ks = 0;
  if (2 * (size_t)pitch_of((size_t)kMoeNW * Gn * rb_s) <= slot) { p.gu_s_rows = kMoeNW * Gn; p.gu_s_ks = 1; }
  else if (LPR == 32) {
    for (int ks : {2, 4, 8, 16})
      if (2 * (size_t)pitch_of((size_t)(kMoeNW / ks) * rb_s) <= slot) { p.gu_s_rows = kMoeNW / ks; p.gu_s_ks = ks; break; }
  }
  if (!p.gu_s_ks) return fail(kErrLimit, "moe_decode: shared gate/up tile does not fit (dim %d)", p.dim);
  p.gu_s_pitch = pitch_of((size_t)p.gu_s_rows * rb_s);
  p.stages = stages;
  p.stage_bytes = (uint32_t)slot;
  auto kern = moe_gu_kernel<TR, TS, LPR>;
  static bool done[64] = {};
  int rc = set_smem(kern, dev, done);
  if (rc) return rc;
  const int tiles = (p.gu_s ? (p.s_hi - p.s_lo + p.gu_s_rows - 1) / p.gu_s_rows : 0) +
                    (p.gu_r ? p.n_routed : 0) * ((p.inter + p.gu_r_rows - 1) / p.gu_r_rows);
  MSB_CUDA(launch_pdl(kern, dim3(std::max(1, std::min(sms, tiles))), dim3((kMoeNW + 1) * 32), fixed + (size_t)stages * slot, st, p));
  MSB_LAUNCH_CHECK("moe_gu_kernel");
  return kOk;
}

template <int TR, int TS, int LPR>
int launch_down(MoeParams& p, int sms, int dev, cudaStream_t st) {
  constexpr int R = kMoeNW / 2;
  const int Ui = p.inter / 32, U = (p.n_routed + 1) * Ui;
  const size_t fixed = ((sizeof(MoeSmemHead) + 127) & ~(size_t)127) + lut_bytes_for(TR) + xq_bytes(U, false, xq_padded(TR) || xq_padded(TS)) + 128;
  const size_t rb_r = row_bytes(TR, p.inter), rb_s = row_bytes(TS, p.inter);
  p.d_rows = R;
  p.d_src_pitch = (uint32_t)((R * rb_r + 15 + 16 + 15) & ~(size_t)15);
  p.d_s_pitch = piece_pitch((uint32_t)units_bytes(TS, (p.s_hi - p.s_lo) / 32));
  const size_t need = std::max((size_t)std::max(1, p.n_routed) * p.d_src_pitch, R * rb_s + 64);
  for (int stages = kMaxStages; stages >= 2; stages--) {
    if (fixed + (size_t)stages * need > (size_t)kSmemLimit) continue;
    const size_t slot = std::min<size_t>(((size_t)kSmemLimit - fixed) / stages, need + 1024) & ~(size_t)127;
    if (slot < need) continue;
    p.stages = stages;
    p.stage_bytes = (uint32_t)slot;
    auto kern = moe_down_kernel<TR, TS, LPR>;
    static bool done[64] = {};
    int rc = set_smem(kern, dev, done);
    if (rc) return rc;
    static_assert(R == 8, "moe_down_blocks() assumes 8-row tiles");
    MSB_CUDA(launch_pdl(kern, dim3(moe_down_blocks(p.dim, sms)), dim3((kMoeNW + 1) * 32), fixed + (size_t)stages * slot, st, p));
    MSB_LAUNCH_CHECK("moe_down_kernel");
    return kOk;
  }
  return fail(kErrLimit, "moe_decode: down staging does not fit (inter %d, %d routed)", p.inter, p.n_routed);
}

template <int TR, int TS>
int launch_gu_lpr(MoeParams& p, int lpr, int sms, int dev, cudaStream_t st) {
  switch (lpr) {
    case 32: return launch_gu<TR, TS, 32>(p, sms, dev, st);
    case 16: return launch_gu<TR, TS, 16>(p, sms, dev, st);
    default: return launch_gu<TR, TS, 8>(p, sms, dev, st);
  }
}
template <int TR, int TS>
int launch_down_lpr(MoeParams& p, int lpr, int sms, int dev, cudaStream_t st) {
  switch (lpr) {
    case 32: return launch_down<TR, TS, 32>(p, sms, dev, st);
    case 16: return launch_down<TR, TS, 16>(p, sms, dev, st);
    default: return launch_down<TR, TS, 8>(p, sms, dev, st);
  }
}
}  // namespace

size_t moe_decode_scratch_bytes(int inter, int max_routed) {
  return sizeof(float) * (size_t)(max_routed + 1) * inter;
}

// part: 0 All, 1 SharedGu, 2 AfterSharedGu, 3 Shared, 4 Routed, 5 SharedDown (the reference's MoePart, quant.hpp:83);
// 6 = gate/up of every expert only, 7 = down of every expert only (the two launches of All, for timing one alone)
int moe_decode(MoeParams p, int t_gate_up, int t_down, int t_shared, int part, size_t scratch_bytes, cudaStream_t st) {
  if (p.n_routed < 0 || p.n_routed > kMaxRouted) return fail(kErrArg, "moe_decode: n_routed %d outside 0..%d", p.n_routed, kMaxRouted);
  if (!routed_type_ok(t_gate_up) || !routed_type_ok(t_down) || !shared_type_ok(t_shared))
    return fail(kErrType, "moe_decode: unsupported type combination (%s, %s, %s)", type_name(t_gate_up), type_name(t_down),
                type_name(t_shared));
  if (p.dim <= 0 || p.inter <= 0 || p.dim % 256 || p.inter % 256) return fail(kErrArg, "moe_decode: dim/inter must be multiples of 256");
  if (scratch_bytes < moe_decode_scratch_bytes(p.inter, p.n_routed)) return fail(kErrScratch, "moe_decode: scratch too small");
  if (part < 0 || part > 7) return fail(kErrArg, "moe_decode: bad part %d", part);
  const bool shared_piece = part == 1 || part == 3 || part == 5;
  if (shared_piece && !p.has_shared) return kOk;
  p.gu_r = part == 0 || part == 2 || part == 4 || part == 6;
  p.gu_s = p.has_shared && (part == 0 || part == 1 || part == 3 || part == 6);
  p.d_r = part == 0 || part == 2 || part == 4 || part == 7;
  p.d_s = p.has_shared && (part == 0 || part == 2 || part == 3 || part == 5 || part == 7);
  if (p.n_routed == 0) p.gu_r = p.d_r = 0;
  if (p.s_lo == 0 && p.s_hi == 0) p.s_hi = p.inter;      // default: the whole shared expert
  if (p.s_lo < 0 || p.s_hi > p.inter || p.s_lo > p.s_hi || p.s_lo % 256 || p.s_hi % 256)
    return fail(kErrArg, "moe_decode: shared-expert range [%d, %d) must be multiples of 256 inside 0..%d", p.s_lo, p.s_hi, p.inter);
  if (p.s_lo == p.s_hi) p.gu_s = p.d_s = 0;              // an empty slice: no shared-expert work on this rank
  if (p.ep_world < 0 || p.ep_world > kMaxEpWorld || (p.ep_world > 0 && (p.ep_rank < 0 || p.ep_rank >= p.ep_world)))
    return fail(kErrArg, "moe_decode: bad expert-parallel world %d / rank %d", p.ep_world, p.ep_rank);
  for (int r = 0; r < p.ep_world; r++)
    if (!p.ep_base[r] || (reinterpret_cast<uintptr_t>(p.ep_base[r]) & 255))
      return fail(kErrArg, "moe_decode: exchange buffer of rank %d missing or not 256-byte aligned", r);
  if (p.ep_world > 0 && !(p.d_r || p.d_s)) {
    // the exchange needs a down launch on every rank, even one without work: it publishes zeros
    p.d_r = 1;
  }
  if (!p.gu_r && !p.gu_s && !p.d_r && !p.d_s) return kOk;
  if ((!p.x && !p.norm_in) || (!p.y && p.ep_world == 0) || !p.h || (p.gu_r && !p.weights)) return fail(kErrArg, "moe_decode: null pointer");
  if (p.norm_in && (!p.norm_w || ((reinterpret_cast<uintptr_t>(p.norm_in) | reinterpret_cast<uintptr_t>(p.norm_w)) & 15)))
    return fail(kErrArg, "moe_decode: norm_in needs a gain vector, both 16-byte aligned");
  int rc = get_tables(&p.tb);
  if (rc) return rc;
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int lpr_gu = lpr_for(p.dim / 32), lpr_d = lpr_for(p.inter / 32);
  if (!lpr_gu || !lpr_d) return fail(kErrArg, "moe_decode: dim/inter not supported");
  unsigned* sched_base = reinterpret_cast<unsigned*>(p.tb.status) + 8;   // [0]: blocks of a down launch that stored their partial
  if (p.d_r || p.d_s) {
    // The down launch keeps the quantised h of every routed expert and of the shared expert in shared memory beside its
    // tables and a two-slot ring: checked here, before the gate/up launch, so that a size that does not fit leaves
    // nothing enqueued (the same arithmetic as launch_down).
    const size_t U = (size_t)(p.n_routed + 1) * (p.inter / 32);
    const size_t fixed = ((sizeof(MoeSmemHead) + 127) & ~(size_t)127) + lut_bytes_for(t_down) +
                         xq_bytes((int)U, false, xq_padded(t_down) || xq_padded(t_shared)) + 128;
    const size_t R = kMoeNW / 2;
    const size_t pitch = (R * row_bytes(t_down, p.inter) + 15 + 16 + 15) & ~(size_t)15;
    const size_t need = std::max((size_t)std::max(1, p.n_routed) * pitch, R * row_bytes(t_shared, p.inter) + 64);
    if (fixed + 2 * need > (size_t)kSmemLimit)
      return fail(kErrLimit, "moe_decode: down staging does not fit (inter %d, %d routed): inter x (routed + 1) x 2.5 bytes of "
                  "quantised h, the tables and two ring slots must fit %d bytes of shared memory", p.inter, p.n_routed, (int)kSmemLimit);
  }
  if (p.gu_r || p.gu_s) {
    p.sched = sched_base;
#define MSB_GU(TR, TS) rc = launch_gu_lpr<TR, TS>(p, lpr_gu, sms, dev, st)
    if (t_gate_up == IQ1_S && t_shared == Q8_0) MSB_GU(IQ1_S, Q8_0);
    else if (t_gate_up == IQ1_S) MSB_GU(IQ1_S, Q6_K);
    else if (t_shared == Q8_0) MSB_GU(IQ2_XXS, Q8_0);
    else MSB_GU(IQ2_XXS, Q6_K);
#undef MSB_GU
    if (rc) return rc;
  }
  if (p.d_r || p.d_s) {
    p.sched = sched_base;
#define MSB_DN(TR, TS) rc = launch_down_lpr<TR, TS>(p, lpr_d, sms, dev, st)
    if (t_down == IQ1_S && t_shared == Q8_0) MSB_DN(IQ1_S, Q8_0);
    else if (t_down == IQ1_S) MSB_DN(IQ1_S, Q6_K);
    else if (t_shared == Q8_0) MSB_DN(IQ2_XXS, Q8_0);
    else MSB_DN(IQ2_XXS, Q6_K);
#undef MSB_DN
    if (rc) return rc;
  }
  return kOk;
}

}  // namespace msb
