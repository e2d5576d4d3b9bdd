// Fused MoE decode for one token: routed experts (IQ1_S / IQ2_XXS) + one shared expert (Q6_K / Q8_0).
//   moe_gu_kernel  : h[e][r] = silu(min(gate_e[r].x, L)) * clamp(up_e[r].x, -L, L) * w_e   (all experts, one launch)
//   moe_down_kernel: y[r] += sum_e down_e[r] . h[e]                                        (all experts, one launch)
// Replaces the reference's q_moe_gu[_t] / q_moe_down[_t] Metal kernels (src/kernels/quant_moe.metal:50-147,175-259)
// behind ms::q::encode_moe_decode / encode_moe_decode_table[_part] (src/kernels/quant.hpp:49-85, quant.mm:264-369).
//
// Work distribution: persistent blocks pull row tiles from a device-side tile counter (big shared-expert tiles
// first), so the split adapts to how many of the routed experts are resident on this GPU (expert parallelism) without
// a host round trip.  A row's partial sums are always formed in the same order, whichever block computes it.
#include <algorithm>
#include "stream_pipe.cuh"
#include "moe_decode_params.cuh"

namespace msb {

struct MoeSmemHead {
  uint64_t full[kMaxStages], empty[kMaxStages];
  int abort_flag;
  int n_local;
  int meta[kMaxStages];
  int local_slot[kMaxRouted];
  const uint8_t* p0[kMaxRouted];   // gate (gu kernel) or down (down kernel) of local routed slot i
  const uint8_t* p1[kMaxRouted];   // up
};

__device__ __forceinline__ float swiglu(float g, float u, float w, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-g)) * u * w;
}

// Resolve which routed slots are handled by this GPU and their matrix addresses.  Thread 0 only.
__device__ __forceinline__ void resolve_local(const MoeParams& p, MoeSmemHead* hd, bool want_routed, bool down) {
  int nl = 0;
  if (want_routed) {
    for (int k = 0; k < p.n_routed; k++) {
      if (p.table) {
        const int id = p.ids ? p.ids[k] : k;          // no ids: the table holds one entry per routed slot
        if (p.ids && (id < p.expert_lo || id >= p.expert_hi)) continue;
        const uint64_t* row = p.table + (size_t)id * 3;
        hd->p0[nl] = reinterpret_cast<const uint8_t*>(down ? row[2] : row[0]);
        hd->p1[nl] = reinterpret_cast<const uint8_t*>(row[1]);
      } else {
        hd->p0[nl] = down ? p.down[k] : p.gate[k];
        hd->p1[nl] = p.up[k];
      }
      hd->local_slot[nl++] = k;
    }
  }
  hd->n_local = nl;
}

__device__ __forceinline__ void finish_block(unsigned* sched) {
  __threadfence();
  const unsigned old = atomicAdd(&sched[1], 1u);
  if (old == gridDim.x - 1) { sched[0] = 0; sched[1] = 0; __threadfence(); }
}

// ---------------------------------------------------------------------------------------------------- gate/up
template <int T, int LPR, int NR>
__device__ __forceinline__ void gu_tile_consume(const MoeParams& p, const Ring& ring, uint32_t& n, const MoeShape& sh,
                                                const uint8_t* G, const uint8_t* Uw, int r0, int U, int warp, int lane,
                                                const XqSmem (&xq)[1], const LaneLuts& L, float* hrow, float w,
                                                bool& ok) {
  constexpr int Gn = 32 / LPR, R = kMoeNW * Gn * NR;
  const uint32_t rb = (uint32_t)row_bytes(T, p.dim);
  float ag[NR][1], au[NR][1];
#pragma unroll
  for (int i = 0; i < NR; i++) { ag[i][0] = 0.f; au[i][0] = 0.f; }
  const int nrows = min(R, p.inter - r0);
  for (int u0 = 0; u0 < U && ok; u0 += sh.chunk) {
    const int nu = min(sh.chunk, U - u0);
    Piece pc;
    pc.row_stride = rb; pc.bytes = units_bytes(T, nu); pc.nrows = nrows;
    pc.src = G + (size_t)r0 * rb + units_bytes(T, u0);
    if (!(ok = consumer_wait(ring, n))) break;
    consume_piece<T, LPR, NR, 1>(ring, n, pc, sh.pitch, warp * Gn * NR, lane, xq, u0, nu, L, ag);
    consumer_release(ring, n, lane); n++;
    pc.src = Uw + (size_t)r0 * rb + units_bytes(T, u0);
    if (!(ok = consumer_wait(ring, n))) break;
    consume_piece<T, LPR, NR, 1>(ring, n, pc, sh.pitch, warp * Gn * NR, lane, xq, u0, nu, L, au);
    consumer_release(ring, n, lane); n++;
  }
  if (!ok) return;
  const int grp = lane / LPR, li = lane % LPR;
#pragma unroll
  for (int i = 0; i < NR; i++) {
    const float g = group_sum<LPR>(ag[i][0]), u = group_sum<LPR>(au[i][0]);
    const int lr = (warp * Gn + grp) * NR + i;
    if (li == 0 && r0 + lr < p.inter) hrow[r0 + lr] = swiglu(g, u, w, p.limit);
  }
}

template <int T, int LPR, int NR>
__device__ __forceinline__ bool gu_tile_produce(const MoeParams& p, const Ring& ring, uint32_t& n, const MoeShape& sh,
                                                const uint8_t* G, const uint8_t* Uw, int r0, int U, int lane, int tile,
                                                MoeSmemHead* hd) {
  constexpr int Gn = 32 / LPR, R = kMoeNW * Gn * NR;
  const uint32_t rb = (uint32_t)row_bytes(T, p.dim);
  const int nrows = min(R, p.inter - r0);
  bool first = true;
  for (int u0 = 0; u0 < U; u0 += sh.chunk) {
    const int nu = min(sh.chunk, U - u0);
    Piece pc;
    pc.row_stride = rb; pc.bytes = units_bytes(T, nu); pc.nrows = nrows;
    for (int m = 0; m < 2; m++, n++) {
      pc.src = (m ? Uw : G) + (size_t)r0 * rb + units_bytes(T, u0);
      if (first) {   // the first piece of a tile carries the tile id for the consumers
        const int s = n % ring.stages;
        if (!mbar_wait(&ring.empty[s], ((n / ring.stages) & 1u) ^ 1u, ring.abort_flag, ring.status, kDevWaitEmpty))
          return false;
        if (lane == 0) *reinterpret_cast<volatile int*>(&hd->meta[s]) = tile;
        __syncwarp();
        first = false;
      }
      if (!produce_piece(ring, n, pc, sh.pitch, lane)) return false;
    }
  }
  return true;
}

template <int TR, int TS, int LPR>
__global__ void __launch_bounds__((kMoeNW + 1) * 32, 1) moe_gu_kernel(const MoeParams p) {
  constexpr int Gn = 32 / LPR;
  constexpr int NR_R = 4, NR_S = 2;
  constexpr int R_R = kMoeNW * Gn * NR_R, R_S = kMoeNW * Gn * NR_S;
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
  xq[0].U = U;
  xq[0].plane = reinterpret_cast<uint4*>(cur);
  xq[0].scale = reinterpret_cast<float*>(cur + (size_t)U * 64);
  xq[0].sumA = reinterpret_cast<int*>(cur + (size_t)U * 68);
  xq[0].sumB = reinterpret_cast<int*>(cur + (size_t)U * 72);
  xq[0].xf = nullptr;
  cur += (size_t)U * 76;
  cur = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(cur) + 127) & ~(uintptr_t)127);
  for (int s = 0; s < kMaxStages; s++) ring.slot[s] = cur + (size_t)s * p.stage_bytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  ring_init(ring, tid, kMoeNW);
  if (tid == 0) resolve_local(p, hd, p.gu_r != 0, false);
  LaneLuts L;
  fill_luts(lut, TR == IQ1_S, TR == IQ2_XXS, false, p.tb, tid, blockDim.x, L, lane);
  quantize_x(p.x, xq[0], tid, blockDim.x);
  __syncthreads();

  const int tiles_s = p.gu_s ? (p.inter + R_S - 1) / R_S : 0;
  const int tiles_r1 = (p.inter + R_R - 1) / R_R;
  const int ntiles = tiles_s + hd->n_local * tiles_r1;
  uint32_t n = 0;
  if (warp == kMoeNW) {
    // ---------------- producer: pull tiles (shared-expert tiles first, they are the largest)
    for (;;) {
      int t = 0;
      if (lane == 0) t = (int)atomicAdd(&p.sched[0], 1u);
      t = __shfl_sync(0xffffffffu, t, 0);
      if (t >= ntiles) break;
      bool ok;
      if (t < tiles_s) {
        ok = gu_tile_produce<TS, LPR, NR_S>(p, ring, n, p.gu_shared, p.sgate, p.sup, t * R_S, U, lane, t, hd);
      } else {
        const int i = (t - tiles_s) / tiles_r1, rt = (t - tiles_s) % tiles_r1;
        ok = gu_tile_produce<TR, LPR, NR_R>(p, ring, n, p.gu_routed, hd->p0[i], hd->p1[i], rt * R_R, U, lane, t, hd);
      }
      if (!ok) return;
    }
    // sentinel: an empty use that tells the consumers to stop
    const int s = n % ring.stages;
    if (!mbar_wait(&ring.empty[s], ((n / ring.stages) & 1u) ^ 1u, ring.abort_flag, ring.status, kDevWaitEmpty)) return;
    if (lane == 0) {
      *reinterpret_cast<volatile int*>(&hd->meta[s]) = -1;
      mbar_arrive(&ring.full[s]);
      finish_block(p.sched);
    }
    return;
  }
  // ---------------- consumers
  for (;;) {
    if (!consumer_wait(ring, n)) return;
    const int t = *reinterpret_cast<volatile int*>(&hd->meta[n % ring.stages]);
    if (t < 0) return;
    bool ok = true;
    if (t < tiles_s) {
      gu_tile_consume<TS, LPR, NR_S>(p, ring, n, p.gu_shared, p.sgate, p.sup, t * R_S, U, warp, lane, xq, L,
                                     p.h + (size_t)p.n_routed * p.inter, 1.0f, ok);
    } else {
      const int i = (t - tiles_s) / tiles_r1, rt = (t - tiles_s) % tiles_r1;
      const int k = hd->local_slot[i];
      gu_tile_consume<TR, LPR, NR_R>(p, ring, n, p.gu_routed, hd->p0[i], hd->p1[i], rt * R_R, U, warp, lane, xq, L,
                                     p.h + (size_t)k * p.inter, __ldg(p.weights + k), ok);
    }
    if (!ok) return;
  }
}

// ---------------------------------------------------------------------------------------------------- down
template <int TR, int TS, int LPR>
__global__ void __launch_bounds__((kMoeNW + 1) * 32, 1) moe_down_kernel(const MoeParams p) {
  constexpr int Gn = 32 / LPR;
  constexpr int NR = 1;
  constexpr int R = kMoeNW * Gn * NR;
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
  xq[0].U = U;
  xq[0].plane = reinterpret_cast<uint4*>(cur);
  xq[0].scale = reinterpret_cast<float*>(cur + (size_t)U * 64);
  xq[0].sumA = reinterpret_cast<int*>(cur + (size_t)U * 68);
  xq[0].sumB = reinterpret_cast<int*>(cur + (size_t)U * 72);
  xq[0].xf = nullptr;
  cur += (size_t)U * 76;
  cur = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(cur) + 127) & ~(uintptr_t)127);
  for (int s = 0; s < kMaxStages; s++) ring.slot[s] = cur + (size_t)s * p.stage_bytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  ring_init(ring, tid, kMoeNW);
  if (tid == 0) resolve_local(p, hd, p.d_r != 0, true);
  LaneLuts L;
  fill_luts(lut, TR == IQ1_S, TR == IQ2_XXS, false, p.tb, tid, blockDim.x, L, lane);
  quantize_x(p.h, xq[0], tid, blockDim.x);
  __syncthreads();

  const int ntiles = (p.dim + R - 1) / R;
  const int n_local = hd->n_local;
  const uint32_t rb_r = (uint32_t)row_bytes(TR, p.inter), rb_s = (uint32_t)row_bytes(TS, p.inter);
  uint32_t n = 0;
  if (warp == kMoeNW) {
    for (;;) {
      int t = 0;
      if (lane == 0) t = (int)atomicAdd(&p.sched[0], 1u);
      t = __shfl_sync(0xffffffffu, t, 0);
      if (t >= ntiles) break;
      const int r0 = t * R, nrows = min(R, p.dim - r0);
      bool first = true;
      for (int e = 0; e < n_local + (p.d_s ? 1 : 0); e++) {
        const bool sh = e == n_local;
        const MoeShape& shp = sh ? p.d_shared : p.d_routed;
        const uint8_t* Wd = sh ? p.sdown : hd->p0[e];
        const uint32_t rb = sh ? rb_s : rb_r;
        for (int u0 = 0; u0 < Ui; u0 += shp.chunk, n++) {
          const int nu = min(shp.chunk, Ui - u0);
          Piece pc;
          pc.row_stride = rb; pc.nrows = nrows;
          pc.bytes = sh ? units_bytes(TS, nu) : units_bytes(TR, nu);
          pc.src = Wd + (size_t)r0 * rb + (sh ? units_bytes(TS, u0) : units_bytes(TR, u0));
          if (first) {
            const int s = n % ring.stages;
            if (!mbar_wait(&ring.empty[s], ((n / ring.stages) & 1u) ^ 1u, ring.abort_flag, ring.status, kDevWaitEmpty))
              return;
            if (lane == 0) *reinterpret_cast<volatile int*>(&hd->meta[s]) = t;
            __syncwarp();
            first = false;
          }
          if (!produce_piece(ring, n, pc, shp.pitch, lane)) return;
        }
      }
    }
    const int s = n % ring.stages;
    if (!mbar_wait(&ring.empty[s], ((n / ring.stages) & 1u) ^ 1u, ring.abort_flag, ring.status, kDevWaitEmpty)) return;
    if (lane == 0) {
      *reinterpret_cast<volatile int*>(&hd->meta[s]) = -1;
      mbar_arrive(&ring.full[s]);
      finish_block(p.sched);
    }
    return;
  }
  const int grp = lane / LPR, li = lane % LPR;
  for (;;) {
    if (!consumer_wait(ring, n)) return;
    const int t = *reinterpret_cast<volatile int*>(&hd->meta[n % ring.stages]);
    if (t < 0) return;
    const int r0 = t * R, nrows = min(R, p.dim - r0);
    float acc[NR][1];
#pragma unroll
    for (int i = 0; i < NR; i++) acc[i][0] = 0.f;
    for (int e = 0; e < n_local + (p.d_s ? 1 : 0); e++) {
      const bool sh = e == n_local;
      const MoeShape& shp = sh ? p.d_shared : p.d_routed;
      const uint8_t* Wd = sh ? p.sdown : hd->p0[e];
      const uint32_t rb = sh ? rb_s : rb_r;
      const int xunit = (sh ? p.n_routed : hd->local_slot[e]) * Ui;
      for (int u0 = 0; u0 < Ui; u0 += shp.chunk, n++) {
        const int nu = min(shp.chunk, Ui - u0);
        Piece pc;
        pc.row_stride = rb; pc.nrows = nrows;
        pc.bytes = sh ? units_bytes(TS, nu) : units_bytes(TR, nu);
        pc.src = Wd + (size_t)r0 * rb + (sh ? units_bytes(TS, u0) : units_bytes(TR, u0));
        if (!consumer_wait(ring, n)) return;
        if (sh) consume_piece<TS, LPR, NR, 1>(ring, n, pc, shp.pitch, warp * Gn * NR, lane, xq, xunit + u0, nu, L, acc);
        else consume_piece<TR, LPR, NR, 1>(ring, n, pc, shp.pitch, warp * Gn * NR, lane, xq, xunit + u0, nu, L, acc);
        consumer_release(ring, n, lane);
      }
    }
#pragma unroll
    for (int i = 0; i < NR; i++) {
      const float v = group_sum<LPR>(acc[i][0]);
      const int lr = (warp * Gn + grp) * NR + i;
      if (li == 0 && r0 + lr < p.dim) p.y[r0 + lr] += v;
    }
  }
}

// ---------------------------------------------------------------------------------------------------- host side
namespace {

bool routed_type_ok(int t) { return t == IQ1_S || t == IQ2_XXS; }
bool shared_type_ok(int t) { return t == Q6_K || t == Q8_0; }

// staged piece shape for R rows of `units` units of type t within a slot of slot_bytes
bool shape_for(int t, int units, int R, int lpr, size_t slot_bytes, MoeShape* out) {
  const bool sb = block_elems(t) == 256;
  const int step = sb ? std::max(lpr, 8) : lpr;
  const long per_row = (long)(slot_bytes / R) - 64;
  if (per_row <= 0) return false;
  const long by_bytes = sb ? per_row / block_bytes(t) * 8 : per_row / units_bytes(t, 1);
  int chunk = (int)std::min<long>(by_bytes, units);
  if (chunk < units && chunk >= step) chunk = chunk / step * step;
  if (sb) chunk = chunk / 8 * 8;
  if (chunk <= 0) return false;
  out->chunk = chunk;
  out->pitch = piece_pitch(units_bytes(t, chunk));
  return true;
}

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
  constexpr int Gn = 32 / LPR, R_R = kMoeNW * Gn * 4, R_S = kMoeNW * Gn * 2;
  const int U = p.dim / 32;
  const size_t fixed = ((sizeof(MoeSmemHead) + 127) & ~(size_t)127) + lut_bytes_for(TR) + (size_t)U * 76 + 128;
  for (int stages = kMaxStages; stages >= 2; stages--) {
    const size_t slot = std::min<size_t>(((size_t)kSmemLimit - fixed) / stages, 48 * 1024) & ~(size_t)127;
    if (!shape_for(TR, U, R_R, LPR, slot, &p.gu_routed) || !shape_for(TS, U, R_S, LPR, slot, &p.gu_shared)) continue;
    p.stages = stages;
    p.stage_bytes = (uint32_t)slot;
    auto kern = moe_gu_kernel<TR, TS, LPR>;
    static bool done[64] = {};
    int rc = set_smem(kern, dev, done);
    if (rc) return rc;
    const int tiles = (p.gu_s ? (p.inter + R_S - 1) / R_S : 0) + (p.gu_r ? p.n_routed : 0) * ((p.inter + R_R - 1) / R_R);
    const int grid = std::max(1, std::min(sms, tiles));
    kern<<<grid, (kMoeNW + 1) * 32, fixed + (size_t)stages * slot, st>>>(p);
    MSB_LAUNCH_CHECK("moe_gu_kernel");
    return kOk;
  }
  return fail(kErrLimit, "moe_decode: gate/up staging does not fit (dim %d)", p.dim);
}

template <int TR, int TS, int LPR>
int launch_down(MoeParams& p, int sms, int dev, cudaStream_t st) {
  constexpr int Gn = 32 / LPR, R = kMoeNW * Gn;
  const int Ui = p.inter / 32, U = (p.n_routed + 1) * Ui;
  const size_t fixed = ((sizeof(MoeSmemHead) + 127) & ~(size_t)127) + lut_bytes_for(TR) + (size_t)U * 76 + 128;
  for (int stages = kMaxStages; stages >= 2; stages--) {
    if (fixed + 8192 > (size_t)kSmemLimit) break;
    const size_t slot = std::min<size_t>(((size_t)kSmemLimit - fixed) / stages, 48 * 1024) & ~(size_t)127;
    if (!shape_for(TR, Ui, R, LPR, slot, &p.d_routed) || !shape_for(TS, Ui, R, LPR, slot, &p.d_shared)) continue;
    p.stages = stages;
    p.stage_bytes = (uint32_t)slot;
    auto kern = moe_down_kernel<TR, TS, LPR>;
    static bool done[64] = {};
    int rc = set_smem(kern, dev, done);
    if (rc) return rc;
    const int tiles = (p.dim + R - 1) / R;
    kern<<<std::max(1, std::min(sms, tiles)), (kMoeNW + 1) * 32, fixed + (size_t)stages * slot, st>>>(p);
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
  if (!p.gu_r && !p.gu_s && !p.d_r && !p.d_s) return kOk;
  if (!p.x || !p.y || !p.h || (p.gu_r && !p.weights)) return fail(kErrArg, "moe_decode: null pointer");
  int rc = get_tables(&p.tb);
  if (rc) return rc;
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int lpr_gu = lpr_for(p.dim / 32), lpr_d = lpr_for(p.inter / 32);
  if (!lpr_gu || !lpr_d) return fail(kErrArg, "moe_decode: dim/inter not supported");
  unsigned* sched_base = reinterpret_cast<unsigned*>(p.tb.status) + 8;
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
    p.sched = sched_base + 2;
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
