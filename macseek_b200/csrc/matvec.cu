// Decode matvec family: y[n][rows] (+)= X[n][cols (* groups)] . W^T with W as raw GGUF block rows.
// Replaces the reference's q_mv / q_mvn Metal kernels (src/kernels/quant_mv.metal:7-39,148-202) behind
// ms::q::encode_matvec / encode_matvec_n (src/kernels/quant.hpp:27-35, quant.mm:70-95,129-156).
//
// Layout of the work: persistent blocks; block b of group g walks row tiles b, b + blocks_per_group, ... of that
// group.  A row tile is R = NW * (32 / LPR) * NR rows; each tile is streamed in K chunks through the TMA ring
// (stream_pipe.cuh).  LPR lanes split the units of a row, partial sums are combined with warp shuffles in a fixed
// order, so a row's result does not depend on the launch shape of other rows.
#include <algorithm>
#include "stream_pipe.cuh"

namespace msb {

struct MvParams {
  const uint8_t* W;
  const float* x;
  float* y;
  int rows, cols, n;            // n activation columns
  int rows_per_group, groups;
  int64_t x_stride, y_stride;   // elements between activation columns / output columns
  uint32_t row_bytes;
  int accumulate;
  int units;                    // cols / 32
  int chunk_units;              // units per staged piece
  int blocks_per_group;
  int tiles_per_group;
  int stages;
  uint32_t pitch;
  uint32_t stage_bytes;
  Tables tb;
};

template <int T, int LPR, int NR, int NC, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, 1) matvec_kernel(const MvParams p) {
  constexpr int G = 32 / LPR;
  constexpr int R = NW * G * NR;
  extern __shared__ __align__(128) uint8_t smem[];
  // [barriers 128 B][luts][xq columns][ring slots]
  Ring ring;
  ring.full = reinterpret_cast<uint64_t*>(smem);
  ring.empty = ring.full + kMaxStages;
  ring.abort_flag = reinterpret_cast<volatile int*>(smem + 64);
  ring.status = p.tb.status;
  ring.stages = p.stages;
  uint8_t* cur = smem + 128;
  uint8_t* lut = cur;
  cur += lut_bytes_for(T);
  XqSmem xq[NC];
  const int U = p.units;
#pragma unroll
  for (int c = 0; c < NC; c++) {
    xq[c].U = U;
    if (is_dense(T)) {
      xq[c].xf = reinterpret_cast<const float*>(cur);
      xq[c].plane = nullptr; xq[c].scale = nullptr; xq[c].sumA = xq[c].sumB = nullptr;
      cur += (size_t)U * 128;
    } else {
      xq[c].plane = reinterpret_cast<uint4*>(cur);
      xq[c].scale = reinterpret_cast<float*>(cur + (size_t)U * 64);
      xq[c].sumA = reinterpret_cast<int*>(cur + (size_t)U * 68);
      xq[c].sumB = reinterpret_cast<int*>(cur + (size_t)U * 72);
      xq[c].xf = nullptr;
      cur += (size_t)U * 76;
    }
  }
  cur = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(cur) + 127) & ~(uintptr_t)127);
  for (int s = 0; s < kMaxStages; s++) ring.slot[s] = cur + (size_t)s * p.stage_bytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = blockIdx.x / p.blocks_per_group, slot = blockIdx.x % p.blocks_per_group;
  ring_init(ring, tid, NW);
  LaneLuts L;
  fill_luts(lut, T == IQ1_S, T == IQ2_XXS, T == IQ4_NL, p.tb, tid, blockDim.x, L, lane);
  // activation of this block's group -> shared (fixed point, or fp32 for dense weights)
#pragma unroll
  for (int c = 0; c < NC; c++) {
    const float* xg = p.x + (size_t)c * p.x_stride + (size_t)group * p.cols;
    if (is_dense(T)) {
      float4* d = reinterpret_cast<float4*>(const_cast<float*>(xq[c].xf));
      for (int i = tid; i < U * 8; i += blockDim.x) d[i] = reinterpret_cast<const float4*>(xg)[i];
    } else {
      quantize_x(xg, xq[c], tid, blockDim.x);
    }
  }
  __syncthreads();

  const int nchunks = (U + p.chunk_units - 1) / p.chunk_units;
  const uint8_t* Wg = p.W + (size_t)group * p.rows_per_group * p.row_bytes;
  uint32_t n = 0;
  if (warp == NW) {
    // ---------------- producer warp
    for (int t = slot; t < p.tiles_per_group; t += p.blocks_per_group) {
      const int r0 = t * R;
      for (int c = 0; c < nchunks; c++, n++) {
        const int u0 = c * p.chunk_units, nu = min(p.chunk_units, U - u0);
        Piece pc;
        pc.src = Wg + (size_t)r0 * p.row_bytes + units_bytes(T, u0);
        pc.row_stride = p.row_bytes;
        pc.bytes = units_bytes(T, nu);
        pc.nrows = min(R, p.rows_per_group - r0);
        if (!produce_piece(ring, n, pc, p.pitch, lane)) return;
      }
    }
    return;
  }
  // ---------------- consumer warps
  const int grp = lane / LPR, li = lane % LPR;
  for (int t = slot; t < p.tiles_per_group; t += p.blocks_per_group) {
    const int r0 = t * R;
    float acc[NR][NC];
#pragma unroll
    for (int i = 0; i < NR; i++)
#pragma unroll
      for (int c = 0; c < NC; c++) acc[i][c] = 0.f;
    for (int c = 0; c < nchunks; c++, n++) {
      const int u0 = c * p.chunk_units, nu = min(p.chunk_units, U - u0);
      Piece pc;
      pc.src = Wg + (size_t)r0 * p.row_bytes + units_bytes(T, u0);
      pc.row_stride = p.row_bytes;
      pc.bytes = units_bytes(T, nu);
      pc.nrows = min(R, p.rows_per_group - r0);
      if (!consumer_wait(ring, n)) return;
      consume_piece<T, LPR, NR, NC>(ring, n, pc, p.pitch, warp * G * NR, lane, xq, u0, nu, L, acc);
      consumer_release(ring, n, lane);
    }
#pragma unroll
    for (int i = 0; i < NR; i++) {
      const int lr = (warp * G + grp) * NR + i;
#pragma unroll
      for (int c = 0; c < NC; c++) {
        const float v = group_sum<LPR>(acc[i][c]);
        if (li == 0 && r0 + lr < p.rows_per_group) {
          float* yp = p.y + (size_t)c * p.y_stride + (size_t)group * p.rows_per_group + r0 + lr;
          *yp = p.accumulate ? *yp + v : v;
        }
      }
    }
  }
}

// ---------------------------------------------------------------- host side
namespace {
constexpr int kNW = 8;

struct Shape { int lpr, nr; };

// lanes per row: the largest of 32/16/8 that wastes the fewest lane iterations on this row length
int pick_lpr(int units, bool superblock) {
  int best = 32;
  double best_eff = 0;
  for (int lpr : {32, 16, 8}) {
    if (superblock && lpr < 8) continue;
    const int iters = (units + lpr - 1) / lpr;
    const double eff = (double)units / (iters * lpr);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = lpr; }
  }
  return best;
}

template <int T, int LPR, int NR, int NC>
int launch_cfg(MvParams& p, cudaStream_t st) {
  constexpr int G = 32 / LPR, R = kNW * G * NR;
  const bool sb = block_elems(T) == 256;
  const size_t fixed = 128 + lut_bytes_for(T) + (size_t)NC * xq_bytes(p.units, is_dense(T)) + 128;
  if (fixed + 2 * 4096 > (size_t)kSmemLimit)
    return fail(kErrLimit, "matvec: cols %d x n %d does not fit in shared memory", p.cols, p.n);
  // chunk: as many units per staged piece as fit in a slot, a multiple of the lane stride (and of a super-block)
  const int step = sb ? std::max(LPR, 8) : LPR;
  int stages = kMaxStages, chunk = 0;
  size_t slot_bytes = 0;
  for (; stages >= 2; stages--) {
    slot_bytes = std::min<size_t>(((size_t)kSmemLimit - fixed) / stages, 48 * 1024) & ~(size_t)127;
    const long per_row = (long)(slot_bytes / R) - 64;          // piece_pitch(b) <= b + 62
    if (per_row <= 0) continue;
    const long by_bytes = sb ? per_row / block_bytes(T) * 8 : per_row / units_bytes(T, 1);
    chunk = (int)std::min<long>(by_bytes, p.units);
    if (chunk < p.units && chunk >= step) chunk = chunk / step * step;   // else: a short chunk, some lanes idle
    if (sb) chunk = chunk / 8 * 8;
    if (chunk > 0) break;
  }
  if (chunk <= 0) return fail(kErrLimit, "matvec: no staging shape fits (type %s cols %d)", type_name(T), p.cols);
  p.chunk_units = chunk;
  p.stages = stages;
  p.pitch = piece_pitch(units_bytes(T, chunk));
  p.stage_bytes = (uint32_t)slot_bytes;
  p.tiles_per_group = (p.rows_per_group + R - 1) / R;
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  p.blocks_per_group = std::max(1, std::min(p.tiles_per_group, sms / p.groups));
  const size_t smem = fixed + (size_t)stages * slot_bytes;
  auto kern = matvec_kernel<T, LPR, NR, NC, kNW>;
  static bool configured[64] = {};
  if (!configured[dev & 63]) {
    MSB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    configured[dev & 63] = true;
  }
  kern<<<p.blocks_per_group * p.groups, (kNW + 1) * 32, smem, st>>>(p);
  MSB_LAUNCH_CHECK("matvec_kernel");
  return kOk;
}

template <int T, int NC>
int launch_type(MvParams& p, cudaStream_t st) {
  const int lpr = pick_lpr(p.units, block_elems(T) == 256);
  constexpr int NR = (T == IQ1_S || T == IQ2_XXS) ? 4 : T == F32 ? 1 : 2;
  constexpr int NRn = NC > 1 ? (NR > 2 ? 2 : NR) : NR;   // fewer rows in flight when several columns share a decode
  switch (lpr) {   // fewer rows per lane group when more groups share a warp: the row tile stays ~32 rows
    case 32: return launch_cfg<T, 32, NRn, NC>(p, st);
    case 16: return launch_cfg<T, 16, (NRn > 1 ? NRn / 2 : 1), NC>(p, st);
    default: return launch_cfg<T, 8, (NRn > 2 ? NRn / 4 : 1), NC>(p, st);
  }
}

template <int NC>
int launch_cols(int t, MvParams& p, cudaStream_t st) {
  switch (t) {
    case F32: return launch_type<F32, NC>(p, st);
    case F16: return launch_type<F16, NC>(p, st);
    case BF16: return launch_type<BF16, NC>(p, st);
    case Q8_0: return launch_type<Q8_0, NC>(p, st);
    case Q5_K: return launch_type<Q5_K, NC>(p, st);
    case Q6_K: return launch_type<Q6_K, NC>(p, st);
    case IQ2_XXS: return launch_type<IQ2_XXS, NC>(p, st);
    case IQ1_S: return launch_type<IQ1_S, NC>(p, st);
    case IQ4_NL: return launch_type<IQ4_NL, NC>(p, st);
  }
  return fail(kErrType, "matvec: unsupported weight type %d", t);
}
}  // namespace

// Y[n x rows] (+)= X[n x cols*groups] . W^T.  n columns are processed four (then two, then one) at a time; each pass
// streams W once.
int matvec_n(int t, const void* W, int rows, int cols, const float* X, int64_t x_stride, float* Y, int64_t y_stride,
             int n, int accumulate, int groups, cudaStream_t st) {
  if (!type_known(t)) return fail(kErrType, "matvec: unsupported weight type %d", t);
  const int qk = block_elems(t) == 1 ? 32 : block_elems(t);
  if (rows <= 0 || cols <= 0 || n <= 0 || groups < 1 || rows % groups != 0 || cols % qk != 0 || cols % 32 != 0)
    return fail(kErrArg, "matvec: bad shape (type %s rows %d cols %d n %d groups %d)", type_name(t), rows, cols, n, groups);
  if (!W || !X || !Y) return fail(kErrArg, "matvec: null pointer");
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 1) || ((x_stride * 4) & 15))
    return fail(kErrArg, "matvec: activations must be 16-byte aligned, weights 2-byte aligned");
  MvParams p{};
  MSB_CUDA(cudaGetLastError());
  int rc = get_tables(&p.tb);
  if (rc) return rc;
  p.W = (const uint8_t*)W;
  p.rows = rows; p.cols = cols;
  p.rows_per_group = rows / groups; p.groups = groups;
  p.x_stride = x_stride; p.y_stride = y_stride;
  p.row_bytes = (uint32_t)row_bytes(t, cols);
  p.accumulate = accumulate;
  p.units = cols / 32;
  for (int c0 = 0; c0 < n;) {
    const int left = n - c0;
    p.x = X + (size_t)c0 * x_stride;
    p.y = Y + (size_t)c0 * y_stride;
    if (left >= 4) { p.n = 4; rc = launch_cols<4>(t, p, st); c0 += 4; }
    else if (left >= 2) { p.n = 2; rc = launch_cols<2>(t, p, st); c0 += 2; }
    else { p.n = 1; rc = launch_cols<1>(t, p, st); c0 += 1; }
    if (rc) return rc;
  }
  return kOk;
}

}  // namespace msb
