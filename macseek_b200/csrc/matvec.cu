// Decode matvec family: y[n][rows] (+)= X[n][cols (* groups)] . W^T with W as raw GGUF block rows.
// Replaces the reference's q_mv / q_mvn Metal kernels (src/kernels/quant_mv.metal:7-39,148-202) behind
// ms::q::encode_matvec / encode_matvec_n (src/kernels/quant.hpp:27-35, quant.mm:70-95,129-156).
//
// Layout of the work: persistent blocks (16 consumer warps + 1 TMA producer warp); block b of group g walks row tiles
// b, b + blocks_per_group, ... of that group.  A row tile is R = NW * (32 / LPR) * NR rows; each tile is streamed in K chunks through the TMA ring
// (stream_pipe.cuh).  LPR lanes split the units of a row, partial sums are combined with warp shuffles in a fixed
// order, so a row's result does not depend on the launch shape of other rows.
#include <algorithm>
#include <cstdlib>
#include "stream_pipe.cuh"

namespace msb {

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
  int chunk_units;              // units per staged piece
  int blocks_per_group;
  int tiles_per_group;
  int stages;
  uint32_t pitch;
  uint32_t stage_bytes;
  Tables tb;
};

struct MvSmemHead {
  uint64_t full[kMaxStages], empty[kMaxStages];
  uint64_t lutbar;
  int abort_flag;
  const uint8_t* src[1];
  float red[32];
};

template <int T, int LPR, int NR, int NC, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, 1) matvec_kernel(const MvParams p) {
  constexpr int G = 32 / LPR;
  constexpr int R = NW * G * NR;
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
  for (int c = 0; c < NC; c++) { xq_bind(xq[c], cur, U, is_dense(T)); cur += xq_bytes(U, is_dense(T)); }
  cur = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(cur) + 127) & ~(uintptr_t)127);
  ring.slot0 = cur; ring.slot_bytes = p.stage_bytes;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = blockIdx.x / p.blocks_per_group, slot = blockIdx.x % p.blocks_per_group;
  ring_init(ring, tid, NW);
  if (tid == 0) { mbar_init(&hd->lutbar, 1); mbar_fence_init(); hd->src[0] = nullptr; }
  __syncthreads();
  LaneLuts L;
  const bool luts_ok = load_luts(lut, T == IQ1_S, T == IQ2_XXS, T == IQ4_NL, p.tb, tid, &hd->lutbar, &hd->abort_flag, L, lane);
  // activation of this block's group -> shared (fixed point, or fp32 for dense weights), optionally RMS-normalised
#pragma unroll
  for (int c = 0; c < NC; c++) {
    const float* xg = p.x + (size_t)c * p.x_stride + (size_t)group * p.cols;
    float mul = 1.f;
    if (p.norm_w) {
      float ss = 0.f;
      for (int i = tid; i < p.cols / 4; i += blockDim.x) {
        const float4 v = reinterpret_cast<const float4*>(xg)[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = warp_sum(ss);
      if (lane == 0) hd->red[warp] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < NW + 1; w++) tot += hd->red[w];
      __syncthreads();
      mul = rsqrtf(tot / (float)p.cols + p.norm_eps);
    }
    if (is_dense(T)) {
      float4* d = reinterpret_cast<float4*>(const_cast<float*>(xq[c].xf));
      for (int i = tid; i < U * 8; i += blockDim.x) {
        float4 v = reinterpret_cast<const float4*>(xg)[i];
        if (p.norm_w) {
          const float4 gw = reinterpret_cast<const float4*>(p.norm_w)[i];
          v.x = v.x * mul * gw.x; v.y = v.y * mul * gw.y; v.z = v.z * mul * gw.z; v.w = v.w * mul * gw.w;
        }
        d[i] = v;
      }
    } else {
      quantize_x(xg, xq[c], tid, blockDim.x, mul, p.norm_w);
    }
  }
  __syncthreads();
  if (!luts_ok) return;

  const int nchunks = (U + p.chunk_units - 1) / p.chunk_units;
  const uint8_t* Wg = p.W + (size_t)group * p.rows_per_group * p.row_bytes;
  uint32_t n = 0;
  if (warp == NW) {
    // ---------------- producer warp
    const uint8_t* srcv[1];
    Piece pc;
    pc.src = srcv; pc.nsrc = 1; pc.rows_per_src = R; pc.row_stride = p.row_bytes;
    for (int t = slot; t < p.tiles_per_group; t += p.blocks_per_group) {
      const int r0 = t * R;
      pc.nrows = min(R, p.rows_per_group - r0);
      for (int c = 0; c < nchunks; c++, n++) {
        const int u0 = c * p.chunk_units, nu = min(p.chunk_units, U - u0);
        srcv[0] = Wg + (size_t)r0 * p.row_bytes + units_bytes(T, u0);
        pc.bytes = units_bytes(T, nu);
        if (!produce_piece(ring, n, pc, p.pitch, lane)) return;
      }
    }
    return;
  }
  // ---------------- consumer warps
  const int grp = lane / LPR, li = lane % LPR;
  const int lr0 = (warp * G + grp) * NR;
  for (int t = slot; t < p.tiles_per_group; t += p.blocks_per_group) {
    const int r0 = t * R;
    float acc[NR][NC];
#pragma unroll
    for (int i = 0; i < NR; i++)
#pragma unroll
      for (int c = 0; c < NC; c++) acc[i][c] = 0.f;
    for (int c = 0; c < nchunks; c++, n++) {
      const int u0 = c * p.chunk_units, nu = min(p.chunk_units, U - u0);
      const uintptr_t a0 = reinterpret_cast<uintptr_t>(Wg) + (size_t)r0 * p.row_bytes + units_bytes(T, u0);
      const saddr_t slot_s = smem_u32(ring.slot(n));
      saddr_t rowp[NR];
#pragma unroll
      for (int i = 0; i < NR; i++)
        rowp[i] = slot_s + (uint32_t)(lr0 + i) * p.pitch + (uint32_t)((a0 + (uintptr_t)(lr0 + i) * p.row_bytes) & 15u);
      if (!consumer_wait(ring, n)) return;
      consume_rows<T, LPR, NR, NC>(rowp, li, xq, u0, nu, L, acc);
      consumer_release(ring, n, lane);
    }
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

// ---------------------------------------------------------------- host side
namespace {
constexpr int kNW = 16;

// lanes per row: the largest of 32/16/8 that wastes the fewest lane iterations on this row length
int pick_lpr(int units) {
  int best = 32;
  double best_eff = 0;
  for (int lpr : {32, 16, 8}) {
    const int iters = (units + lpr - 1) / lpr;
    const double eff = (double)units / (iters * lpr);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = lpr; }
  }
  return best;
}

template <int T, int LPR, int NR, int NC>
int launch_cfg(MvParams& p, cudaStream_t st, int dev, int sms) {
  constexpr int G = 32 / LPR, R = kNW * G * NR;
  const size_t fixed = ((sizeof(MvSmemHead) + 127) & ~(size_t)127) + lut_bytes_for(T) + (size_t)NC * xq_bytes(p.units, is_dense(T)) + 128;
  if (fixed + 2 * 4096 > (size_t)kSmemLimit)
    return fail(kErrLimit, "matvec: cols %d x n %d does not fit in shared memory", p.cols, p.n);
  int stages = kMaxStages, chunk = 0;
  size_t slot_bytes = 0;
  static const int env_chunk = getenv("MSB_MV_CHUNK") ? atoi(getenv("MSB_MV_CHUNK")) : 0;   // tuning probes
  static const int env_stages = getenv("MSB_MV_STAGES") ? atoi(getenv("MSB_MV_STAGES")) : 0;
  for (stages = env_stages ? env_stages : kMaxStages; stages >= 2; stages--) {
    slot_bytes = std::min<size_t>(((size_t)kSmemLimit - fixed) / stages, env_chunk ? 200 * 1024 : 48 * 1024) & ~(size_t)127;
    chunk = chunk_units_for(T, p.units, R, LPR, slot_bytes);
    if (env_chunk && chunk > env_chunk) chunk = env_chunk;
    if (chunk > 0) break;
  }
  if (chunk <= 0) return fail(kErrLimit, "matvec: no staging shape fits (type %s cols %d)", type_name(T), p.cols);
  p.chunk_units = chunk;
  p.stages = stages;
  p.pitch = piece_pitch(units_bytes(T, chunk));
  p.stage_bytes = (uint32_t)slot_bytes;
  p.tiles_per_group = (p.rows_per_group + R - 1) / R;
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

// rows per lane group: as many as the type's decode cost warrants (they share the activation registers), but few
// enough that the matrix still spreads over every SM
template <int T, int LPR, int NC>
int launch_rows(MvParams& p, cudaStream_t st, int dev, int sms) {
  constexpr int G = 32 / LPR;
  constexpr int kMaxNR = (T == IQ1_S || T == IQ2_XXS) ? 4 : 2;
  const int want_tiles = 2 * sms / p.groups;
  int nr = NC > 1 ? std::min(kMaxNR, 2) : kMaxNR;
  while (nr > 1 && (p.rows_per_group + kNW * G * nr - 1) / (kNW * G * nr) < want_tiles) nr >>= 1;
  if (T == F32) nr = 1;
  static const int env_nr = getenv("MSB_MV_NR") ? atoi(getenv("MSB_MV_NR")) : 0;
  if (env_nr) nr = env_nr;
  if (nr >= 4) {
    if constexpr (kMaxNR >= 4 && NC == 1) return launch_cfg<T, LPR, 4, NC>(p, st, dev, sms);
  }
  if (nr >= 2) return launch_cfg<T, LPR, 2, NC>(p, st, dev, sms);
  return launch_cfg<T, LPR, 1, NC>(p, st, dev, sms);
}

template <int T, int NC>
int launch_type(MvParams& p, cudaStream_t st, int dev, int sms) {
  switch (pick_lpr(p.units)) {
    case 32: return launch_rows<T, 32, NC>(p, st, dev, sms);
    case 16: return launch_rows<T, 16, NC>(p, st, dev, sms);
    default: return launch_rows<T, 8, NC>(p, st, dev, sms);
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
             int n, int accumulate, int groups, const float* norm_w, float norm_eps, cudaStream_t st) {
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
  for (int c0 = 0; c0 < n;) {
    const int left = n - c0;
    p.x = X + (size_t)c0 * x_stride;
    p.y = Y + (size_t)c0 * y_stride;
    if (left >= 4) { p.n = 4; rc = launch_cols<4>(t, p, st, dev, sms); c0 += 4; }
    else if (left >= 2) { p.n = 2; rc = launch_cols<2>(t, p, st, dev, sms); c0 += 2; }
    else { p.n = 1; rc = launch_cols<1>(t, p, st, dev, sms); c0 += 1; }
    if (rc) return rc;
  }
  return kOk;
}

}  // namespace msb
