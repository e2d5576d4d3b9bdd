// Sparse attention, decode: one query token, 64 heads, K == V rows gathered from the window ring and from the
// compressed KV cache by the indexer's top-k list.
//   logits = rope(q_h) . row * D^-0.5 ; softmax with the per-head sink logit in the denominator only ;
//   out_h = sum_r p_r row_r ; inverse rope on the last 64 dims of out   (math spec: tests/ref/attn_ref.cpp:204-230)
// Replaces the reference's attn_sparse_h8/h16 + attn_sparse_combine Metal kernels (src/kernels/attn_sparse.metal:
// 21-288) behind ms::attn::encode_sparse (src/kernels/attn.hpp:128-129, attn.mm:419-445).
//
// Split-K flash decoding on mma.sync m16n8k16 (f16 or bf16 rows, fp32 accumulation): block (head group of 16, row
// split); 4 warps share the 32-row tile staged in shared memory with cp.async gathers.  Each warp contracts a quarter
// of D for Q.K^T (partials summed through shared memory in a fixed order) and owns a quarter of D of the output.
// q and the probabilities are fed as two terms (hi + lo) of the row element type, so no operand precision is lost.
#include <algorithm>
#include "msb_common.cuh"

namespace msb {

constexpr int kSaRows = 32;      // rows per tile
constexpr int kSaHeadsPerBlock = 16;

struct SparseParams {
  const float* q;        // [H][D] pre-rope
  const float* cs;       // [32][2] (cos, sin) of the query position
  const float* sinks;    // [H]
  const uint8_t* win;    // [n_win][D] elements
  const uint8_t* cache;  // [cap][D] elements
  const int* topk;       // [k] row indices into cache, -1 = none
  float* part_o;         // [splits][H][D]
  float* part_ml;        // [splits][H][2]
  float* out;            // [H][D]
  int n_win, k, H, splits, rows_per_split;
};

template <bool BF>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (BF) { __nv_bfloat162 v = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&v); }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <bool BF>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if (BF) return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
// hi = E(a, b), lo = E(a - hi.a, b - hi.b)
template <bool BF>
__device__ __forceinline__ void split2(float a, float b, uint32_t& hi, uint32_t& lo) {
  hi = pack2<BF>(a, b);
  const float2 h = unpack2<BF>(hi);
  lo = pack2<BF>(a - h.x, b - h.y);
}
template <bool BF>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D, bool BF>
__global__ void __launch_bounds__(128, 1) sparse_partial_kernel(const SparseParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int KS = D / 64;            // k-steps of 16 dims per warp (each warp contracts D / 4 dims)
  constexpr int NTW = D / 32;           // 8-wide output tiles per warp (each warp owns D / 4 output dims)
  constexpr int PITCH = D * 2 + 16;     // bytes per staged row (+16: rows start on different bank groups)
  constexpr int CH = D * 2 / 16;        // 16-byte chunks per row
  constexpr int NT = kSaRows / 8;       // score tiles per row tile
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* rows[2] = {smem, smem + kSaRows * PITCH};
  float* spart = reinterpret_cast<float*>(smem + 2 * kSaRows * PITCH);   // [4 warps][NT][32 lanes][4]
  int* rowvalid = reinterpret_cast<int*>(spart + 4 * NT * 32 * 4);       // [2][kSaRows]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int hg = blockIdx.x, split = blockIdx.y;
  const int total = p.n_win + p.k;
  const int v0 = split * p.rows_per_split, v1 = min(total, v0 + p.rows_per_split);
  const int nit = v1 > v0 ? (v1 - v0 + kSaRows - 1) / kSaRows : 0;
  const int kbase = 16 * KS * warp;     // first contracted dim of this warp == first output dim of this warp

  // four threads per row: the row's source is resolved once per thread (one dependent load, all rows in parallel),
  // then the thread copies every fourth 16-byte chunk of it
  auto gather = [&](int it, int buf) {
    const int r = tid >> 2, v = v0 + it * kSaRows + r;
    const uint8_t* src = nullptr;
    if (v < v1) {
      if (v < p.n_win) src = p.win + (size_t)v * D * 2;
      else {
        const int idx = __ldg(p.topk + (v - p.n_win));
        if (idx >= 0) src = p.cache + (size_t)idx * D * 2;
      }
    }
    uint8_t* dst = rows[buf] + r * PITCH;
#pragma unroll
    for (int c = tid & 3; c < CH; c += 4) {
      if (src) cp_async16(smem_u32(dst + c * 16), src + c * 16);
      else *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(0, 0, 0, 0);
    }
    if ((tid & 3) == 0) rowvalid[buf * kSaRows + r] = src != nullptr;
    cp_async_commit();
  };

  // ---- query fragments for this warp's contraction range, roped, as hi + lo terms.  The 16 heads' queries pass
  // through the (still unused) second row buffer with coalesced 16-byte loads.  Every independent global read of the
  // prologue is requested before the first dependent one: the queries and the rope factors first, then the first
  // tile's rows (whose addresses wait for the selected indices), so that one round trip covers them all.
  constexpr int kQ4 = kSaHeadsPerBlock * D / 4 / 128;   // 16-byte pieces per thread (16 or 18)
  static_assert(kSaHeadsPerBlock * D / 4 % 128 == 0, "query staging assumes a whole number of pieces per thread");
  float4 qv[kQ4];
  {
    const float4* src = reinterpret_cast<const float4*>(p.q + (size_t)hg * kSaHeadsPerBlock * D);
#pragma unroll
    for (int i = 0; i < kQ4; i++) qv[i] = src[tid + 128 * i];
  }
  float rc[KS][2], rs[KS][2];     // cos / sin of the rope pair this lane holds at (k-step s, half j); (1, 0) outside
#pragma unroll
  for (int s = 0; s < KS; s++)
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const int d = kbase + 16 * s + 8 * j + 2 * t;
      const bool roped = d >= D - 64;
      rc[s][j] = roped ? p.cs[d - (D - 64)] : 1.f;
      rs[s][j] = roped ? p.cs[d - (D - 64) + 1] : 0.f;
    }
  if (nit > 0) gather(0, 0);
  {
    float4* qs4 = reinterpret_cast<float4*>(rows[1]);
#pragma unroll
    for (int i = 0; i < kQ4; i++) qs4[tid + 128 * i] = qv[i];
  }
  __syncthreads();
  uint32_t qh[KS][4], ql[KS][4];
  {
    const float* qs = reinterpret_cast<const float*>(rows[1]);
#pragma unroll
    for (int s = 0; s < KS; s++)
#pragma unroll
      for (int j = 0; j < 2; j++)
#pragma unroll
        for (int r = 0; r < 2; r++) {
          const int d = kbase + 16 * s + 8 * j + 2 * t;
          const float2 v = *reinterpret_cast<const float2*>(qs + (g + 8 * r) * D + d);
          float a = v.x, b = v.y;
          if (d >= D - 64) {
            const float c = rc[s][j], sn = rs[s][j];
            const float ra = a * c - b * sn, rb = a * sn + b * c;
            a = ra; b = rb;
          }
          split2<BF>(a, b, qh[s][j * 2 + r], ql[s][j * 2 + r]);
        }
  }
  __syncthreads();   // the second row buffer is free again

  float o[NTW][4];
#pragma unroll
  for (int i = 0; i < NTW; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const float scale = 1.0f / sqrtf((float)D);

  for (int it = 0; it < nit; it++) {
    const int buf = it & 1;
    if (it + 1 < nit) { gather(it + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const uint32_t rbase = smem_u32(rows[buf]);
    // ---- partial scores over this warp's dims: S[16 heads x 32 rows]
    float sp[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      sp[nt][0] = sp[nt][1] = sp[nt][2] = sp[nt][3] = 0.f;
      const uint32_t rowaddr = rbase + (nt * 8 + (lane & 7)) * PITCH + (kbase + 8 * (lane >> 3)) * 2;
#pragma unroll
      for (int s = 0; s + 1 < KS; s += 2) {
        uint32_t b[4];
        ldsm_x4(b, rowaddr + 32 * s);
        mma16816<BF>(sp[nt], qh[s], b[0], b[1]);
        mma16816<BF>(sp[nt], ql[s], b[0], b[1]);
        mma16816<BF>(sp[nt], qh[s + 1], b[2], b[3]);
        mma16816<BF>(sp[nt], ql[s + 1], b[2], b[3]);
      }
      if (KS & 1) {
        uint32_t b[2];
        ldsm_x2(b, rbase + (nt * 8 + (lane & 7)) * PITCH + (kbase + 16 * (KS - 1) + 8 * ((lane >> 3) & 1)) * 2);
        mma16816<BF>(sp[nt], qh[KS - 1], b[0], b[1]);
        mma16816<BF>(sp[nt], ql[KS - 1], b[0], b[1]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
      *reinterpret_cast<float4*>(spart + ((warp * NT + nt) * 32 + lane) * 4) = make_float4(sp[nt][0], sp[nt][1], sp[nt][2], sp[nt][3]);
    __syncthreads();
    // ---- full scores (same summation order in every warp), masking, online softmax
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      float4 a = *reinterpret_cast<const float4*>(spart + ((0 * NT + nt) * 32 + lane) * 4);
#pragma unroll
      for (int w = 1; w < 4; w++) {
        const float4 b = *reinterpret_cast<const float4*>(spart + ((w * NT + nt) * 32 + lane) * 4);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      const bool va = rowvalid[buf * kSaRows + nt * 8 + 2 * t] != 0, vb = rowvalid[buf * kSaRows + nt * 8 + 2 * t + 1] != 0;
      sp[nt][0] = va ? a.x * scale : -INFINITY; sp[nt][1] = vb ? a.y * scale : -INFINITY;
      sp[nt][2] = va ? a.z * scale : -INFINITY; sp[nt][3] = vb ? a.w * scale : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(sp[nt][0], sp[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(sp[nt][2], sp[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float f0 = (n0 == -INFINITY) ? 1.f : expf(m0 - n0), f1 = (n1 == -INFINITY) ? 1.f : expf(m1 - n1);
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      sp[nt][0] = sp[nt][0] == -INFINITY ? 0.f : expf(sp[nt][0] - n0);
      sp[nt][1] = sp[nt][1] == -INFINITY ? 0.f : expf(sp[nt][1] - n0);
      sp[nt][2] = sp[nt][2] == -INFINITY ? 0.f : expf(sp[nt][2] - n1);
      sp[nt][3] = sp[nt][3] == -INFINITY ? 0.f : expf(sp[nt][3] - n1);
      sum0 += sp[nt][0] + sp[nt][1];
      sum1 += sp[nt][2] + sp[nt][3];
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * f0 + sum0; l1 = l1 * f1 + sum1;
    m0 = n0; m1 = n1;
#pragma unroll
    for (int i = 0; i < NTW; i++) { o[i][0] *= f0; o[i][1] *= f0; o[i][2] *= f1; o[i][3] *= f1; }
    // ---- O += P . V over this warp's output dims
#pragma unroll
    for (int j = 0; j < kSaRows / 16; j++) {
      uint32_t ph[4], pl[4];
      split2<BF>(sp[2 * j][0], sp[2 * j][1], ph[0], pl[0]);
      split2<BF>(sp[2 * j][2], sp[2 * j][3], ph[1], pl[1]);
      split2<BF>(sp[2 * j + 1][0], sp[2 * j + 1][1], ph[2], pl[2]);
      split2<BF>(sp[2 * j + 1][2], sp[2 * j + 1][3], ph[3], pl[3]);
      // matrices of one x4.trans: (rows 0-7, tile i), (rows 8-15, tile i), (rows 0-7, tile i+1), (rows 8-15, tile i+1)
      const uint32_t vaddr = rbase + (16 * j + 8 * ((lane >> 3) & 1) + (lane & 7)) * PITCH + (kbase + 8 * (lane >> 4)) * 2;
#pragma unroll
      for (int i = 0; i < NTW; i += 2) {
        uint32_t b[4];
        ldsm_x4_t(b, vaddr + 32 * (i / 2));
        mma16816<BF>(o[i], ph, b[0], b[1]);
        mma16816<BF>(o[i], pl, b[0], b[1]);
        mma16816<BF>(o[i + 1], ph, b[2], b[3]);
        mma16816<BF>(o[i + 1], pl, b[2], b[3]);
      }
    }
    __syncthreads();   // everyone is done with rows[buf], spart and rowvalid before they are overwritten
  }
  // ---- partial results of this split
  const int h0 = hg * kSaHeadsPerBlock + g, h1 = h0 + 8;
  float* po0 = p.part_o + ((size_t)split * p.H + h0) * D + kbase;
  float* po1 = p.part_o + ((size_t)split * p.H + h1) * D + kbase;
#pragma unroll
  for (int i = 0; i < NTW; i++) {
    *reinterpret_cast<float2*>(po0 + 8 * i + 2 * t) = make_float2(o[i][0], o[i][1]);
    *reinterpret_cast<float2*>(po1 + 8 * i + 2 * t) = make_float2(o[i][2], o[i][3]);
  }
  if (warp == 0 && t == 0) {
    float* ml = p.part_ml + ((size_t)split * p.H) * 2;
    ml[2 * h0] = m0; ml[2 * h0 + 1] = l0;
    ml[2 * h1] = m1; ml[2 * h1 + 1] = l1;
  }
}

// combine the splits of one head, add the sink to the denominator, inverse rope on the last 64 dims.  A head's D
// outputs are spread over 4 blocks (D / 4 threads each): the kernel streams splits x H x D partials and is bounded by
// how many of those loads are in flight, so it wants every SM, not one block per head.
template <int D>
__global__ void __launch_bounds__(D / 4) sparse_combine_kernel(const SparseParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DQ = D / 4;
  __shared__ float xs[DQ];
  __shared__ float fs[1024];      // per-split rescale factors exp(m_s - M)
  __shared__ float ls[1024];
  const int h = blockIdx.x, t = threadIdx.x, d = blockIdx.y * DQ + t;
  // this thread's partial outputs of the first kPre splits are requested before anything else: one memory latency for
  // all of them, under the staging of (m, l) below, instead of a batch of loads per 16 splits afterwards
  constexpr int kPre = 72;
  const float* po = p.part_o + (size_t)h * D + d;
  const size_t stride = (size_t)p.H * D;
  float pv[kPre];
#pragma unroll
  for (int s = 0; s < kPre; s++) pv[s] = s < p.splits ? __ldcg(po + (size_t)s * stride) : 0.f;
  const float sink = p.sinks[h];
  // every thread needs M and the denominator: stage (m, l) of all splits once, then every thread reduces them from
  // shared memory in the same order
  for (int s = t; s < p.splits; s += DQ) {
    const float2 ml = *reinterpret_cast<const float2*>(p.part_ml + ((size_t)s * p.H + h) * 2);
    fs[s] = ml.x; ls[s] = ml.y;
  }
  __syncthreads();
  float M = sink;
  for (int s = 0; s < p.splits; s++) M = fmaxf(M, fs[s]);
  __syncthreads();
  for (int s = t; s < p.splits; s += DQ) { const float m = fs[s]; fs[s] = (m == -INFINITY) ? 0.f : expf(m - M); }
  __syncthreads();
  float den = expf(sink - M);
  for (int s = 0; s < p.splits; s++) den += ls[s] * fs[s];
  float acc = 0.f;
#pragma unroll
  for (int s = 0; s < kPre; s++)
    if (s < p.splits) acc += pv[s] * fs[s];
#pragma unroll 16
  for (int s = kPre; s < p.splits; s++) acc += po[(size_t)s * stride] * fs[s];
  xs[t] = acc / den;
  __syncthreads();
  float v = xs[t];
  if (d >= D - 64) {    // rope pairs (d, d ^ 1) sit in the same block: DQ is even
    const int i = (d - (D - 64)) >> 1;
    const float c = p.cs[2 * i], sn = -p.cs[2 * i + 1];
    const float a = xs[t & ~1], b2 = xs[t | 1];
    v = (d & 1) ? a * sn + b2 * c : a * c - b2 * sn;
  }
  p.out[(size_t)h * D + d] = v;
}

// ---------------------------------------------------------------- host side
static int splits_for(int total_rows, int H, int sms) {
  const int tiles = std::max(1, (total_rows + kSaRows - 1) / kSaRows);
  const int hg = H / kSaHeadsPerBlock;
  // two blocks fit an SM: one row tile per block while that gives at most two blocks per SM (the chain gather ->
  // scores -> softmax -> output is latency-bound, so more blocks beat longer ones)
  return std::max(1, std::min(std::min(tiles, 1024), std::max(1, 2 * sms / hg)));
}
size_t sparse_scratch_bytes(int total_rows_max, int H, int D) {
  const int splits = std::max(1, (total_rows_max + kSaRows - 1) / kSaRows);   // upper bound, any device
  return sizeof(float) * (size_t)std::min(splits, 1024) * H * (D + 2);   // at most 1024 splits (combine kernel)
}

template <int D, bool BF>
static int launch_sparse(SparseParams& p, cudaStream_t st, int dev) {
  constexpr int PITCH = D * 2 + 16;
  const size_t smem = 2 * kSaRows * PITCH + 4 * (kSaRows / 8) * 32 * 4 * sizeof(float) + 2 * kSaRows * sizeof(int);
  auto kern = sparse_partial_kernel<D, BF>;
  static bool done[64] = {};
  if (!done[dev & 63]) {
    MSB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    done[dev & 63] = true;
  }
  MSB_CUDA(launch_pdl(kern, dim3(dim3(p.H / kSaHeadsPerBlock, p.splits)), dim3(128), smem, st, p));
  MSB_CUDA(launch_pdl(sparse_combine_kernel<D>, dim3(p.H, 4), dim3(D / 4), 0, st, p));
  MSB_LAUNCH_CHECK("sparse attention");
  return kOk;
}

// elem_type: MSB_F16 (1) or MSB_BF16 (30)
int sparse_decode(const float* q, const float* cs, const float* sinks, int elem_type, const void* win, int n_win,
                  const void* cache, const int* topk, int k, int H, int D, float* out, void* scratch,
                  size_t scratch_bytes, cudaStream_t st) {
  if (H <= 0 || H % kSaHeadsPerBlock || (D != 512 && D != 576)) return fail(kErrArg, "sparse: H %d D %d unsupported", H, D);
  if (elem_type != F16 && elem_type != BF16) return fail(kErrType, "sparse: rows must be F16 or BF16");
  if (n_win < 0 || k < 0 || n_win + k <= 0) return fail(kErrArg, "sparse: no rows");
  if (!q || !cs || !sinks || !out || !scratch || (n_win && !win) || (k && (!cache || !topk)))
    return fail(kErrArg, "sparse: null pointer");
  if ((reinterpret_cast<uintptr_t>(win) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15))
    return fail(kErrArg, "sparse: row buffers must be 16-byte aligned");
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  SparseParams p;
  p.q = q; p.cs = cs; p.sinks = sinks; p.win = (const uint8_t*)win; p.cache = (const uint8_t*)cache; p.topk = topk;
  p.out = out; p.n_win = n_win; p.k = k; p.H = H;
  const int total = n_win + k;
  p.splits = splits_for(total, H, sms);
  const int tiles = (total + kSaRows - 1) / kSaRows;
  p.rows_per_split = ((tiles + p.splits - 1) / p.splits) * kSaRows;
  p.splits = (total + p.rows_per_split - 1) / p.rows_per_split;
  const size_t need = sizeof(float) * (size_t)p.splits * H * (D + 2);
  if (scratch_bytes < need) return fail(kErrScratch, "sparse: scratch too small (%zu < %zu)", scratch_bytes, need);
  p.part_o = reinterpret_cast<float*>(scratch);
  p.part_ml = p.part_o + (size_t)p.splits * H * D;
  if (D == 512) return elem_type == BF16 ? launch_sparse<512, true>(p, st, dev) : launch_sparse<512, false>(p, st, dev);
  return elem_type == BF16 ? launch_sparse<576, true>(p, st, dev) : launch_sparse<576, false>(p, st, dev);
}

}  // namespace msb
