// Sampling head over the vocabulary row(s) of logits -- the reference's ms::arch::encode_argmax (greedy, or Gumbel-max =
// exact temperature sampling), encode_topk (k <= 64, with the full-row log-sum-exp for a CPU top-p sampler) and
// encode_log_softmax (src/kernels/arch.hpp:109-122, arch_sample.metal:15-213), and the CPU sampler sample_top_p
// (arch.mm:322-342).  Off the per-token critical path except argmax; written for determinism: every reduction has a
// fixed tree, ties go to the lower index, repeated calls give identical bits.
//
// Each kernel is one launch: grid (groups, rows); a group reduces a contiguous chunk of its row, stores a partial, and
// the group that takes the row's last ticket merges the partials (then resets the ticket for the next call).
#include <algorithm>
#include <cmath>
#include "msb_common.cuh"

namespace msb {

namespace {
constexpr int kSampT = 1024;          // threads per group
constexpr int kSampK = 64;            // largest k of the top-k
constexpr int kSampMaxGroups = 64;    // groups per row (a group holds 4 candidates per thread: chunk <= 4096)

__device__ __forceinline__ uint32_t hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
// Gumbel(0,1) noise of element i under (s0, s1): two rounds of the 32-bit mixer, 24 bits -> u in (0,1), -log(-log u)
// (arch_sample.metal:15-26)
__device__ __forceinline__ float gumbel(uint32_t i, uint32_t s0, uint32_t s1) {
  uint32_t x = hash32(i * 0x9E3779B9u ^ s0);
  x = hash32(x ^ (s1 * 0x85EBCA6Bu + 0x632BE5ABu));
  const float u = ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(-logf(u));
}
__device__ __forceinline__ bool better(float v, uint32_t i, float w, uint32_t j) { return v > w || (v == w && i < j); }

struct BlockRed {          // shared scratch of the block-wide reductions
  float v[32];
  uint32_t i[32];
  float m[32], s[32];
  int last;
};

// block-wide (value, index) argmax, ties -> lower index; every thread gets the result
__device__ __forceinline__ void block_argmax(float& v, uint32_t& i, BlockRed& r, int tid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (better(ov, oi, v, i)) { v = ov; i = oi; }
  }
  if ((tid & 31) == 0) { r.v[tid >> 5] = v; r.i[tid >> 5] = i; }
  __syncthreads();
  v = r.v[tid & 31]; i = r.i[tid & 31];          // kSampT / 32 = 32 warps: one partial per lane
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (better(ov, oi, v, i)) { v = ov; i = oi; }
  }
  __syncthreads();
}
// (max, sum of exp(x - max)) pairs
__device__ __forceinline__ void lse_combine(float& m, float& s, float m2, float s2) {
  const float M = fmaxf(m, m2);
  s = s * expf(m - M) + s2 * expf(m2 - M);
  m = M;
}
__device__ __forceinline__ void block_lse(float& m, float& s, BlockRed& r, int tid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lse_combine(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
  if ((tid & 31) == 0) { r.m[tid >> 5] = m; r.s[tid >> 5] = s; }
  __syncthreads();
  m = r.m[tid & 31]; s = r.s[tid & 31];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lse_combine(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
  __syncthreads();
}
// the row's last group to arrive (its partial is stored and fenced before the ticket)
__device__ __forceinline__ bool last_group(unsigned* ticket, int groups, BlockRed& r, int tid) {
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    r.last = atomicAdd(ticket, 1u) == (unsigned)groups - 1;
  }
  __syncthreads();
  if (r.last) __threadfence();
  return r.last != 0;
}

struct SampleParams {
  const float* logits;
  int rows, V, groups, chunk, k;
  float inv_temp;
  uint32_t seed_lo, seed_hi;
  int use_gumbel;
  float* part_v;        // argmax: [rows][groups] (value); top-k: [rows][groups][64]
  uint32_t* part_i;     // same shapes
  float2* part_ms;      // top-k: [rows][groups] (max, sum)
  unsigned* ticket;     // [rows]
  int* out_idx;         // argmax [rows]; top-k [rows][64]
  float* out_val;       // argmax [rows] (may be null); top-k [rows][64]
  float* out_lse;       // top-k [rows]
};

__global__ void __launch_bounds__(kSampT) argmax_rows_kernel(const SampleParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ BlockRed r;
  const int tid = threadIdx.x, g = blockIdx.x, row = blockIdx.y;
  const float* l = p.logits + (size_t)row * p.V;
  const int b = g * p.chunk, e = min(p.V, b + p.chunk);
  const uint32_t s0 = p.seed_lo + (uint32_t)row * 0x2545F491u;
  float bv = -INFINITY;
  uint32_t bi = 0xffffffffu;
  for (int i = b + tid; i < e; i += kSampT) {
    const float v = p.use_gumbel ? l[i] * p.inv_temp + gumbel((uint32_t)i, s0, p.seed_hi) : l[i];
    if (better(v, (uint32_t)i, bv, bi)) { bv = v; bi = (uint32_t)i; }
  }
  block_argmax(bv, bi, r, tid);
  if (tid == 0) { p.part_v[row * p.groups + g] = bv; p.part_i[row * p.groups + g] = bi; }
  if (!last_group(p.ticket + row, p.groups, r, tid)) return;
  bv = -INFINITY; bi = 0xffffffffu;
  for (int k = tid; k < p.groups; k += kSampT) {
    const float v = reinterpret_cast<volatile float*>(p.part_v)[row * p.groups + k];
    const uint32_t i = reinterpret_cast<volatile uint32_t*>(p.part_i)[row * p.groups + k];
    if (better(v, i, bv, bi)) { bv = v; bi = i; }
  }
  block_argmax(bv, bi, r, tid);
  if (tid == 0) {
    p.out_idx[row] = (int)bi;
    if (p.out_val) p.out_val[row] = bv;
    p.ticket[row] = 0;
  }
}

// the top k (descending, ties -> lower index) of up to 4 * kSampT (value, index) pairs held 4 per thread
__device__ __forceinline__ void extract_topk(float (&v)[4], uint32_t (&ix)[4], int k, BlockRed& r, int tid, float* out_v,
                                             uint32_t* out_i) {
  for (int round = 0; round < k; round++) {
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;
#pragma unroll
    for (int q = 0; q < 4; q++)
      if (ix[q] != 0xffffffffu && better(v[q], ix[q], bv, bi)) { bv = v[q]; bi = ix[q]; }
    block_argmax(bv, bi, r, tid);
#pragma unroll
    for (int q = 0; q < 4; q++)
      if (ix[q] == bi) { v[q] = -INFINITY; ix[q] = 0xffffffffu; }
    if (tid == 0) { out_v[round] = bv; out_i[round] = bi; }
  }
}

__global__ void __launch_bounds__(kSampT) topk_lse_kernel(const SampleParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ BlockRed r;
  const int tid = threadIdx.x, g = blockIdx.x, row = blockIdx.y;
  const float* l = p.logits + (size_t)row * p.V;
  const int b = g * p.chunk, e = min(p.V, b + p.chunk);
  float v[4];
  uint32_t ix[4];
  float m = -INFINITY, s = 0.f;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const int i = b + tid + q * kSampT;
    const bool ok = i < e;
    v[q] = ok ? l[i] : -INFINITY;
    ix[q] = ok ? (uint32_t)i : 0xffffffffu;
    if (ok) {
      if (s == 0.f) { m = v[q] * p.inv_temp; s = 1.f; }
      else lse_combine(m, s, v[q] * p.inv_temp, 1.f);
    }
  }
  // an empty thread carries (m, s) = (-inf, 0): give it a finite max so that exp(m - M) is exp(-inf) = 0, not NaN
  if (s == 0.f) m = -3.0e38f;
  block_lse(m, s, r, tid);
  if (tid == 0) p.part_ms[row * p.groups + g] = make_float2(m, s);
  const size_t pb = ((size_t)row * p.groups + g) * kSampK;
  extract_topk(v, ix, p.k, r, tid, p.part_v + pb, p.part_i + pb);
  if (!last_group(p.ticket + row, p.groups, r, tid)) return;
  // merge: groups * k candidates, 4 per thread
  const int nc = p.groups * p.k;
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const int c = tid + q * kSampT;
    const bool ok = c < nc;
    const int gg = ok ? c / p.k : 0, rr = ok ? c - gg * p.k : 0;
    const size_t o = ((size_t)row * p.groups + gg) * kSampK + rr;
    v[q] = ok ? reinterpret_cast<volatile float*>(p.part_v)[o] : -INFINITY;
    ix[q] = ok ? reinterpret_cast<volatile uint32_t*>(p.part_i)[o] : 0xffffffffu;
  }
  m = -3.0e38f; s = 0.f;
  for (int k = tid; k < p.groups; k += kSampT) {
    const float qm = reinterpret_cast<volatile float*>(p.part_ms)[2 * (row * p.groups + k)];
    const float qs = reinterpret_cast<volatile float*>(p.part_ms)[2 * (row * p.groups + k) + 1];
    lse_combine(m, s, qm, qs);
  }
  block_lse(m, s, r, tid);
  if (tid == 0) p.out_lse[row] = m + logf(s);
  extract_topk(v, ix, p.k, r, tid, p.out_val + (size_t)row * kSampK, reinterpret_cast<uint32_t*>(p.out_idx) + (size_t)row * kSampK);
  if (tid == 0) p.ticket[row] = 0;
}

// out[r][i] = in[r][i] - logsumexp(in[r]); one group per row; out may alias in
__global__ void __launch_bounds__(kSampT) log_softmax_kernel(const float* in, float* out, int V) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ BlockRed r;
  const int tid = threadIdx.x, row = blockIdx.x;
  const float* x = in + (size_t)row * V;
  float m = -3.0e38f, s = 0.f;
  for (int i = tid; i < V; i += kSampT) {
    const float v = x[i];
    if (v > m) { s = s * expf(m - v) + 1.f; m = v; }
    else s += expf(v - m);
  }
  block_lse(m, s, r, tid);
  const float lse = m + logf(s);
  float* y = out + (size_t)row * V;
  for (int i = tid; i < V; i += kSampT) y[i] = x[i] - lse;
}

int groups_for(int V) { return std::max(1, std::min(kSampMaxGroups, (V + 4 * kSampT - 1) / (4 * kSampT))); }
}  // namespace

// scratch: tickets [rows] | part_ms [rows][G] | part_v [rows][G][64] | part_i [rows][G][64]; must start at zero (the
// kernels leave the tickets at zero again)
size_t sample_scratch_bytes(int rows) {
  if (rows <= 0) return 0;
  const size_t R = (size_t)rows, G = kSampMaxGroups;
  return 256 + ((R * 4 + 255) & ~(size_t)255) + R * G * 8 + 2 * R * G * kSampK * 4;
}

static int fill_scratch(SampleParams& p, int rows, void* scratch, size_t scratch_bytes) {
  if (!scratch || scratch_bytes < sample_scratch_bytes(rows)) return fail(kErrScratch, "sampling: scratch too small");
  if (reinterpret_cast<uintptr_t>(scratch) & 15) return fail(kErrArg, "sampling: scratch must be 16-byte aligned");
  uint8_t* c = static_cast<uint8_t*>(scratch);
  const size_t R = (size_t)rows, G = kSampMaxGroups;
  p.ticket = reinterpret_cast<unsigned*>(c); c += (R * 4 + 255) & ~(size_t)255;
  p.part_ms = reinterpret_cast<float2*>(c); c += R * G * 8;
  p.part_v = reinterpret_cast<float*>(c); c += R * G * kSampK * 4;
  p.part_i = reinterpret_cast<uint32_t*>(c);
  return kOk;
}

int argmax_rows(const float* logits, int rows, int V, int* out_idx, float* out_val, float temperature, uint64_t seed,
                void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (rows <= 0 || V <= 0 || !logits || !out_idx) return fail(kErrArg, "argmax_rows: bad arguments");
  SampleParams p{};
  int rc = fill_scratch(p, rows, scratch, scratch_bytes);
  if (rc) return rc;
  p.logits = logits; p.rows = rows; p.V = V;
  p.groups = std::max(1, std::min(kSampMaxGroups, (V + 2047) / 2048));
  p.chunk = (V + p.groups - 1) / p.groups;
  p.inv_temp = temperature > 0.f ? 1.f / temperature : 1.f;
  p.seed_lo = (uint32_t)seed; p.seed_hi = (uint32_t)(seed >> 32);
  p.use_gumbel = temperature > 0.f ? 1 : 0;
  p.out_idx = out_idx; p.out_val = out_val;
  MSB_CUDA(launch_pdl(argmax_rows_kernel, dim3(p.groups, rows), dim3(kSampT), 0, st, p));
  MSB_LAUNCH_CHECK("argmax_rows_kernel");
  return kOk;
}

int sample_topk(const float* logits, int rows, int V, int k, float temperature, float* out_v, int* out_i, float* out_lse,
                void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (rows <= 0 || V <= 0 || !logits || !out_v || !out_i || !out_lse) return fail(kErrArg, "sample_topk: bad arguments");
  if (k < 1 || k > kSampK) return fail(kErrArg, "sample_topk: k %d outside 1..%d", k, kSampK);
  if ((size_t)V > (size_t)kSampMaxGroups * 4 * kSampT) return fail(kErrLimit, "sample_topk: V %d beyond %d", V, kSampMaxGroups * 4 * kSampT);
  SampleParams p{};
  int rc = fill_scratch(p, rows, scratch, scratch_bytes);
  if (rc) return rc;
  p.logits = logits; p.rows = rows; p.V = V; p.k = k;
  p.groups = groups_for(V);
  p.chunk = (V + p.groups - 1) / p.groups;
  p.inv_temp = temperature > 0.f ? 1.f / temperature : 1.f;
  p.out_idx = out_i; p.out_val = out_v; p.out_lse = out_lse;
  MSB_CUDA(launch_pdl(topk_lse_kernel, dim3(p.groups, rows), dim3(kSampT), 0, st, p));
  MSB_LAUNCH_CHECK("topk_lse_kernel");
  return kOk;
}

int log_softmax(const float* in, float* out, int rows, int V, cudaStream_t st) {
  if (rows <= 0 || V <= 0 || !in || !out) return fail(kErrArg, "log_softmax: bad arguments");
  MSB_CUDA(launch_pdl(log_softmax_kernel, dim3(rows), dim3(kSampT), 0, st, in, out, V));
  MSB_LAUNCH_CHECK("log_softmax_kernel");
  return kOk;
}

// CPU: temperature + top-p sampling from sample_topk's output.  p_i = exp(v_i / T - lse); the smallest prefix whose
// cumulative mass reaches top_p is kept and renormalised; u in [0, 1) picks inside it (arch.mm:322-342).
int sample_top_p(const float* vals, const int* ids, int k, float lse, float temperature, float top_p, double u) {
  if (temperature <= 0.0f || k <= 1) return ids[0];
  if (k > kSampK) k = kSampK;
  const double inv_t = 1.0 / temperature;
  double probs[kSampK];
  double cum = 0.0;
  int keep = k;
  for (int i = 0; i < k; i++) {
    probs[i] = std::exp((double)vals[i] * inv_t - (double)lse);
    cum += probs[i];
    if (cum >= top_p) { keep = i + 1; break; }
  }
  double tot = 0.0;
  for (int i = 0; i < keep; i++) tot += probs[i];
  const double target = u * tot;
  double acc = 0.0;
  for (int i = 0; i < keep; i++) {
    acc += probs[i];
    if (target < acc) return ids[i];
  }
  return ids[keep - 1];
}

}  // namespace msb
