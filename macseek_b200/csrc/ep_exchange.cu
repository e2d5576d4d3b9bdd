// Expert-parallel exchange of the MoE decode output: allocation / peer mapping of the per-rank exchange buffers and the
// combine kernel that adds the ranks' partial outputs into the hidden state.
//
// The reference model sums the ranks' routed outputs with an all-reduce (reference/inference/model.py:903-904).  Here
// the MoE down launch of every rank stores its partial row sums straight into slot `rank` of EVERY rank's exchange
// buffer (peer-mapped memory over NVLink, plain st.global); each of its blocks then adds 1, with release semantics at
// system scope, to its rank's arrival counter of the current exchange in every rank's buffer (one cache line per source
// rank).  ep_combine_kernel on each rank waits (bounded) until every source rank's blocks have arrived, adds the slots in rank order -- so all ranks compute
// bit-identical sums -- zeroes the counter and advances the epoch.  Slots and counters are double-buffered by the
// parity of the rank's epoch counter: a rank can run at most one exchange ahead of a peer, because finishing exchange k
// needs every peer's arrivals of k, and a peer writes parity p again only after this rank's combine of the previous
// exchange on p has finished (it needs this rank's contribution to the exchange in between).
#include <algorithm>
#include <cstring>
#include "moe_decode_params.cuh"

namespace msb {

static long long g_peer_wait_cycles = 2000000000LL;    // ~1 s of SM clock
void set_peer_wait_cycles(long long c) { g_peer_wait_cycles = c > 0 ? c : 2000000000LL; }

struct EpCombineParams {
  uint8_t* base;       // this rank's exchange buffer
  float* h;            // [dim], h += sum over ranks of their partial
  int world, dim;
  unsigned expected;   // arrivals per source rank in one exchange: the blocks of a down launch
  int* status;
  long long wait_cycles;
};

// One block: no ticket, no second grid-wide step.  1024 threads x 4 elements cover dim 4096 in one pass.
__global__ void __launch_bounds__(1024) ep_combine_kernel(const EpCombineParams p) {
  pdl_launch_dependents();
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  pdl_wait();       // the down launch of this rank (and through it the epoch's previous combine) precedes us in the stream
  __syncthreads();
  const unsigned E = *reinterpret_cast<volatile unsigned*>(p.base);
  const int par = (int)(E & 1u);
  if (threadIdx.x < p.world) {
    unsigned* cnt = ep_arrivals(p.base, par, threadIdx.x);        // thread r waits for rank r's blocks
    // a device-side failure recorded earlier means a partial may never arrive: do not wait again
    bool ok = *reinterpret_cast<volatile int*>(p.status) == 0;
    if (ok) {
      const long long t0 = clock64();
      for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
        if (v == p.expected) break;
        if (clock64() - t0 > p.wait_cycles) { ok = false; atomicCAS(p.status, 0, kDevPeerWait); break; }
        __nanosleep(32);
      }
    }
    if (!ok) failed = 1;
  }
  __syncthreads();
  if (!failed) {
    const float* slots = reinterpret_cast<const float*>(p.base + kEpSlotsOff) + (size_t)par * p.world * p.dim;
    for (int i = threadIdx.x * 4; i < p.dim; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(p.h + i);
      float4 s[kMaxEpWorld];
#pragma unroll
      for (int r = 0; r < kMaxEpWorld; r++)
        if (r < p.world) s[r] = __ldcg(reinterpret_cast<const float4*>(slots + (size_t)r * p.dim + i));
#pragma unroll
      for (int r = 0; r < kMaxEpWorld; r++)          // rank order on every rank
        if (r < p.world) { v.x += s[r].x; v.y += s[r].y; v.z += s[r].z; v.w += s[r].w; }
      *reinterpret_cast<float4*>(p.h + i) = v;
    }
  }
  // the counter goes back to zero for the next exchange on this parity and the epoch advances; a failed exchange does
  // both too, so that the ranks' parities stay aligned if the caller clears the failure and carries on
  __syncthreads();
  if (threadIdx.x < p.world) *reinterpret_cast<volatile unsigned*>(ep_arrivals(p.base, par, threadIdx.x)) = 0u;
  if (threadIdx.x == 0) {
    *reinterpret_cast<volatile unsigned*>(p.base) = E + 1u;
    __threadfence();
  }
}

int ep_combine(uint8_t* const* base, int world, int rank, float* h, int dim, cudaStream_t st) {
  if (world < 1 || world > kMaxEpWorld || rank < 0 || rank >= world) return fail(kErrArg, "ep_combine: bad world %d / rank %d", world, rank);
  if (!base || !base[rank] || !h || dim <= 0 || dim % 4) return fail(kErrArg, "ep_combine: null pointer or bad dim");
  if (reinterpret_cast<uintptr_t>(h) & 15) return fail(kErrArg, "ep_combine: h must be 16-byte aligned");
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  int dev = 0, sms = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  MSB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  EpCombineParams p;
  p.base = base[rank]; p.h = h; p.world = world; p.dim = dim; p.status = tb.status;
  // every rank's down launch runs moe_down_blocks(dim) blocks (identical GPUs), each of which arrives once
  p.expected = (unsigned)moe_down_blocks(dim, sms);
  p.wait_cycles = g_peer_wait_cycles;
  MSB_CUDA(launch_pdl(ep_combine_kernel, dim3(1), dim3(1024), 0, st, p));
  MSB_LAUNCH_CHECK("ep_combine_kernel");
  return kOk;
}

// ---- exchange buffers: plain cudaMalloc allocations (so that they can be exported), zero-filled
int ep_alloc(size_t bytes, void** out) {
  if (!out || bytes == 0) return fail(kErrArg, "ep_alloc: bad arguments");
  void* d = nullptr;
  MSB_CUDA(cudaMalloc(&d, bytes));
  cudaError_t e = cudaMemset(d, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { cudaFree(d); return cuda_fail(e, "ep_alloc"); }
  *out = d;
  return kOk;
}
int ep_free(void* p) {
  if (p) MSB_CUDA(cudaFree(p));
  return kOk;
}
int ipc_export(void* p, unsigned char* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (!p || !handle64) return fail(kErrArg, "ipc_export: null pointer");
  cudaIpcMemHandle_t h;
  MSB_CUDA(cudaIpcGetMemHandle(&h, p));
  memcpy(handle64, &h, 64);
  return kOk;
}
int ipc_import(const unsigned char* handle64, void** out) {
  if (!handle64 || !out) return fail(kErrArg, "ipc_import: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  MSB_CUDA(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return kOk;
}
int ipc_release(void* p) {
  if (p) MSB_CUDA(cudaIpcCloseMemHandle(p));
  return kOk;
}

}  // namespace msb
