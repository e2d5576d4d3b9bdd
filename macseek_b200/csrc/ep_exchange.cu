// Expert-parallel exchange of the MoE decode output: allocation / peer mapping of the per-rank exchange buffers and the
// combine kernel that adds the ranks' partial outputs into the hidden state.
//
// The reference model sums the ranks' routed outputs with an all-reduce (reference/inference/model.py:903-904).  Here
// the MoE down launch of every rank stores its partial row sums straight into slot `rank` of EVERY rank's exchange
// buffer (peer-mapped memory over NVLink, plain st.global) and then raises flag `rank` there; ep_combine_kernel on each
// rank waits (bounded) for the `world` flags of the current exchange and adds the slots in rank order, so all ranks
// compute bit-identical sums.  Slots and flags are double-buffered by the parity of the rank's epoch counter: a rank
// can run at most one exchange ahead of a peer, because finishing exchange k needs every peer's flag k.
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
  int* status;
  unsigned* ticket;
  long long wait_cycles;
};

__global__ void __launch_bounds__(256) ep_combine_kernel(const EpCombineParams p) {
  pdl_launch_dependents();
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  pdl_wait();       // the down launch of this rank (and through it the epoch's previous combine) precedes us in the stream
  __syncthreads();
  const unsigned E = *reinterpret_cast<volatile unsigned*>(p.base);
  const int par = (int)(E & 1u);
  if (threadIdx.x < p.world) {
    const unsigned* flag = reinterpret_cast<const unsigned*>(p.base + kEpFlagsOff) + par * kMaxEpWorld + threadIdx.x;
    // a device-side failure recorded earlier means a partial may never arrive: do not wait again
    bool ok = *reinterpret_cast<volatile int*>(p.status) == 0;
    if (ok) {
      const long long t0 = clock64();
      for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v == E + 1u) break;
        if (clock64() - t0 > p.wait_cycles) { ok = false; atomicCAS(p.status, 0, kDevPeerWait); break; }
        __nanosleep(64);
      }
    }
    if (!ok) failed = 1;
  }
  __syncthreads();
  if (!failed) {
    const float* slots = reinterpret_cast<const float*>(p.base + kEpSlotsOff) + (size_t)par * p.world * p.dim;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < p.dim; i += gridDim.x * blockDim.x) {
      float v = p.h[i];
      for (int r = 0; r < p.world; r++) v += __ldcg(slots + (size_t)r * p.dim + i);     // rank order on every rank
      p.h[i] = v;
    }
  }
  // the last block to finish advances the epoch (every block has read E by then); a failed exchange advances it too,
  // so that the ranks' parities stay aligned if the caller clears the failure and carries on
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.ticket, 1u) == gridDim.x - 1) {
      *p.ticket = 0;
      *reinterpret_cast<volatile unsigned*>(p.base) = E + 1u;
      __threadfence();
    }
  }
}

int ep_combine(uint8_t* const* base, int world, int rank, float* h, int dim, cudaStream_t st) {
  if (world < 1 || world > kMaxEpWorld || rank < 0 || rank >= world) return fail(kErrArg, "ep_combine: bad world %d / rank %d", world, rank);
  if (!base || !base[rank] || !h || dim <= 0) return fail(kErrArg, "ep_combine: null pointer or bad dim");
  Tables tb;
  int rc = get_tables(&tb);
  if (rc) return rc;
  EpCombineParams p;
  p.base = base[rank]; p.h = h; p.world = world; p.dim = dim; p.status = tb.status;
  p.ticket = reinterpret_cast<unsigned*>(tb.status) + 13;
  p.wait_cycles = g_peer_wait_cycles;
  const int blocks = std::max(1, std::min(8, (dim + 1023) / 1024));
  MSB_CUDA(launch_pdl(ep_combine_kernel, dim3(blocks), dim3(256), 0, st, p));
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
