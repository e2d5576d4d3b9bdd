// Launch parameters of the fused MoE decode kernels (moe_decode.cu), shared with the C entry points.
#pragma once
#include "msb_common.cuh"

namespace msb {

constexpr int kMaxRouted = 16;
constexpr int kMoeNW = 16;
constexpr int kMaxEpWorld = 8;


struct MoeParams {
  int dim, inter, n_routed, has_shared;
  int gu_r, gu_s, d_r, d_s;               // which pieces this launch covers
  const uint8_t* gate[kMaxRouted];
  const uint8_t* up[kMaxRouted];
  const uint8_t* down[kMaxRouted];
  const uint8_t *sgate, *sup, *sdown;
  const uint64_t* table;                  // optional [n_experts][3] device addresses {gate, up, down}
  const int* ids;                         // device [n_routed] expert ids (with table)
  int expert_lo, expert_hi;               // experts resident on this GPU (with table)
  const float* weights;                   // device [n_routed]
  const float* x;
  // not null: the gate/up launch ignores x and computes RMSNorm(norm_in) * norm_w itself, before the grid dependency
  // resolves.  norm_in must have been complete before the PREVIOUS kernel of the stream started (the fused-norm router
  // over the same vector is that kernel: it releases its dependents only after its own dependency resolved).
  const float* norm_in;
  const float* norm_w;
  float norm_eps;
  float* y;
  float* h;                               // [n_routed + 1][inter]
  unsigned* sched;                        // [1] expert-parallel exchange: blocks of the down launch that have stored their
                                          // partial; zero between launches
  float limit;
  // tile shapes (whole rows, every piece one contiguous bulk copy per source)
  int gu_r_rows;                          // routed gate/up tile rows (each warp owns whole rows)
  uint32_t gu_r_pitch, gu_s_pitch;        // shared-memory distance between a tile's gate rows and its up rows
  int gu_s_rows, gu_s_ks;                 // shared gate/up tile rows, warps sharing a row
  int d_rows;                             // down tile rows (two warps share a row)
  uint32_t d_src_pitch;                   // shared-memory distance between the experts' row blocks of a down piece
  uint32_t d_s_pitch;                     // distance between the shared expert's staged row pieces when only a K range is read
  uint32_t stage_bytes;
  int stages;
  // Rows [s_lo, s_hi) of the shared expert's gate / up matrices, and the same range of the K dimension of its down
  // matrix, are computed by this launch (multiples of 256; 0 .. inter = all of it).  Under expert parallelism rank r
  // takes the r-th slice, so the ranks' partial outputs add up to the whole shared expert.
  int s_lo, s_hi;
  // Expert-parallel exchange (ep_world > 0): the down launch does not touch y; it stores its row sums into slot ep_rank
  // of every rank's exchange buffer (peer-mapped memory, plain stores); every block then adds 1 to the exchange's arrival counter there.
  int ep_world, ep_rank;
  uint8_t* ep_base[kMaxEpWorld];
  Tables tb;
};

// Exchange buffer of one rank (zero-filled at creation):
//   +0    u32 epoch E: combines completed on this rank; slot / counter parity of the current exchange = E & 1
//   +128  arrival counters [2][kMaxEpWorld], one 128-byte line each: counter [parity][r] counts the blocks of rank r's
//         down launch whose partial rows of this exchange are in place; complete at moe_down_blocks(); zeroed again by
//         the combine
//   +4096 f32 slots[2][world][dim]
constexpr size_t kEpFlagsOff = 128, kEpCounterStride = 128, kEpSlotsOff = 4096;
__host__ __device__ inline unsigned* ep_arrivals(uint8_t* base, int parity, int src_rank) {
  return reinterpret_cast<unsigned*>(base + kEpFlagsOff + (size_t)(parity * kMaxEpWorld + src_rank) * kEpCounterStride);
}
// blocks of one moe_down_kernel launch (8-row tiles over dim, at most one block per SM): what each rank contributes to
// an exchange's arrival count
inline int moe_down_blocks(int dim, int sms) { const int tiles = (dim + 7) / 8; return tiles < sms ? (tiles > 1 ? tiles : 1) : sms; }
inline size_t ep_exchange_bytes(int dim, int world) { return kEpSlotsOff + sizeof(float) * 2 * (size_t)world * dim; }

size_t moe_decode_scratch_bytes(int inter, int max_routed);
// part: 0 All, 1 SharedGu, 2 AfterSharedGu, 3 Shared, 4 Routed, 5 SharedDown
int moe_decode(MoeParams p, int t_gate_up, int t_down, int t_shared, int part, size_t scratch_bytes, cudaStream_t st);

}  // namespace msb
