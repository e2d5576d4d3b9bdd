// Launch parameters of the fused MoE decode kernels (moe_decode.cu), shared with the C entry points.
#pragma once
#include "msb_common.cuh"

namespace msb {

constexpr int kMaxRouted = 16;
constexpr int kMoeNW = 16;


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
  unsigned* sched;                        // [2] counter of tiles handed out after each block's first (tile = its
                                          // block index), finished-block counter; both zero between launches
  float limit;
  // tile shapes (whole rows, every piece one contiguous bulk copy per source)
  int gu_r_rows;                          // routed gate/up tile rows (each warp owns whole rows)
  uint32_t gu_r_pitch, gu_s_pitch;        // shared-memory distance between a tile's gate rows and its up rows
  int gu_s_rows, gu_s_ks;                 // shared gate/up tile rows, warps sharing a row
  int d_rows;                             // down tile rows (two warps share a row)
  uint32_t d_src_pitch;                   // shared-memory distance between the experts' row blocks of a down piece
  uint32_t stage_bytes;
  int stages;
  Tables tb;
};

size_t moe_decode_scratch_bytes(int inter, int max_routed);
// part: 0 All, 1 SharedGu, 2 AfterSharedGu, 3 Shared, 4 Routed, 5 SharedDown
int moe_decode(MoeParams p, int t_gate_up, int t_down, int t_shared, int part, size_t scratch_bytes, cudaStream_t st);

}  // namespace msb
