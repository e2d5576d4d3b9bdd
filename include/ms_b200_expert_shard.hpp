// Expert-parallel weight placement straight from GGUF file offsets: rank r of N reads, for every layer, the byte ranges
// of experts [r E / N, (r + 1) E / N) of the three stacked expert tensors into ONE device arena per layer and builds the
// [n_experts][3] address table that msb_moe_decode_ids / msb_moe_decode_ep resolve on the GPU.  What the reference's
// src/store (SSD streaming, slot arena, eviction) becomes when every expert fits in HBM: the file is read once.
// Expert ranges are the reference model's contiguous split (reference/inference/model.py:869-872).
#pragma once
#include <memory>
#include "ms_b200_attn_state.hpp"
#include "ms_b200_gguf.hpp"

namespace ms {

struct ExpertShardLayer {
  Buffer arena;                  // gate range | up range | down range of the resident experts, each contiguous
  Buffer table;                  // u64 [n_experts][3] device addresses {gate, up, down}; 0 for experts not resident here
  q::QType t_gate_up = q::QType::IQ1_S, t_down = q::QType::IQ2_XXS;
  int dim = 0, inter = 0;
};

struct ExpertShard {
  int n_layers = 0, n_experts = 0, expert_lo = 0, expert_hi = 0;
  std::vector<ExpertShardLayer> layers;
  uint64_t bytes = 0;            // device bytes of all arenas

  static std::pair<int, int> expert_range(int n_experts, int world, int rank) {
    if (world <= 0 || rank < 0 || rank >= world || n_experts % world) die("ExpertShard: experts do not split over the ranks");
    const int per = n_experts / world;
    return {rank * per, (rank + 1) * per};
  }

  // Reads through a host staging buffer of `chunk` bytes (file -> host -> device, one blocking copy per chunk).
  static ExpertShard load(const Gguf& g, const ExpertLayout& L, int rank, int world, size_t chunk = (size_t)64 << 20) {
    ExpertShard S;
    S.n_layers = L.n_layers; S.n_experts = L.n_experts;
    const std::pair<int, int> r = expert_range(L.n_experts, world, rank);
    S.expert_lo = r.first; S.expert_hi = r.second;
    const int n_local = S.expert_hi - S.expert_lo;
    std::unique_ptr<char[]> stage(new char[chunk]);
    for (int l = 0; l < L.n_layers; l++) {
      const ExpertLayerLayout& ll = L.layers[l];
      ExpertShardLayer out;
      if (ll.mat[0].type != ll.mat[1].type || ll.mat[0].len != ll.mat[1].len) die("ExpertShard: gate and up differ in type or size");
      out.t_gate_up = (q::QType)(int)ll.mat[0].type; out.t_down = (q::QType)(int)ll.mat[2].type;
      out.dim = (int)ll.mat[0].cols; out.inter = (int)ll.mat[0].rows;
      if (ll.mat[2].cols != out.inter || ll.mat[2].rows != out.dim) die("ExpertShard: down matrix shape does not match gate / up");
      // every matrix must start on a 2-byte boundary for the kernels; strides of whole GGUF blocks are even
      size_t off[3], total = 0;
      for (int k = 0; k < 3; k++) { off[k] = total; total += ((size_t)n_local * ll.mat[k].stride + 255) & ~(size_t)255; }
      out.arena = Device::get().alloc(total ? total : 256);
      for (int k = 0; k < 3; k++) {
        const ExpertMat& m = ll.mat[k];
        const uint64_t begin = m.base + (uint64_t)S.expert_lo * m.stride, len = (uint64_t)n_local * m.stride;
        if (begin + len > m.file_size) die("ExpertShard: expert range past the end of the file");
        for (uint64_t done = 0; done < len; done += chunk) {
          const size_t n = (size_t)std::min<uint64_t>(chunk, len - done);
          if (pread_full(g.fd(m.split), stage.get(), n, begin + done) != (long long)n) die("ExpertShard: short read");
          upload(out.arena.sub(off[k] + done, n), stage.get(), n);
        }
      }
      std::vector<uint64_t> tb((size_t)L.n_experts * 3, 0);
      const uint64_t base = (uint64_t)(uintptr_t)out.arena.ptr();
      for (int e = S.expert_lo; e < S.expert_hi; e++)
        for (int k = 0; k < 3; k++) tb[(size_t)e * 3 + k] = base + off[k] + (uint64_t)(e - S.expert_lo) * ll.mat[k].stride;
      out.table = Device::get().alloc(tb.size() * 8);
      upload(out.table, tb.data(), tb.size() * 8);
      S.bytes += total;
      S.layers.push_back(out);
    }
    return S;
  }
  void release() {
    for (ExpertShardLayer& l : layers) { Device::get().release(l.arena); Device::get().release(l.table); }
    layers.clear();
  }
};

}  // namespace ms
