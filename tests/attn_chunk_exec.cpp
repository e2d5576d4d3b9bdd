// Chunked attention side through include/ms_b200_attn_state.hpp: encode_layer(e, S, io, 0, n) over a chunk of n tokens
// (two layers: a KV / index source with ratio 2 and a layer that shares its caches and top-k lists) against the same
// tokens fed one at a time into a second state.
//   attn_chunk_exec <blob> <out> <n>
// blob (f32): kv_norm[512] sinks[64] c_norm[512] idx_knorm[128] idx_wk(bf16 [128][512], 32768 floats' worth of bytes / 2)
//   then q0[n][64][512] q1[n][64][512] kv[n][512] c_kv[n][512] c_gate[n][512] idx_q[n][32][128] idx_w[n][32]
// out: f32 A[2][n][64][512], f32 B[2][n][64][512], i32 lists[n][512] (state A, source layer), u16 ckv rows [n / 2][512]
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "ms_b200_attn_state.hpp"

using namespace ms;

int main(int argc, char** argv) {
  if (argc < 4) return 1;
  const int n = std::atoi(argv[3]);
  FILE* f = std::fopen(argv[1], "rb");
  if (!f) return 2;
  std::fseek(f, 0, SEEK_END);
  const long bytes = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  std::vector<char> blob((size_t)bytes);
  if (std::fread(blob.data(), 1, blob.size(), f) != blob.size()) return 2;
  std::fclose(f);
  Device& dev = Device::get();
  Buffer w = dev.alloc(blob.size());
  upload(w, blob.data(), blob.size());
  size_t off = 0;
  auto take = [&](size_t nbytes) { Buffer b = w.sub(off, nbytes); off += nbytes; return b; };
  const int D = 512, H = 64, IH = 32, ID = 128;
  Buffer kv_norm = take(D * 4), sinks = take(H * 4), c_norm = take(D * 4), idx_knorm = take(ID * 4), idx_wk = take((size_t)ID * D * 2);
  Buffer q0 = take((size_t)n * H * D * 4), q1 = take((size_t)n * H * D * 4), kv = take((size_t)n * D * 4), c_kv = take((size_t)n * D * 4),
         c_gate = take((size_t)n * D * 4), idx_q = take((size_t)n * IH * ID * 4), idx_w = take((size_t)n * IH * 4);
  attn::Shape sh;
  sh.layers = 2;
  attn::Roles roles;
  roles.kv_source = {0, 0}; roles.index_source = {0, 0}; roles.ratio = {2, 2};
  attn::Options oa, ob;
  oa.max_pos = ob.max_pos = 1024; oa.actq = ob.actq = true;
  oa.max_chunk = n; ob.max_chunk = 1;
  attn::State A, B;
  attn::init(A, oa, sh, roles); attn::reset(A);
  attn::init(B, ob, sh, roles); attn::reset(B);
  Buffer outA = dev.alloc((size_t)2 * n * H * D * 4), outB = dev.alloc((size_t)2 * n * H * D * 4);
  auto io_for = [&](int layer, const Buffer& out) {
    attn::LayerIO io;
    io.layer = layer; io.q = layer == 0 ? q0 : q1; io.kv = kv; io.kv_norm = kv_norm; io.sinks = sinks;
    io.out = out.sub((size_t)layer * n * H * D * 4, (size_t)n * H * D * 4);
    io.c_kv = c_kv; io.c_gate = c_gate; io.c_norm = c_norm; io.idx_wk = idx_wk; io.idx_knorm = idx_knorm; io.idx_q = idx_q; io.idx_w = idx_w;
    return io;
  };
  Enc e;
  // A: one call per layer for the whole chunk
  attn::encode_layer(e, A, io_for(0, outA), 0, n);
  attn::encode_layer(e, A, io_for(1, outA), 0, n);
  // B: token by token, both layers per token
  for (int t = 0; t < n; t++)
    for (int layer = 0; layer < 2; layer++) {
      attn::LayerIO io = io_for(layer, outB), one = io;
      one.q = attn::tok_row(io.q, t, (size_t)H * D); one.kv = attn::tok_row(io.kv, t, D); one.out = attn::tok_row(io.out, t, (size_t)H * D);
      one.c_kv = attn::tok_row(io.c_kv, t, D); one.c_gate = attn::tok_row(io.c_gate, t, D);
      one.idx_q = attn::tok_row(io.idx_q, t, (size_t)IH * ID); one.idx_w = attn::tok_row(io.idx_w, t, IH);
      attn::encode_layer(e, B, one, t, 1);
    }
  e.wait();
  FILE* out = std::fopen(argv[2], "wb");
  std::vector<float> v((size_t)2 * n * H * D);
  download(v.data(), outA, v.size() * 4); std::fwrite(v.data(), 4, v.size(), out);
  download(v.data(), outB, v.size() * 4); std::fwrite(v.data(), 4, v.size(), out);
  std::vector<int> lists((size_t)n * sh.topk);
  download(lists.data(), A.topk[0], lists.size() * 4); std::fwrite(lists.data(), 4, lists.size(), out);
  std::vector<uint16_t> rows((size_t)(n / 2) * D);
  download(rows.data(), A.ckv[0], rows.size() * 2); std::fwrite(rows.data(), 2, rows.size(), out);
  std::fclose(out);
  return 0;
}
