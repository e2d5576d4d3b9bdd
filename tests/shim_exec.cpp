// Runs two calls through the C++ shim (include/ms_b200_shim.hpp) on the GPU and writes their outputs to a file: the
// test compares them with the same calls made through ctypes.  Inputs come from files written by the test.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_runtime_api.h>
#include "ms_b200_shim.hpp"

static std::vector<char> slurp(const char* path) {
  FILE* f = std::fopen(path, "rb");
  if (!f) { std::perror(path); std::exit(2); }
  std::fseek(f, 0, SEEK_END);
  long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  std::vector<char> v((size_t)n);
  if (std::fread(v.data(), 1, (size_t)n, f) != (size_t)n) std::exit(2);
  std::fclose(f);
  return v;
}
static ms::Buffer upload(const std::vector<char>& v, size_t extra = 0) {
  void* d = nullptr;
  if (cudaMalloc(&d, v.size() + extra) != cudaSuccess) std::exit(3);
  cudaMemset(d, 0, v.size() + extra);
  cudaMemcpy(d, v.data(), v.size(), cudaMemcpyHostToDevice);
  return ms::Buffer{d, 0, v.size() + extra};
}
static ms::Buffer zeros(size_t bytes) { return upload(std::vector<char>(), bytes); }

int main(int argc, char** argv) {
  if (argc < 8) return 1;
  const int rows = std::atoi(argv[1]), cols = std::atoi(argv[2]), len = std::atoi(argv[3]);
  ms::Enc e;
  // (1) ms::q::encode_matvec, Q6_K
  ms::Buffer W = upload(slurp(argv[4])), x = upload(slurp(argv[5])), y = zeros((size_t)rows * 4);
  ms::q::encode_matvec(e, ms::q::QType::Q6_K, W, rows, cols, x, y);
  // (2) ms::attn::encode_index_decode on one KV source of reference shape (32 heads, F16 keys, top-512)
  ms::attn::DecodeCaches c;
  c.ikey = upload(slurp(argv[6]));
  std::vector<char> qw = slurp(argv[7]);      // iq [32][128] then iw [32] then rope row (64 floats)
  ms::Buffer all = upload(qw);
  ms::Buffer iq = all.sub(0, 32 * 128 * 4), iw = all.sub(32 * 128 * 4, 32 * 4);
  c.rope = all.sub(32 * 128 * 4 + 32 * 4, 64 * 4);
  c.topk_list = zeros(512 * 4);
  c.dec_scores = zeros((size_t)len * 4 + 64);
  c.q_prep = zeros(32 * 128 * 4);
  c.w_prep = zeros(32 * 4);
  c.topk_scratch = zeros(msb_topk_scratch_bytes(len));
  ms::attn::encode_index_decode(e, c, iq, iw, /*pos=*/0, len, /*actq=*/true);
  e.wait();
  std::vector<float> yh((size_t)rows);
  std::vector<int> tk(512);
  cudaMemcpy(yh.data(), y.ptr(), yh.size() * 4, cudaMemcpyDeviceToHost);
  cudaMemcpy(tk.data(), c.topk_list.ptr(), tk.size() * 4, cudaMemcpyDeviceToHost);
  FILE* f = std::fopen(argv[8], "wb");
  std::fwrite(yh.data(), 4, yh.size(), f);
  std::fwrite(tk.data(), 4, tk.size(), f);
  std::fclose(f);
  return 0;
}
