// Host-side status text and the per-device codebook tables of libmacseek_b200.
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>
#include "quant_blocks.cuh"
#include "iq_grids_packed.h"

namespace msb {

static thread_local char t_err[512] = "";
const char* last_error_text() { return t_err; }

bool pdl_enabled() {
  static const bool on = [] { const char* e = getenv("MSB_PDL"); return !(e && e[0] == '0'); }();
  return on;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof t_err, fmt, ap);
  va_end(ap);
  return code;
}
int cuda_fail(cudaError_t e, const char* what) {
  return fail(kErrCuda, "CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
}
const char* type_name(int t) {
  switch (t) {
    case F32: return "F32"; case F16: return "F16"; case BF16: return "BF16"; case Q8_0: return "Q8_0";
    case Q5_K: return "Q5_K"; case Q6_K: return "Q6_K"; case IQ2_XXS: return "IQ2_XXS"; case IQ1_S: return "IQ1_S";
    case IQ4_NL: return "IQ4_NL";
  }
  return "?";
}

// GGUF IQ4_NL value table (16 signed levels)
static const int8_t kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

namespace {
constexpr int kMaxDev = 64;
struct DevTables { bool ready = false; Tables t{}; float* noalloc = nullptr; };
// scratch of msb_moe_decode_noalloc: static device memory, (kMaxRouted + 1) x 4096 floats = 272 KB per device
__device__ __align__(256) float g_noalloc_moe_scratch[(size_t)kNoAllocFloats];
DevTables g_tables[kMaxDev];
std::mutex g_mu;

struct HostImage {
  std::vector<uint32_t> iq2_grid;   // 2 words per entry
  std::vector<uint32_t> iq2_sign;   // 2 words per entry
  std::vector<uint16_t> iq4_pair;
  std::vector<int8_t> iq1s_i8;
  std::vector<uint32_t> iq1s_sel;   // 2 words per entry
  std::vector<uint32_t> iq2_sel;    // 2 words per entry
  std::vector<uint32_t> iq2_sign16; // 4 words per entry
  std::vector<uint32_t> img_iq1s, img_iq2g, img_iq2s, img_iq4;
  HostImage() : iq2_grid(512), iq2_sign(256), iq4_pair(256), iq1s_i8(2048 * 8), iq1s_sel(2048 * 2, 0), iq2_sel(256 * 2, 0), iq2_sign16(128 * 4, 0) {
    img_iq1s.assign(2048 * kIq1sCopies, 0);
    for (int i = 0; i < 2048; i++) {
      uint32_t w = 0;
      for (int j = 0; j < 8; j++) {
        const uint32_t f = (kMsbIq1sPacked[i] >> (2 * j)) & 3;   // value + 1
        iq1s_i8[i * 8 + j] = (int8_t)((int)f - 1);
        w |= f << (8 * (j % 4) + 4 * (j / 4));                    // element j: byte j % 4, high nibble for j >= 4
      }
      for (int c = 0; c < kIq1sCopies; c++) img_iq1s[i * kIq1sCopies + c] = w;
      // selectors: code c (0..2) of an element picks bytes (2c, 2c+1) of the 8-byte pool of three halfs
      for (int j = 0; j < 4; j++) {
        const uint32_t ca = (kMsbIq1sPacked[i] >> (4 * j)) & 3, cb = (kMsbIq1sPacked[i] >> (4 * j + 2)) & 3;
        const uint32_t sel = (2 * ca) | ((2 * ca + 1) << 4) | ((2 * cb) << 8) | ((2 * cb + 1) << 12);
        iq1s_sel[2 * i + j / 2] |= sel << (16 * (j % 2));
      }
    }
    static const uint32_t lv[4] = {8, 25, 43, 0};
    for (int i = 0; i < 256; i++)
      for (int j = 0; j < 8; j++) iq2_grid[2 * i + j / 4] |= lv[(kMsbIq2xxsPacked[i] >> (2 * j)) & 3] << (8 * (j % 4));
    for (int i = 0; i < 256; i++)
      for (int j = 0; j < 4; j++) {
        const uint32_t ca = (kMsbIq2xxsPacked[i] >> (4 * j)) & 3, cb = (kMsbIq2xxsPacked[i] >> (4 * j + 2)) & 3;
        const uint32_t sel = (2 * ca) | ((2 * ca + 1) << 4) | ((2 * cb) << 8) | ((2 * cb + 1) << 12);
        iq2_sel[2 * i + j / 2] |= sel << (16 * (j % 2));
      }
    for (int i = 0; i < 128; i++) {
      const int bits = i | ((__builtin_popcount((unsigned)i) & 1) << 7);
      for (int j = 0; j < 8; j++)
        if ((bits >> j) & 1) {
          iq2_sign[2 * i + j / 4] |= 0xFFu << (8 * (j % 4));
          iq2_sign16[4 * i + j / 2] |= 0x8000u << (16 * (j % 2));
        }
    }
    for (int b = 0; b < 256; b++)
      iq4_pair[b] = (uint16_t)((uint8_t)kIq4nl[b & 15] | ((uint16_t)(uint8_t)kIq4nl[b >> 4] << 8));
    img_iq2g.assign(256 * kIq2Copies, 0);
    img_iq2s.assign(128 * kIq2Copies, 0);
    img_iq4.assign(256 * 8, 0);
    for (int i = 0; i < 256; i++) {
      uint32_t w = 0;                                             // nibble j = magnitude code of element j
      for (int j = 0; j < 8; j++) w |= ((kMsbIq2xxsPacked[i] >> (2 * j)) & 3u) << (4 * j);
      for (int c = 0; c < kIq2Copies; c++) img_iq2g[i * kIq2Copies + c] = w;
    }
    for (int i = 0; i < 128; i++) {
      const int bits = i | ((__builtin_popcount((unsigned)i) & 1) << 7);
      uint32_t w = 0;                                             // nibble j = 3 where element j is negative
      for (int j = 0; j < 8; j++)
        if ((bits >> j) & 1) w |= 3u << (4 * j);
      for (int c = 0; c < kIq2Copies; c++) img_iq2s[i * kIq2Copies + c] = w;
    }
    for (int i = 0; i < 256; i++)
      for (int c = 0; c < 8; c++) img_iq4[i * 8 + c] = iq4_pair[i];
  }
};

template <typename T>
cudaError_t upload(const std::vector<T>& v, const void** out) {
  void* d = nullptr;
  cudaError_t e = cudaMalloc(&d, v.size() * sizeof(T));
  if (e != cudaSuccess) return e;
  e = cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
  *out = d;
  return e;
}
}  // namespace

int get_tables(Tables* out) {
  int dev = 0;
  MSB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDev) return fail(kErrArg, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  DevTables& d = g_tables[dev];
  if (!d.ready) {
    static const HostImage img;
    Tables t{};
    const void** slots[] = {(const void**)&t.img_iq1s, (const void**)&t.img_iq2g, (const void**)&t.img_iq2s, (const void**)&t.img_iq4,
                            (const void**)&t.iq2xxs_grid, (const void**)&t.iq2_signmask, (const void**)&t.iq4nl_pair,
                            (const void**)&t.iq1s_i8, (const void**)&t.iq1s_sel, (const void**)&t.iq2_sel, (const void**)&t.iq2_sign16};
    cudaError_t e = cudaSuccess;
    auto up = [&](auto& v, int k) { if (e == cudaSuccess) e = upload(v, slots[k]); };
    up(img.img_iq1s, 0); up(img.img_iq2g, 1); up(img.img_iq2s, 2); up(img.img_iq4, 3); up(img.iq2_grid, 4); up(img.iq2_sign, 5);
    up(img.iq4_pair, 6); up(img.iq1s_i8, 7); up(img.iq1s_sel, 8); up(img.iq2_sel, 9); up(img.iq2_sign16, 10);
    if (e == cudaSuccess) e = cudaMalloc((void**)&t.status, 2048);     // status word, scheduling counters, argmax partials
    if (e == cudaSuccess) e = cudaMemset(t.status, 0, 2048);
    void* na = nullptr;
    // the first symbol look-up loads the module that holds the array: done here, never on the allocation-free path
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&na, g_noalloc_moe_scratch);
    if (e != cudaSuccess) {
      // nothing half-built survives: a later call starts over instead of leaking what was uploaded so far
      for (const void** sl : slots) if (*sl) cudaFree(const_cast<void*>(*sl));
      if (t.status) cudaFree(t.status);
      return cuda_fail(e, "get_tables");
    }
    d.t = t;
    d.noalloc = static_cast<float*>(na);
    d.ready = true;
  }
  *out = d.t;
  return kOk;
}

// Whether this device's tables and status buffer already exist (nothing is created here).
bool tables_ready() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return false;
  std::lock_guard<std::mutex> lk(g_mu);
  return g_tables[dev].ready;
}

// The allocation-free MoE entry point's scratch on the current device, or nullptr when msb_init() has not run there.
// A pure read of what get_tables() cached: no CUDA call that could create anything, safe during a stream capture.
float* noalloc_scratch(size_t* bytes) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_tables[dev].ready) return nullptr;
  if (bytes) *bytes = sizeof(float) * (size_t)kNoAllocFloats;
  return g_tables[dev].noalloc;
}

}  // namespace msb
