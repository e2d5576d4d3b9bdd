// GGUF block decoders for sm_100a.  Two families per type:
//   dequant8<T>  : exact dequantisation of 8 consecutive elements (bit-identical with the reference's CPU
//                  ref::dequant_row, tests/ref/dequant.cpp:34-120: same float association, no FMA contraction).
//   decode_unit<T> / dot_unit<T> : dot product of one 32-element unit of a weight row (staged in shared memory, 2-byte aligned) with
//                  the activation.  Quantised types multiply integer codes with a 16-bit fixed-point copy of the
//                  activation (two int8 limbs, dp4a), exact in int32 inside the unit, scaled and accumulated in fp32.
//                  Dense types (F32/F16/BF16) use fp32 FMAs.
// Block layouts as in the reference's src/kernels/quant_blocks.h:56,73,110,145 (IQ1_S {f16 d; u8 qs[32]; u16 qh[8]},
// IQ2_XXS {f16 d; u16 qs[32]}, Q6_K {ql[128]; qh[64]; i8 sc[16]; f16 d}, Q5_K {f16 d,dmin; sc[12]; qh[32]; qs[128]},
// Q8_0 {f16 d; i8 qs[32]}, IQ4_NL {f16 d; u8 qs[16]}).
#pragma once
#include "msb_common.cuh"

namespace msb {

// Shared-memory lookup tables hold 4-bit codes, eight per 32-bit entry (element k of an entry's 8 in the low nibble of
// byte k for k < 4, element k + 4 in the high nibble), and are replicated so that lanes of a warp hit disjoint banks:
// copy c of entry i is the word at i * copies + c.
//   IQ1_S  : nibble = grid value + 1 (0..2).  (entry & 0x0F0F0F0F) is a dp4a operand for elements 0..3 and
//            (entry & 0xF0F0F0F0) one for elements 4..7 scaled by 16, which an exact shift removes from the integer sum.
//   IQ2_XXS: grid nibble = magnitude code 0..2 (8, 25, 43), sign nibble = 3 for a negative element; their sum selects a
//            byte of the pool {8, 25, 43, -8, -25, -43} with one byte-permute per four elements.  Here the nibbles are in
//            element order (nibble k = element k), the order the permute's selector wants.
constexpr int kIq1sCopies = 8;    // 2048 x 4 B x 8  = 64 KB: four lanes share a copy
constexpr int kIq2Copies = 32;    // 256 x 4 B x 32 = 32 KB (grid) + 128 x 4 B x 32 = 16 KB (signs): one copy per lane
constexpr int kIq4Copies = 8;     // 256 x 4 B x 8  = 8 KB
constexpr size_t kIq1sLutBytes = 2048 * 4 * kIq1sCopies;
constexpr size_t kIq2GridLutBytes = 256 * 4 * kIq2Copies;
constexpr size_t kIq2SignLutBytes = 128 * 4 * kIq2Copies;
constexpr size_t kIq4LutBytes = 256 * 4 * kIq4Copies;

__host__ __device__ constexpr size_t lut_bytes_for(int t) {
  return t == IQ1_S ? kIq1sLutBytes : t == IQ2_XXS ? kIq2GridLutBytes + kIq2SignLutBytes : t == IQ4_NL ? kIq4LutBytes : 0;
}
__host__ __device__ constexpr bool is_dense(int t) { return t == F32 || t == F16 || t == BF16; }
// bytes of `units` 32-element units of one row (units a multiple of 8 for the 256-element super-block types)
__host__ __device__ constexpr int units_bytes(int t, int units) {
  return block_elems(t) == 256 ? (units / 8) * block_bytes(t) : block_elems(t) == 32 ? units * block_bytes(t)
                                                                                     : units * 32 * block_bytes(t);
}

#ifdef __CUDACC__
// Every hot-path shared-memory read goes through explicit ld.shared with 32-bit shared-space addresses: pointers that
// travel through structs lose their address space and would otherwise compile to generic loads.
typedef uint32_t saddr_t;
// Loads are explicit ld.shared instructions on 32-bit shared-space addresses (no generic-address arithmetic).  They are
// volatile asm statements: the compiler keeps them in program order relative to the mbarrier waits and named barriers
// (also volatile asm), and the assembler schedules them freely among the arithmetic.
__device__ __forceinline__ uint32_t lds_u8(saddr_t a) { uint32_t v; asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds_u16(saddr_t a) { uint32_t v; asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds_u32(saddr_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint2 lds_u64(saddr_t a) {
  uint2 v; asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v;
}
__device__ __forceinline__ uint4 lds_u128(saddr_t a) {
  uint4 v; asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v;
}
__device__ __forceinline__ float4 lds_f128(saddr_t a) {
  float4 v; asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a)); return v;
}

struct LaneLuts {      // per-lane shared-space base addresses (already offset to the lane's copy)
  saddr_t iq1s, iq2g, iq2s, iq4;
};

// Quantised activation in shared memory: U units of 32 elements.  x ~= scale * (256 * hi + lo), hi signed bytes,
// lo unsigned bytes.  plane[0][.] / plane[1][.] = hi bytes of elements 0..15 / 16..31, plane[2..3] = lo bytes.
// meta[.] = {scale, scale * sum of the fixed-point values, (int) sum over elements 0..15, (int) sum over 16..31}.
// In the padded form (used when a Q6_K or IQ1_S matrix reads it) unit u sits at slot u + u/8 of each array: one 16-byte slot
// of padding per 8 units, so that lanes that each walk their own half super-block (unit stride 4) reach distinct banks,
// as lanes on consecutive units do in either form.
struct XqSmem {
  uint4* plane;     // [4][S], S = xq_slots(U)
  float4* meta;     // [S]
  const float* xf;  // dense types: fp32 copy of x [32 U]
  saddr_t plane_s, meta_s, xf_s;   // the same locations as shared-space addresses
  int U, S;
  uint32_t padmask;   // all ones in the padded form, else 0
};
__host__ __device__ constexpr bool xq_padded(int t) { return t == Q6_K || t == IQ1_S; }
__host__ __device__ inline int xq_pos_padded(int u) { return u + (u >> 3); }
__host__ __device__ inline int xq_slots(int U, bool padded) { return padded ? U + ((U + 7) >> 3) : U; }
__host__ __device__ inline size_t xq_bytes(int U, bool dense, bool padded) {
  return dense ? (size_t)U * 128 : (size_t)xq_slots(U, padded) * 80;
}
__device__ __forceinline__ int xq_pos(const XqSmem& x, int u) { return u + (int)((uint32_t)(u >> 3) & x.padmask); }
__device__ __forceinline__ void xq_bind(XqSmem& x, uint8_t* base, int U, bool dense, bool padded) {
  x.U = U;
  x.S = xq_slots(U, padded);
  x.padmask = padded ? 0xFFFFFFFFu : 0u;
  x.plane_s = x.xf_s = smem_u32(base);
  x.meta_s = x.plane_s + (uint32_t)x.S * 64u;
  if (dense) { x.xf = reinterpret_cast<const float*>(base); x.plane = nullptr; x.meta = nullptr; }
  else { x.plane = reinterpret_cast<uint4*>(base); x.meta = reinterpret_cast<float4*>(base + (size_t)x.S * 64); x.xf = nullptr; }
}
struct XRegs { uint32_t h[8], l[8]; float s, sx; int sa, sb; };

__device__ __forceinline__ void load_xq(const XqSmem& x, int u, XRegs& r) {
  const uint32_t pos = (uint32_t)xq_pos(x, u);
  const saddr_t pa = x.plane_s + 16u * pos, st = 16u * (uint32_t)x.S;
  const uint4 a = lds_u128(pa), b = lds_u128(pa + st), c = lds_u128(pa + 2 * st), d = lds_u128(pa + 3 * st);
  const float4 m = lds_f128(x.meta_s + 16u * pos);
  r.h[0] = a.x; r.h[1] = a.y; r.h[2] = a.z; r.h[3] = a.w; r.h[4] = b.x; r.h[5] = b.y; r.h[6] = b.z; r.h[7] = b.w;
  r.l[0] = c.x; r.l[1] = c.y; r.l[2] = c.z; r.l[3] = c.w; r.l[4] = d.x; r.l[5] = d.y; r.l[6] = d.z; r.l[7] = d.w;
  r.s = m.x; r.sx = m.y; r.sa = __float_as_int(m.z); r.sb = __float_as_int(m.w);
}

// Quantise units of x (global or shared fp32, 16-byte aligned; unit u = elements [32 u, 32 u + 32)) into `q`, optionally
// scaling every element by `mul` first (fused RMSNorm: mul = rstd, and by gain[i] when gain is given).  Called by all
// `nthreads` threads of the block (a multiple of 32); 4 threads cooperate on one unit (8 elements each).  The v-th unit
// handled is unit_of(v), v = 0 .. n_units - 1 (a map lets a caller quantise only the rows it will read).  Caller
// synchronises afterwards.
template <class Map>
__device__ __forceinline__ void quantize_units(const float* __restrict__ x, const XqSmem& q, int tid, int nthreads, float mul,
                                               const float* __restrict__ gain, int n_units, Map unit_of) {
  const int lane4 = tid & 3;
  for (int base = 0; base < n_units * 4; base += nthreads) {
    const int item = base + tid;           // one item = 8 elements
    const bool live = item < n_units * 4;  // whole quads are live or not
    const int u = live ? unit_of(item >> 2) : 0;
    const int at = 32 * u + 8 * lane4;
    float v[8];
    if (live) {
      const float4 a = *reinterpret_cast<const float4*>(x + at);
      const float4 b = *reinterpret_cast<const float4*>(x + at + 4);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
      if (gain) {
        const float4 ga = *reinterpret_cast<const float4*>(gain + at);
        const float4 gb = *reinterpret_cast<const float4*>(gain + at + 4);
        v[0] = v[0] * mul * ga.x; v[1] = v[1] * mul * ga.y; v[2] = v[2] * mul * ga.z; v[3] = v[3] * mul * ga.w;
        v[4] = v[4] * mul * gb.x; v[5] = v[5] * mul * gb.y; v[6] = v[6] * mul * gb.z; v[7] = v[7] * mul * gb.w;
      } else if (mul != 1.f) {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] *= mul;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float inv = amax > 0.f ? 32767.f / amax : 0.f;
    // round to the nearest integer in [-32767, 32767] by adding 1.5 * 2^23: the sum's low 16 mantissa bits are the
    // two's-complement value (high byte signed, low byte unsigned), picked out with byte permutes; no clamp is needed,
    // |v * inv| <= 32767 (1 + 2^-22) rounds to at most 32767
    constexpr float kMagic = 12582912.f;
    uint32_t f[8];
#pragma unroll
    for (int i = 0; i < 8; i++) f[i] = __float_as_uint(fmaf(v[i], inv, kMagic));
    uint32_t hw[2], lw[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
      hw[j] = __byte_perm(__byte_perm(f[4 * j], f[4 * j + 1], 0x0051), __byte_perm(f[4 * j + 2], f[4 * j + 3], 0x0051), 0x5410);
      lw[j] = __byte_perm(__byte_perm(f[4 * j], f[4 * j + 1], 0x0040), __byte_perm(f[4 * j + 2], f[4 * j + 3], 0x0040), 0x5410);
    }
    // sum of the 8 fixed-point values = 256 * (sum of the signed high bytes) + (sum of the unsigned low bytes)
    const int sum = 256 * dp4a_ss(hw[1], 0x01010101u, dp4a_ss(hw[0], 0x01010101u, 0)) +
                    dp4a_uu(lw[1], 0x01010101u, dp4a_uu(lw[0], 0x01010101u, 0));
    const int pair = sum + __shfl_xor_sync(0xffffffffu, sum, 1);   // lanes (0,1): elements 0..15, (2,3): 16..31
    const int other = __shfl_xor_sync(0xffffffffu, pair, 2);
    if (live) {
      const int pos = xq_pos(q, u);
      uint2* ph = reinterpret_cast<uint2*>(&q.plane[(lane4 >> 1) * q.S + pos]) + (lane4 & 1);
      uint2* pl = reinterpret_cast<uint2*>(&q.plane[(2 + (lane4 >> 1)) * q.S + pos]) + (lane4 & 1);
      *ph = make_uint2(hw[0], hw[1]);
      *pl = make_uint2(lw[0], lw[1]);
      if (lane4 == 0) {
        const float sc = amax * (1.0f / 32767.f);
        q.meta[pos] = make_float4(sc, sc * (float)(pair + other), __int_as_float(pair), __int_as_float(other));
      }
    }
  }
}
__device__ __forceinline__ void quantize_x(const float* __restrict__ x, const XqSmem& q, int tid, int nthreads,
                                           float mul = 1.f, const float* __restrict__ gain = nullptr) {
  quantize_units(x, q, tid, nthreads, mul, gain, q.U, [](int v) { return v; });
}

__device__ __forceinline__ uint32_t lds_u32_a2(saddr_t p) { return lds_u16(p) | (lds_u16(p + 2) << 16); }
__device__ __forceinline__ float lds_half(saddr_t p) { return __half2float(__ushort_as_half((unsigned short)lds_u16(p))); }
// N consecutive little-endian 32-bit words starting at a 2-byte aligned shared address (reads one word past the end
// when the address is not 4-byte aligned; stage buffers are padded for that).
template <int N>
__device__ __forceinline__ void load_words(saddr_t p, uint32_t (&w)[N]) {
  const saddr_t a = p & ~3u;
  const uint32_t sh = (p & 2u) * 8u;
  uint32_t t[N + 1];
#pragma unroll
  for (int i = 0; i <= N; i++) t[i] = lds_u32(a + 4u * i);
#pragma unroll
  for (int i = 0; i < N; i++) w[i] = __funnelshift_r(t[i], t[i + 1], sh);
}

// ---------------------------------------------------------------- decode_unit / dot_unit: one 32-element unit of a row
// decode_unit turns the unit into 8 words of byte codes (element 4i+k in byte k of w[i]) plus the scalars needed to
// finish; dot_unit multiplies them with one quantised activation column.  Splitting the two lets several activation
// columns share one decode.
template <int T> struct Dec { uint32_t w[8]; float a, b; };
template <> struct Dec<Q6_K> { uint32_t w[8]; float a, s0, s1; };

template <int T>
__device__ __forceinline__ void decode_unit(saddr_t rowp, int u, const LaneLuts& L, Dec<T>& d);
template <int T>
__device__ __forceinline__ float dot_unit(const Dec<T>& d, const XRegs& x);

// ---- IQ1_S, one half super-block (4 units = 128 elements) of NRT rows against NC activation columns.
// weight = d (2 s_u + 1) (g + delta_u), g in {-1, 0, 1}, delta_u = +-1/8 per unit.  With the table's codes c = g + 1 and
// the unit's fixed-point activation x = xs_u * xi:
//   row . x = d * sum_u xs_u/8 * [ 8 (2 s_u + 1) sum_k c_k xi_k  +  (2 s_u + 1) (8 delta_u - 8) sum_k xi_k ]
// the bracket is an exact integer (8 delta - 8 = -7 or -9), converted to float once per unit and row.  A look-up returns
// 8 codes as nibbles; e = w & 0x0F0F0F0F multiplies elements 0..3, w - e (elements 4..7 scaled by 16) the other four,
// and an exact shift takes the 16 out of that partial sum.
// `blk[i]` = shared address of row i's block (2-byte aligned), `u0` = the half block's first unit in the activation.
__device__ __forceinline__ uint32_t sub_fma_pipe(uint32_t w, uint32_t e) {   // w - e as a multiply-add
  uint32_t o;
  asm("mad.lo.u32 %0, %1, 0xFFFFFFFF, %2;" : "=r"(o) : "r"(e), "r"(w));
  return o;
}
template <int NRT, int NC>
__device__ __forceinline__ void iq1s_half_block(const saddr_t (&blk)[NRT], int half, const XqSmem (&xq)[NC], int u0,
                                                const LaneLuts& L, float (&acc)[NRT][NC]) {
  uint32_t q[NRT][4], hw[NRT][2];
  float part[NRT][NC];
#pragma unroll
  for (int i = 0; i < NRT; i++) {
    load_words<4>(blk[i] + 2 + 16 * half, q[i]);
    load_words<2>(blk[i] + 34 + 8 * half, hw[i]);
#pragma unroll
    for (int c = 0; c < NC; c++) part[i][c] = 0.f;
  }
#pragma unroll
  for (int u = 0; u < 4; u++) {
    XRegs x[NC];
    float xs8[NC];
    int xi[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) { load_xq(xq[c], u0 + u, x[c]); xs8[c] = 0.125f * x[c].s; xi[c] = x[c].sa + x[c].sb; }
#pragma unroll
    for (int i = 0; i < NRT; i++) {
      // qh of the unit in the low 16 bits (for even u the next unit's word rides along above them; every use masks)
      const uint32_t h = (u & 1) ? (hw[i][u >> 1] >> 16) : hw[i][u >> 1];
      uint32_t w[4];
#pragma unroll
      for (int l = 0; l < 4; l++) {
        // entry address = lut + 4 copies * ((8-bit code) + 256 * (3 high bits)); the lane's copy is folded into L.iq1s
        const uint32_t hi = (h & (7u << (3 * l))) * ((1024u * kIq1sCopies) >> (3 * l)) + L.iq1s;
        w[l] = lds_u32(__byte_perm(q[i][u], 0, 0x4440 | l) * (4u * kIq1sCopies) + hi);
      }
      const int sc = (int)(((h >> 11) & 14u) | 1u);
      const int sg = (h & 0x8000u) ? -9 * sc : -7 * sc;
#pragma unroll
      for (int c = 0; c < NC; c++) {
        int he = 0, le = 0, ho = 0, lo = 0;
#pragma unroll
        for (int l = 0; l < 4; l++) {
          const uint32_t e = w[l] & 0x0F0F0F0Fu, o = sub_fma_pipe(w[l], e);
          he = dp4a_us(e, x[c].h[2 * l], he); le = dp4a_uu(e, x[c].l[2 * l], le);
          ho = dp4a_us(o, x[c].h[2 * l + 1], ho); lo = dp4a_uu(o, x[c].l[2 * l + 1], lo);
        }
        const int S = (he * 256 + le) + ((ho * 256 + lo) >> 4);
        part[i][c] = fmaf(xs8[c], (float)(8 * sc * S + sg * xi[c]), part[i][c]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NRT; i++) {
    const float d = lds_half(blk[i]);
#pragma unroll
    for (int c = 0; c < NC; c++) acc[i][c] = fmaf(d, part[i][c], acc[i][c]);
  }
}

// ---- IQ2_XXS: the grid entry's magnitude codes (0..2) plus 3 for a negative element select a byte of the pool
// {8, 25, 43, -8, -25, -43}: one addition and two byte-permutes per 8 elements
template <>
__device__ __forceinline__ void decode_unit<IQ2_XXS>(saddr_t rowp, int u, const LaneLuts& L, Dec<IQ2_XXS>& d) {
  constexpr uint32_t kPoolA = 0xF82B1908u, kPoolB = 0x0000D5E7u;   // bytes 8, 25, 43, -8 | -25, -43
  const saddr_t blk = rowp + (uint32_t)(u >> 3) * 66u;
  const saddr_t a8 = blk + 2 + 8 * (u & 7);
  const uint32_t q = lds_u32_a2(a8), a1 = lds_u32_a2(a8 + 4);
#pragma unroll
  for (int l = 0; l < 4; l++) {
    const uint32_t g = lds_u32(L.iq2g + __byte_perm(q, 0, 0x4440 | l) * (4 * kIq2Copies));
    const uint32_t m = lds_u32(L.iq2s + ((a1 >> (7 * l)) & 127u) * (4 * kIq2Copies));
    const uint32_t sel = g + m;
    d.w[2 * l] = __byte_perm(kPoolA, kPoolB, sel);
    d.w[2 * l + 1] = __byte_perm(kPoolA, kPoolB, sel >> 16);
  }
  d.a = lds_half(blk) * (0.5f + (float)(a1 >> 28)) * 0.25f;
  d.b = 0.f;
}
template <int T>
__device__ __forceinline__ float dot_signed(const Dec<T>& d, const XRegs& x) {
  int sh = 0, sl = 0, th = 0, tl = 0;
#pragma unroll
  for (int i = 0; i < 8; i += 2) {
    sh = dp4a_ss(d.w[i], x.h[i], sh); sl = dp4a_su(d.w[i], x.l[i], sl);
    th = dp4a_ss(d.w[i + 1], x.h[i + 1], th); tl = dp4a_su(d.w[i + 1], x.l[i + 1], tl);
  }
  return d.a * x.s * (float)((sh + th) * 256 + (sl + tl));
}
template <>
__device__ __forceinline__ float dot_unit<IQ2_XXS>(const Dec<IQ2_XXS>& d, const XRegs& x) { return dot_signed(d, x); }

// ---- Q8_0: the int8 codes as they are
template <>
__device__ __forceinline__ void decode_unit<Q8_0>(saddr_t rowp, int u, const LaneLuts&, Dec<Q8_0>& d) {
  const saddr_t blk = rowp + (uint32_t)u * 34u;
  load_words<8>(blk + 2, d.w);
  d.a = lds_half(blk);
  d.b = 0.f;
}
template <>
__device__ __forceinline__ float dot_unit<Q8_0>(const Dec<Q8_0>& d, const XRegs& x) { return dot_signed(d, x); }

// ---- IQ4_NL: nibble -> signed level through the byte-pair table
template <>
__device__ __forceinline__ void decode_unit<IQ4_NL>(saddr_t rowp, int u, const LaneLuts& L, Dec<IQ4_NL>& d) {
  const saddr_t blk = rowp + (uint32_t)u * 18u;
  uint32_t q[4];
  load_words<4>(blk + 2, q);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    uint32_t r[4];
#pragma unroll
    for (int k = 0; k < 4; k++)
      r[k] = lds_u32(L.iq4 + ((q[i] >> (8 * k)) & 0xFFu) * (4 * kIq4Copies));
    const uint32_t t01 = __byte_perm(r[0], r[1], 0x5140), t23 = __byte_perm(r[2], r[3], 0x5140);
    d.w[i] = __byte_perm(t01, t23, 0x5410);       // low nibbles  -> elements 4i .. 4i+3
    d.w[4 + i] = __byte_perm(t01, t23, 0x7632);   // high nibbles -> elements 16+4i ..
  }
  d.a = lds_half(blk);
  d.b = 0.f;
}
template <>
__device__ __forceinline__ float dot_unit<IQ4_NL>(const Dec<IQ4_NL>& d, const XRegs& x) { return dot_signed(d, x); }

// ---- Q6_K: codes 0..63 unsigned, two int8 scales per unit; sum (q - 32) x = sum q x - 32 sum x
template <>
__device__ __forceinline__ void decode_unit<Q6_K>(saddr_t rowp, int u, const LaneLuts&, Dec<Q6_K>& d) {
  const saddr_t blk = rowp + (uint32_t)(u >> 3) * 210u;
  const int j = u & 7, half = j >> 2, q = j & 3;
  uint32_t a[8], b[8];
  load_words<8>(blk + 64 * half + 32 * (q & 1), a);
  load_words<8>(blk + 128 + 32 * half, b);
  const int nsh = 4 * (q >> 1), hsh = 2 * q;
#pragma unroll
  for (int i = 0; i < 8; i++) d.w[i] = ((a[i] >> nsh) & 0x0F0F0F0Fu) | (((b[i] >> hsh) & 0x03030303u) << 4);
  const uint32_t sc = lds_u16(blk + 192 + 8 * half + 2 * q);   // two int8 scales (the address is even)
  d.a = lds_half(blk + 208);
  d.s0 = (float)(int8_t)(sc & 0xFFu);
  d.s1 = (float)(int8_t)(sc >> 8);
}
template <>
__device__ __forceinline__ float dot_unit<Q6_K>(const Dec<Q6_K>& d, const XRegs& x) {
  int h0 = 0, l0 = 0, h1 = 0, l1 = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    h0 = dp4a_us(d.w[i], x.h[i], h0); l0 = dp4a_uu(d.w[i], x.l[i], l0);
    h1 = dp4a_us(d.w[4 + i], x.h[4 + i], h1); l1 = dp4a_uu(d.w[4 + i], x.l[4 + i], l1);
  }
  return d.a * x.s * (d.s0 * (float)(h0 * 256 + l0 - 32 * x.sa) + d.s1 * (float)(h1 * 256 + l1 - 32 * x.sb));
}

// Q6_K, one half super-block (128 elements: units 4h .. 4h+3 of the block) of NRT rows against NC activation columns.
// The half's 64 ql bytes and 32 qh bytes are each read once: ql[0..31] serves sub-blocks 0 (low nibbles) and 2 (high),
// ql[32..63] sub-blocks 1 and 3, and qh supplies bits 4..5 of all four.  With m = 0x0F0F0F0F and
// hx = (qh >> 0 or 2) & 0x33333333 the code words are (ql & m) | ((hx << 4) & ~m) and ((ql >> 4) & m) | (hx & ~m): one
// shift and one three-input logic operation per word.  `blk[i]` = shared address of row i's block (2-byte aligned),
// `u0` = index of the half's first unit in the activation.
template <int NRT, int NC>
__device__ __forceinline__ void q6k_half_block(const saddr_t (&blk)[NRT], int half, const XqSmem (&xq)[NC], int u0,
                                               float (&acc)[NRT][NC]) {
  constexpr uint32_t m = 0x0F0F0F0Fu;
  uint32_t scw[NRT][2];
  float d[NRT], part[NRT][NC];
  uint32_t hk[NRT][8];
#pragma unroll
  for (int i = 0; i < NRT; i++) {
    load_words<2>(blk[i] + 192 + 8 * half, scw[i]);
    d[i] = lds_half(blk[i] + 208);
    load_words<8>(blk[i] + 128 + 32 * half, hk[i]);
#pragma unroll
    for (int c = 0; c < NC; c++) part[i][c] = 0.f;
  }
#pragma unroll
  for (int P = 0; P < 2; P++) {
    uint32_t ql[NRT][8], hx[NRT][8];
#pragma unroll
    for (int i = 0; i < NRT; i++) {
      load_words<8>(blk[i] + 64 * half + 32 * P, ql[i]);
#pragma unroll
      for (int g = 0; g < 8; g++) hx[i][g] = (P == 0 ? hk[i][g] : (hk[i][g] >> 2)) & 0x33333333u;
    }
#pragma unroll
    for (int jj = 0; jj < 2; jj++) {
      const int j = P + 2 * jj;                       // sub-block (unit) inside the half
      const uint32_t pos = (uint32_t)xq_pos_padded(u0 + j);
      float sub[NRT][NC];
#pragma unroll
      for (int i = 0; i < NRT; i++)
#pragma unroll
        for (int c = 0; c < NC; c++) sub[i][c] = 0.f;
      float xs[NC];
#pragma unroll
      for (int is = 0; is < 2; is++) {
        uint32_t w[NRT][4];
#pragma unroll
        for (int i = 0; i < NRT; i++)
#pragma unroll
          for (int k = 0; k < 4; k++) {
            const int g = 4 * is + k;
            w[i][k] = jj == 0 ? ((ql[i][g] & m) | ((hx[i][g] << 4) & ~m)) : (((ql[i][g] >> 4) & m) | (hx[i][g] & ~m));
          }
#pragma unroll
        for (int c = 0; c < NC; c++) {
          const uint32_t st = 16u * (uint32_t)xq[c].S;
          const uint4 xh = lds_u128(xq[c].plane_s + 16u * pos + st * is);
          const uint4 xl = lds_u128(xq[c].plane_s + 16u * pos + st * (2 + is));
          const float4 mt = lds_f128(xq[c].meta_s + 16u * pos);
          xs[c] = mt.x;
          const int s16 = __float_as_int(is == 0 ? mt.z : mt.w);
#pragma unroll
          for (int i = 0; i < NRT; i++) {
            int h = dp4a_us(w[i][0], xh.x, 0), l = dp4a_uu(w[i][0], xl.x, 0);
            h = dp4a_us(w[i][1], xh.y, h); l = dp4a_uu(w[i][1], xl.y, l);
            h = dp4a_us(w[i][2], xh.z, h); l = dp4a_uu(w[i][2], xl.z, l);
            h = dp4a_us(w[i][3], xh.w, h); l = dp4a_uu(w[i][3], xl.w, l);
            const int sidx = 2 * j + is;
            const float sc = (float)(int8_t)((scw[i][sidx >> 2] >> (8 * (sidx & 3))) & 0xFFu);
            sub[i][c] = fmaf(sc, (float)(h * 256 + l - 32 * s16), sub[i][c]);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < NRT; i++)
#pragma unroll
        for (int c = 0; c < NC; c++) part[i][c] = fmaf(xs[c], sub[i][c], part[i][c]);
    }
  }
#pragma unroll
  for (int i = 0; i < NRT; i++)
#pragma unroll
    for (int c = 0; c < NC; c++) acc[i][c] = fmaf(d[i], part[i][c], acc[i][c]);
}

// ---- Q5_K: codes 0..31 unsigned, y = (d * scale) q - dmin * min
template <>
__device__ __forceinline__ void decode_unit<Q5_K>(saddr_t rowp, int u, const LaneLuts&, Dec<Q5_K>& d) {
  const saddr_t blk = rowp + (uint32_t)(u >> 3) * 176u;
  const int j = u & 7;
  const saddr_t sc = blk + 4;
  uint32_t scale, mn;
  if (j < 4) { scale = lds_u8(sc + j) & 63u; mn = lds_u8(sc + j + 4) & 63u; }
  else {
    const uint32_t hi = lds_u8(sc + j + 4);
    scale = (hi & 0xFu) | ((lds_u8(sc + j - 4) >> 6) << 4);
    mn = (hi >> 4) | ((lds_u8(sc + j) >> 6) << 4);
  }
  uint32_t a[8], b[8];
  load_words<8>(blk + 48 + 32 * (j >> 1), a);
  load_words<8>(blk + 16, b);
  const int nsh = 4 * (j & 1);
#pragma unroll
  for (int i = 0; i < 8; i++) d.w[i] = ((a[i] >> nsh) & 0x0F0F0F0Fu) | (((b[i] >> j) & 0x01010101u) << 4);
  d.a = lds_half(blk) * (float)scale;
  d.b = lds_half(blk + 2) * (float)mn;
}
template <>
__device__ __forceinline__ float dot_unit<Q5_K>(const Dec<Q5_K>& d, const XRegs& x) {
  int sh = 0, sl = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) { sh = dp4a_us(d.w[i], x.h[i], sh); sl = dp4a_uu(d.w[i], x.l[i], sl); }
  return d.a * (x.s * (float)(sh * 256 + sl)) - d.b * x.sx;
}

// ---------------------------------------------------------------- exact dequantisation of 8 consecutive elements
// `blk` points at the block in GLOBAL memory (2-byte aligned), e8 = index of the 8-element group inside the block.
__device__ __forceinline__ uint32_t ldg_u16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); }
__device__ __forceinline__ float ldg_half(const uint8_t* p) { return __half2float(__ushort_as_half((unsigned short)ldg_u16(p))); }

template <int T>
__device__ __forceinline__ void dequant8(const uint8_t* blk, int e8, const Tables& tb, float (&y)[8]);

template <>
__device__ __forceinline__ void dequant8<Q8_0>(const uint8_t* blk, int e8, const Tables&, float (&y)[8]) {
  const float d = ldg_half(blk);
#pragma unroll
  for (int j = 0; j < 8; j++) y[j] = __fmul_rn((float)(int8_t)__ldg(blk + 2 + 8 * e8 + j), d);
}
template <>
__device__ __forceinline__ void dequant8<IQ4_NL>(const uint8_t* blk, int e8, const Tables& tb, float (&y)[8]) {
  const float d = ldg_half(blk);
  const int hi = e8 >> 1, off = 8 * (e8 & 1);      // elements 0..15 = low nibbles of qs[0..15], 16..31 = high nibbles
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const uint32_t pr = __ldg(tb.iq4nl_pair + __ldg(blk + 2 + off + j));
    y[j] = __fmul_rn(d, (float)(int8_t)(hi ? (pr >> 8) : (pr & 0xFF)));
  }
}
template <>
__device__ __forceinline__ void dequant8<IQ1_S>(const uint8_t* blk, int e8, const Tables& tb, float (&y)[8]) {
  const int ib = e8 >> 2, l = e8 & 3;
  const uint32_t qh = ldg_u16(blk + 34 + 2 * ib);
  const float dl = __fmul_rn(ldg_half(blk), (float)(2 * ((qh >> 12) & 7u) + 1));
  const float delta = (qh & 0x8000u) ? -0.125f : 0.125f;
  const uint32_t idx = __ldg(blk + 2 + 4 * ib + l) | (((qh >> (3 * l)) & 7u) << 8);
  const uint2 gv = __ldg(reinterpret_cast<const uint2*>(tb.iq1s_i8 + idx * 8));   // the entry's 8 signed bytes at once
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const int8_t gj = (int8_t)(((j < 4 ? gv.x : gv.y) >> (8 * (j & 3))) & 0xFFu);
    y[j] = __fmul_rn(dl, __fadd_rn((float)gj, delta));
  }
}
template <>
__device__ __forceinline__ void dequant8<IQ2_XXS>(const uint8_t* blk, int e8, const Tables& tb, float (&y)[8]) {
  const int ib = e8 >> 2, l = e8 & 3;
  const uint8_t* a8 = blk + 2 + 8 * ib;
  const uint32_t a1 = ldg_u16(a8 + 4) | (ldg_u16(a8 + 6) << 16);
  const float db = __fmul_rn(__fmul_rn(ldg_half(blk), __fadd_rn(0.5f, (float)(a1 >> 28))), 0.25f);
  const uint2 g = __ldg(tb.iq2xxs_grid + __ldg(a8 + l));
  const uint2 m = __ldg(tb.iq2_signmask + ((a1 >> (7 * l)) & 127u));
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const uint32_t gv = ((j < 4 ? g.x : g.y) >> (8 * (j & 3))) & 0xFFu;
    const bool neg = ((j < 4 ? m.x : m.y) >> (8 * (j & 3))) & 1u;
    y[j] = __fmul_rn(__fmul_rn(db, (float)gv), neg ? -1.f : 1.f);
  }
}
template <>
__device__ __forceinline__ void dequant8<Q6_K>(const uint8_t* blk, int e8, const Tables&, float (&y)[8]) {
  // element e = 128*half + 32*q + l  (q = 0..3, l = 0..31): ql byte 64*half + 32*(q&1) + l, nibble q>>1;
  // qh byte 128 + 32*half + l, bits 2q..2q+1; scale sc[8*half + 2*q + l/16]
  const int e = 8 * e8, half = e >> 7, q = (e >> 5) & 3, l0 = e & 31;
  const float d = ldg_half(blk + 208);
  const float sc = (float)(int8_t)__ldg(blk + 192 + 8 * half + 2 * q + (l0 >> 4));
  const float ds = __fmul_rn(d, sc);
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const uint32_t ql = __ldg(blk + 64 * half + 32 * (q & 1) + l0 + j), qh = __ldg(blk + 128 + 32 * half + l0 + j);
    const int v = (int)(((ql >> (4 * (q >> 1))) & 0xFu) | (((qh >> (2 * q)) & 3u) << 4)) - 32;
    y[j] = __fmul_rn(ds, (float)v);
  }
}
template <>
__device__ __forceinline__ void dequant8<Q5_K>(const uint8_t* blk, int e8, const Tables&, float (&y)[8]) {
  const int e = 8 * e8, j = e >> 5, l0 = e & 31;          // sub-block j = 0..7
  const uint8_t* sc = blk + 4;
  uint32_t scale, mn;
  if (j < 4) { scale = __ldg(sc + j) & 63u; mn = __ldg(sc + j + 4) & 63u; }
  else {
    scale = (__ldg(sc + j + 4) & 0xFu) | ((__ldg(sc + j - 4) >> 6) << 4);
    mn = (__ldg(sc + j + 4) >> 4) | ((__ldg(sc + j) >> 6) << 4);
  }
  const float d1 = __fmul_rn(ldg_half(blk), (float)scale), m1 = __fmul_rn(ldg_half(blk + 2), (float)mn);
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const uint32_t ql = __ldg(blk + 48 + 32 * (j >> 1) + l0 + i), qh = __ldg(blk + 16 + l0 + i);
    const int v = (int)((ql >> (4 * (j & 1))) & 0xFu) + (int)((qh >> j) & 1u) * 16;
    y[i] = __fsub_rn(__fmul_rn(d1, (float)v), m1);
  }
}
#endif  // __CUDACC__

}  // namespace msb
