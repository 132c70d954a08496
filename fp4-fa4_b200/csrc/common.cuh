// Shared device/host helpers: status plumbing, number-format conversions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/fa4b.h"

namespace fa4b {

void set_error(const char* fmt, ...);
int sm_count();  // multiprocessors of the current device, cached per device; 0 when the query fails

#define FA4B_REQUIRE(cond, status, ...)        \
  do {                                         \
    if (!(cond)) {                             \
      ::fa4b::set_error(__VA_ARGS__);          \
      return (status);                         \
    }                                          \
  } while (0)

#define FA4B_CUDA(call)                                                          \
  do {                                                                           \
    cudaError_t e__ = (call);                                                    \
    if (e__ != cudaSuccess) {                                                    \
      ::fa4b::set_error("%s failed: %s", #call, cudaGetErrorString(e__));        \
      return FA4B_CUDA_ERROR;                                                    \
    }                                                                            \
  } while (0)

constexpr float kFltMin = 1.17549435e-38f;
constexpr float kNvfp4GlobalDiv = 2688.0f;  // 6 * 448

// ---- conversions ------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) { return __uint_as_float(b16 << 16); }

// two f32 -> one byte of two E2M1 codes; `lo` lands in the low nibble
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// two f32 -> two E4M3 bytes (lo in bits 0-7)
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t cvt_e5m2x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// four f32 -> four bytes of one register (a in bits 0-7): the two conversions write its halves, nothing merges them afterwards
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  uint32_t r;
  asm("{ .reg .b16 lo, hi; cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1; cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3; mov.b32 %0, {lo, hi}; }"
      : "=r"(r)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}
__device__ __forceinline__ uint32_t cvt_e5m2x4(float a, float b, float c, float d) {
  uint32_t r;
  asm("{ .reg .b16 lo, hi; cvt.rn.satfinite.e5m2x2.f32 lo, %2, %1; cvt.rn.satfinite.e5m2x2.f32 hi, %4, %3; mov.b32 %0, {lo, hi}; }"
      : "=r"(r)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
  uint32_t h2;
  uint16_t in = (uint16_t)byte;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffff)));
}
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  float mag;
  switch (code & 7u) {
    case 0: mag = 0.f; break;
    case 1: mag = .5f; break;
    case 2: mag = 1.f; break;
    case 3: mag = 1.5f; break;
    case 4: mag = 2.f; break;
    case 5: mag = 3.f; break;
    case 6: mag = 4.f; break;
    default: mag = 6.f; break;
  }
  return (code & 8u) ? -mag : mag;
}

// one byte of two E2M1 codes -> packed f16 pair (low nibble first)
__device__ __forceinline__ uint32_t e2m1x2_to_f16x2(uint32_t byte) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(r) : "r"(byte));
  return r;
}
__device__ __forceinline__ uint32_t hadd2_bits(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// ---- packed FP32 pairs (sm_100 executes fma/add/mul on two floats per instruction) ----
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack2u(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x of a packed pair on the FMA pipe instead of the exponential unit (which delivers 16 results per clock and
// SM and bounds the forward's softmax): n = floor(x) from a round-down add of 1.5 * 2^23 (the low significand bits of
// the sum are n), f = x - n in [0, 1) exactly, 2^f by a degree-3 polynomial (relative minimax fit on [0, 1], error
// <= 7.5e-5 -- an E4M3 probability keeps 3 significand bits), and n added into the exponent field.  x is clamped
// at -125 so that the exponent field stays positive.  The idea of the reference's exponential emulation
// (tk_fa4/fp4_fa4_fwd/stage2_ex2_alu_helpers.cuh:7-50); coefficients fitted for this build.
constexpr float kEx2C0 = 0.9999251961708069f, kEx2C1 = 0.6958335638046265f, kEx2C2 = 0.22606715559959412f, kEx2C3 = 0.07802452147006989f;
__device__ __forceinline__ uint64_t ex2_poly2(uint64_t x2) {
  float a, b;
  unpack2(x2, a, b);
  x2 = pack2(fmaxf(a, -125.0f), fmaxf(b, -125.0f));
  uint64_t t;
  asm("add.rm.ftz.f32x2 %0, %1, %2;" : "=l"(t) : "l"(x2), "l"(pack2(12582912.0f, 12582912.0f)));
  const uint64_t n = add2(t, pack2(-12582912.0f, -12582912.0f));   // exact
  const uint64_t f = fma2(n, pack2(-1.0f, -1.0f), x2);            // exact
  uint64_t p = fma2(f, pack2(kEx2C3, kEx2C3), pack2(kEx2C2, kEx2C2));
  p = fma2(f, p, pack2(kEx2C1, kEx2C1));
  p = fma2(f, p, pack2(kEx2C0, kEx2C0));
  uint32_t t0, t1, p0, p1;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(t0), "=r"(t1) : "l"(t));
  asm("mov.b64 {%0, %1}, %2;" : "=r"(p0), "=r"(p1) : "l"(p));
  return pack2u(p0 + (t0 << 23), p1 + (t1 << 23));
}
// which of a row's key columns take the polynomial: 6 of every 16 (pairs 1, 4 and 6 of each eight pairs), the share the
// reference moves off the exponential unit (hao_direct_config.inc:47-50); the oracle applies the same rule to the same keys
__device__ __host__ constexpr bool ex2_pair_on_fma(int pair) { return (pair & 7) == 1 || (pair & 7) == 4 || (pair & 7) == 6; }

// byte offset of the scale of (row, kblock) inside its 512-byte page
__device__ __host__ __forceinline__ uint32_t page_offset(uint32_t row, uint32_t kblock) {
  return (row & 31u) * 16u + ((row & 127u) >> 5) * 4u + (kblock & 3u);
}

// ---- division by a block's step without a divide per element ------------------------------
// q = RN(x / d) from r = RN(1 / d):  q0 = RN(x r),  e = x - d q0 (exact in one FMA),  q = RN(q0 + e r).
// That is the correctly rounded quotient whenever r is the correctly rounded reciprocal and d's
// significand is not all ones (Markstein's theorem); callers send such a d down the division path.
__device__ __forceinline__ uint64_t div2_exact(uint64_t x2, uint64_t r2, uint64_t neg_d2) {
  const uint64_t q0 = mul2(x2, r2);
  return fma2(fma2(q0, neg_d2, x2), r2, q0);
}
__device__ __forceinline__ bool significand_all_ones(float d) { return (__float_as_uint(d) & 0x7FFFFFu) == 0x7FFFFFu; }
// two bf16 in one word -> packed f32 pair (low half first)
__device__ __forceinline__ uint64_t bf16x2_to_f32x2(uint32_t w) { return pack2u(w << 16, w & 0xFFFF0000u); }
// |a|, |b| element-wise maximum of packed bf16 pairs
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t acc, uint32_t w) {
  const __nv_bfloat162 m = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&acc), __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w)));
  return *reinterpret_cast<const uint32_t*>(&m);
}
// max(m, |a|, |b|) in one three-input maximum (the absolute values fold into its operands)
__device__ __forceinline__ float absmax3(float m, uint64_t pair) {
  float a, b, r;
  unpack2(pair, a, b);
  asm("{ .reg .f32 aa, bb; abs.f32 aa, %2; abs.f32 bb, %3; max.f32 %0, %1, aa, bb; }" : "=f"(r) : "f"(m), "f"(a), "f"(b));
  return r;
}
// four packed f32 pairs -> eight E2M1 codes in one word (element 0 in the low nibble of byte 0); the four
// conversions write the bytes of one register, so no masks or merges follow them
__device__ __forceinline__ uint32_t e2m1_pack8(uint64_t q0, uint64_t q1, uint64_t q2, uint64_t q3) {
  uint32_t r;
  asm("{ .reg .b8 t0, t1, t2, t3; .reg .f32 a0, a1, b0, b1, c0, c1, d0, d1;\n\t"
      "mov.b64 {a0, a1}, %1; mov.b64 {b0, b1}, %2; mov.b64 {c0, c1}, %3; mov.b64 {d0, d1}, %4;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t0, a1, a0;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t1, b1, b0;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t2, c1, c0;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t3, d1, d0;\n\t"
      "mov.b32 %0, {t0, t1, t2, t3}; }"
      : "=r"(r)
      : "l"(q0), "l"(q1), "l"(q2), "l"(q3));
  return r;
}
// eight packed f32 pairs -> sixteen E2M1 codes (two words)
__device__ __forceinline__ void e2m1_pack16(const uint64_t (&q)[8], uint32_t& lo, uint32_t& hi) {
  lo = e2m1_pack8(q[0], q[1], q[2], q[3]);
  hi = e2m1_pack8(q[4], q[5], q[6], q[7]);
}
// NVFP4 scale byte E4M3(clamp(bamax / 6 / g)) from one multiplication by inv6g ~ 1 / (6 g).  The
// product is within 3 ulp of the twice-rounded quotient; every E4M3 rounding boundary has zero low
// 19 significand bits, so a product more than 16 ulp away from such a pattern rounds to the same
// byte, and the rare closer one takes the two divisions.  A zero (or vanishing) product is byte 0
// either way and stays on the short path: all-zero blocks are common.
__device__ __forceinline__ uint32_t nvfp4_scale_byte(float bamax, float g, float inv6g) {
  float s = bamax * inv6g;
  const uint32_t u = __float_as_uint(s) + 16u;
  if ((u & 0x7FFFFu) <= 32u && u > 32u) s = (bamax / 6.0f) / g;
  return cvt_e4m3x2(s, 0.f) & 0xffu;
}
// per-tensor table over the 127 scale bytes: step d = max(E4M3(byte) g, FLT_MIN) and r = RN(1 / d)
// (r = 0 marks a step whose significand is all ones: divide).  128 threads fill it.
struct StepTable {
  float2 e[128];  // .x = d, .y = r: one shared-memory read per block
};
__device__ __forceinline__ void fill_step_table(StepTable& tab, float g, int t) {
  if (t < 128) {
    const float dec = (t < 127) ? e4m3_to_f32((uint32_t)t) : 0.f;
    const float d = fmaxf(dec * g, kFltMin);
    tab.e[t] = make_float2(d, significand_all_ones(d) ? 0.f : __frcp_rn(d));
  }
}
// sixteen values (eight packed pairs, largest magnitude `bamax`) divided by the step of scale byte
// `sb`.  A block whose quotients could overflow (a step clamped to FLT_MIN under values of ordinary
// size) divides: inf - inf in the correction would lose the sign that saturation keeps.
__device__ __forceinline__ void nvfp4_codes16(const uint64_t (&x)[8], float bamax, const StepTable& tab, uint32_t sb, uint32_t& lo,
                                              uint32_t& hi) {
  const float2 e = tab.e[sb];
  const float d = e.x, r = e.y;
  uint64_t q[8];
  if (r != 0.f && bamax * r < 1.0e38f) {
    const uint64_t r2 = pack2(r, r), nd2 = pack2(-d, -d);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = div2_exact(x[i], r2, nd2);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float a, c;
      unpack2(x[i], a, c);
      q[i] = pack2(a / d, c / d);
    }
  }
  e2m1_pack16(q, lo, hi);
}

// Encode-centric recipe of the TK quantiser (TK_quantisation/nvfp4_v6/core.cuh:47-60, 86-101;
// fused_amax_quantize.cuh:235-256): the block's multiplier M = E4M3(6 / (bamax * S_enc)) is what is rounded, the
// stored scale is E4M3(1 / M), and every element is one multiplication by M * S_enc before the E2M1 rounding.
// Per-tensor table over the 127 multiplier bytes: .x = M * S_enc, .y = the stored scale byte (as an integer's bits).
struct EncodeTable {
  float2 e[128];
};
__device__ __forceinline__ void fill_encode_table(EncodeTable& tab, float s_enc, int t) {
  if (t < 128) {
    const float m = (t < 127) ? e4m3_to_f32((uint32_t)t) : 0.f;
    tab.e[t] = make_float2(m * s_enc, __uint_as_float(cvt_e4m3x2(1.0f / m, 0.f) & 0xffu));
  }
}
// The multiplier byte from an approximate quotient (two instructions, within 2 ulp for the magnitudes a block can
// have); the quotient that lands within 16 ulp of an E4M3 rounding boundary (zero low 19 bits) is divided properly.
__device__ __forceinline__ void nvfp4_codes16_encode(const uint64_t (&x)[8], float bamax, float s_enc, const EncodeTable& tab, uint32_t& sb,
                                                     uint32_t& lo, uint32_t& hi) {
  const float v = bamax * s_enc;
  float u = fminf(__fdividef(6.0f, v), 3.4028235e38f);
  const uint32_t ub = __float_as_uint(u) + 16u;
  if ((ub & 0x7FFFFu) <= 32u || !(v >= 1.0e-30f)) u = fminf(6.0f / v, 3.4028235e38f);
  const uint32_t mbyte = bamax <= 1.0e-9f ? 0x7eu : (cvt_e4m3x2(u, 0.f) & 0xffu);
  const float2 e = tab.e[mbyte];
  sb = __float_as_uint(e.y);
  const uint64_t c2 = pack2(e.x, e.x);
  uint64_t q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = mul2(x[i], c2);
  e2m1_pack16(q, lo, hi);
}

}  // namespace fa4b
