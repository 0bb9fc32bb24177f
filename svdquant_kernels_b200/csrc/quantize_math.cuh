// Per-group arithmetic of the activation quantizer, shared by both fused kernels.
//
// Results follow baseline/kernels/quantize_w4a4_act_fuse_lora/ref.py:40-48 and
// baseline/kernels/_nvfp4.py:27-41, :82-91 of the reference bit for bit; none of it
// runs a per-element IEEE divide.  Two fp32 lanes at a time where the hardware has
// a packed instruction (mul / fma on f32x2), three-input |max| for the group amax,
// and a 128-entry table in shared memory for the two constants that depend on the
// scale byte.
//
// Smoothing divide.  x / s must equal the IEEE quotient.  With r_hi = RU(1/s) (rounded up) and
// r_lo = RN(1/s - r_hi) <= 0, r_hi + r_lo equals 1/s to 2^-47, and q = fma(x, r_hi, RN(x * r_lo)) is
// the correctly rounded quotient for operands of at most 11 significant bits: such a quotient is
// never closer than 2^-36 (relative) to a midpoint between two fp32 numbers, unless it is exactly
// representable (checked exhaustively over mantissa pairs on the CPU).  Rounding r_hi UP makes r_lo
// non-positive (-0 when 1/s is exact), which is what turns a -0 input into a +0 quotient:
// (-0) * r_lo = +0 and (-0) * r_hi + (+0) = +0, as the reference's sign rule needs.  Nothing may
// over- or underflow: the table builder sets a flag when a smooth value lies outside the safe range,
// and then stores {s0, s1, -, -} for the kernels to divide with __fdiv_rn.  Per column pair the table
// holds {r_hi0, r_hi1, r_lo0, r_lo1}.
//
// Codes.  The scale byte is J * 2^E (J = 1..15), so m = trunc(4 v / 2^E) is an integer
// with v's sign and the E2M1 code is the number of n in {1,3,5,7,10,14,20} with
// n J <= |m|.  m / (4 J) lies on a rounding bound of E2M1 exactly when |m| = n J and at
// least 1/(4 J) away from every bound otherwise, so RN(m * RN(1/(4 J)) * (1 + 2^-20))
// is strictly above the bound in the first case and on the right side of it in the
// second, and the hardware conversion cvt.rn.satfinite.e2m1x2.f32 of it returns the
// reference's code, sign included (checked exhaustively over J and m on the CPU).
// Groups whose scale byte is 0 (everything non-zero saturates) or the 448 clamp
// (ratios are unbounded) compare against the seven exact products instead.
#pragma once

#include "nvfp4_math.cuh"


namespace svdq {
namespace qmath {

// Widen a pair of 16-bit values.  CANON adds +0 first, which turns -0 into +0 and changes nothing
// else (the reference gives a zero the sign bit only when the value tests < 0).  The smoothing
// divide of the fast path does the same by itself (see above), so only the other paths ask for it.
template <typename T, bool CANON> __device__ __forceinline__ float2 unpack2(uint32_t v);
template <> __device__ __forceinline__ float2 unpack2<__half, true>(uint32_t v) {
  return __half22float2(__hadd2(*reinterpret_cast<__half2*>(&v), __float2half2_rn(0.0f)));
}
template <> __device__ __forceinline__ float2 unpack2<__half, false>(uint32_t v) {
  return __half22float2(*reinterpret_cast<__half2*>(&v));
}
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16, true>(uint32_t v) {
  const __nv_bfloat162 c = __hadd2(*reinterpret_cast<__nv_bfloat162*>(&v), __float2bfloat162_rn(0.0f));
  const uint32_t u = *reinterpret_cast<const uint32_t*>(&c);
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16, false>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
}

template <typename T, bool CANON>
__device__ __forceinline__ void unpack_group(const uint4& lo16, const uint4& hi16, float2 (&f)[8]) {
  const uint32_t w[8] = {lo16.x, lo16.y, lo16.z, lo16.w, hi16.x, hi16.y, hi16.z, hi16.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = unpack2<T, CANON>(w[j]);
}

// Smoothing divide of one 16-element group; tb points at the group's eight table entries in shared
// memory (the same address in every lane of a quad column): {r_hi0, r_hi1, r_lo0, r_lo1}, or
// {s0, s1, -, -} when the launch divides with __fdiv_rn.
__device__ __forceinline__ void smooth_divide(float2 (&f)[8], const float4* tb, bool use_fdiv) {
  if (!use_fdiv) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 t = tb[j];
      f[j] = __ffma2_rn(f[j], make_float2(t.x, t.y), __fmul2_rn(f[j], make_float2(t.z, t.w)));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 t = tb[j];
      f[j].x = __fadd_rn(__fdiv_rn(f[j].x, t.x), 0.0f);           // an underflow to -0 counts as +0
      f[j].y = __fadd_rn(__fdiv_rn(f[j].y, t.y), 0.0f);
    }
  }
}

// Two rows of the same 16 columns: every table entry is loaded once.  A 16-byte shared-memory load costs
// four wavefronts of the load/store unit however many lanes share its address, and that unit (x loads, table
// loads, the stores, the MMA's operand reads and the TMA's writes all pass through it) is what the fused
// quantizer saturates.
__device__ __forceinline__ void smooth_divide2(float2 (&f0)[8], float2 (&f1)[8], const float4* tb, bool use_fdiv) {
  if (!use_fdiv) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 t = tb[j];
      const float2 hi = make_float2(t.x, t.y), lo = make_float2(t.z, t.w);
      f0[j] = __ffma2_rn(f0[j], hi, __fmul2_rn(f0[j], lo));
      f1[j] = __ffma2_rn(f1[j], hi, __fmul2_rn(f1[j], lo));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 t = tb[j];
      f0[j].x = __fadd_rn(__fdiv_rn(f0[j].x, t.x), 0.0f);          // an underflow to -0 counts as +0
      f0[j].y = __fadd_rn(__fdiv_rn(f0[j].y, t.y), 0.0f);
      f1[j].x = __fadd_rn(__fdiv_rn(f1[j].x, t.x), 0.0f);
      f1[j].y = __fadd_rn(__fdiv_rn(f1[j].y, t.y), 0.0f);
    }
  }
}

// Table entry of one column pair (see above); `exact_divide` selects the {s0, s1} form.
__device__ __forceinline__ float4 smooth_table_entry(float s0, float s1, bool exact_divide) {
  if (exact_divide) return make_float4(s0, s1, 0.0f, 0.0f);
  const float h0 = __frcp_ru(s0), h1 = __frcp_ru(s1);
  const float e0 = fmaf(-s0, h0, 1.0f), e1 = fmaf(-s1, h1, 1.0f);   // exact: 1 - s * r_hi, <= 0
  return make_float4(h0, h1, e0 == 0.0f ? -0.0f : __fmul_rn(e0, h0), e1 == 0.0f ? -0.0f : __fmul_rn(e1, h1));
}

// {2^(2-E), RN(1/(4 J)) (1 + 2^-20)} of scale byte sb = J 2^E; {0, 0} for the two bytes that take the compare path
__device__ __forceinline__ float2 scale_constants(uint32_t sb) {
  if (sb == 0u || sb >= 0x7Eu) return make_float2(0.0f, 0.0f);
  const uint32_t e = sb >> 3, m3 = sb & 7u;
  const uint32_t J = e ? 8u + m3 : m3;
  const float mult = __uint_as_float((e ? 139u - e : 138u) << 23);
  const float rj = __fmul_rn(__frcp_rn(static_cast<float>(4u * J)), 1.00000095367431640625f);
  return make_float2(mult, rj);
}
constexpr int kScaleLutEntries = 128;
__device__ __forceinline__ void fill_scale_lut(float2* lut, int tid, int nthreads) {
  for (int i = tid; i < kScaleLutEntries; i += nthreads) lut[i] = scale_constants(static_cast<uint32_t>(i));
}

__device__ __forceinline__ float max3abs(float a, float b, float c) {
  float r;
  asm("max.abs.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Four pairs of floats -> eight E2M1 codes in one word (element 2j in bits 8j..8j+3, element 2j+1
// above it), round to nearest, saturating, sign included.
__device__ __forceinline__ uint32_t cvt_e2m1x8(float2 a, float2 b, float2 c, float2 d) {
  uint32_t r;
  asm("{\n\t.reg .b8 q0, q1, q2, q3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 q0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 q1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 q2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 q3, %8, %7;\n\t"
      "mov.b32 %0, {q0, q1, q2, q3};\n\t}"
      : "=r"(r)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y), "f"(d.x), "f"(d.y));
  return r;
}

// amax of a 16-element group -> scale byte: e4m3(clamp(amax / 6, 1e-12, 448)), the divide correctly rounded
__device__ __forceinline__ uint32_t group_scale_byte(const float2 (&f)[8]) {
  const float m0 = max3abs(f[0].x, f[0].y, f[1].x), m1 = max3abs(f[1].y, f[2].x, f[2].y);
  const float m2 = max3abs(f[3].x, f[3].y, f[4].x), m3 = max3abs(f[4].y, f[5].x, f[5].y);
  const float m4 = max3abs(f[6].x, f[6].y, f[7].x);
  const float amax = fmaxf(max3abs(m0, m1, m2), max3abs(m3, m4, f[7].y));
  // amax / 6, correctly rounded (amax is finite and >= 0; tiny quotients are clamped away below)
  const float r6 = 0.16666667163372039794921875f;   // RN(1/6)
  const float s0 = amax * r6;
  float s = fmaf(fmaf(-6.0f, s0, amax), r6, s0);
  s = fminf(fmaxf(s, 1e-12f), 448.0f);
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3));
}

// Main path of the codes: k = {2^(2-E), ~1/(4J)} of the group's scale byte.
// m = trunc(4 v / 2^E) keeps the sign of v (also as -0 for a small negative v, whose code is
// "negative zero" in the reference too; v itself is never -0 here: inputs were made +0 and
// quotients cannot underflow in this path)
__device__ __forceinline__ void group_codes_fast(const float2 (&f)[8], float2 k, uint32_t& code_lo, uint32_t& code_hi) {
  const float2 mult = make_float2(k.x, k.x), rj = make_float2(k.y, k.y);
  float2 w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 t = __fmul2_rn(f[j], mult);
    w[j] = __fmul2_rn(make_float2(truncf(t.x), truncf(t.y)), rj);
  }
  code_lo = cvt_e2m1x8(w[0], w[1], w[2], w[3]);
  code_hi = cvt_e2m1x8(w[4], w[5], w[6], w[7]);
}

// Zero scale (everything non-zero saturates) or the 448 clamp (ratios are unbounded): compare path
__device__ __forceinline__ void group_codes_compare(const float2 (&f)[8], uint32_t sb, uint32_t& code_lo, uint32_t& code_hi) {
  float sf = e4m3_to_f32(static_cast<uint8_t>(sb));
  sf = (sf == 0.0f) ? __uint_as_float(4u) : sf;     // 2^-147 * {.25 .. 5}: positive, below any normal number
  GroupBounds gb;
  gb.p[0] = sf * 0.25f; gb.p[1] = sf * 0.75f; gb.p[2] = sf * 1.25f; gb.p[3] = sf * 1.75f;
  gb.p[4] = sf * 2.5f;  gb.p[5] = sf * 3.5f;  gb.p[6] = sf * 5.0f;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) lo += (e2m1_code(f[j].x, gb) << (8 * j)) + (e2m1_code(f[j].y, gb) << (8 * j + 4));
#pragma unroll
  for (int j = 0; j < 4; ++j) hi += (e2m1_code(f[4 + j].x, gb) << (8 * j)) + (e2m1_code(f[4 + j].y, gb) << (8 * j + 4));
  code_lo = lo; code_hi = hi;
}

// Division by a per-column constant with its reciprocal at hand: q0 = RN(a r), e = a - s q0 (exact in one
// fma), q = RN(q0 + e r).  With r = RN(1 / s) this is the correctly rounded a / s whenever nothing over- or
// underflows on the way (Markstein's correction step; it needs a correctly rounded reciprocal and a divisor
// whose significand is not all ones, which a 16-bit s cannot be).  svdq_selftest_divide checks it against
// __fdiv_rn for every fp32 significand of a and every 11-bit significand of s; powers of two scale through
// all three steps exactly.  Arguments: the pair of dividends, the NEGATED divisors and the reciprocals.
__device__ __forceinline__ float2 divide_by_constant2(float2 a, float2 neg_s, float2 r) {
  const float2 q0 = __fmul2_rn(a, r);
  const float2 e = __ffma2_rn(neg_s, q0, a);
  return __ffma2_rn(e, r, q0);
}

// quantize_group with the scale byte already worked out
__device__ __forceinline__ void quantize_group_with(float2 (&f)[8], uint32_t sb, uint32_t& code_lo, uint32_t& code_hi) {
  const float2 k = scale_constants(sb);
  if (k.x != 0.0f) group_codes_fast(f, k, code_lo, code_hi);
  else group_codes_compare(f, sb, code_lo, code_hi);
}

// One 16-element group (smoothed, fp32): amax, scale byte, eight code bytes.  scale_lut: the table
// fill_scale_lut made in shared memory, or null to work the two constants out on the spot.
__device__ __forceinline__ void quantize_group(float2 (&f)[8], const float2* scale_lut,
                                               uint32_t& code_lo, uint32_t& code_hi, uint32_t& sbyte) {
  const uint32_t sb = group_scale_byte(f);
  sbyte = sb;
  const float2 k = scale_lut != nullptr ? scale_lut[sb] : scale_constants(sb);
  if (k.x != 0.0f) group_codes_fast(f, k, code_lo, code_hi);
  else group_codes_compare(f, sb, code_lo, code_hi);
}

}  // namespace qmath
}  // namespace svdq
