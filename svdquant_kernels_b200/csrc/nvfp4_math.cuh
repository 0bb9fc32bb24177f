// Scalar NVFP4 arithmetic shared by the quantizer kernels.
//
// The rules restate baseline/kernels/_nvfp4.py:27-41 and :82-91 of the
// reference so that codes and scales come out bit-identical:
//   scale  = e4m3( clamp(amax / 6, 1e-12, 448) )        (IEEE fp32 divide, RNE cast)
//   q      = v / float(scale)                           (IEEE fp32 divide)
//   code   = #{ bounds b in {.25,.75,1.25,1.75,2.5,3.5,5} : |q| >= b }  |  (q < 0) << 3
//
// The per-element divide by the scale is never executed.  With s an e4m3 value
// (4 significant bits) and b a bound (3 significant bits) the product s*b is
// exact in fp32, and RN(|v| / s) >= b holds exactly when |v| >= s*b: the
// quotients that round up to b from below would need |v| strictly between two
// adjacent fp32 numbers.  So each group compares |v| with seven exact products.
// A zero scale (amax/6 below 2^-10) makes every non-zero v an infinity (code 7)
// and every zero a NaN (code 0); the smallest denormal as bound reproduces that.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace svdq {

__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(float v) { return v; }

// e4m3 byte of clamp(amax/6, 1e-12, 448); round-to-nearest-even incl. subnormals.
__device__ __forceinline__ uint8_t scale_byte_from_amax(float amax) {
  float s = __fdiv_rn(amax, 6.0f);
  s = fminf(fmaxf(s, 1e-12f), 448.0f);
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3));
}

// exact value of a non-negative e4m3 byte
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  uint32_t e = (b >> 3) & 0xF, m = b & 7;
  if (e == 0) return static_cast<float>(m) * 0.001953125f;  // m * 2^-9
  return __uint_as_float(((e + 120u) << 23) | (m << 20));
}

struct GroupBounds {
  float p[7];
};

__device__ __forceinline__ GroupBounds bounds_for_scale(float s) {
  GroupBounds g;
  if (s == 0.0f) {
    const float tiny = __uint_as_float(1u);  // any non-zero magnitude saturates
#pragma unroll
    for (int i = 0; i < 7; ++i) g.p[i] = tiny;
  } else {
    g.p[0] = s * 0.25f; g.p[1] = s * 0.75f; g.p[2] = s * 1.25f; g.p[3] = s * 1.75f;
    g.p[4] = s * 2.5f;  g.p[5] = s * 3.5f;  g.p[6] = s * 5.0f;
  }
  return g;
}

// 4-bit code of one value: three dependent compares instead of seven.
__device__ __forceinline__ uint32_t e2m1_code(float v, const GroupBounds& g) {
  const float a = fabsf(v);
  const bool c4 = a >= g.p[3];
  const float mid = c4 ? g.p[5] : g.p[1];
  const bool c2 = a >= mid;
  const float hi = c2 ? g.p[6] : g.p[4];
  const float lo = c2 ? g.p[2] : g.p[0];
  const bool c1 = a >= (c4 ? hi : lo);
  uint32_t idx = (c4 ? 4u : 0u) + (c2 ? 2u : 0u) + (c1 ? 1u : 0u);
  return idx | ((v < 0.0f) ? 8u : 0u);
}

// lora_act in the 16-bit form the GEMM's dense MMA consumes (same format as lora_up):
//   fp16: one copy, round to nearest even, magnitudes beyond 65504 clamp to it
//   bf16: hi = bf16(v) and lo = bf16(v - hi), stored as two [rows, R] planes; hi + lo carries
//         16 significant bits of v with bf16's full exponent range.  A third plane holds v as
//         fp16 (clamped like the fp16 form): where a whole row block is known to fit fp16 the
//         GEMM multiplies that plane with an fp16 copy of lora_up in one pass instead of two.
//         Behind the planes: one 32-bit word per 32 rows, non-zero if some value of those rows
//         does not fit (see lora16_flags)
__device__ __forceinline__ __half f32_to_f16_sat(float v) {
  return __float2half_rn(fminf(fmaxf(v, -65504.0f), 65504.0f));
}
__device__ __forceinline__ void f32_to_bf16_hi_lo(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(v);
  lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}
// writes element `idx` (of `plane` elements per plane) of the 16-bit form of v
template <typename T>
__device__ __forceinline__ void store_lora16(void* base, size_t idx, size_t plane, float v);
template <>
__device__ __forceinline__ void store_lora16<__half>(void* base, size_t idx, size_t, float v) {
  static_cast<__half*>(base)[idx] = f32_to_f16_sat(v);
}
template <>
__device__ __forceinline__ void store_lora16<__nv_bfloat16>(void* base, size_t idx, size_t plane, float v) {
  __nv_bfloat16 hi, lo;
  f32_to_bf16_hi_lo(v, hi, lo);
  static_cast<__nv_bfloat16*>(base)[idx] = hi;
  static_cast<__nv_bfloat16*>(base)[plane + idx] = lo;
  reinterpret_cast<__half*>(base)[2 * plane + idx] = f32_to_f16_sat(v);
}
// four consecutive elements at once (idx % 4 == 0)
template <typename T>
__device__ __forceinline__ void store_lora16x4(void* base, size_t idx, size_t plane, float4 v);
template <>
__device__ __forceinline__ void store_lora16x4<__half>(void* base, size_t idx, size_t, float4 v) {
  __half2 a = __floats2half2_rn(fminf(fmaxf(v.x, -65504.0f), 65504.0f), fminf(fmaxf(v.y, -65504.0f), 65504.0f));
  __half2 b = __floats2half2_rn(fminf(fmaxf(v.z, -65504.0f), 65504.0f), fminf(fmaxf(v.w, -65504.0f), 65504.0f));
  *reinterpret_cast<uint2*>(static_cast<__half*>(base) + idx) =
      make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}
template <>
__device__ __forceinline__ void store_lora16x4<__nv_bfloat16>(void* base, size_t idx, size_t plane, float4 v) {
  __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
  const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
  __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2bfloat162_rn(v.z - f1.x, v.w - f1.y);
  __nv_bfloat16* p = static_cast<__nv_bfloat16*>(base);
  *reinterpret_cast<uint2*>(p + idx) = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
  *reinterpret_cast<uint2*>(p + plane + idx) = make_uint2(*reinterpret_cast<uint32_t*>(&l0), *reinterpret_cast<uint32_t*>(&l1));
  store_lora16x4<__half>(p + 2 * plane, idx, plane, v);
}
// bf16 form only: the per-32-row "does not fit fp16" words behind the three planes
__host__ __device__ __forceinline__ uint32_t* lora16_flags(void* base, size_t plane) {
  return reinterpret_cast<uint32_t*>(static_cast<uint16_t*>(base) + 3 * plane);
}
__host__ __device__ __forceinline__ const uint32_t* lora16_flags(const void* base, size_t plane) {
  return reinterpret_cast<const uint32_t*>(static_cast<const uint16_t*>(base) + 3 * plane);
}
// 16-bit elements of the whole form for `rows` x R values
__host__ __device__ __forceinline__ size_t lora16_elems(size_t rows, size_t R, bool bf16) {
  return bf16 ? 3 * rows * R + 2 * ((rows + 31) / 32) : rows * R;
}
// true if v survives the fp16 plane (finite and within range)
__device__ __forceinline__ bool fits_f16(float4 v) {
  return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))) <= 65504.0f;
}

// byte offset of (row m, group g) inside the 128-row x 4-group scale atoms the
// tensor core reads (cute_kernels/gemm_w4a4/kernel.py:194-225 builds the same
// order with a transpose + permute): atoms of 512 bytes ordered (m/128, g/4).
__host__ __device__ __forceinline__ size_t sf_swizzled_offset(uint32_t m, uint32_t g, uint32_t groups) {
  return (static_cast<size_t>(m >> 7) * (groups >> 2) + (g >> 2)) * 512u + (m & 31u) * 16u + ((m >> 5) & 3u) * 4u + (g & 3u);
}

}  // namespace svdq
