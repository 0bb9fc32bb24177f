// Shape-agnostic quantizer kernels: the NVFP4 row packer (used for weights at
// load time and as the path for activation shapes the fused kernel does not
// take) and a plain LoRA-down projection.  CUDA-core only; the fused
// tensor-core kernel lives in quantize_fused.cu.
//
// Reference behaviour restated: baseline/kernels/_nvfp4.py:60-95 (row packer)
// and baseline/kernels/quantize_w4a4_act_fuse_lora/ref.py:36-48 (raw-x LoRA-down,
// smooth divide only on the quantised branch, zero rows up to the padded height).
#include "nvfp4_math.cuh"
#include "svdq_internal.h"

namespace svdq {

template <typename T>
struct Vec16;  // 16 consecutive elements
template <>
struct Vec16<__half> {
  uint4 a, b;
  __device__ __forceinline__ float get(int i) const {
    const __half* h = reinterpret_cast<const __half*>(this);
    return __half2float(h[i]);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  uint4 a, b;
  __device__ __forceinline__ float get(int i) const {
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(this);
    return __bfloat162float(h[i]);
  }
};
template <>
struct Vec16<float> {
  float4 a, b, c, d;
  __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float*>(this)[i]; }
};

// One thread per (row, 16-group).  Consecutive threads take consecutive groups
// of a row, so loads are 32 B per thread and contiguous across the warp.
template <typename T>
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const T* __restrict__ x, const T* __restrict__ smooth, uint8_t* __restrict__ codes,
                     uint8_t* __restrict__ scales, uint8_t* __restrict__ scales_swz, int rows, int rows_pad, int K) {
  const int groups = K >> 4;
  const long long total = static_cast<long long>(rows_pad) * groups;
  for (long long item = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; item < total;
       item += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(item / groups);
    const int g = static_cast<int>(item - static_cast<long long>(m) * groups);
    uint2 packed = make_uint2(0u, 0u);
    uint8_t sbyte = 0;
    if (m < rows) {
      const Vec16<T> v = *reinterpret_cast<const Vec16<T>*>(x + static_cast<size_t>(m) * K + g * 16);
      float f[16];
      if (smooth != nullptr) {
        const Vec16<T> s = *reinterpret_cast<const Vec16<T>*>(smooth + g * 16);
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = __fdiv_rn(v.get(i), s.get(i));
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = v.get(i);
      }
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
      sbyte = scale_byte_from_amax(amax);
      const GroupBounds gb = bounds_for_scale(e4m3_to_f32(sbyte));
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) lo |= e2m1_code(f[i], gb) << (4 * i);
#pragma unroll
      for (int i = 0; i < 8; ++i) hi |= e2m1_code(f[8 + i], gb) << (4 * i);
      packed = make_uint2(lo, hi);
    }
    *reinterpret_cast<uint2*>(codes + static_cast<size_t>(m) * (K >> 1) + g * 8) = packed;
    scales[static_cast<size_t>(g) * rows_pad + m] = sbyte;
    if (scales_swz != nullptr) scales_swz[sf_swizzled_offset(m, g, groups)] = sbyte;
  }
}

// out[m, r] = sum_k x[m, k] * w[k, r] in fp32; rows >= M are written as zeros.
// 8 rows per block; threads stride over r so the w reads are coalesced.
template <typename T>
__global__ void __launch_bounds__(128)
lora_down_kernel(const T* __restrict__ x, const T* __restrict__ w, float* __restrict__ out, void* __restrict__ out16,
                 int M, int M_pad, int K, int R) {
  constexpr int ROWS = 8, KC = 128;
  __shared__ float xs[ROWS][KC];
  const int m0 = blockIdx.x * ROWS;
  for (int r0 = 0; r0 < R; r0 += blockDim.x) {
    const int r = r0 + threadIdx.x;
    float acc[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) acc[i] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += KC) {
      __syncthreads();
      for (int i = threadIdx.x; i < ROWS * KC; i += blockDim.x) {
        const int rr = i / KC, kk = i % KC;
        const int m = m0 + rr, k = k0 + kk;
        xs[rr][kk] = (m < M && k < K) ? to_f32(x[static_cast<size_t>(m) * K + k]) : 0.0f;
      }
      __syncthreads();
      if (r < R) {
        const int kmax = min(KC, K - k0);
        for (int kk = 0; kk < kmax; ++kk) {
          const float wv = to_f32(w[static_cast<size_t>(k0 + kk) * R + r]);
#pragma unroll
          for (int i = 0; i < ROWS; ++i) acc[i] = fmaf(xs[i][kk], wv, acc[i]);
        }
      }
    }
    if (r < R) {
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        const int m = m0 + i;
        if (m < M_pad) {
          out[static_cast<size_t>(m) * R + r] = acc[i];
          if (out16 != nullptr) store_lora16<T>(out16, static_cast<size_t>(m) * R + r, static_cast<size_t>(M_pad) * R, acc[i]);
        }
      }
    }
  }
}

// canonical [groups, rows] scale bytes -> 128x4 atom order
__global__ void swizzle_scales_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int groups, int rows) {
  const long long total = static_cast<long long>(groups) * rows;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i / rows), m = static_cast<int>(i % rows);
    dst[sf_swizzled_offset(m, g, groups)] = src[i];
  }
}

// fp32 lora_act -> the 16-bit form of type T (see store_lora16)
template <typename T>
__global__ void cast_lora16_kernel(const float* __restrict__ src, void* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    store_lora16<T>(dst, static_cast<size_t>(i), static_cast<size_t>(n), src[i]);
}

static int grid_for(long long items, int block) {
  long long g = (items + block - 1) / block;
  const long long cap = 148ll * 16;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

int launch_quantize_rows(const void* x, const void* smooth, void* codes, void* scales, void* scales_swz, int rows,
                         int rows_pad, int K, int dtype, cudaStream_t stream) {
  const long long items = static_cast<long long>(rows_pad) * (K / 16);
  if (items == 0) return SVDQ_OK;
  const int grid = grid_for(items, 256);
  uint8_t* c = static_cast<uint8_t*>(codes);
  uint8_t* s = static_cast<uint8_t*>(scales);
  uint8_t* sw = static_cast<uint8_t*>(scales_swz);
  switch (dtype) {
    case SVDQ_DTYPE_F16:
      quantize_rows_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), static_cast<const __half*>(smooth), c, s, sw, rows, rows_pad, K);
      break;
    case SVDQ_DTYPE_BF16:
      quantize_rows_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(smooth), c, s, sw, rows, rows_pad, K);
      break;
    case SVDQ_DTYPE_F32:
      quantize_rows_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<const float*>(smooth), c, s, sw, rows, rows_pad, K);
      break;
    default:
      return SVDQ_ERR_DTYPE;
  }
  return cudaGetLastError() == cudaSuccess ? SVDQ_OK : SVDQ_ERR_LAUNCH;
}

// The CUDA-core paths do not look at magnitudes: they mark every row block of a bf16 form as
// "does not fit fp16", which sends the GEMM down its two-pass bf16 route.
static int mark_lora16_unfit(void* out16, int rows, int R, int dtype, cudaStream_t stream) {
  if (out16 == nullptr || dtype != SVDQ_DTYPE_BF16 || rows == 0) return SVDQ_OK;
  uint32_t* flags = lora16_flags(out16, static_cast<size_t>(rows) * R);
  return cudaMemsetAsync(flags, 0xFF, sizeof(uint32_t) * ((rows + 31) / 32), stream) == cudaSuccess ? SVDQ_OK : SVDQ_ERR_CUDA;
}

int launch_lora_down(const void* x, const void* w, float* out, void* out16, int M, int M_pad, int K, int R, int dtype,
                     cudaStream_t stream) {
  if (M_pad == 0 || R == 0) return SVDQ_OK;
  const int grid = (M_pad + 7) / 8;
  if (dtype == SVDQ_DTYPE_F16)
    lora_down_kernel<__half><<<grid, 128, 0, stream>>>(static_cast<const __half*>(x), static_cast<const __half*>(w), out, out16, M, M_pad, K, R);
  else if (dtype == SVDQ_DTYPE_BF16)
    lora_down_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), out, out16, M, M_pad, K, R);
  else
    return SVDQ_ERR_DTYPE;
  if (cudaGetLastError() != cudaSuccess) return SVDQ_ERR_LAUNCH;
  return mark_lora16_unfit(out16, M_pad, R, dtype, stream);
}

int launch_swizzle_scales(const void* src, void* dst, int groups, int rows, cudaStream_t stream) {
  const long long n = static_cast<long long>(groups) * rows;
  if (n == 0) return SVDQ_OK;
  swizzle_scales_kernel<<<grid_for(n, 256), 256, 0, stream>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), groups, rows);
  return cudaGetLastError() == cudaSuccess ? SVDQ_OK : SVDQ_ERR_LAUNCH;
}

int launch_cast_f32(const float* src, void* dst, int rows, int R, int dtype, cudaStream_t stream) {
  const long long n = static_cast<long long>(rows) * R;
  if (n == 0) return SVDQ_OK;
  if (dtype == SVDQ_DTYPE_F16)
    cast_lora16_kernel<__half><<<grid_for(n, 256), 256, 0, stream>>>(src, dst, n);
  else if (dtype == SVDQ_DTYPE_BF16)
    cast_lora16_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, stream>>>(src, dst, n);
  else
    return SVDQ_ERR_DTYPE;
  if (cudaGetLastError() != cudaSuccess) return SVDQ_ERR_LAUNCH;
  return mark_lora16_unfit(dst, rows, R, dtype, stream);
}

}  // namespace svdq
