// extern "C" surface of libsvdq_b200.so (declared in include/svdq_b200.h):
// argument validation, dispatch between the fused and the generic quantizer,
// the device status word, and the host-buffer "plan" used for end-to-end runs.
#include <cstring>
#include <mutex>
#include <new>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <vector>

#include "nvfp4_math.cuh"
#include "sm100.cuh"
#include "svdq_internal.h"

namespace svdq {

int read_and_clear_status(unsigned int out[4]) {
  if (cudaDeviceSynchronize() != cudaSuccess) return SVDQ_ERR_CUDA;
  if (cudaMemcpyFromSymbol(out, g_status_word, sizeof(unsigned int) * 4) != cudaSuccess) return SVDQ_ERR_CUDA;
  if (out[0] != 0 || out[3] != 0) {
    const unsigned int zero[4] = {0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_status_word, zero, sizeof(zero)) != cudaSuccess) return SVDQ_ERR_CUDA;
  }
  return out[0] == 0 ? SVDQ_OK : SVDQ_ERR_DEVICE;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace svdq

using namespace svdq;

extern "C" {

const char* svdq_status_string(int status) {
  switch (status) {
    case SVDQ_OK: return "ok";
    case SVDQ_ERR_NULL: return "a required pointer is NULL";
    case SVDQ_ERR_SHAPE: return "size outside the operator's contract";
    case SVDQ_ERR_DTYPE: return "unsupported element type";
    case SVDQ_ERR_ALIGN: return "pointer not 16-byte aligned";
    case SVDQ_ERR_LAUNCH: return "CUDA launch or descriptor creation failed";
    case SVDQ_ERR_DEVICE: return "a kernel gave up on a bounded wait";
    case SVDQ_ERR_UNSUPPORTED: return "shape not supported by the requested kernel";
    case SVDQ_ERR_CUDA: return "CUDA runtime call failed";
    default: return "unknown status";
  }
}

int svdq_version(void) { return 100; }

int svdq_prepare_smooth(const void* smooth, void* smooth_table, int K, int dtype, void* stream) {
  if (dtype != SVDQ_DTYPE_F16 && dtype != SVDQ_DTYPE_BF16) return SVDQ_ERR_DTYPE;
  if (K <= 0 || K % 16 != 0) return SVDQ_ERR_SHAPE;
  if (smooth == nullptr || smooth_table == nullptr) return SVDQ_ERR_NULL;
  if (!aligned16(smooth_table)) return SVDQ_ERR_ALIGN;
  return launch_smooth_table(smooth, smooth_table, K, dtype, static_cast<cudaStream_t>(stream));
}

static int quantize_entry(const void* x, const void* lora_down, const void* smooth, const void* smooth_table, void* act,
                          void* ascales, float* lora_act, void* ascales_swz, void* lora_act16, int M, int K, int R,
                          int M_pad, int dtype, int flags, void* workspace, size_t workspace_bytes, void* stream) {
  if (dtype != SVDQ_DTYPE_F16 && dtype != SVDQ_DTYPE_BF16) return SVDQ_ERR_DTYPE;
  if (M < 0 || K <= 0 || R < 0 || M_pad < M || K % 16 != 0) return SVDQ_ERR_SHAPE;
  if (M_pad == 0) return SVDQ_OK;
  if (act == nullptr || ascales == nullptr || (M > 0 && x == nullptr)) return SVDQ_ERR_NULL;
  if (R > 0 && (lora_down == nullptr || lora_act == nullptr)) return SVDQ_ERR_NULL;
  if (!aligned16(x) || !aligned16(act) || !aligned16(smooth) || !aligned16(lora_down) || !aligned16(lora_act) ||
      !aligned16(ascales_swz) || !aligned16(lora_act16) || !aligned16(smooth_table) || !aligned16(workspace))
    return SVDQ_ERR_ALIGN;
  if (smooth == nullptr && smooth_table != nullptr) return SVDQ_ERR_NULL;
  if (ascales_swz != nullptr && (M_pad % 128 != 0 || K % 64 != 0)) return SVDQ_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the fused kernels read the smoothing factors from the prepared table; without one they cannot smooth
  const bool table_ok = smooth == nullptr || smooth_table != nullptr;
  const bool fused_ok = M > 0 && quantize_fused_supported(M, K, R, M_pad) && table_ok;
  if (flags == SVDQ_QUANT_FORCE_FUSED && !fused_ok) return SVDQ_ERR_UNSUPPORTED;
  if (flags >= SVDQ_QUANT_FORCE_STREAM) {
    // The streaming form (128- or 256-row tiles, K ranks met in the workspace) runs only on request: on
    // every benchmark shape it measured a few per cent behind the cluster form (c1 21.2 vs 18.9 us,
    // c3 55.6 vs 55.0 us), because both are bound by the quantize warps, not by their data movement.
    const int tm = (flags >> 8) & 0x1FF, ks = (flags >> 4) & 0xF;
    if (M <= 0 || !table_ok) return SVDQ_ERR_UNSUPPORTED;
    return launch_quantize_stream(x, lora_down, smooth_table, act, ascales, lora_act, ascales_swz, lora_act16, M, K, R,
                                  M_pad, dtype, workspace, workspace != nullptr ? workspace_bytes : 0, tm, ks, st);
  }
  if (fused_ok && flags != SVDQ_QUANT_FORCE_GENERIC)
    return launch_quantize_fused(x, lora_down, smooth_table, act, ascales, lora_act, ascales_swz, lora_act16, M, K, R,
                                 M_pad, dtype, st);
  int rc = launch_quantize_rows(x, smooth, act, ascales, ascales_swz, M, M_pad, K, dtype, st);
  if (rc != SVDQ_OK) return rc;
  return launch_lora_down(x, lora_down, lora_act, lora_act16, M, M_pad, K, R, dtype, st);
}

int svdq_quantize_w4a4_act_fuse_lora(const void* x, const void* lora_down, const void* smooth,
                                     const void* smooth_table, void* act,
                                     void* ascales, float* lora_act, void* ascales_swz, void* lora_act16, int M,
                                     int K, int R, int M_pad, int dtype, int flags, void* stream) {
  return quantize_entry(x, lora_down, smooth, smooth_table, act, ascales, lora_act, ascales_swz, lora_act16, M, K, R, M_pad,
                        dtype, flags, nullptr, 0, stream);
}

unsigned long long svdq_quantize_workspace_bytes(int M, int K, int R, int M_pad) {
  return static_cast<unsigned long long>(quantize_stream_workspace_bytes(M, K, R, M_pad));
}

int svdq_quantize_w4a4_act_fuse_lora_ws(const void* x, const void* lora_down, const void* smooth,
                                        const void* smooth_table, void* act, void* ascales, float* lora_act,
                                        void* ascales_swz, void* lora_act16, int M, int K, int R, int M_pad, int dtype,
                                        int flags, void* workspace, unsigned long long workspace_bytes, void* stream) {
  return quantize_entry(x, lora_down, smooth, smooth_table, act, ascales, lora_act, ascales_swz, lora_act16, M, K, R, M_pad,
                        dtype, flags, workspace, static_cast<size_t>(workspace_bytes), stream);
}

int svdq_quantize_nvfp4_rows(const void* x, void* codes, void* scales, void* scales_swz, int rows, int rows_pad, int K,
                             int dtype, void* stream) {
  if (rows < 0 || rows_pad < rows || K <= 0 || K % 16 != 0) return SVDQ_ERR_SHAPE;
  if (rows_pad == 0) return SVDQ_OK;
  if (codes == nullptr || scales == nullptr || (rows > 0 && x == nullptr)) return SVDQ_ERR_NULL;
  if (!aligned16(x) || !aligned16(codes) || !aligned16(scales_swz)) return SVDQ_ERR_ALIGN;
  if (scales_swz != nullptr && (rows_pad % 128 != 0 || K % 64 != 0)) return SVDQ_ERR_SHAPE;
  return launch_quantize_rows(x, nullptr, codes, scales, scales_swz, rows, rows_pad, K, dtype,
                              static_cast<cudaStream_t>(stream));
}

int svdq_swizzle_scales(const void* scales, void* scales_swz, int k_groups, int rows, void* stream) {
  if (k_groups < 0 || rows < 0 || rows % 128 != 0 || k_groups % 4 != 0) return SVDQ_ERR_SHAPE;
  if (k_groups == 0 || rows == 0) return SVDQ_OK;
  if (scales == nullptr || scales_swz == nullptr) return SVDQ_ERR_NULL;
  return launch_swizzle_scales(scales, scales_swz, k_groups, rows, static_cast<cudaStream_t>(stream));
}

long long svdq_lora_act16_elems(int rows, int R, int dtype) {
  if (rows < 0 || R < 0 || (dtype != SVDQ_DTYPE_F16 && dtype != SVDQ_DTYPE_BF16)) return -1;
  return static_cast<long long>(lora16_elems(static_cast<size_t>(rows), static_cast<size_t>(R), dtype == SVDQ_DTYPE_BF16));
}

int svdq_cast_lora_act(const float* src, void* dst, int rows, int R, int dtype, void* stream) {
  if (rows < 0 || R < 0) return SVDQ_ERR_SHAPE;
  if (rows == 0 || R == 0) return SVDQ_OK;
  if (src == nullptr || dst == nullptr) return SVDQ_ERR_NULL;
  if (!aligned16(dst)) return SVDQ_ERR_ALIGN;
  return launch_cast_f32(src, dst, rows, R, dtype, static_cast<cudaStream_t>(stream));
}

int svdq_lora_up_to_f16(const void* lora_up_bf16_host, void* out_f16_host, long long count) {
  if (count < 0) return SVDQ_ERR_SHAPE;
  if (count > 0 && (lora_up_bf16_host == nullptr || out_f16_host == nullptr)) return SVDQ_ERR_NULL;
  const uint16_t* src = static_cast<const uint16_t*>(lora_up_bf16_host);
  __half* dst = static_cast<__half*>(out_f16_host);
  for (long long i = 0; i < count; ++i) {
    const uint32_t bits = static_cast<uint32_t>(src[i]) << 16;
    float v;
    memcpy(&v, &bits, 4);
    if (!(v >= -65504.0f && v <= 65504.0f)) return SVDQ_ERR_UNSUPPORTED;     // out of fp16 range or NaN: no copy
    dst[i] = __float2half_rn(v);
  }
  return SVDQ_OK;
}

int svdq_quantizer_max_active_clusters(int R, int k_split, int dtype) {
  if (k_split != 1 && k_split != 2 && k_split != 4 && k_split != 8) return -1;
  return quantize_fused_max_clusters(R, k_split, dtype);
}

int svdq_gemm_w4a4_supported(int M, int N, int K, int R) { return gemm_supported(M, N, K, R) ? 1 : 0; }

static int gemm_entry(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                      const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales,
                      const void* bias, void* y, int M, int N, int K, int R, int dtype, int variant, void* workspace,
                      size_t workspace_bytes, void* stream) {
  if (dtype != SVDQ_DTYPE_F16 && dtype != SVDQ_DTYPE_BF16) return SVDQ_ERR_DTYPE;
  if (!gemm_supported(M, N, K, R)) return SVDQ_ERR_SHAPE;
  if (act == nullptr || wgt == nullptr || ascales_swz == nullptr || wscales_swz == nullptr || y == nullptr)
    return SVDQ_ERR_NULL;
  if ((lora_act16 == nullptr) != (lora_up == nullptr)) return SVDQ_ERR_NULL;
  if (R > 0 && lora_act16 == nullptr) return SVDQ_ERR_NULL;
  if (lora_act16 == nullptr) R = 0;
  if (!aligned16(act) || !aligned16(wgt) || !aligned16(ascales_swz) || !aligned16(wscales_swz) ||
      !aligned16(lora_act16) || !aligned16(lora_up) || !aligned16(lora_up_f16) || !aligned16(y) || !aligned16(workspace))
    return SVDQ_ERR_ALIGN;
  GemmTp extra;
  extra.ws = workspace;
  extra.ws_bytes = workspace != nullptr ? workspace_bytes : 0;
  return launch_gemm_w4a4(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, lora_up_f16, wcscales, bias, y, M, N,
                          K, R, dtype, variant, extra, static_cast<cudaStream_t>(stream));
}

int svdq_gemm_w4a4(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                   const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales,
                   const void* bias, void* y, int M, int N, int K, int R, int dtype, int variant, void* stream) {
  return gemm_entry(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, lora_up_f16, wcscales, bias, y, M, N, K, R,
                    dtype, variant, nullptr, 0, stream);
}

int svdq_gemm_w4a4_next(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                        const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales,
                        const void* bias, void* y, const void* smooth_next, void* qout, void* oscales, void* oscales_swz,
                        int M, int N, int K, int R, int dtype, int variant, void* stream) {
  if (dtype != SVDQ_DTYPE_F16 && dtype != SVDQ_DTYPE_BF16) return SVDQ_ERR_DTYPE;
  if (!gemm_supported(M, N, K, R)) return SVDQ_ERR_SHAPE;
  if (act == nullptr || wgt == nullptr || ascales_swz == nullptr || wscales_swz == nullptr || y == nullptr ||
      smooth_next == nullptr || qout == nullptr || oscales == nullptr)
    return SVDQ_ERR_NULL;
  if ((lora_act16 == nullptr) != (lora_up == nullptr)) return SVDQ_ERR_NULL;
  if (R > 0 && lora_act16 == nullptr) return SVDQ_ERR_NULL;
  if (lora_act16 == nullptr) R = 0;
  if (!aligned16(act) || !aligned16(wgt) || !aligned16(ascales_swz) || !aligned16(wscales_swz) ||
      !aligned16(lora_act16) || !aligned16(lora_up) || !aligned16(lora_up_f16) || !aligned16(y) || !aligned16(qout))
    return SVDQ_ERR_ALIGN;
  if (oscales_swz != nullptr && N % 64 != 0) return SVDQ_ERR_SHAPE;
  GemmTp extra;
  extra.smooth_next = smooth_next; extra.qout = qout; extra.oscales = oscales; extra.oscales_swz = oscales_swz;
  return launch_gemm_w4a4(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, lora_up_f16, wcscales, bias, y, M, N,
                          K, R, dtype, variant, extra, static_cast<cudaStream_t>(stream));
}

unsigned long long svdq_gemm_w4a4_workspace_bytes(int M, int N, int K, int R) {
  return static_cast<unsigned long long>(gemm_split_workspace_bytes(M, N, K, R));
}

int svdq_gemm_w4a4_ws(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                      const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales,
                      const void* bias, void* y, int M, int N, int K, int R, int dtype, int variant, void* workspace,
                      unsigned long long workspace_bytes, void* stream) {
  return gemm_entry(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, lora_up_f16, wcscales, bias, y, M, N, K, R,
                    dtype, variant, workspace, static_cast<size_t>(workspace_bytes), stream);
}

int svdq_gemm_w4a4_columns(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                           const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales,
                           const void* bias, void* y_full, void* const* y_full_peers, int n_peers, int N_total,
                           int col0, int M, int N, int K, int R, int dtype, int variant, void* stream) {
  if (dtype != SVDQ_DTYPE_F16 && dtype != SVDQ_DTYPE_BF16) return SVDQ_ERR_DTYPE;
  if (!gemm_supported(M, N, K, R)) return SVDQ_ERR_SHAPE;
  if (act == nullptr || wgt == nullptr || ascales_swz == nullptr || wscales_swz == nullptr || y_full == nullptr)
    return SVDQ_ERR_NULL;
  if ((lora_act16 == nullptr) != (lora_up == nullptr)) return SVDQ_ERR_NULL;
  if (R > 0 && lora_act16 == nullptr) return SVDQ_ERR_NULL;
  if (lora_act16 == nullptr) R = 0;
  if (n_peers < 0 || n_peers > 7 || (n_peers > 0 && y_full_peers == nullptr)) return SVDQ_ERR_SHAPE;
  if (N_total < N || col0 < 0 || col0 + N > N_total) return SVDQ_ERR_SHAPE;
  if (!aligned16(act) || !aligned16(wgt) || !aligned16(ascales_swz) || !aligned16(wscales_swz) ||
      !aligned16(lora_act16) || !aligned16(lora_up) || !aligned16(lora_up_f16) || !aligned16(y_full))
    return SVDQ_ERR_ALIGN;
  GemmTp tp;
  tp.col0 = col0; tp.y_ld = N_total; tp.n_peers = n_peers;
  for (int d = 0; d < n_peers; ++d) {
    if (y_full_peers[d] == nullptr) return SVDQ_ERR_NULL;
    if (!aligned16(y_full_peers[d])) return SVDQ_ERR_ALIGN;
    tp.y_peer[d] = y_full_peers[d];
  }
  return launch_gemm_w4a4(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, lora_up_f16, wcscales, bias, y_full,
                          M, N, K, R, dtype, variant, tp, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// split-K GEMM on a workspace that is part of the library image
// ---------------------------------------------------------------------------
// Room for the ticket counters and 148 partial tiles of 128 x 128 fp32 (tiles x splits never exceeds the
// SM count, 148 on this part): 9.25 MiB of device memory per device that loads the library, there
// whether or not the entry point below is ever called.  Static storage: zero when the module is loaded.
constexpr size_t kStaticWsPartials = 148;
constexpr size_t kStaticWsBytes = kSplitTicketBytes + kStaticWsPartials * (128 * 128 * 4);
static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes];

// The array's address on each device, looked up once (cudaGetSymbolAddress) under a mutex: first calls
// may come from several host threads at once.
static std::mutex g_static_ws_mutex;
static void* g_static_ws_addr[64] = {};

static int static_ws_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SVDQ_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_static_ws_mutex);
  if (g_static_ws_addr[dev] == nullptr) {
    void* a = nullptr;
    if (cudaGetSymbolAddress(&a, g_static_ws) != cudaSuccess || a == nullptr) { cudaGetLastError(); return SVDQ_ERR_CUDA; }
    g_static_ws_addr[dev] = a;
  }
  *out = g_static_ws_addr[dev];
  return SVDQ_OK;
}

// A kernel that gave up on a bounded wait may have left ticket counters of the static workspace
// non-zero; every later split call on it would then draw tickets that never reach "last" and write
// no output.  Reading a failure therefore also puts the counters of the current device's array back
// to zero (the device is idle here: the read synchronised it).  Nothing is allocated.
int svdq_device_status(unsigned int out[4]) {
  unsigned int tmp[4] = {0, 0, 0, 0};
  int rc = read_and_clear_status(tmp);
  if (rc == SVDQ_ERR_DEVICE) {
    void* ws = nullptr;
    if (static_ws_address(&ws) != SVDQ_OK || cudaMemset(ws, 0, kSplitTicketBytes) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess)
      rc = SVDQ_ERR_CUDA;
  }
  if (out != nullptr)
    for (int i = 0; i < 4; ++i) out[i] = tmp[i];
  return rc;
}

int svdq_gemm_w4a4_static_ws(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                             const void* lora_act16, const void* lora_up, const void* lora_up_f16,
                             const void* wcscales, const void* bias, void* y, int M, int N, int K, int R, int dtype,
                             int variant, void* stream) {
  if (!gemm_supported(M, N, K, R)) return SVDQ_ERR_SHAPE;
  // what this call would park in the workspace: the library's own plan, or the forced split count
  size_t need = 0;
  if (variant == 0) need = gemm_split_workspace_bytes(M, N, K, R);
  else if (variant >= 10000)
    need = kSplitTicketBytes + static_cast<size_t>(M / 128) * (N / 128) * (variant / 10000) * (128 * 128 * 4);
  if (need > kStaticWsBytes) return SVDQ_ERR_UNSUPPORTED;
  // the array's address on the current device, looked up once per device and kept
  void* ws = nullptr;
  const int rc = static_ws_address(&ws);
  if (rc != SVDQ_OK) return rc;
  return gemm_entry(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, lora_up_f16, wcscales, bias, y, M, N, K, R,
                    dtype, variant, ws, kStaticWsBytes, stream);
}

// ---------------------------------------------------------------------------
// self-test of the bounded wait
// ---------------------------------------------------------------------------
}  // extern "C"

namespace svdq {
// One warp waits on a barrier of its own that nothing ever arrives on, with the same mbar_wait the
// kernels use but a caller-given limit; when the limit runs out the wait records its code in the
// status word and returns false, the kernel notes what it saw and ends normally.
__global__ void wait_expiry_selftest_kernel(unsigned long long limit_ns, unsigned int* seen) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  const WaitCtx ctx{&abort_flag};
  const bool ok = mbar_wait(&bar, 0, ctx, kDevWaitMisc, 0x5E1Fu, limit_ns);
  // a second wait in an aborted CTA returns at once
  const bool again = mbar_wait(&bar, 0, ctx, kDevWaitMisc, 0x5E20u, limit_ns);
  if (threadIdx.x == 0 && seen != nullptr) *seen = (ok ? 1u : 0u) | (again ? 2u : 0u) | (abort_flag ? 4u : 0u);
}
}  // namespace svdq

extern "C" {

int svdq_selftest_wait_expiry(unsigned long long limit_ns, unsigned int* seen_device, void* stream) {
  if (limit_ns == 0 || limit_ns > 100000000ull) return SVDQ_ERR_SHAPE;      // at most 0.1 s
  wait_expiry_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, seen_device);
  return cudaGetLastError() == cudaSuccess ? SVDQ_OK : SVDQ_ERR_LAUNCH;
}

// Every fp32 significand of a (2^23, a in [1, 2)) against every 11-bit significand of s (2^10, s in [1, 2)):
// qmath::divide_by_constant2 with r = __frcp_rn(s) must equal __fdiv_rn(a, s).  Block b takes s = 1 + b / 1024.
__global__ void divide_selftest_kernel(unsigned long long* mismatches) {
  const float sv = __uint_as_float(0x3f800000u | (static_cast<uint32_t>(blockIdx.x) << 13));
  const float r = __frcp_rn(sv);
  const float2 ns = make_float2(-sv, -sv), rr = make_float2(r, r);
  unsigned int bad = 0;
  for (uint32_t m = threadIdx.x * 2u; m < (1u << 23); m += blockDim.x * 2u) {
    const float a0 = __uint_as_float(0x3f800000u | m), a1 = __uint_as_float(0x3f800000u | (m + 1u));
    const float2 q = svdq::qmath::divide_by_constant2(make_float2(a0, a1), ns, rr);
    bad += (q.x != __fdiv_rn(a0, sv)) + (q.y != __fdiv_rn(a1, sv));
  }
  if (bad) atomicAdd(mismatches, static_cast<unsigned long long>(bad));
}

int svdq_selftest_divide(unsigned long long* mismatches_device, void* stream) {
  if (mismatches_device == nullptr) return SVDQ_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(mismatches_device, 0, sizeof(unsigned long long), st) != cudaSuccess) return SVDQ_ERR_CUDA;
  divide_selftest_kernel<<<1024, 1024, 0, st>>>(mismatches_device);
  return cudaGetLastError() == cudaSuccess ? SVDQ_OK : SVDQ_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// host-buffer plan
// ---------------------------------------------------------------------------
// Two slots of per-call buffers and three streams (host->device, compute, device->host), so that the
// copies of neighbouring calls overlap the kernels and each other (PCIe is full duplex).  A slot's
// life: x copy -> quantizer + GEMM -> y copy; events hand it from stream to stream and keep a slot's
// next use behind its previous one.
constexpr int kPlanSlots = 2;

struct PlanSlot {
  void *x, *act, *ascales, *ascales_swz, *lora_act16, *y;
  float* lora_act;
  void *x_pin, *y_pin;                                           // pinned staging for pageable caller buffers
  cudaEvent_t x_ready, computed, y_done;
  void* y_user;                                                  // pageable destination still to be filled from y_pin
  size_t y_bytes;
  bool busy;
};

struct svdq_linear_plan {
  int max_M, max_M_pad, K, N, R, dtype;
  cudaStream_t s_in, s_run, s_out;
  PlanSlot slot[kPlanSlots];
  unsigned long long submitted;
  void *wgt, *wscales_swz, *lora_down, *lora_up, *lora_up_f16, *smooth, *smooth_table, *wc, *bias;  // resident weights
  void* split_ws;                                                // split-K workspace of the GEMM (few-row calls, long K), or null
  size_t split_ws_bytes;
  void* quant_ws;                                                // workspace of the quantizer's streaming form, or null
  size_t quant_ws_bytes;
};

static bool is_pinned_host(const void* ptr) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, ptr) != cudaSuccess) { cudaGetLastError(); return false; }
  return a.type == cudaMemoryTypeHost;
}

static int dev_upload(void** dst, const void* src, size_t bytes, cudaStream_t st) {
  *dst = nullptr;
  if (src == nullptr || bytes == 0) return SVDQ_OK;
  if (cudaMalloc(dst, bytes) != cudaSuccess) return SVDQ_ERR_CUDA;
  if (cudaMemcpyAsync(*dst, src, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) return SVDQ_ERR_CUDA;
  return SVDQ_OK;
}

int svdq_linear_plan_create(svdq_linear_plan** out, int max_M, int K, int N, int R, int dtype, const void* wgt_host,
                            const void* wscales_host, const void* lora_down_host, const void* lora_up_host,
                            const void* smooth_host, const void* wcscales_host, const void* bias_host) {
  if (out == nullptr || wgt_host == nullptr || wscales_host == nullptr) return SVDQ_ERR_NULL;
  if (dtype != SVDQ_DTYPE_F16 && dtype != SVDQ_DTYPE_BF16) return SVDQ_ERR_DTYPE;
  const int max_M_pad = (max_M + 255) / 256 * 256;
  if (max_M <= 0 || !gemm_supported(max_M_pad, N, K, R)) return SVDQ_ERR_SHAPE;
  if (R > 0 && (lora_down_host == nullptr || lora_up_host == nullptr)) return SVDQ_ERR_NULL;
  svdq_linear_plan* p = new (std::nothrow) svdq_linear_plan();
  if (p == nullptr) return SVDQ_ERR_CUDA;
  p->max_M = max_M; p->max_M_pad = max_M_pad; p->K = K; p->N = N; p->R = R; p->dtype = dtype;
  int rc = SVDQ_OK;
  bool bad = cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking) != cudaSuccess;
  bad = bad || cudaStreamCreateWithFlags(&p->s_run, cudaStreamNonBlocking) != cudaSuccess;
  bad = bad || cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking) != cudaSuccess;
  const size_t mp = static_cast<size_t>(max_M_pad);
  for (int i = 0; i < kPlanSlots && !bad; ++i) {
    PlanSlot& q = p->slot[i];
    bad = bad || cudaMalloc(&q.x, static_cast<size_t>(max_M) * K * 2) != cudaSuccess;
    bad = bad || cudaMalloc(&q.act, mp * K / 2) != cudaSuccess;
    bad = bad || cudaMalloc(&q.ascales, mp * K / 16) != cudaSuccess;
    bad = bad || cudaMalloc(&q.ascales_swz, mp * K / 16) != cudaSuccess;
    bad = bad || cudaMalloc(&q.lora_act, mp * (R > 0 ? R : 1) * 4) != cudaSuccess;
    bad = bad || cudaMalloc(&q.lora_act16, 2 * lora16_elems(mp, R > 0 ? R : 1, dtype == SVDQ_DTYPE_BF16) + 16) != cudaSuccess;
    bad = bad || cudaMalloc(&q.y, mp * N * 2) != cudaSuccess;
    bad = bad || cudaMallocHost(&q.x_pin, static_cast<size_t>(max_M) * K * 2) != cudaSuccess;
    bad = bad || cudaMallocHost(&q.y_pin, mp * N * 2) != cudaSuccess;
    bad = bad || cudaEventCreateWithFlags(&q.x_ready, cudaEventDisableTiming) != cudaSuccess;
    bad = bad || cudaEventCreateWithFlags(&q.computed, cudaEventDisableTiming) != cudaSuccess;
    bad = bad || cudaEventCreateWithFlags(&q.y_done, cudaEventDisableTiming) != cudaSuccess;
  }
  if (bad) rc = SVDQ_ERR_CUDA;
  cudaStream_t st = p->s_run;
  void* wscales_dev = nullptr;
  if (rc == SVDQ_OK) rc = dev_upload(&p->wgt, wgt_host, static_cast<size_t>(N) * K / 2, st);
  if (rc == SVDQ_OK) rc = dev_upload(&wscales_dev, wscales_host, static_cast<size_t>(N) * K / 16, st);
  if (rc == SVDQ_OK && cudaMalloc(&p->wscales_swz, static_cast<size_t>(N) * K / 16) != cudaSuccess) rc = SVDQ_ERR_CUDA;
  if (rc == SVDQ_OK) rc = launch_swizzle_scales(wscales_dev, p->wscales_swz, K / 16, N, st);
  if (rc == SVDQ_OK) rc = dev_upload(&p->lora_down, lora_down_host, static_cast<size_t>(K) * R * 2, st);
  if (rc == SVDQ_OK) rc = dev_upload(&p->lora_up, lora_up_host, static_cast<size_t>(N) * R * 2, st);
  std::vector<uint16_t> lu16;                      // must outlive the asynchronous upload below
  if (rc == SVDQ_OK && dtype == SVDQ_DTYPE_BF16 && R > 0) {
    // fp16 copy of a bf16 lora_up for the single-pass LoRA route (skipped if a value does not fit)
    lu16.resize(static_cast<size_t>(N) * R);
    if (svdq_lora_up_to_f16(lora_up_host, lu16.data(), static_cast<long long>(lu16.size())) == SVDQ_OK)
      rc = dev_upload(&p->lora_up_f16, lu16.data(), lu16.size() * 2, st);
  }
  if (rc == SVDQ_OK) rc = dev_upload(&p->smooth, smooth_host, static_cast<size_t>(K) * 2, st);
  if (rc == SVDQ_OK && p->smooth != nullptr) {
    if (cudaMalloc(&p->smooth_table, static_cast<size_t>(K) * 8 + 16) != cudaSuccess) rc = SVDQ_ERR_CUDA;
    if (rc == SVDQ_OK) rc = launch_smooth_table(p->smooth, p->smooth_table, K, dtype, st);
  }
  if (rc == SVDQ_OK) rc = dev_upload(&p->wc, wcscales_host, static_cast<size_t>(N) * 2, st);
  if (rc == SVDQ_OK) rc = dev_upload(&p->bias, bias_host, static_cast<size_t>(N) * 2, st);
  if (rc == SVDQ_OK && gemm_split_plan(256, N, K, R) > 1) {
    // a call with few rows may take the split-K form: tiles x splits never exceeds the SM count
    p->split_ws_bytes = kSplitTicketBytes + static_cast<size_t>(sm_count()) * (128 * 128 * 4);
    if (cudaMalloc(&p->split_ws, p->split_ws_bytes) != cudaSuccess ||
        cudaMemsetAsync(p->split_ws, 0, kSplitTicketBytes, st) != cudaSuccess) rc = SVDQ_ERR_CUDA;
  }
  if (rc == SVDQ_OK && R > 0) {
    // calls of any height up to max_M: room for eight K ranks of the tallest one
    p->quant_ws_bytes = 2048 + static_cast<size_t>(8) * max_M_pad * 128 * 4;
    if (cudaMalloc(&p->quant_ws, p->quant_ws_bytes) != cudaSuccess ||
        cudaMemsetAsync(p->quant_ws, 0, 2048, st) != cudaSuccess) rc = SVDQ_ERR_CUDA;
  }
  if (rc == SVDQ_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = SVDQ_ERR_CUDA;
  if (wscales_dev != nullptr) cudaFree(wscales_dev);
  if (rc != SVDQ_OK) {
    svdq_linear_plan_destroy(p);
    return rc;
  }
  *out = p;
  return SVDQ_OK;
}

// Finish the call that last used slot `i`: wait for its y copy and, for a pageable y, move the rows
// out of the staging buffer.
static int plan_retire(svdq_linear_plan* p, int i) {
  PlanSlot& q = p->slot[i];
  if (!q.busy) return SVDQ_OK;
  q.busy = false;
  if (cudaEventSynchronize(q.y_done) != cudaSuccess) return SVDQ_ERR_CUDA;
  if (q.y_user != nullptr) { memcpy(q.y_user, q.y_pin, q.y_bytes); q.y_user = nullptr; }
  return SVDQ_OK;
}

int svdq_linear_plan_submit(svdq_linear_plan* p, const void* x_host, void* y_host, int M) {
  if (p == nullptr || x_host == nullptr || y_host == nullptr) return SVDQ_ERR_NULL;
  if (M <= 0 || M > p->max_M) return SVDQ_ERR_SHAPE;
  const int i = static_cast<int>(p->submitted % kPlanSlots);
  int rc = plan_retire(p, i);                      // at most kPlanSlots calls are in flight
  if (rc != SVDQ_OK) return rc;
  PlanSlot& q = p->slot[i];
  const int M_pad = (M + 255) / 256 * 256;
  const size_t xbytes = static_cast<size_t>(M) * p->K * 2, ybytes = static_cast<size_t>(M) * p->N * 2;
  // page-locked caller buffers are copied from and to directly; pageable ones go through the slot's staging
  const void* x_src = x_host;
  if (!is_pinned_host(x_host)) { memcpy(q.x_pin, x_host, xbytes); x_src = q.x_pin; }
  const bool y_pinned = is_pinned_host(y_host);
  bool bad = false;
  // x copy: after the kernels of the slot's previous call have read the old x (stream order on s_run
  // plus this wait; `computed` of a never-used slot is complete by definition)
  bad = bad || cudaStreamWaitEvent(p->s_in, q.computed, 0) != cudaSuccess;
  bad = bad || cudaMemcpyAsync(q.x, x_src, xbytes, cudaMemcpyHostToDevice, p->s_in) != cudaSuccess;
  bad = bad || cudaEventRecord(q.x_ready, p->s_in) != cudaSuccess;
  // kernels: after x has landed and the slot's previous y has left the device
  bad = bad || cudaStreamWaitEvent(p->s_run, q.x_ready, 0) != cudaSuccess;
  bad = bad || cudaStreamWaitEvent(p->s_run, q.y_done, 0) != cudaSuccess;
  if (bad) return SVDQ_ERR_CUDA;
  rc = svdq_quantize_w4a4_act_fuse_lora_ws(q.x, p->lora_down, p->smooth, p->smooth_table, q.act, q.ascales, q.lora_act,
                                           q.ascales_swz, q.lora_act16, M, p->K, p->R, M_pad, p->dtype, SVDQ_QUANT_AUTO,
                                           p->quant_ws, p->quant_ws_bytes, p->s_run);
  if (rc != SVDQ_OK) return rc;
  rc = svdq_gemm_w4a4_ws(q.act, p->wgt, q.ascales_swz, p->wscales_swz, p->R > 0 ? q.lora_act16 : nullptr,
                         p->R > 0 ? p->lora_up : nullptr, p->R > 0 ? p->lora_up_f16 : nullptr, p->wc, p->bias, q.y, M_pad,
                         p->N, p->K, p->R, p->dtype, 0, p->split_ws, p->split_ws_bytes, p->s_run);
  if (rc != SVDQ_OK) return rc;
  bad = bad || cudaEventRecord(q.computed, p->s_run) != cudaSuccess;
  // y copy
  bad = bad || cudaStreamWaitEvent(p->s_out, q.computed, 0) != cudaSuccess;
  bad = bad || cudaMemcpyAsync(y_pinned ? y_host : q.y_pin, q.y, ybytes, cudaMemcpyDeviceToHost, p->s_out) != cudaSuccess;
  bad = bad || cudaEventRecord(q.y_done, p->s_out) != cudaSuccess;
  if (bad) return SVDQ_ERR_CUDA;
  q.y_user = y_pinned ? nullptr : y_host;
  q.y_bytes = ybytes;
  q.busy = true;
  ++p->submitted;
  return SVDQ_OK;
}

int svdq_linear_plan_wait(svdq_linear_plan* p) {
  if (p == nullptr) return SVDQ_ERR_NULL;
  // oldest first
  for (int k = 0; k < kPlanSlots; ++k) {
    const int rc = plan_retire(p, static_cast<int>((p->submitted + k) % kPlanSlots));
    if (rc != SVDQ_OK) return rc;
  }
  return SVDQ_OK;
}

int svdq_linear_plan_forward_host(svdq_linear_plan* p, const void* x_host, void* y_host, int M) {
  const int rc = svdq_linear_plan_submit(p, x_host, y_host, M);
  return rc != SVDQ_OK ? rc : svdq_linear_plan_wait(p);
}

void svdq_linear_plan_destroy(svdq_linear_plan* p) {
  if (p == nullptr) return;
  if (p->s_in != nullptr) cudaStreamSynchronize(p->s_in);
  if (p->s_run != nullptr) cudaStreamSynchronize(p->s_run);
  if (p->s_out != nullptr) cudaStreamSynchronize(p->s_out);
  for (PlanSlot& q : p->slot) {
    void* dev[] = {q.x, q.act, q.ascales, q.ascales_swz, q.lora_act, q.lora_act16, q.y};
    for (void* d : dev)
      if (d != nullptr) cudaFree(d);
    if (q.x_pin != nullptr) cudaFreeHost(q.x_pin);
    if (q.y_pin != nullptr) cudaFreeHost(q.y_pin);
    if (q.x_ready != nullptr) cudaEventDestroy(q.x_ready);
    if (q.computed != nullptr) cudaEventDestroy(q.computed);
    if (q.y_done != nullptr) cudaEventDestroy(q.y_done);
  }
  void* dev[] = {p->wgt, p->wscales_swz, p->lora_down, p->lora_up, p->lora_up_f16, p->smooth, p->smooth_table, p->wc, p->bias,
                 p->split_ws, p->quant_ws};
  for (void* d : dev)
    if (d != nullptr) cudaFree(d);
  if (p->s_in != nullptr) cudaStreamDestroy(p->s_in);
  if (p->s_run != nullptr) cudaStreamDestroy(p->s_run);
  if (p->s_out != nullptr) cudaStreamDestroy(p->s_out);
  delete p;
}

}  // extern "C"
