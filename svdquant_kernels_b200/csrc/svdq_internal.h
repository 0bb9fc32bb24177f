// Internal launch prototypes shared by the translation units of libsvdq_b200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/svdq_b200.h"

namespace svdq {

// quantize_generic.cu
int launch_quantize_rows(const void* x, const void* smooth, void* codes, void* scales, void* scales_swz, int rows,
                         int rows_pad, int K, int dtype, cudaStream_t stream);
int launch_lora_down(const void* x, const void* w, float* out, void* out16, int M, int M_pad, int K, int R, int dtype,
                     cudaStream_t stream);
int launch_swizzle_scales(const void* src, void* dst, int groups, int rows, cudaStream_t stream);
int launch_cast_f32(const float* src, void* dst, int rows, int R, int dtype, cudaStream_t stream);

// quantize_fused.cu
bool quantize_fused_supported(int M, int K, int R, int M_pad);
int launch_smooth_table(const void* smooth, void* table, int K, int dtype, cudaStream_t stream);
int launch_quantize_fused(const void* x, const void* lora_down, const void* smooth_table, void* act, void* ascales,
                          float* lora_act, void* ascales_swz, void* lora_act16, int M, int K, int R, int M_pad,
                          int dtype, cudaStream_t stream);

int quantize_fused_max_clusters(int R, int ks, int dtype);

// quantize_stream.cu : the form for tall activations (128- or 256-row tiles, K split met in a workspace)
bool quantize_stream_plan(int M, int K, int R, int M_pad, int* tm_out, int* ks_out);
size_t quantize_stream_workspace_bytes(int M, int K, int R, int M_pad);
int launch_quantize_stream(const void* x, const void* lora_down, const void* smooth_table, void* act, void* ascales,
                           float* lora_act, void* ascales_swz, void* lora_act16, int M, int K, int R, int M_pad,
                           int dtype, void* ws, size_t ws_bytes, int tm, int ks, cudaStream_t stream);

// gemm_w4a4.cu
bool gemm_supported(int M, int N, int K, int R);
// Column-sharded form: y is the local [M, y_ld] matrix, this launch fills columns [col0, col0 + N)
// of it and of the same matrix of n_peers other GPUs (peer-mapped pointers).  y_ld = 0: plain call.
struct GemmTp {
  int col0 = 0, y_ld = 0, n_peers = 0;
  void* y_peer[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  // split-K workspace (plain form only): ticket counters (zero between launches), then fp32 partial tiles
  void* ws = nullptr;
  size_t ws_bytes = 0;
  int interleave = 0;            // LoRA slabs spread among the main slabs (1) or after them (0)
  // next-layer quantisation in the epilogue (plain form only): smooth_next [N] in the output type, qout
  // [M, N/2], oscales [N/16, M] and optionally the tensor-core twin of oscales
  const void* smooth_next = nullptr;
  void* qout = nullptr;
  void* oscales = nullptr;
  void* oscales_swz = nullptr;
};
constexpr size_t kSplitTicketBytes = 1024;     // 256 ticket counters
constexpr int kSplitMaxTiles = 74;             // split-K is for problems with at most this many 128 x 128 tiles
constexpr int kSplitMax = 6;                   // CTAs per tile at most
int gemm_split_plan(int M, int N, int K, int R);
size_t gemm_split_workspace_bytes(int M, int N, int K, int R);
int launch_gemm_w4a4(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                     const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales,
                     const void* bias, void* y, int M, int N, int K, int R, int dtype, int variant,
                     const GemmTp& tp, cudaStream_t stream);

// tensormap.cu : cuTensorMapEncodeTiled resolved through the runtime at first use
enum TmapSwizzle { kTmapSwizzleNone = 0, kTmapSwizzle128 = 1 };
// 2-D row-major tensor [rows, cols] of `elem_bytes`-sized elements; box = [box_rows, box_cols].
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, TmapSwizzle swz);
int sm_count();

// status word (defined once in gemm_w4a4.cu via sm100.cuh's extern declaration)
int read_and_clear_status(unsigned int out[4]);

}  // namespace svdq
