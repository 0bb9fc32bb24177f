// Persistent, warp-specialised NVFP4 block-scaled GEMM with the LoRA-up product
// accumulated into the same tensor-memory accumulator and the per-column
// affine fused into the epilogue.
//
//   y = cast( (deq(act) deq(wgt)^T + lora_act lora_up^T) * wcscales + bias )
//
// Math order follows baseline/kernels/gemm_w4a4/ref.py:61-78 of the reference
// (LoRA added before the affine; multiply and add rounded separately in fp32).
// The reference's own kernel for this op is
// cute_kernels/gemm_w4a4/kernel_v2_fa4.py:841-1589.
//
// Work decomposition (one CTA per SM, 192 threads):
//   warps 0-3  epilogue: tensor memory -> registers -> affine -> 16-bit -> global
//   warp  4    producer: TMA loads into a ring of shared-memory stages
//   warp  5    MMA issuer: scale copies smem->TMEM, tcgen05.mma, commits
// A stage holds one 256-element K slab: A 128 x 128 B, B BN x 128 B (both
// 128-byte swizzled, K-major, two E2M1 codes per byte) and their scale atoms.
// The LoRA-up product reuses the very same ring: a slab of 64 rank elements of
// lora_act (128 rows x 128 B) and lora_up (BN rows x 128 B) has exactly the
// byte footprint of a main slab, so it is just ceil(R/64) more ring passes per
// output tile, issued as dense 16-bit MMAs into the same accumulator.
#include "sm100.cuh"
#include "svdq_internal.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <type_traits>
#include <cstdlib>

namespace svdq {

namespace gemm {

constexpr int BM = 128;          // rows of y per CTA tile
constexpr int BK = 256;          // K elements per stage (128 bytes of codes per row)
constexpr int A_BYTES = BM * 128;
constexpr int SFA_BYTES = BM * (BK / 16);  // 2048
constexpr int NUM_THREADS = 192;

template <int BN>
struct Cfg {
  static constexpr int B_BYTES = BN * 128;
  static constexpr int SFB_BYTES = BN * (BK / 16);
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int ACC_STAGES = (BN <= 128) ? 2 : 1;
  static constexpr int STAGES = (BN <= 128) ? 6 : 4;
  static constexpr int SFA_COLS = 16;                 // 4 k-blocks x 4 columns
  static constexpr int SFB_COLS = 4 * (BN / 32);      // 4 k-blocks x BN/32 columns
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 2048 /*affine*/ + 256 /*barriers*/;
};

struct Params {
  const uint8_t* sfa;   // swizzled activation scales
  const uint8_t* sfb;   // swizzled weight scales
  const void* wc;       // [N] or null
  const void* bias;     // [N] or null
  void* y;              // [M, N]
  int M, N, K, R;
  int tiles_m, tiles_n;
  int dbg;   // TEMP diagnostic switches
};

__device__ __forceinline__ uint32_t pack2(__half a, __half b) {
  __half2 h = __halves2half2(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack2(__nv_bfloat16 a, __nv_bfloat16 b) {
  __nv_bfloat162 h = __halves2bfloat162(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <typename T> __device__ __forceinline__ float as_f32(T v);
template <> __device__ __forceinline__ float as_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float as_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <int BN, typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_w4a4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmLA, const __grid_constant__ CUtensorMap tmLU, const Params p) {
  using C = Cfg<BN>;
  constexpr bool kBf16 = sizeof(OutT) == 2 && !std::is_same<OutT, __half>::value;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tail = smem + C::STAGES * C::STAGE_BYTES;
  float* affine = reinterpret_cast<float*>(tail);                 // [2][BN] : wcscales, bias of the current tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 2048);
  uint64_t* full = bars;                                          // [STAGES]
  uint64_t* empty = bars + C::STAGES;                             // [STAGES]
  uint64_t* acc_full = bars + 2 * C::STAGES;                      // [ACC_STAGES]
  uint64_t* acc_empty = acc_full + C::ACC_STAGES;                 // [ACC_STAGES]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + C::ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx ctx{abort_flag};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < C::ACC_STAGES; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB);
    if (p.R > 0) { tma_prefetch_desc(&tmLA); tma_prefetch_desc(&tmLU); }
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sfa = tmem_base + C::ACC_STAGES * BN;
  const uint32_t tmem_sfb = tmem_sfa + C::SFA_COLS;

  const int kt_main = (p.K + BK - 1) / BK;   // the last slab may hold fewer than four 64-element k-blocks
  const int kt_lora = (p.R + 63) / 64;
  const int kt_all = kt_main + kt_lora;
  const int total_tiles = p.tiles_m * p.tiles_n;
  const int k_groups4 = p.K / 64;   // scale atoms along K

  if (warp == 4) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mb = tile % p.tiles_m, nb = tile / p.tiles_m;
        const int m0 = mb * BM, n0 = nb * BN;
        for (int kt = 0; kt < kt_all; ++kt, ++it) {
          const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, ctx, kDevWaitEmpty, it)) { ok = false; break; }
          uint8_t* st = smem + s * C::STAGE_BYTES;
          if (p.dbg & 8) { mbar_arrive(&full[s]); continue; }
          if (kt < kt_main) {
            // codes past K are zero-filled by TMA (and still counted); scale atoms past K are not fetched
            const uint32_t nkb = min(4, k_groups4 - kt * 4);
            mbar_arrive_expect_tx(&full[s], A_BYTES + C::B_BYTES + nkb * 512u * (1 + BN / 128));
            tma_load_2d(st, &tmA, kt * 128, m0, &full[s]);
            tma_load_2d(st + A_BYTES, &tmB, kt * 128, n0, &full[s]);
            bulk_load_1d(st + A_BYTES + C::B_BYTES, p.sfa + (static_cast<size_t>(mb) * k_groups4 + kt * 4) * 512, nkb * 512u, &full[s]);
#pragma unroll
            for (int h = 0; h < BN / 128; ++h)
              bulk_load_1d(st + A_BYTES + C::B_BYTES + SFA_BYTES + h * 2048,
                           p.sfb + (static_cast<size_t>(nb * (BN / 128) + h) * k_groups4 + kt * 4) * 512, nkb * 512u, &full[s]);
          } else {
            const int r0 = (kt - kt_main) * 64;
            mbar_arrive_expect_tx(&full[s], A_BYTES + C::B_BYTES);
            tma_load_2d(st, &tmLA, r0, m0, &full[s]);
            tma_load_2d(st + A_BYTES, &tmLU, r0, n0, &full[s]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint64_t kDescAB = smem_desc_base(0, 1024, kSwizzle128B);   // K-major, 8-row groups 1024 B apart
      constexpr uint64_t kDescSF = smem_desc_base(0, 128, kSwizzleNone);    // 8 x 16 B core matrices, 128 B apart
      constexpr uint32_t kIdescMain = idesc_nvfp4(BM, BN);
      constexpr uint32_t kIdescLora = idesc_f16(kBf16, BM, BN, false, false);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
        const uint32_t as = tcount % C::ACC_STAGES, aph = (tcount / C::ACC_STAGES) & 1;
        if (!mbar_wait(&acc_empty[as], aph ^ 1, ctx, kDevWaitAccFree, tcount)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + as * BN;
        for (int kt = 0; kt < kt_all; ++kt, ++it) {
          const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&full[s], ph, ctx, kDevWaitFull, it)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
          if (kt < kt_main) {
            const uint32_t sfa_addr = b_addr + C::B_BYTES;
            const uint32_t sfb_addr = sfa_addr + SFA_BYTES;
            const int nkb = (p.dbg & 4) ? 0 : min(4, k_groups4 - kt * 4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (j < nkb && !((p.dbg & 2) && kt > 0)) {
                tmem_cp_scales<1>(tmem_sfa + j * 4, smem_desc(kDescSF, sfa_addr + j * 512));
#pragma unroll
                for (int h = 0; h < BN / 128; ++h)
                  tmem_cp_scales<1>(tmem_sfb + j * (BN / 32) + h * 4, smem_desc(kDescSF, sfb_addr + h * 2048 + j * 512));
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (j < nkb) mma_nvfp4<1>(tmem_acc, smem_desc(kDescAB, a_addr + j * 32), smem_desc(kDescAB, b_addr + j * 32),
                           kIdescMain, tmem_sfa + j * 4, tmem_sfb + j * (BN / 32), (kt | j) != 0 ? 1u : 0u);
          } else {
            const int r0 = (kt - kt_main) * 64;
            const int nk = (p.dbg & 4) ? 0 : min(4, (p.R - r0) / 16);
            for (int j = 0; j < nk; ++j)
              mma_f16<1>(tmem_acc, smem_desc(kDescAB, a_addr + j * 32), smem_desc(kDescAB, b_addr + j * 32),
                         kIdescLora, (kt | j) != 0 ? 1u : 0u);
          }
          tc_commit(&empty[s]);          // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(&acc_full[as]);  // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (warps 0-3) ------------------------------
    OutT* y = static_cast<OutT*>(p.y);
    const OutT* wc = static_cast<const OutT*>(p.wc);
    const OutT* bias = static_cast<const OutT*>(p.bias);
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
      const int mb = tile % p.tiles_m, nb = tile / p.tiles_m;
      const int m0 = mb * BM, n0 = nb * BN;
      const uint32_t as = tcount % C::ACC_STAGES, aph = (tcount / C::ACC_STAGES) & 1;
      // stage this tile's per-column affine terms (previous tile's readers are done: see the barrier below)
      for (int c = threadIdx.x; c < BN; c += 128) {
        affine[c] = wc != nullptr ? as_f32<OutT>(wc[n0 + c]) : 1.0f;
        affine[BN + c] = bias != nullptr ? as_f32<OutT>(bias[n0 + c]) : 0.0f;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!mbar_wait(&acc_full[as], aph, ctx, kDevWaitAcc, tcount)) ok = false;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + as * BN;
      const size_t row = static_cast<size_t>(m0 + warp * 32 + lane);
      OutT* yrow = y + row * p.N + n0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c0, v);
        tmem_ld_wait();
        uint32_t o[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float a = __uint_as_float(v[2 * i]), b = __uint_as_float(v[2 * i + 1]);
          if (wc != nullptr) { a = __fmul_rn(a, affine[c0 + 2 * i]); b = __fmul_rn(b, affine[c0 + 2 * i + 1]); }
          if (bias != nullptr) { a = __fadd_rn(a, affine[BN + c0 + 2 * i]); b = __fadd_rn(b, affine[BN + c0 + 2 * i + 1]); }
          o[i] = pack2(from_f32<OutT>(a), from_f32<OutT>(b));
        }
        uint4* dst = reinterpret_cast<uint4*>(yrow + c0);
        if (!(p.dbg & 1)) {
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
      // affine[] may be overwritten after this barrier; it also makes the four warps agree on whether to go on
      uint32_t any_failed;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\tsetp.eq.u32 p, %1, 0;\n\t"
          "bar.red.or.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
          : "=r"(any_failed) : "r"(ok ? 1u : 0u) : "memory");
      ok = any_failed == 0;
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // give copies that were already in flight time to land before the CTA's memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 50000ull) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace gemm

bool gemm_supported(int M, int N, int K, int R) {
  return M > 0 && N > 0 && K > 0 && M % 128 == 0 && N % 128 == 0 && K % 64 == 0 && R >= 0 && R % 16 == 0;
}

template <int BN, typename OutT>
static int launch_gemm_t(const void* act, const void* wgt, const void* sfa, const void* sfb, const void* la,
                         const void* lu, const void* wc, const void* bias, void* y, int M, int N, int K, int R,
                         cudaStream_t stream) {
  using C = gemm::Cfg<BN>;
  CUtensorMap tmA, tmB, tmLA, tmLU;
  int rc;
  if ((rc = make_tmap_2d(&tmA, act, 1, M, K / 2, K / 2, gemm::BM, 128, kTmapSwizzle128)) != SVDQ_OK) return rc;
  if ((rc = make_tmap_2d(&tmB, wgt, 1, N, K / 2, K / 2, BN, 128, kTmapSwizzle128)) != SVDQ_OK) return rc;
  if (R > 0) {
    if ((rc = make_tmap_2d(&tmLA, la, 2, M, R, static_cast<uint64_t>(R) * 2, gemm::BM, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
    if ((rc = make_tmap_2d(&tmLU, lu, 2, N, R, static_cast<uint64_t>(R) * 2, BN, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
  } else {
    tmLA = tmA; tmLU = tmB;
  }
  gemm::Params p;
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.wc = wc; p.bias = bias; p.y = y;
  p.M = M; p.N = N; p.K = K; p.R = R;
  p.tiles_m = M / gemm::BM; p.tiles_n = N / BN;
  { const char* e = getenv("SVDQ_DEBUG"); p.dbg = e ? atoi(e) : 0; }
  auto kern = gemm::gemm_w4a4_kernel<BN, OutT>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) return SVDQ_ERR_LAUNCH;
    configured = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, gemm::NUM_THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, tmLA, tmLU, p);
  return cudaGetLastError() == cudaSuccess ? SVDQ_OK : SVDQ_ERR_LAUNCH;
}

int launch_gemm_w4a4(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                     const void* lora_act16, const void* lora_up, const void* wcscales, const void* bias, void* y,
                     int M, int N, int K, int R, int dtype, int variant, cudaStream_t stream) {
  if (!gemm_supported(M, N, K, R)) return SVDQ_ERR_SHAPE;
  const bool wide = (variant == 0) ? (N % 256 == 0) : (variant == 256);
  if (wide && N % 256 != 0) return SVDQ_ERR_SHAPE;
  if (dtype == SVDQ_DTYPE_F16) {
    return wide ? launch_gemm_t<256, __half>(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, wcscales, bias, y, M, N, K, R, stream)
                : launch_gemm_t<128, __half>(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, wcscales, bias, y, M, N, K, R, stream);
  } else if (dtype == SVDQ_DTYPE_BF16) {
    return wide ? launch_gemm_t<256, __nv_bfloat16>(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, wcscales, bias, y, M, N, K, R, stream)
                : launch_gemm_t<128, __nv_bfloat16>(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, wcscales, bias, y, M, N, K, R, stream);
  }
  return SVDQ_ERR_DTYPE;
}

}  // namespace svdq
