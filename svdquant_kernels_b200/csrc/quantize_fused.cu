// Fused activation quantizer + LoRA-down for sm_100a: one pass over x.
//
//   act, ascales = nvfp4( x / smooth )        bit-exact with the reference oracle
//   lora_act     = x @ lora_down              fp32, tcgen05 dense 16-bit MMA
//
// Replaces the reference's Triton kernel
// (triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:115-286); results
// follow baseline/kernels/quantize_w4a4_act_fuse_lora/ref.py:19-50.
//
// Decomposition.  A cluster of KS CTAs owns one tile of 128 rows; CTA k of the
// cluster owns a contiguous range of 64-column slabs of K.  Per slab the
// producer warp TMA-loads the x tile (128 x 64, 128-byte swizzle) and the
// matching lora_down slab (64 x R) into one ring stage.  Two consumers read
// the same stage: the MMA warp accumulates x_tile @ lora_down_slab into a
// [128 x R] fp32 accumulator in tensor memory, and the quantize warps turn the
// tile into codes and scales.  x is read from HBM exactly once.  At the end the
// KS partial accumulators are summed in a fixed order through distributed
// shared memory (no atomics, no zero-fill, no scratch in global memory).
//
// Exact arithmetic.  x / smooth must equal the IEEE quotient.  It is computed
// as q0 = x*r, e = fma(-s, q0, x), q = fma(e, r, q0) with r = RN(1/s) held in
// shared memory; for operands with at most 11 significant bits this is the
// correctly rounded quotient (checked exhaustively over mantissas).  Columns
// whose smooth lies outside [2^-60, 2^60] switch the CTA to __fdiv_rn.
#include "nvfp4_math.cuh"
#include "sm100.cuh"
#include "svdq_internal.h"
#include <cstdlib>

namespace svdq {
namespace qf {

constexpr int TILE_M = 128;
constexpr int SLAB_K = 64;                 // columns per ring stage (128 bytes of 16-bit x)
constexpr int X_BYTES = TILE_M * 128;      // 16 KB
constexpr int QUANT_WARPS = 8;
constexpr int NUM_THREADS = (2 + QUANT_WARPS) * 32;
constexpr int MAX_KRANGE = 4096;           // columns per CTA whose (smooth, 1/smooth) fit the table

template <int RP>
struct Cfg {
  static constexpr int W_BYTES = SLAB_K * RP * 2;                 // lora_down slab
  static constexpr int STAGE_BYTES = X_BYTES + W_BYTES;
  static constexpr int STAGES = RP <= 64 ? 7 : (RP <= 128 ? 6 : 4);
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int TABLE_BYTES = MAX_KRANGE * 8;              // float2 {smooth, 1/smooth}
  static constexpr int SMEM_BYTES = 1024 + RING_BYTES + TABLE_BYTES + 256;
  static constexpr int TMEM_COLS = RP < 32 ? 32 : RP;             // power of two >= 32
  static_assert(TILE_M * RP * 4 <= RING_BYTES, "partial accumulator must fit in the ring");
};

struct Params {
  const void* smooth;     // [K] or null
  uint8_t* act;           // [M_pad, K/2]
  uint8_t* scales;        // [K/16, M_pad]
  uint8_t* scales_swz;    // atom order or null
  float* lora;            // [M_pad, R]
  void* lora16;           // [M_pad, R] or null
  int M, K, R, M_pad;
  int dbg;   // TEMP diagnostic switches
};

template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t v);
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<__half2*>(&v));
}
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
}
template <typename T> __device__ __forceinline__ uint32_t pack2_rn(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2_rn<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2_rn<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// float4 slot of (row, c4) in the partial-accumulator buffer; the XOR spreads the
// 32 rows a warp writes at once over all bank groups.
__device__ __forceinline__ uint32_t partial_slot(uint32_t row, uint32_t c4, uint32_t rp4) {
  return row * rp4 + (c4 ^ (row & 7u));
}

template <typename T, int RP>
__global__ void __launch_bounds__(NUM_THREADS, 1)
quantize_fused_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const Params p) {
  using C = Cfg<RP>;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float2* table = reinterpret_cast<float2*>(smem + C::RING_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::RING_BYTES + C::TABLE_BYTES);
  uint64_t* full = bars;                       // [STAGES]  producer -> consumers
  uint64_t* empty = bars + C::STAGES;          // [STAGES]  consumers -> producer
  uint64_t* acc_done = bars + 2 * C::STAGES;   // MMA -> epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* slow_div = abort_flag + 1;
  const WaitCtx ctx{abort_flag};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ks = gridDim.y;               // cluster = (1, KS, 1): blockIdx.y is the rank along K
  const uint32_t krank = blockIdx.y;
  const int m0 = blockIdx.x * TILE_M;

  // slabs owned by this CTA
  const int n_slabs = p.K / SLAB_K;
  const int base = n_slabs / ks, rem = n_slabs % ks;
  const int slab_begin = static_cast<int>(krank) * base + (static_cast<int>(krank) < rem ? static_cast<int>(krank) : rem);
  const int my_slabs = base + (static_cast<int>(krank) < rem ? 1 : 0);
  const int k_begin = slab_begin * SLAB_K;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *slow_div = 0;
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1 + QUANT_WARPS / 2); }
    mbar_init(acc_done, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmX);
    if (p.R > 0) tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  __syncthreads();   // slow_div initialised before anyone may raise it
  // {smooth, 1/smooth} of this CTA's columns
  if (p.smooth != nullptr) {
    const T* sm = static_cast<const T*>(p.smooth);
    for (int i = threadIdx.x; i < my_slabs * SLAB_K; i += NUM_THREADS) {
      const float s = to_f32(sm[k_begin + i]);
      table[i] = make_float2(s, __frcp_rn(s));
      const float a = fabsf(s);
      if (!(a >= 8.6736174e-19f && a <= 1.1529215e18f)) *slow_div = 1;   // outside [2^-60, 2^60] or NaN
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_acc = *tmem_slot;
  const bool use_fdiv = *slow_div != 0;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      for (int i = 0; i < my_slabs; ++i) {
        const uint32_t s = i % C::STAGES, ph = (i / C::STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, ctx, kDevWaitEmpty, i)) break;
        uint8_t* st = smem + s * C::STAGE_BYTES;
        const int k0 = k_begin + i * SLAB_K;
        mbar_arrive_expect_tx(&full[s], p.R > 0 ? C::STAGE_BYTES : X_BYTES);
        tma_load_2d(st, &tmX, k0, m0, &full[s]);
        if (p.R > 0) {
#pragma unroll
          for (int b = 0; b < RP / 64; ++b) tma_load_2d(st + X_BYTES + b * (SLAB_K * 128), &tmW, b * 64, k0, &full[s]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint64_t kDescA = smem_desc_base(0, 1024, kSwizzle128B);               // x tile, K-major
      constexpr uint64_t kDescB = smem_desc_base(SLAB_K * 128, 1024, kSwizzle128B);    // lora_down slab, R-major
      constexpr uint32_t kIdesc = idesc_f16(kBf16, TILE_M, RP, false, true);
      bool ok = true;
      for (int i = 0; i < my_slabs && ok; ++i) {
        const uint32_t s = i % C::STAGES, ph = (i / C::STAGES) & 1;
        if (!mbar_wait(&full[s], ph, ctx, kDevWaitFull, i)) { ok = false; break; }
        tc_fence_after_sync();
        if (p.R > 0 && !(p.dbg & 64)) {
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + X_BYTES;
#pragma unroll
          for (int j = 0; j < SLAB_K / 16; ++j)
            mma_f16<1>(tmem_acc, smem_desc(kDescA, a_addr + j * 32), smem_desc(kDescB, b_addr + j * 2048), kIdesc,
                       (i | j) != 0 ? 1u : 0u);
        }
        if (p.R > 0) tc_commit(&empty[s]); else mbar_arrive(&empty[s]);
      }
      if (ok && p.R > 0) tc_commit(acc_done);
    }
    __syncwarp();
  } else {
    // ------------------------------ quantize warps ------------------------------
    const int qw = warp - 2;                  // 0..7
    const int half_id = qw >> 2;              // which alternate slab this warp group takes
    const int row = (qw & 3) * 32 + lane;     // row of the tile
    const int m = m0 + row;
    const int groups = p.K >> 4;
    const uint32_t xor7 = static_cast<uint32_t>(row & 7);
    uint8_t* act_row = p.act + static_cast<size_t>(m) * (p.K >> 1);
    for (int i = half_id; i < my_slabs; i += 2) {
      const uint32_t s = i % C::STAGES, ph = (i / C::STAGES) & 1;
      if (!mbar_wait(&full[s], ph, ctx, kDevWaitFull, 0x10000 + i)) break;
      const uint8_t* xrow = smem + s * C::STAGE_BYTES + row * 128;
      uint4 raw[8];
#pragma unroll
      for (uint32_t c = 0; c < 8; ++c) raw[c] = *reinterpret_cast<const uint4*>(xrow + ((c ^ xor7) << 4));
      // the stage is no longer needed by this warp
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);

      if (p.dbg & 16) continue;
      const int kl = i * SLAB_K;              // column offset inside this CTA's range
      uint32_t codes[8];
      uint32_t sbytes = 0;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float f[16];
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw[2 * g]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 v = unpack2<T>(w[j]);
          f[2 * j] = v.x; f[2 * j + 1] = v.y;
        }
        if (p.smooth != nullptr) {
          const float4* tb = reinterpret_cast<const float4*>(table + kl + g * 16);
          if (!use_fdiv) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 t = tb[j];          // {s0, r0, s1, r1}
              float q0 = f[2 * j] * t.y;
              float e0 = fmaf(-t.x, q0, f[2 * j]);
              f[2 * j] = fmaf(e0, t.y, q0);
              float q1 = f[2 * j + 1] * t.w;
              float e1 = fmaf(-t.z, q1, f[2 * j + 1]);
              f[2 * j + 1] = fmaf(e1, t.w, q1);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 t = tb[j];
              f[2 * j] = __fdiv_rn(f[2 * j], t.x);
              f[2 * j + 1] = __fdiv_rn(f[2 * j + 1], t.z);
            }
          }
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(f[j]));
        const uint8_t sb = scale_byte_from_amax(amax);
        sbytes |= static_cast<uint32_t>(sb) << (8 * g);
        const GroupBounds gb = bounds_for_scale(e4m3_to_f32(sb));
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) lo |= e2m1_code(f[j], gb) << (4 * j);
#pragma unroll
        for (int j = 0; j < 8; ++j) hi |= e2m1_code(f[8 + j], gb) << (4 * j);
        codes[2 * g] = lo; codes[2 * g + 1] = hi;
      }
      const int k0 = k_begin + kl;
      if ((p.dbg & 32) && codes[0] != 0x12345678u) continue;
      uint4* dst = reinterpret_cast<uint4*>(act_row + (k0 >> 1));
      dst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
      dst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
      const int g0 = k0 >> 4;
#pragma unroll
      for (int g = 0; g < 4; ++g) p.scales[static_cast<size_t>(g0 + g) * p.M_pad + m] = static_cast<uint8_t>(sbytes >> (8 * g));
      if (p.scales_swz != nullptr)
        *reinterpret_cast<uint32_t*>(p.scales_swz + sf_swizzled_offset(m, g0, groups)) = sbytes;
    }
    // every quantize warp is done reading the ring before it is reused below
    asm volatile("bar.sync 2, %0;" ::"n"(QUANT_WARPS * 32) : "memory");
  }

  // ------------------------------ LoRA epilogue ------------------------------
  if (p.R > 0) {
    constexpr uint32_t RP4 = RP / 4;
    float4* partial = reinterpret_cast<float4*>(smem);       // reuses the ring
    if (warp >= 2) {
      const int qw = warp - 2;
      const int quarter = warp & 3;                           // TMEM lanes this warp may read
      const int chalf = (qw >> 2);                            // column half
      const uint32_t row = quarter * 32 + lane;
      const bool ok = mbar_wait(acc_done, 0, ctx, kDevWaitAcc, 0);
      tc_fence_after_sync();
      constexpr int COLS_PER_WARP = RP / 2;
#pragma unroll 1
      for (int c0 = chalf * COLS_PER_WARP; c0 < (chalf + 1) * COLS_PER_WARP; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, v);
        tmem_ld_wait();
        if (ks > 1) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            partial[partial_slot(row, (c0 >> 2) + j, RP4)] =
                make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
        } else if (ok) {
          const size_t gm = static_cast<size_t>(m0 + row);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int c = c0 + 4 * j;
            if (c < p.R) {
              *reinterpret_cast<float4*>(p.lora + gm * p.R + c) =
                  make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
              if (p.lora16 != nullptr)
                *reinterpret_cast<uint2*>(static_cast<T*>(p.lora16) + gm * p.R + c) =
                    make_uint2(pack2_rn<T>(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1])),
                               pack2_rn<T>(__uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
            }
          }
        }
      }
    }
    if (ks > 1) {
      tc_fence_before_sync();
      cluster_sync_all();                                     // every CTA's partial is in its shared memory
      // CTA k sums rows [k*128/KS, (k+1)*128/KS) over the cluster, in rank order
      const uint32_t rows_per = TILE_M / ks;
      const uint32_t row_lo = krank * rows_per;
      const uint32_t items = rows_per * RP4;
      const uint32_t base_addr = smem_u32(partial);
      for (uint32_t it = threadIdx.x; it < items; it += NUM_THREADS) {
        const uint32_t row = row_lo + it / RP4, c4 = it % RP4;
        const uint32_t off = base_addr + partial_slot(row, c4, RP4) * 16u;
        float4 acc = ld_cluster_f4(map_to_cta(off, 0));
        for (uint32_t j = 1; j < ks; ++j) {
          const float4 t = ld_cluster_f4(map_to_cta(off, j));
          acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
        }
        const int c = c4 * 4;
        if (c < p.R) {
          const size_t gm = static_cast<size_t>(m0 + row);
          *reinterpret_cast<float4*>(p.lora + gm * p.R + c) = acc;
          if (p.lora16 != nullptr)
            *reinterpret_cast<uint2*>(static_cast<T*>(p.lora16) + gm * p.R + c) =
                make_uint2(pack2_rn<T>(acc.x, acc.y), pack2_rn<T>(acc.z, acc.w));
        }
      }
      cluster_sync_all();                                     // nobody leaves while its memory is being read
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 50000ull) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_acc, C::TMEM_COLS);
  }
}

}  // namespace qf

// How many CTAs share one row tile along K (0 = no admissible split).
static int pick_k_split(int M_pad, int K) {
  const int tiles = M_pad / qf::TILE_M;
  const int slabs = K / qf::SLAB_K;
  const int sms = sm_count();
  int best = 0;
  double best_cost = 1e30;
  for (int ks : {1, 2, 4}) {
    if (ks > slabs) continue;
    if (((slabs + ks - 1) / ks) * qf::SLAB_K > qf::MAX_KRANGE) continue;
    const int ctas = tiles * ks;
    const int waves = (ctas + sms - 1) / sms;
    const double cost = static_cast<double>(waves) * ((slabs + ks - 1) / ks) + 2.0 * (ks > 1);
    if (cost < best_cost) { best_cost = cost; best = ks; }
  }
  return best;
}

bool quantize_fused_supported(int M, int K, int R, int M_pad) {
  if (M <= 0 || K <= 0 || M_pad < M) return false;
  if (M_pad % qf::TILE_M != 0 || K % qf::SLAB_K != 0) return false;
  if (R < 0 || R > 256 || R % 8 != 0) return false;
  return pick_k_split(M_pad, K) != 0;
}

template <typename T, int RP>
static int launch_qf(const void* x, const void* w, const qf::Params& p, cudaStream_t stream) {
  using C = qf::Cfg<RP>;
  CUtensorMap tmX, tmW;
  int rc;
  if ((rc = make_tmap_2d(&tmX, x, 2, p.M, p.K, static_cast<uint64_t>(p.K) * 2, qf::TILE_M, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
  if (p.R > 0) {
    if ((rc = make_tmap_2d(&tmW, w, 2, p.K, p.R, static_cast<uint64_t>(p.R) * 2, qf::SLAB_K, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
  } else {
    tmW = tmX;
  }
  auto kern = qf::quantize_fused_kernel<T, RP>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) return SVDQ_ERR_LAUNCH;
    configured = true;
  }
  int ks = pick_k_split(p.M_pad, p.K);
  { const char* e = getenv("SVDQ_KS"); if (e) ks = atoi(e); }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.M_pad / qf::TILE_M, ks, 1);
  cfg.blockDim = dim3(qf::NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = ks;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, tmX, tmW, p) != cudaSuccess) return SVDQ_ERR_LAUNCH;
  return SVDQ_OK;
}

template <typename T, int RP>
static int max_clusters_t(int ks) {
  using C = qf::Cfg<RP>;
  auto kern = qf::quantize_fused_kernel<T, RP>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(64, ks, 1);
  cfg.blockDim = dim3(qf::NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = ks; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return -1; }
  return n;
}

int quantize_fused_max_clusters(int R, int ks, int dtype) {
  const int rp = R <= 64 ? 64 : (R <= 128 ? 128 : 256);
  if (dtype == SVDQ_DTYPE_F16) return rp == 64 ? max_clusters_t<__half, 64>(ks) : rp == 128 ? max_clusters_t<__half, 128>(ks) : max_clusters_t<__half, 256>(ks);
  return rp == 64 ? max_clusters_t<__nv_bfloat16, 64>(ks) : rp == 128 ? max_clusters_t<__nv_bfloat16, 128>(ks) : max_clusters_t<__nv_bfloat16, 256>(ks);
}

int launch_quantize_fused(const void* x, const void* lora_down, const void* smooth, void* act, void* ascales,
                          float* lora_act, void* ascales_swz, void* lora_act16, int M, int K, int R, int M_pad,
                          int dtype, cudaStream_t stream) {
  if (!quantize_fused_supported(M, K, R, M_pad)) return SVDQ_ERR_UNSUPPORTED;
  qf::Params p;
  p.smooth = smooth;
  p.act = static_cast<uint8_t*>(act);
  p.scales = static_cast<uint8_t*>(ascales);
  p.scales_swz = static_cast<uint8_t*>(ascales_swz);
  p.lora = lora_act;
  p.lora16 = lora_act16;
  p.M = M; p.K = K; p.R = R; p.M_pad = M_pad;
  { const char* e = getenv("SVDQ_DEBUG"); p.dbg = e ? atoi(e) : 0; }
  const int rp = R <= 64 ? 64 : (R <= 128 ? 128 : 256);
  if (dtype == SVDQ_DTYPE_F16) {
    if (rp == 64) return launch_qf<__half, 64>(x, lora_down, p, stream);
    if (rp == 128) return launch_qf<__half, 128>(x, lora_down, p, stream);
    return launch_qf<__half, 256>(x, lora_down, p, stream);
  } else if (dtype == SVDQ_DTYPE_BF16) {
    if (rp == 64) return launch_qf<__nv_bfloat16, 64>(x, lora_down, p, stream);
    if (rp == 128) return launch_qf<__nv_bfloat16, 128>(x, lora_down, p, stream);
    return launch_qf<__nv_bfloat16, 256>(x, lora_down, p, stream);
  }
  return SVDQ_ERR_DTYPE;
}

}  // namespace svdq
