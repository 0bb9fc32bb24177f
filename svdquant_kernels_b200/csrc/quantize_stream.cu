// Fused activation quantizer + LoRA-down for sm_100a, the form for tall activations
// (thousands of rows): one pass over x, no thread-block clusters.
//
//   act, ascales = nvfp4( x / smooth )        bit-exact with the reference oracle
//   lora_act     = x @ lora_down              fp32, tcgen05 dense 16-bit MMA
//
// Same results as quantize_fused.cu (which stays the form for a few hundred rows); replaces the
// reference's Triton kernel (triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:115-286);
// results follow baseline/kernels/quantize_w4a4_act_fuse_lora/ref.py:19-50.
//
// Why a second form.  With 64-row tiles every 8 KB slab of x drags a 16 KB slab of lora_down
// through shared memory and four small MMAs through the tensor pipe, and both cost more than the
// HBM time of the slab: the kernel ran at 58 % of the copy bandwidth however few instructions the
// quantize warps executed.  Here a CTA owns TM = 128 or 256 rows and 1/KS of K, so a lora_down slab
// serves two to four times as many rows, and the LoRA product is computed transposed,
//     lora_act^T [R x TM] += lora_down_slab^T [R x 16] * x_tile^T [16 x TM]
// (A = lora_down slab, M = 128 = R padded, MN-major; B = x tile, N = TM, K-major), so that one MMA
// instruction covers all TM rows: 4 MMAs per 64-column slab whatever TM is.
//
// The KS partial sums of a row tile meet in a caller-owned workspace in global memory (they stay in
// L2): every CTA parks its fp32 partial [TM x 128], raises the tile's arrival counter and waits
// (bounded) until all KS have arrived; CTA k then adds rows [k TM/KS, (k+1) TM/KS) of the KS
// partials in rank order - the sum does not depend on timing - and writes lora_act and its 16-bit
// twin.  All CTAs of a launch are resident at once (the host only chooses KS > 1 when tiles x KS
// fits the SM count), so the wait cannot starve; the counters return to zero before the launch
// ends.  Four auxiliary warps (TMA producer, MMA issuer, two helpers) do this exchange while the
// sixteen quantize warps are still busy with the last slabs.
#include "nvfp4_math.cuh"
#include "quantize_math.cuh"
#include "sm100.cuh"
#include "svdq_internal.h"

#include <cstdlib>
#include <type_traits>

namespace svdq {
namespace qs {

constexpr int SLAB_K = 64;                 // columns per ring stage (128 bytes of 16-bit x per row)
constexpr int RP = 128;                    // LoRA rank padded to the MMA's M
constexpr int W_BYTES = SLAB_K * RP * 2;   // lora_down slab: 16 KB
constexpr int QUANT_WARPS = 16;
constexpr int AUX_WARPS = 4;               // producer, MMA issuer, two helpers; together they drain the accumulator
constexpr int NUM_THREADS = (AUX_WARPS + QUANT_WARPS) * 32;
constexpr int TB_BYTES = SLAB_K * 8;       // table entries of a slab's columns
constexpr int TB_GROUP_STRIDE = 144;       // spacing of the four 128-byte group pieces in a stage
constexpr int kTicketBytes = 2048;         // arrival counters [256], then completion counters [256]

template <int TM>
struct Cfg {
  static constexpr int X_BYTES = TM * 128;
  static constexpr int STAGE_BYTES = X_BYTES + W_BYTES + 1024;   // + table slab, padded to the 1 KB swizzled tiles need
  static constexpr int QUANT_GROUPS = 256 / TM;                  // groups of warps that take slabs in turn
  static constexpr int GROUP_WARPS = QUANT_WARPS / QUANT_GROUPS; // each warp: 16 rows of the tile
  static constexpr int STAGES_RAW = (232448 - 1024 - 512 - 1024) / STAGE_BYTES;
  // a multiple of the group count, so that a group always meets the same stages (see quantize_fused.cu)
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : (STAGES_RAW / QUANT_GROUPS) * QUANT_GROUPS;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = 1024 + RING_BYTES + 512 + 1024;   // ring, barriers, scale-constant table
  static constexpr int TMEM_COLS = TM;
  static_assert(TM == 128 || TM == 256, "tile height");
  static_assert(GROUP_WARPS * 16 == TM, "16 rows per quantize warp");
  static_assert(STAGES >= 2 * QUANT_GROUPS, "ring too shallow");
};

struct Params {
  const float2* table;    // [K/2] entries of qmath::smooth_table_entry followed by one flag word, or null (no smoothing)
  uint8_t* act;           // [M_pad, K/2]
  uint8_t* scales;        // [K/16, M_pad]
  uint8_t* scales_swz;    // atom order or null
  float* lora;            // [M_pad, R]
  void* lora16;           // 16-bit form of lora or null
  unsigned int* tickets;  // workspace head (KS > 1)
  float* partials;        // workspace body: [tiles][KS][TM][128] fp32
  int M, K, R, M_pad, ks;
};

// Bounded wait until *flag >= target (flag in global memory, raised by other CTAs of this launch).
__device__ __forceinline__ bool wait_counter(const unsigned int* flag, unsigned int target, const WaitCtx& ctx, unsigned int tag) {
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) return true;
    if (*ctx.abort_flag) return false;
    __nanosleep(40);
    if ((++spins & 0x3F) == 0) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > SVDQ_WAIT_LIMIT_NS) { report_failure(ctx, kDevWaitMisc, tag); return false; }
    }
  }
}

// CTA `krank` of a row tile adds rows [krank TM/KS, (krank+1) TM/KS) of the tile's KS partial sums
// (fp32 [TM][128] each, KS of them back to back at `first`) in rank order and writes lora_act and its
// 16-bit twin.  All KS loads of an item are in flight together (one round trip to L2 per item pair,
// not per partial).  Returns a bit per 32-row block of the tile in which a value did not fit fp16.
template <typename T, int TM, int KS>
__device__ __forceinline__ uint32_t add_partials(const Params& p, const float4* first, int m0, int krank, int tid, size_t plane) {
  constexpr int rows_per = TM / KS;
  const int row_lo = krank * rows_per;
  const int r4 = p.R >> 2;                    // float4 per row that carry rank columns
  uint32_t unfit = 0u;
  for (int it = tid; it < rows_per * r4; it += AUX_WARPS * 32) {
    const int row = row_lo + it / r4, c4 = it % r4;
    const float4* src = first + row * (RP / 4) + c4;
    float4 t[KS];
#pragma unroll
    for (int j = 0; j < KS; ++j) t[j] = __ldcg(src + static_cast<size_t>(j) * (TM * RP / 4));
    float4 acc = t[0];
#pragma unroll
    for (int j = 1; j < KS; ++j) { acc.x += t[j].x; acc.y += t[j].y; acc.z += t[j].z; acc.w += t[j].w; }
    const size_t idx = static_cast<size_t>(m0 + row) * p.R + c4 * 4;
    *reinterpret_cast<float4*>(p.lora + idx) = acc;
    if (p.lora16 != nullptr) {
      store_lora16x4<T>(p.lora16, idx, plane, acc);
      if (std::is_same<T, __nv_bfloat16>::value && !fits_f16(acc)) unfit |= 1u << (row >> 5);
    }
  }
  return unfit;
}

template <typename T, int TM>
__global__ void __launch_bounds__(NUM_THREADS, 1)
quantize_stream_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const Params p) {
  using C = Cfg<TM>;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::RING_BYTES);
  uint64_t* full = bars;                       // [STAGES]  producer -> consumers
  uint64_t* empty = bars + C::STAGES;          // [STAGES]  consumers -> producer
  uint64_t* acc_done = bars + 2 * C::STAGES;   // MMA -> epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* lora_unfit = tmem_slot + 2;        // [8] bf16 form: per 32 rows of the tile, some value does not fit fp16
  float2* scale_lut = reinterpret_cast<float2*>(smem + C::RING_BYTES + 512);
  const WaitCtx ctx{abort_flag};

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  auto uwait = [&](uint64_t* bar, uint32_t parity, unsigned int code, unsigned int tag) -> bool {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, code, tag)) != 0;
  };
  const int ks = p.ks;
  const int tile = blockIdx.x, krank = blockIdx.y;
  const int m0 = tile * TM;
  const bool has_lora = p.R > 0;
  const bool has_table = p.table != nullptr;

  // slabs owned by this CTA
  const int n_slabs = p.K / SLAB_K;
  const int base = n_slabs / ks, rem = n_slabs % ks;
  const int slab_begin = krank * base + (krank < rem ? krank : rem);
  const int my_slabs = base + (krank < rem ? 1 : 0);
  const int k_begin = slab_begin * SLAB_K;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1 + C::GROUP_WARPS); }
    mbar_init(acc_done, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmX);
    if (has_lora) tma_prefetch_desc(&tmW);
  }
  if (threadIdx.x < 8) lora_unfit[threadIdx.x] = 0u;
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  qmath::fill_scale_lut(scale_lut, threadIdx.x, NUM_THREADS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_acc = *tmem_slot;
  // set-up done; what follows reads and writes global memory
  pdl_trigger();
  pdl_wait();
  const bool use_fdiv = has_table && reinterpret_cast<const uint32_t*>(p.table + p.K)[0] != 0u;

  bool aux_ok = true;
  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    const uint32_t stage_bytes = C::X_BYTES + (has_lora ? W_BYTES : 0) + (has_table ? TB_BYTES : 0);
    for (int i = 0; i < my_slabs; ++i) {
      const uint32_t s = i % C::STAGES, ph = (i / C::STAGES) & 1;
      if (!uwait(&empty[s], ph ^ 1, kDevWaitEmpty, i)) { aux_ok = false; break; }
      uint8_t* st = smem + s * C::STAGE_BYTES;
      const int k0 = k_begin + i * SLAB_K;
      if (elect_one()) {
        mbar_arrive_expect_tx(&full[s], stage_bytes);
        tma_load_2d(st, &tmX, k0, m0, &full[s]);
        if (has_lora) {
          // two boxes of 64 rank columns; columns past R (and a whole box past R) arrive as zeros
          tma_load_2d(st + C::X_BYTES, &tmW, 0, k0, &full[s]);
          tma_load_2d(st + C::X_BYTES + SLAB_K * 128, &tmW, 64, k0, &full[s]);
        }
        if (has_table) {
#pragma unroll
          for (int gq = 0; gq < 4; ++gq)
            bulk_load_1d(st + C::X_BYTES + W_BYTES + gq * TB_GROUP_STRIDE, p.table + k0 + gq * 16, 128, &full[s]);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // D^T [128 x TM] += A [128 x 16] * B [16 x TM]: A = lora_down slab (rank-major rows of 128 bytes,
    // i.e. M-major, two 64-column boxes 8 KB apart), B = x tile (K-major, 8-row groups 1 KB apart).
    constexpr uint64_t kDescA = smem_desc_base(SLAB_K * 128, 1024, kSwizzle128B);
    constexpr uint64_t kDescB = smem_desc_base(0, 1024, kSwizzle128B);
    constexpr uint32_t kIdesc = idesc_f16(kBf16, kBf16, RP, TM, true, false);
    for (int i = 0; i < my_slabs; ++i) {
      const uint32_t s = i % C::STAGES, ph = (i / C::STAGES) & 1;
      if (!uwait(&full[s], ph, kDevWaitFull, i)) { aux_ok = false; break; }
      tc_fence_after_sync();
      const uint32_t x_addr = smem_u32(smem + s * C::STAGE_BYTES);
      const uint32_t w_addr = x_addr + C::X_BYTES;
      if (elect_one()) {
        if (has_lora) {
#pragma unroll
          for (int j = 0; j < SLAB_K / 16; ++j)
            mma_f16<1>(tmem_acc, smem_desc(kDescA, w_addr + j * 2048), smem_desc(kDescB, x_addr + j * 32), kIdesc,
                       (i | j) != 0 ? 1u : 0u);
          tc_commit(&empty[s]);
          if (i == my_slabs - 1) tc_commit(acc_done);
        } else {
          mbar_arrive(&empty[s]);
        }
      }
      __syncwarp();
    }
  } else if (warp >= AUX_WARPS) {
    // ------------------------------ quantize warps ------------------------------
    // Group grp takes slabs grp, grp + QUANT_GROUPS, ...; its warp wq owns rows 16 wq .. 16 wq + 15 of the
    // tile.  Lane l works on 16-column group l % 4 of rows l / 4 and l / 4 + 8 of those, so the four
    // lanes of a quad hold one row's whole 64-column stretch of the slab: their 8-byte code stores
    // fill one 32-byte sector, and their scale bytes are adjacent in the atom layout.
    const int qw = warp - AUX_WARPS;
    const int grp = qw / C::GROUP_WARPS;
    const int wq = qw % C::GROUP_WARPS;
    const int g = lane & 3;
    const int row_base = 16 * wq + (lane >> 2);
    const int groups = p.K >> 4;
    uint8_t* const act_base = p.act + static_cast<size_t>(m0) * (p.K >> 1);
    for (int i = grp; i < my_slabs; i += C::QUANT_GROUPS) {
      const uint32_t s = i % C::STAGES, ph = (i / C::STAGES) & 1;
      if (!mbar_wait(&full[s], ph, ctx, kDevWaitFull, 0x10000 + i)) break;
      const uint8_t* st = smem + s * C::STAGE_BYTES;
      uint4 raw[2][2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const uint32_t row = row_base + 8 * rr;
        const uint8_t* xrow = st + row * 128;
        raw[rr][0] = *reinterpret_cast<const uint4*>(xrow + (((2 * g) ^ (row & 7)) << 4));
        raw[rr][1] = *reinterpret_cast<const uint4*>(xrow + (((2 * g + 1) ^ (row & 7)) << 4));
      }
      float2 f[2][8];
      if (has_table && !use_fdiv) {
        qmath::unpack_group<T, false>(raw[0][0], raw[0][1], f[0]);
        qmath::unpack_group<T, false>(raw[1][0], raw[1][1], f[1]);
      } else {
        qmath::unpack_group<T, true>(raw[0][0], raw[0][1], f[0]);
        qmath::unpack_group<T, true>(raw[1][0], raw[1][1], f[1]);
      }
      if (has_table) {
        const float4* tb = reinterpret_cast<const float4*>(st + C::X_BYTES + W_BYTES + g * TB_GROUP_STRIDE);
        qmath::smooth_divide(f[0], tb, use_fdiv);
        qmath::smooth_divide(f[1], tb, use_fdiv);
      }
      // Hand the stage back: the ring was read through the generic proxy and will be overwritten through
      // the async proxy (TMA); an mbarrier arrival does not wait for earlier shared-memory loads.
      __threadfence_block();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);

      const int k0 = k_begin + i * SLAB_K + g * 16;
      const int gi = k0 >> 4;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int row = row_base + 8 * rr;
        // one group after the other, each stored as soon as it is done: running both groups' scale chains
        // side by side and keeping their results in registers until the end measured 5-8 % slower
        uint32_t c_lo, c_hi, s_b;
        qmath::quantize_group(f[rr], scale_lut, c_lo, c_hi, s_b);
        *reinterpret_cast<uint2*>(act_base + static_cast<size_t>(row) * (p.K >> 1) + (k0 >> 1)) = make_uint2(c_lo, c_hi);
        p.scales[static_cast<size_t>(gi) * p.M_pad + m0 + row] = static_cast<uint8_t>(s_b);
        if (p.scales_swz != nullptr) p.scales_swz[sf_swizzled_offset(m0 + row, gi, groups)] = static_cast<uint8_t>(s_b);
      }
    }
  }

  // ------------------------------ LoRA epilogue (warps 0-3) ------------------------------
  // The accumulator holds lora_act^T: lane = rank index r, column = row of the tile.  Warp w may read
  // lanes 32 w .. 32 w + 31.
  if (has_lora && warp < AUX_WARPS) {
    const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_done, 0, ctx, kDevWaitAcc, 0)) != 0 && aux_ok;
    tc_fence_after_sync();
    const int r = warp * 32 + lane;
    const size_t plane = static_cast<size_t>(p.M_pad) * p.R;
    float* part = p.partials + (static_cast<size_t>(tile) * ks + krank) * (TM * RP);
#pragma unroll 1
    for (int c0 = 0; c0 < TM; c0 += 32) {
      uint32_t v[32];
      tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
      tmem_ld_wait();
      if (ks > 1) {
        // partial [row][r]: a warp writes 32 consecutive floats of one row per instruction
        // (warps whose 32 rank indices all lie past R have nothing to contribute)
        if (warp * 32 < p.R) {
#pragma unroll
          for (int j = 0; j < 32; ++j) __stcg(part + (c0 + j) * RP + r, __uint_as_float(v[j]));
        }
      } else if (ok && r < p.R) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float val = __uint_as_float(v[j]);
          const size_t idx = static_cast<size_t>(m0 + c0 + j) * p.R + r;
          p.lora[idx] = val;
          if (p.lora16 != nullptr) {
            store_lora16<T>(p.lora16, idx, plane, val);
            if (kBf16 && !(fabsf(val) <= 65504.0f)) atomicOr(&lora_unfit[(c0 + j) >> 5], 1u);
          }
        }
      }
    }
    if (ks > 1) {
      const int tid = threadIdx.x;                 // 0 .. 127
      unsigned int* arrive = p.tickets + tile;
      unsigned int* done = p.tickets + 256 + tile;
      __threadfence();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      bool all_here = true;
      if (tid == 0) {
        if (ok) atomicAdd(arrive, 1u);
        all_here = wait_counter(arrive, static_cast<unsigned int>(ks), ctx, 0x30000 + tile);
        if (!all_here) *abort_flag = 1;
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      all_here = *abort_flag == 0;
      if (all_here) {
        __threadfence();
        // rows [krank TM/KS, (krank+1) TM/KS) of the KS partials, added in rank order
        const float4* first = reinterpret_cast<const float4*>(p.partials + static_cast<size_t>(tile) * ks * (TM * RP));
        uint32_t unfit = 0u;
        if (ks == 2) unfit = add_partials<T, TM, 2>(p, first, m0, krank, tid, plane);
        else if (ks == 4) unfit = add_partials<T, TM, 4>(p, first, m0, krank, tid, plane);
        else unfit = add_partials<T, TM, 8>(p, first, m0, krank, tid, plane);
        if (kBf16 && unfit != 0u) {
#pragma unroll
          for (int b = 0; b < 8; ++b)
            if (unfit & (1u << b)) atomicOr(&lora_unfit[b], 1u);
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (tid == 0) {
          // the last CTA of the tile to finish reading puts both counters back to zero
          if (atomicAdd(done, 1u) == static_cast<unsigned int>(ks - 1)) { *arrive = 0u; *done = 0u; }
        }
      }
    } else {
      asm volatile("bar.sync 2, 128;" ::: "memory");
    }
    if (kBf16 && p.lora16 != nullptr) {
      // one word per 32 rows; this CTA wrote rows [row_lo, row_lo + TM / KS) of the tile
      uint32_t* flags = lora16_flags(p.lora16, plane);
      const int rows_per = TM / ks, row_lo = krank * rows_per;
      if (threadIdx.x < rows_per / 32) flags[(m0 + row_lo) / 32 + threadIdx.x] = lora_unfit[row_lo / 32 + threadIdx.x];
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

}  // namespace qs

// Tile height and K split of the streaming form for this problem; false if it does not apply
// (then the cluster form of quantize_fused.cu, or the generic kernels, take the call).
bool quantize_stream_plan(int M, int K, int R, int M_pad, int* tm_out, int* ks_out) {
  if (M <= 0 || K <= 0 || M_pad < M || K % qs::SLAB_K != 0) return false;
  if (R < 0 || R > qs::RP || R % 8 != 0) return false;
  const int sms = sm_count();
  const int slabs = K / qs::SLAB_K;
  int best_tm = 0, best_ks = 0;
  double best_cost = 1e30;
  for (int tm : {256, 128}) {
    if (M_pad % tm != 0) continue;
    const int tiles = M_pad / tm;
    for (int ks : {1, 2, 4, 8}) {
      if (ks > slabs || tm / ks < 32) continue;
      if (ks > 1 && (tiles * ks > sms || tiles > 256)) continue;
      const int waves = (tiles * ks + sms - 1) / sms;
      // time in slab-rows: a CTA streams ceil(slabs / ks) slabs of tm rows per wave; the exchange of the
      // partial sums costs about as much as streaming tm x 1.5 rows of one slab per rank met
      const double cost = static_cast<double>(waves) * ((slabs + ks - 1) / ks) * tm + (ks > 1 ? 1.5 * tm : 0.0);
      if (cost < best_cost) { best_cost = cost; best_tm = tm; best_ks = ks; }
    }
  }
  if (best_tm == 0) return false;
  *tm_out = best_tm; *ks_out = best_ks;
  return true;
}

size_t quantize_stream_workspace_bytes(int M, int K, int R, int M_pad) {
  int tm, ks;
  if (R <= 0 || !quantize_stream_plan(M, K, R, M_pad, &tm, &ks) || ks == 1) return 0;
  return qs::kTicketBytes + static_cast<size_t>(ks) * M_pad * qs::RP * 4;
}

template <typename T, int TM>
static int launch_qs(const void* x, const void* w, const qs::Params& p, cudaStream_t stream) {
  using C = qs::Cfg<TM>;
  CUtensorMap tmX, tmW;
  int rc;
  if ((rc = make_tmap_2d(&tmX, x, 2, p.M, p.K, static_cast<uint64_t>(p.K) * 2, TM, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
  if (p.R > 0) {
    if ((rc = make_tmap_2d(&tmW, w, 2, p.K, p.R, static_cast<uint64_t>(p.R) * 2, qs::SLAB_K, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
  } else {
    tmW = tmX;
  }
  auto kern = qs::quantize_stream_kernel<T, TM>;
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SVDQ_ERR_CUDA;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) return SVDQ_ERR_LAUNCH;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.M_pad / TM, p.ks, 1);
  cfg.blockDim = dim3(qs::NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, tmX, tmW, p) != cudaSuccess) return SVDQ_ERR_LAUNCH;
  return SVDQ_OK;
}

// tm / ks: 0 = planned; otherwise forced (tests and tuning), checked against the same limits
int launch_quantize_stream(const void* x, const void* lora_down, const void* smooth_table, void* act, void* ascales,
                           float* lora_act, void* ascales_swz, void* lora_act16, int M, int K, int R, int M_pad,
                           int dtype, void* ws, size_t ws_bytes, int tm, int ks, cudaStream_t stream) {
  int ptm = 0, pks = 0;
  if (!quantize_stream_plan(M, K, R, M_pad, &ptm, &pks)) return SVDQ_ERR_UNSUPPORTED;
  // tuning overrides (tile height 128 / 256, K split 1 / 2 / 4 / 8), checked like forced arguments
  if (tm == 0 && ks == 0) {
    if (const char* e = getenv("SVDQ_QUANT_TILE")) tm = atoi(e);
    if (const char* e = getenv("SVDQ_QUANT_KSPLIT")) ks = atoi(e);
  }
  if (tm == 0) tm = ptm;
  if (ks == 0) ks = (tm == ptm) ? pks : 1;
  if ((tm != 128 && tm != 256) || M_pad % tm != 0) return SVDQ_ERR_UNSUPPORTED;
  if ((ks != 1 && ks != 2 && ks != 4 && ks != 8) || ks > K / qs::SLAB_K || tm / ks < 32) return SVDQ_ERR_UNSUPPORTED;
  const int tiles = M_pad / tm;
  if (ks > 1 && (tiles * ks > sm_count() || tiles > 256)) return SVDQ_ERR_UNSUPPORTED;
  if (ks > 1 && R > 0) {
    if (ws == nullptr || ws_bytes < qs::kTicketBytes + static_cast<size_t>(ks) * M_pad * qs::RP * 4) return SVDQ_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(ws) % 16 != 0) return SVDQ_ERR_ALIGN;
  }
  if (reinterpret_cast<uintptr_t>(smooth_table) % 16 != 0) return SVDQ_ERR_ALIGN;
  qs::Params p;
  p.table = static_cast<const float2*>(smooth_table);
  p.act = static_cast<uint8_t*>(act);
  p.scales = static_cast<uint8_t*>(ascales);
  p.scales_swz = static_cast<uint8_t*>(ascales_swz);
  p.lora = lora_act;
  p.lora16 = lora_act16;
  p.tickets = static_cast<unsigned int*>(ws);
  p.partials = ws != nullptr ? reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + qs::kTicketBytes) : nullptr;
  p.M = M; p.K = K; p.R = R; p.M_pad = M_pad; p.ks = ks;
  if (dtype == SVDQ_DTYPE_F16)
    return tm == 256 ? launch_qs<__half, 256>(x, lora_down, p, stream) : launch_qs<__half, 128>(x, lora_down, p, stream);
  if (dtype == SVDQ_DTYPE_BF16)
    return tm == 256 ? launch_qs<__nv_bfloat16, 256>(x, lora_down, p, stream) : launch_qs<__nv_bfloat16, 128>(x, lora_down, p, stream);
  return SVDQ_ERR_DTYPE;
}

}  // namespace svdq
