// Fused activation quantizer + LoRA-down for sm_100a: one pass over x.
//
//   act, ascales = nvfp4( x / smooth )        bit-exact with the reference oracle
//   lora_act     = x @ lora_down              fp32, tcgen05 dense 16-bit MMA
//
// Replaces the reference's Triton kernel
// (triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:115-286); results
// follow baseline/kernels/quantize_w4a4_act_fuse_lora/ref.py:19-50.
//
// Decomposition.  A cluster of KS (1, 2, 4 or 8) CTAs owns one tile of 64 rows; CTA k
// owns a contiguous range of 64-column slabs of K.  Per slab one producer warp
// TMA-loads the x tile (64 x 64, 128-byte swizzle) with the slab's 64 entries of
// the smoothing table (four 128-byte bulk copies) into a stage of the x ring, a
// second one the matching lora_down slab (64 x R) into a ring of its own.
// Two kinds of consumers read an x stage: two MMA-issuing warps (even and odd
// slabs) accumulate x_tile @ lora_down_slab into [64 x R] fp32 accumulators in
// tensor memory, one each, and sixteen quantize warps turn the tile into codes
// and scales.  x is read from HBM exactly once.  With KS > 1 the partial
// accumulators are summed in a fixed order (two ranks: through the copy engine
// into the partner's shared memory; more: through distributed shared memory
// loads): no atomics, no zero-fill, no scratch in global
// memory.  Large inputs run with KS = 2; clusters of 4 and 8 are for inputs of
// a few hundred rows, where pairs would leave most SMs idle (256 x 10240:
// 36.0 -> 12.9 us), and are taken only if all of them are resident at once.  (64-row tiles with pairs, not 128-row tiles with quads: a B200 keeps
// at most 33 four-CTA clusters of this size resident, one short of the 34 row
// tiles of a 4352-row activation, while 68 pairs fit in one wave.  128-row tiles
// whose K ranks meet through global memory were measured too: what they save in
// lora_down traffic and MMA count, the 9 MB of partial sums that all CTAs write
// at the same moment costs again.)
//
// Lane mapping.  The four lanes of a quad hold one row's four 16-column groups
// of the slab, so their 8-byte code stores fill one 32-byte sector and their
// scale bytes are adjacent in the atom layout; with a lane per row and a warp
// per group the same stores touched 32 sectors each and cost 4 us more.
//
// Codes.  The scale byte is J * 2^E (J = 1..15), so floor(4 |v| / 2^E) is an
// integer m and the E2M1 code is the number of n in {1,3,5,7,10,14,20} with
// n J <= m.  m / (4 J) times (1 + 2^-20) is never on the wrong side of a
// rounding bound of E2M1, so the hardware float -> E2M1 conversion of it
// (cvt.rn.satfinite.e2m1x2.f32) yields exactly that count, with the sign, two
// codes per instruction; see quantize_group.
//
// Exact arithmetic.  x / smooth must equal the IEEE quotient.  It is computed
// as fma(x, r_hi, RN(x * r_lo)) with r_hi + r_lo = 1/s to 2^-47 from the table
// (quantize_math.cuh); for operands with at most 11 significant bits this is the
// correctly rounded quotient (checked exhaustively over mantissas), provided
// nothing over- or underflows: the table builder raises a flag when a smooth
// value lies outside [2^-60, 2^60] (2^16 for bf16) and the kernel then divides
// with __fdiv_rn.  amax / 6 uses a three-step form q0 = a*r, q = fma(fma(-6, q0, a), r, q0)
// (checked exhaustively as well).
#include "nvfp4_math.cuh"
#include "quantize_math.cuh"
#include "sm100.cuh"
#include "svdq_internal.h"

#include <type_traits>

namespace svdq {
namespace qf {

constexpr int TILE_M = 64;
constexpr int SLAB_K = 64;                 // columns per ring stage (128 bytes of 16-bit x)
constexpr int X_BYTES = TILE_M * 128;      // 8 KB
#ifndef SVDQ_QUANT_GROUPS
#define SVDQ_QUANT_GROUPS 4
#endif
constexpr int QUANT_GROUPS = SVDQ_QUANT_GROUPS;   // groups of 4 warps take slabs round-robin
constexpr int QUANT_WARPS = 4 * QUANT_GROUPS;
#ifndef SVDQ_DIRECT_EXCHANGE
#define SVDQ_DIRECT_EXCHANGE 1
#endif
constexpr bool kDirectExchange = SVDQ_DIRECT_EXCHANGE != 0;
constexpr int AUX_WARPS = 4;                // x producer, MMA issuer (even slabs), lora_down producer, MMA issuer (odd slabs); with two K ranks they exchange the LoRA sums
constexpr int NUM_THREADS = (AUX_WARPS + QUANT_WARPS) * 32;
constexpr int TB_BYTES = SLAB_K * 8;       // {smooth, 1/smooth} of a slab's columns
constexpr int TB_GROUP_STRIDE = 144;       // spacing of the four 128-byte group pieces in a stage


template <int RP>
struct Cfg {
  // Two rings.  An x stage holds a 64 x 64 tile of x (8 KB) and the slab's 64 table entries; it is read by
  // the MMA and by one quantize group and released by both.  A lora_down slab (64 x RP, 16 KB at rank
  // 128) would make that stage three times as large and the ring a third as deep, and the stage would stay
  // held for the slab's four MMAs; in a ring of its own, which only the MMA reads, a few stages are enough
  // (the slabs come out of L2) and the x ring gets the rest of the shared memory.
  static constexpr int X_STAGE_BYTES = X_BYTES + 1024;            // tile + table slab, padded to the 1 KB swizzled tiles need
  static constexpr int W_BYTES = SLAB_K * RP * 2;                 // lora_down slab
  static constexpr int W_STAGES = RP > 128 ? 3 : 4;
  static constexpr int W_RING_BYTES = W_STAGES * W_BYTES;
  static constexpr int RECV_BYTES = (TILE_M / 2) * RP * 4;        // two K ranks: the peer's partial sums of this CTA's 32 rows
  static constexpr int STAGES_RAW = (232448 - 1024 - 512 - 1024 - RECV_BYTES - W_RING_BYTES) / X_STAGE_BYTES;
  // A multiple of the group count: a group then always meets the same stages, and the slab it waits
  // for is the direct successor (in that stage) of one it consumed itself.  A one-bit phase parity
  // cannot tell "one revolution behind" from "one ahead"; this rule makes the second impossible.
  static constexpr int STAGES = ((STAGES_RAW > 16 ? 16 : STAGES_RAW) / QUANT_GROUPS) * QUANT_GROUPS;
  static constexpr int RING_BYTES = STAGES * X_STAGE_BYTES;
  static constexpr int BARS_OFF = RING_BYTES + W_RING_BYTES;
  static constexpr int SMEM_BYTES = 1024 + BARS_OFF + 512 + 1024 + RECV_BYTES;   // rings, barriers, scale-constant table, receive buffer
  // Two accumulators: slabs alternate between two issuing warps (see the MMA issuers), each with its own.
  static constexpr int TMEM_COLS = 2 * (RP < 32 ? 32 : RP);       // power of two >= 64
  static constexpr int EPI_COLS = RP / 4 < 32 ? 32 : RP / 4;      // accumulator columns per epilogue warp
  static_assert(TILE_M * RP * 4 <= RING_BYTES, "partial accumulator must fit in the x ring");
  static_assert(STAGES >= QUANT_GROUPS && STAGES % QUANT_GROUPS == 0, "ring depth");
  static_assert((2 * STAGES + 2 * W_STAGES + 3) * 8 + 64 <= 512, "barrier block");
  static_assert(2 * RECV_BYTES <= W_RING_BYTES, "the exchange stages both halves of the accumulator in the lora_down ring");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct Params {
  const float2* table;    // [K/2] entries of qmath::smooth_table_entry followed by one flag word, or null (no smoothing)
  uint8_t* act;           // [M_pad, K/2]
  uint8_t* scales;        // [K/16, M_pad]
  uint8_t* scales_swz;    // atom order or null
  float* lora;            // [M_pad, R]
  void* lora16;           // 16-bit form of lora (fp16 [M_pad, R] or bf16 [2, M_pad, R]) or null
  int M, K, R, M_pad;
};

// float4 slot of (row, c4) in the partial-accumulator buffer; the XOR spreads the
// rows a warp writes at once over all bank groups.
__device__ __forceinline__ uint32_t partial_slot(uint32_t row, uint32_t c4, uint32_t rp4) {
  return row * rp4 + (c4 ^ (row & 7u));
}

using qmath::quantize_group;
using qmath::smooth_divide;
using qmath::unpack_group;

template <typename T, int RP>
__global__ void __launch_bounds__(NUM_THREADS, 1)
quantize_fused_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const Params p) {
  using C = Cfg<RP>;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;

  extern __shared__ uint8_t smem_raw[];
  // 1 KB alignment by pointer arithmetic (not an integer round trip) so that the compiler keeps
  // the shared address space and emits shared-memory loads and stores
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* wring = smem + C::RING_BYTES;       // lora_down slabs
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BARS_OFF);
  uint64_t* full = bars;                       // [STAGES]    x stage filled
  uint64_t* empty = bars + C::STAGES;          // [STAGES]    x stage consumed (MMA + one quantize group)
  uint64_t* wfull = bars + 2 * C::STAGES;      // [W_STAGES]  lora_down slab landed
  uint64_t* wempty = wfull + C::W_STAGES;      // [W_STAGES]  lora_down slab consumed (MMA)
  uint64_t* acc_done = wempty + C::W_STAGES;   // MMA -> epilogue
  uint64_t* recv_bar = acc_done + 1;           // two K ranks: the peer's partial sums have landed in `recv`
  uint64_t* ack_bar = recv_bar + 1;            // two K ranks: the peer has received what this CTA sent
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ack_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* lora_unfit = tmem_slot + 2;        // bf16 form: some LoRA value this CTA wrote does not fit fp16
  float2* scale_lut = reinterpret_cast<float2*>(smem + C::BARS_OFF + 512);   // per scale byte: {2^(2-E), ~1/(4J)}
  float4* recv = reinterpret_cast<float4*>(smem + C::BARS_OFF + 512 + 1024);  // [32 rows][RP / 4], slots as partial_slot
  const WaitCtx ctx{abort_flag};

  // warp index through a shuffle: provably warp-uniform, so the role branches are convergent code
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  auto uwait = [&](uint64_t* bar, uint32_t parity, unsigned int code, unsigned int tag) -> bool {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, code, tag)) != 0;
  };
  const uint32_t ks = gridDim.y;               // cluster = (1, KS, 1): blockIdx.y is the rank along K
  const uint32_t krank = blockIdx.y;
  const int m0 = blockIdx.x * TILE_M;
  const bool has_lora = p.R > 0;
  const bool has_table = p.table != nullptr;

  // slabs owned by this CTA
  const int n_slabs = p.K / SLAB_K;
  const int base = n_slabs / static_cast<int>(ks), rem = n_slabs % static_cast<int>(ks);
  const int slab_begin = static_cast<int>(krank) * base + (static_cast<int>(krank) < rem ? static_cast<int>(krank) : rem);
  const int my_slabs = base + (static_cast<int>(krank) < rem ? 1 : 0);
  const int k_begin = slab_begin * SLAB_K;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *lora_unfit = 0u;
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1 + QUANT_WARPS / QUANT_GROUPS); }
    for (int s = 0; s < C::W_STAGES; ++s) { mbar_init(&wfull[s], 1); mbar_init(&wempty[s], 1); }
    mbar_init(acc_done, my_slabs > 1 ? 2 : 1);     // one arrival per MMA issuer that has slabs
    mbar_init(recv_bar, 1);                    // armed below with the bytes of the peer's two copies
    mbar_init(ack_bar, 1);
    if (kDirectExchange && ks == 2 && has_lora) mbar_arrive_expect_tx(recv_bar, C::RECV_BYTES);
    fence_barrier_init();
    tma_prefetch_desc(&tmX);
    if (has_lora) tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  qmath::fill_scale_lut(scale_lut, threadIdx.x, NUM_THREADS);
  tc_fence_before_sync();
  __syncthreads();
  // Two K ranks hand their partial sums to each other through the copy engine, counted on the partner's
  // barrier, so that barrier must exist (and be armed) before either touches it.  (The CTAs of a cluster
  // start together; this costs a fraction of a microsecond, before the wait for the kernel ahead.)
  if (kDirectExchange && ks == 2 && has_lora) cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_acc = *tmem_slot;
  // set-up done; what follows reads and writes global memory
  pdl_trigger();
  pdl_wait();
  // out-of-range smooth anywhere in K (flag word behind the table) selects the IEEE divide
  const bool use_fdiv = has_table && reinterpret_cast<const uint32_t*>(p.table + p.K)[0] != 0u;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    const uint32_t stage_bytes = X_BYTES + (has_table ? TB_BYTES : 0);
    for (int i = 0; i < my_slabs; ++i) {
      const uint32_t s = i % C::STAGES, ph = (i / C::STAGES) & 1;
      if (!uwait(&empty[s], ph ^ 1, kDevWaitEmpty, i)) break;
      uint8_t* st = smem + s * C::X_STAGE_BYTES;
      const int k0 = k_begin + i * SLAB_K;
      if (elect_one()) {
        mbar_arrive_expect_tx(&full[s], stage_bytes);
        tma_load_2d(st, &tmX, k0, m0, &full[s]);
        if (has_table) {
          // one 128-byte piece per 16-column group, 144 bytes apart: the four groups a quad of lanes
          // reads at once then sit in different banks
#pragma unroll
          for (int gq = 0; gq < 4; ++gq)
            bulk_load_1d(st + X_BYTES + gq * TB_GROUP_STRIDE, p.table + k0 + gq * 16, 128, &full[s]);
        }
      }
      __syncwarp();
    }
  } else if (warp == 2) {
    // ------------------------------ lora_down producer ------------------------------
    if (has_lora) {
      for (int i = 0; i < my_slabs; ++i) {
        const uint32_t s = i % C::W_STAGES, ph = (i / C::W_STAGES) & 1;
        if (!uwait(&wempty[s], ph ^ 1, kDevWaitEmpty, 0x50000 + i)) break;
        uint8_t* st = wring + s * C::W_BYTES;
        const int k0 = k_begin + i * SLAB_K;
        if (elect_one()) {
          mbar_arrive_expect_tx(&wfull[s], C::W_BYTES);
#pragma unroll
          for (int b = 0; b < RP / 64; ++b) tma_load_2d(st + b * (SLAB_K * 128), &tmW, b * 64, k0, &wfull[s]);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------ MMA issuers ------------------------------
    // Two warps, even and odd slabs, each into an accumulator of its own (added up in the epilogue, always in
    // the same order).  One thread's loop - two barrier waits, four MMAs, three commits - takes about 0.3 us
    // per slab whatever the tensor pipe has to do (it is busy a quarter of the time), which made a single
    // issuer the slowest agent of the kernel: the x ring ran full behind it and the epilogue started late.
    constexpr uint64_t kDescA = smem_desc_base(0, 1024, kSwizzle128B);               // x tile, K-major
    constexpr uint64_t kDescB = smem_desc_base(SLAB_K * 128, 1024, kSwizzle128B);    // lora_down slab, R-major (its own ring)
    constexpr uint32_t kIdesc = idesc_f16(kBf16, kBf16, TILE_M, RP, false, true);
    const int issuer = warp >> 1;                                  // 0 or 1
    const uint32_t acc = tmem_acc + issuer * RP;
    const int last = ((my_slabs - 1 - issuer) & ~1) + issuer;      // this issuer's last slab (negative: none)
    bool ok = true;
    for (int i = issuer; i < my_slabs && ok; i += 2) {
      const uint32_t s = i % C::STAGES, ph = (i / C::STAGES) & 1;
      if (!uwait(&full[s], ph, kDevWaitFull, i)) { ok = false; break; }
      const uint32_t sw = i % C::W_STAGES;
      if (has_lora && !uwait(&wfull[sw], (i / C::W_STAGES) & 1, kDevWaitFull, 0x50000 + i)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t a_addr = smem_u32(smem + s * C::X_STAGE_BYTES);
      const uint32_t b_addr = smem_u32(wring + sw * C::W_BYTES);
      if (elect_one()) {
        if (has_lora) {
#pragma unroll
          for (int j = 0; j < SLAB_K / 16; ++j)
            mma_f16<1>(acc, smem_desc(kDescA, a_addr + j * 32), smem_desc(kDescB, b_addr + j * 2048), kIdesc,
                       (i != issuer || j != 0) ? 1u : 0u);
        }
        if (has_lora) { tc_commit(&empty[s]); tc_commit(&wempty[sw]); if (i == last) tc_commit(acc_done); }
        else mbar_arrive(&empty[s]);
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
    const int grp = qw >> 2;
    const int wq = qw & 3;
    const int g = lane & 3;                   // 16-column group inside the slab
    const int row_base = 16 * wq + (lane >> 2);
    const int groups = p.K >> 4;
    uint8_t* const act_base = p.act + static_cast<size_t>(m0) * (p.K >> 1);
    for (int i = grp; i < my_slabs; i += QUANT_GROUPS) {
      const uint32_t s = i % C::STAGES, ph = (i / C::STAGES) & 1;
      if (!mbar_wait(&full[s], ph, ctx, kDevWaitFull, 0x10000 + i)) break;
      const uint8_t* st = smem + s * C::X_STAGE_BYTES;
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
        unpack_group<T, false>(raw[0][0], raw[0][1], f[0]);
        unpack_group<T, false>(raw[1][0], raw[1][1], f[1]);
      } else {
        unpack_group<T, true>(raw[0][0], raw[0][1], f[0]);
        unpack_group<T, true>(raw[1][0], raw[1][1], f[1]);
      }
      if (has_table) {
        // {smooth, 1/smooth} of this lane's 16 columns landed with the slab
        const float4* tb = reinterpret_cast<const float4*>(st + X_BYTES + g * TB_GROUP_STRIDE);
        qmath::smooth_divide2(f[0], f[1], tb, use_fdiv);
      }
      // Hand the stage back.  The ring was read through the generic proxy and will be overwritten
      // through the async proxy (TMA); mbarrier arrivals are performed by a separate unit and do not
      // wait for earlier shared-memory loads, so without these fences the refill can overtake the reads.
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
    // every quantize warp is done reading the ring before it is reused below
    asm volatile("bar.sync 2, %0;" ::"n"(QUANT_WARPS * 32) : "memory");
  }

  // 32 accumulator columns of this warp's lanes: the even slabs' accumulator plus, if there is more than one
  // slab, the odd slabs' (always in this order)
  auto acc_ld = [&](uint32_t taddr, uint32_t (&v)[32]) {
    tmem_ld_32x32(taddr, v);
    if (my_slabs > 1) {
      uint32_t w[32];
      tmem_ld_32x32(taddr + RP, w);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), __uint_as_float(w[j])));
    } else {
      tmem_ld_wait();
    }
  };

  // ------------------------------ LoRA epilogue ------------------------------
  // The 64 accumulator rows live in lanes 0-15 of each 32-lane quarter of tensor memory:
  // row r is lane (r % 16) + 32 * (r / 16).
  if (kDirectExchange && has_lora && ks == 2) {
    // Two K ranks (the form for tall activations): CTA k owns rows [32 k, 32 k + 32) of the tile.  The four
    // auxiliary warps do the whole exchange while the quantize warps are still busy with the last slabs:
    // warp w reads rows 16 w .. 16 w + 15 of the accumulator (lanes 0-15 of its quarter of tensor
    // memory) into the lora_down ring, which is free once the last MMA has retired.  Rows of the partner
    // then go to the partner's receive buffer with one copy-engine transfer per warp, counted on the
    // partner's barrier (remote stores by the 16 lanes took 1.3 us of issue slots that the quantize warps
    // wanted); own rows wait there for the partner's.  Then all four warps add the two partial sums (two
    // terms: the order does not matter) and write the finished rows out, consecutive lanes taking
    // consecutive 16 bytes of a row.
    if (warp < AUX_WARPS) {
      constexpr uint32_t RP4 = RP / 4;
      constexpr uint32_t HALF_BYTES = 16u * RP * 4u;                 // one warp's 16 rows
      const bool ok = __all_sync(0xffffffffu, mbar_wait(acc_done, 0, ctx, kDevWaitAcc, 0)) != 0;
      tc_fence_after_sync();
      const bool mine = static_cast<uint32_t>(warp >> 1) == krank;
      const uint32_t row_local = 16u * (warp & 1) + (lane & 15);     // row within the owner's 32
      const uint32_t taddr = tmem_acc + (static_cast<uint32_t>(warp * 32) << 16);
      float4* send = reinterpret_cast<float4*>(wring);                // [32 rows][RP / 4], slots as partial_slot
      float4* own = reinterpret_cast<float4*>(wring + C::RECV_BYTES);
      float4* dst = mine ? own : send;
#pragma unroll 1
      for (int c0 = 0; c0 < RP; c0 += 32) {
        uint32_t v[32];
        acc_ld(taddr + c0, v);
        if (lane < 16) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            dst[partial_slot(row_local, (c0 >> 2) + j, RP4)] =
                make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
        }
      }
      if (!mine) {
        fence_proxy_async_smem();                                     // the copy engine reads what the lanes wrote
        __syncwarp();
        if (lane == 0 && ok) {
          const uint32_t off = (warp & 1) * HALF_BYTES;
          bulk_copy_smem_to_cluster(map_to_cta(smem_u32(recv) + off, krank ^ 1u), smem_u32(send) + off, HALF_BYTES,
                                    map_to_cta(smem_u32(recv_bar), krank ^ 1u));
        }
      }
      tc_fence_before_sync();
      asm volatile("bar.sync 3, %0;" ::"n"(AUX_WARPS * 32) : "memory");       // own rows are staged
      // Every thread that will read the receive buffer observes the barrier itself: that is what makes
      // the copy engine's writes visible to it.
      const bool got = __all_sync(0xffffffffu, mbar_wait(recv_bar, 0, ctx, kDevWaitMisc, 0x40000)) != 0;
      // both halves are here: the partner may give up the memory they were copied from
      if (warp == 0 && lane == 0 && got) mbar_arrive_cluster(ack_bar, krank ^ 1u);
      if (*abort_flag == 0) {
        const uint32_t r4 = static_cast<uint32_t>(p.R) >> 2;
        const size_t row0 = static_cast<size_t>(m0) + 32u * krank;
        for (uint32_t it = threadIdx.x; it < 32u * r4; it += AUX_WARPS * 32) {
          const uint32_t row = it / r4, c4 = it - row * r4;
          const uint32_t slot = partial_slot(row, c4, RP4);
          const float4 a = own[slot], b = recv[slot];
          const float4 o = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
          const size_t idx = (row0 + row) * p.R + 4u * c4;
          *reinterpret_cast<float4*>(p.lora + idx) = o;
          if (p.lora16 != nullptr) {
            store_lora16x4<T>(p.lora16, idx, static_cast<size_t>(p.M_pad) * p.R, o);
            if (kBf16 && !fits_f16(o)) atomicOr(lora_unfit, 1u);
          }
        }
      }
      if (kBf16 && p.lora16 != nullptr) {
        asm volatile("bar.sync 3, %0;" ::"n"(AUX_WARPS * 32) : "memory");
        if (threadIdx.x == 0) lora16_flags(p.lora16, static_cast<size_t>(p.M_pad) * p.R)[m0 / 32 + krank] = *lora_unfit;
      }
      // the partner has everything this CTA sent: only then may the memory it was copied from go away
      if (warp == 0) (void)__all_sync(0xffffffffu, mbar_wait_cluster(ack_bar, 0, ctx, kDevWaitMisc, 0x41000));
    }
  } else if (has_lora) {
    constexpr uint32_t RP4 = RP / 4;
    float4* partial = reinterpret_cast<float4*>(smem);       // reuses the ring
    if (warp >= AUX_WARPS) {
      const int qw = warp - AUX_WARPS;
      const int quarter = warp & 3;                           // TMEM lanes this warp may read
      const int cpart = qw >> 2;                              // column part
      if (cpart * C::EPI_COLS < RP) {
        const bool ok = mbar_wait(acc_done, 0, ctx, kDevWaitAcc, 0);
        tc_fence_after_sync();
        const uint32_t row = quarter * 16 + (lane & 15);
#pragma unroll 1
        for (int c0 = cpart * C::EPI_COLS; c0 < (cpart + 1) * C::EPI_COLS; c0 += 32) {
          uint32_t v[32];
          acc_ld(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, v);
          if (lane < 16) {
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
                  if (p.lora16 != nullptr) {
                    const float4 o = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                 __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                    store_lora16x4<T>(p.lora16, gm * p.R + c, static_cast<size_t>(p.M_pad) * p.R, o);
                    if (kBf16 && !fits_f16(o)) atomicOr(lora_unfit, 1u);
                  }
                }
              }
            }
          }
        }
      }
    }
    if (ks > 1) {
      tc_fence_before_sync();
      __syncwarp();
      cluster_sync_all();                                     // every CTA's partial is in its shared memory
      // CTA k sums rows [k*64/KS, (k+1)*64/KS) over the cluster, in rank order
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
          if (p.lora16 != nullptr) {
            store_lora16x4<T>(p.lora16, gm * p.R + c, static_cast<size_t>(p.M_pad) * p.R, acc);
            if (kBf16 && !fits_f16(acc)) atomicOr(lora_unfit, 1u);
          }
        }
      }
      cluster_sync_all();                                     // nobody leaves while its memory is being read
      if (kBf16 && p.lora16 != nullptr) {
        // One "does not fit fp16" word per 32 rows, and KS / 2 CTAs wrote rows of the same block: the
        // first of them gathers the others' verdicts (all final since the barrier above) and stores
        // the exact word; nobody leaves before that read is over.
        const uint32_t share = ks / 2;
        if (threadIdx.x == 0 && krank % share == 0) {
          uint32_t unfit = 0u;
          for (uint32_t j = 0; j < share; ++j) unfit |= ld_cluster_u32(map_to_cta(smem_u32(lora_unfit), krank + j));
          lora16_flags(p.lora16, static_cast<size_t>(p.M_pad) * p.R)[m0 / 32 + krank / share] = unfit;
        }
        cluster_sync_all();
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (kBf16 && has_lora && p.lora16 != nullptr && threadIdx.x == 0 && ks == 1) {
    // one word per 32 rows: this CTA wrote rows [m0, m0 + 64) alone
    uint32_t* flags = lora16_flags(p.lora16, static_cast<size_t>(p.M_pad) * p.R);
    const uint32_t unfit = *lora_unfit;
    flags[m0 / 32] = unfit; flags[m0 / 32 + 1] = unfit;
  }
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

// Per column pair one table entry (qmath::smooth_table_entry), then one flag word: 1 if any smooth value
// lies outside [2^-60, 2^60] (2^16 for bf16; negative, zero and NaN count as outside), where the two-step
// divide could over- or underflow or leave a zero with the wrong sign; the entries then hold the smooth
// values themselves and the kernels divide with __fdiv_rn.
template <typename T>
__global__ void smooth_table_kernel(const T* __restrict__ smooth, float2* __restrict__ table, int K) {
  // upper bound: 2^60 for fp16 inputs; 2^16 for bf16 inputs, whose smallest subnormal (2^-133)
  // divided by anything larger would underflow to a signed zero
  constexpr float kMaxSmooth = std::is_same<T, __nv_bfloat16>::value ? 65536.0f : 1.1529215e18f;
  __shared__ int bad;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < K; i += blockDim.x) {
    const float s = to_f32(smooth[i]);
    if (!(s >= 8.6736174e-19f && s <= kMaxSmooth)) bad = 1;      // also: negative, zero or NaN
  }
  __syncthreads();
  const bool exact_divide = bad != 0;
  float4* pairs = reinterpret_cast<float4*>(table);
  for (int i = threadIdx.x; i < K / 2; i += blockDim.x)
    pairs[i] = qmath::smooth_table_entry(to_f32(smooth[2 * i]), to_f32(smooth[2 * i + 1]), exact_divide);
  if (threadIdx.x == 0) *reinterpret_cast<uint2*>(table + K) = make_uint2(exact_divide ? 1u : 0u, 0u);
}

}  // namespace qf

// How many CTAs share one row tile along K (0 = no admissible split).
// Clusters of 4 and 8 serve inputs of a few hundred to a couple of thousand rows, where two CTAs per
// row tile would leave most SMs idle; they are taken only if all of them can be resident at once
// (max4 / max8: clusters of that size the device can hold).  Cost in slabs; the constant is the
// cluster reduction of the LoRA partial sums.
static int pick_k_split(int M_pad, int K, int max4, int max8) {
  const int tiles = M_pad / qf::TILE_M;
  const int slabs = K / qf::SLAB_K;
  const int sms = sm_count();
  int best = 0;
  double best_cost = 1e30;
  for (int ks : {1, 2, 4, 8}) {
    if (ks > slabs) continue;
    const int ctas = tiles * ks;
    if (ks > 2 && (ctas > sms || tiles > (ks == 4 ? max4 : max8))) continue;
    const int waves = (ctas + sms - 1) / sms;
    const double cost = static_cast<double>(waves) * ((slabs + ks - 1) / ks) + (ks == 1 ? 0.0 : ks == 2 ? 2.0 : 1.0 + 0.5 * ks);
    if (cost < best_cost) { best_cost = cost; best = ks; }
  }
  return best;
}

template <typename T, int RP> static int max_clusters_t(int ks);

bool quantize_fused_supported(int M, int K, int R, int M_pad) {
  if (M <= 0 || K <= 0 || M_pad < M) return false;
  if (M_pad % qf::TILE_M != 0 || K % qf::SLAB_K != 0) return false;
  if (R < 0 || R > 256 || R % 8 != 0) return false;
  return pick_k_split(M_pad, K, 0, 0) != 0;
}

int launch_smooth_table(const void* smooth, void* table, int K, int dtype, cudaStream_t stream) {
  if (dtype == SVDQ_DTYPE_F16)
    qf::smooth_table_kernel<__half><<<1, 1024, 0, stream>>>(static_cast<const __half*>(smooth), static_cast<float2*>(table), K);
  else if (dtype == SVDQ_DTYPE_BF16)
    qf::smooth_table_kernel<__nv_bfloat16><<<1, 1024, 0, stream>>>(static_cast<const __nv_bfloat16*>(smooth), static_cast<float2*>(table), K);
  else
    return SVDQ_ERR_DTYPE;
  return cudaGetLastError() == cudaSuccess ? SVDQ_OK : SVDQ_ERR_LAUNCH;
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
  // the attribute is per device: remember which devices of this process have it
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SVDQ_ERR_CUDA;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) return SVDQ_ERR_LAUNCH;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  static int cap4[64], cap8[64];
  static bool capped[64] = {};
  if (dev >= 0 && dev < 64 && !capped[dev]) {
    cap4[dev] = max_clusters_t<T, RP>(4);
    cap8[dev] = max_clusters_t<T, RP>(8);
    capped[dev] = true;
  }
  const bool known = dev >= 0 && dev < 64;
  int ks = pick_k_split(p.M_pad, p.K, known ? cap4[dev] : 0, known ? cap8[dev] : 0);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.M_pad / qf::TILE_M, ks, 1);
  cfg.blockDim = dim3(qf::NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = ks;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
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

int launch_quantize_fused(const void* x, const void* lora_down, const void* smooth_table, void* act, void* ascales,
                          float* lora_act, void* ascales_swz, void* lora_act16, int M, int K, int R, int M_pad,
                          int dtype, cudaStream_t stream) {
  if (!quantize_fused_supported(M, K, R, M_pad)) return SVDQ_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(smooth_table) % 16 != 0) return SVDQ_ERR_ALIGN;   // bulk copies start on 16-byte boundaries
  qf::Params p;
  p.table = static_cast<const float2*>(smooth_table);
  p.act = static_cast<uint8_t*>(act);
  p.scales = static_cast<uint8_t*>(ascales);
  p.scales_swz = static_cast<uint8_t*>(ascales_swz);
  p.lora = lora_act;
  p.lora16 = lora_act16;
  p.M = M; p.K = K; p.R = R; p.M_pad = M_pad;
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
