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
// Work decomposition (384 threads per CTA, one CTA per SM):
//   warps 0-7  epilogue: tensor memory -> registers -> affine -> 16 bit ->
//              swizzled shared memory -> TMA store (a 32-row x BN/2 strip per warp)
//   warp  8    producer: TMA loads into a ring of shared-memory stages
//   warp  9    MMA issuer: tcgen05.mma + commits
//   warps 10-11 scale copiers: tcgen05.cp of the stage's scale atoms into a
//              multi-buffered scale area of tensor memory, a few slabs ahead;
//              each warp takes two of the slab's four k-blocks
// Issuing one tcgen05.cp costs its thread about 30 cycles (measured), and a
// 256-wide slab needs 12 scale copies next to its 4 MMAs, which together with
// the waits is more than the 512 cycles the slab's MMAs run for; so the two
// kinds are issued by different warps and handshake through mbarriers: each
// copier's commit is one of the arrivals the stage's "full" barrier waits for
// (beside the producer's, which carries the operand bytes), so the MMA issuer
// waits once per slab and finds operands in shared memory and scales in tensor
// memory.  All single-lane roles stay converged and elect one lane per
// instruction, so descriptors and addresses live in uniform registers.
//
// CG = 1: a CTA computes a 128 x BN tile.
// CG = 2: two CTAs of a cluster compute a 256 x BN tile with cta_group::2
//         MMAs.  Each CTA loads its own 128 rows of A and its own BN/2 rows of
//         B (nothing is fetched twice), its own activation scales, and the
//         weight scales of all BN columns.  Loads of both CTAs complete on the
//         leader's "full" barrier; the leader issues the MMAs and its commits
//         arrive on the barriers of both CTAs.
//
// A stage holds one 256-element K slab: A 128 x 128 B, B rows x 128 B (both
// 128-byte swizzled, K-major, two E2M1 codes per byte) and their scale atoms.
// The scale atoms are requested first and complete on a barrier of their own,
// which is all the scale copiers wait for: a stage's scales are in tensor
// memory by the time its operand tiles land.
// The LoRA-up product reuses the very same ring: a slab of 64 rank elements of
// lora_act (128 rows x 128 B) and lora_up (B rows x 128 B) has exactly the byte
// footprint of a main slab, so it is ceil(R/64) more ring passes per output
// tile, issued as dense 16-bit MMAs into the same accumulator.  Both operands
// of a dense MMA must have the same 16-bit format (an fp16 x bf16 pair is an
// illegal instruction on this part), so lora_act arrives in the output type:
// fp16 as one rounded copy, bf16 as a hi + lo pair (lora_act = hi + lo to 16
// significant bits) that takes two passes over the same lora_up slab - a single
// bf16 copy would put the LoRA term's 2^-9 rounding error above the 1e-3 bound.
// For bf16 the quantizer also provides lora_act as an fp16 plane with a word per 32
// rows telling whether those rows fit fp16; given an fp16 copy of lora_up, a tile
// whose rows all fit takes a single fp16 pass instead (decided per tile by every
// role from the same words, so all agree on the tile's slab count).
//
// Column-sharded form (n_peers > 0): the launch fills N columns of a wider result
// that every GPU holds in full; each finished strip also leaves the staging buffer
// as one TMA store per peer, into the peers' copies over NVLink (lane stores of 16
// bytes measured the same: the link, not the store path, sets the pace).
//
// Split-K form (SK = true, one CTA per 128 x 128 tile part): for problems with few tiles and a
// long K, S CTAs share a tile's slabs.  Each parks its fp32 partial tile in a caller-owned
// workspace (thread t writes float4 j at [j][t], so every access is a whole line per warp and a
// thread later reads back exactly the places its namesakes wrote), fences, and draws a ticket
// from the tile's counter; the CTA that draws ticket S - 1 adds the S partials in split order -
// the result does not depend on who finished first - runs the epilogue and zeroes the counter.
// No CTA waits for another, so nothing depends on the CTAs of a tile running together.
#include "nvfp4_math.cuh"
#include "quantize_math.cuh"
#include "sm100.cuh"
#include "svdq_internal.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdlib>
#include <type_traits>

namespace svdq {

namespace gemm {

constexpr int BM = 128;          // rows of y per CTA
constexpr int BK = 256;          // K elements per stage (128 bytes of codes per row)
constexpr int A_BYTES = BM * 128;
constexpr int SFA_BYTES = BM * (BK / 16);  // 2048
constexpr int EPI_WARPS = 8;
constexpr int SF_WARPS = 2;       // scale copiers: each takes two of a slab's four k-blocks
constexpr int NUM_THREADS = (EPI_WARPS + 2 + SF_WARPS) * 32;
constexpr int STORE_BUF_BYTES = 32 * 128;  // one 32-row x 64-column strip of y

template <int CG, int BN, bool NEXT = false>
struct Cfg {
  static constexpr int B_ROWS = BN / CG;                           // rows of B this CTA loads
  static constexpr int B_BYTES = B_ROWS * 128;
  static constexpr int SFB_BYTES = BN * (BK / 16);
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int ACC_STAGES = (BN <= 128) ? 2 : 1;
  // One 32-row x 64-column staging strip per epilogue warp.  The accumulator is drained into
  // registers in one burst and released before any staging happens, so a second strip would only
  // take shared memory away from the load ring.
  static constexpr int GROUPS_PER_WARP = BN / 128;                 // 64-column strips each epilogue warp handles per tile
  static constexpr int STORE_BUFS = 1;
  static constexpr int STORE_BYTES = EPI_WARPS * STORE_BUFS * STORE_BUF_BYTES;
  // per-column rows of the current tile: wcscales, bias and, for the next layer's quantisation, -smooth_next and
  // 1 / smooth_next (that fourth kilobyte would cost the plain 256 x 256 form its fifth ring stage)
  static constexpr int AFFINE_BYTES = NEXT ? 4096 : 3072;
  static constexpr int TAIL_BYTES = AFFINE_BYTES + 512 /*barriers*/;
  static constexpr int STAGES_RAW = (232448 - 1024 - STORE_BYTES - TAIL_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SFA_COLS = 16;                 // 4 k-blocks x 4 columns
  static constexpr int SFB_COLS = 4 * (BN / 32);      // 4 k-blocks x BN/32 columns
  static constexpr int SF_COLS = SFA_COLS + SFB_COLS; // one scale buffer
  // Scale buffers in tensor memory.  Copies and MMAs execute in issue order on one pipe, and an MMA
  // may only be issued once its scales have landed, so the copier has to run several slabs ahead of
  // the MMA issuer or every slab pays a copy + wake-up bubble.
  static constexpr int SF_BUFS_FIT = (512 - ACC_STAGES * BN) / SF_COLS;
  static constexpr int SF_BUFS = SF_BUFS_FIT > 6 ? 6 : SF_BUFS_FIT;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STORE_BYTES + TAIL_BYTES;
  static_assert(ACC_STAGES * BN + SF_BUFS * SF_COLS <= TMEM_COLS, "tensor memory budget");
  static_assert(STAGES >= 3, "ring too shallow");
  static_assert((3 * STAGES + 2 * ACC_STAGES + 2 * SF_BUFS) * 8 + 16 <= 512, "barrier block");
};

// Column-sharded form: one tensor map per peer's copy of the result (same geometry as this GPU's).
struct PeerMaps {
  CUtensorMap m[7];
};

struct Params {
  const void* wc;       // [N] or null
  const void* bias;     // [N] or null
  const uint32_t* la_flags;   // bf16 only: per 32 rows of lora_act, non-zero = does not fit fp16; null = always two-pass
  int M, N, K, R;
  int tiles_m, tiles_n; // in units of (CG*128) x BN
  // Column-sharded (tensor-parallel) form: this launch computes columns [col0, col0 + N) of a
  // [M, y_ld] result that every rank holds in full.  The local copy is written through tmY (built over
  // the local full matrix); each finished strip is also stored, by TMA from the same staging buffer,
  // into the same place of every peer's matrix (peer-mapped memory, one tensor map per peer).
  int col0, y_ld, n_peers;
  // Split-K form (SK kernels only): a tile's slabs are shared by `splits` CTAs; each writes its fp32
  // partial tile to ws_partials[(tile * splits + split) * BM * BN], takes a ticket from
  // ws_tickets[tile], and the CTA that draws the last ticket adds the partials in split order, runs
  // the epilogue and puts the ticket counter back to zero.
  int splits;
  int interleave;       // 1: LoRA slabs spread evenly among the main slabs of a tile; 0: after them
  int stride1, stride2; // interleaved: positions between LoRA slabs of a tile with one / two LoRA passes
  float4* ws_partials;
  unsigned int* ws_tickets;
  // Next-layer quantisation (NEXT kernels only): the fp32 result, before its cast, divided by
  // smooth_next [N] and packed as NVFP4 rows: qout [M, N/2], oscales [N/16, M] (+ the tensor-core twin).
  const void* smooth_next;
  uint8_t* qout;
  uint8_t* oscales;
  uint8_t* oscales_swz;
};

__device__ __forceinline__ uint32_t pack2(__half a, __half b) {
  __half2 h = __halves2half2(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack2(__nv_bfloat16 a, __nv_bfloat16 b) {
  __nv_bfloat162 h = __halves2bfloat162(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ uint32_t pack2f(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2f<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2f<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <typename T> __device__ __forceinline__ float as_f32(T v);
template <> __device__ __forceinline__ float as_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float as_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Next layer's quantisation of one 16-column group of one row: the 16 fp32 results (already scaled and
// biased) are divided by smooth_next and packed as NVFP4.  ns4 / r4: the group's four entries of the
// -smooth_next and 1 / smooth_next rows.  Returns {codes 0-7, codes 8-15, scale byte, -}.
// Not inlined on purpose: the epilogue calls it eight times per tile from fully unrolled code (the
// accumulator lives in registers, which only constant indices can address), and eight copies of the
// division, the scale and both code paths made the epilogue too large for the instruction cache (the top
// stall reason was "no instruction", at 17 % issue utilisation).
__device__ __noinline__ uint4 next_group_codes(float2 a0, float2 a1, float2 a2, float2 a3, float2 a4, float2 a5,
                                               float2 a6, float2 a7, const float4* ns4, const float4* r4, int tile_fdiv) {
  const float2 a[8] = {a0, a1, a2, a3, a4, a5, a6, a7};
  float2 q[8];
  // IEEE divide of the uncast fp32 values, as the reference does; + 0 turns a -0 quotient into +0 (the
  // reference gives a zero the sign bit only when the value tests < 0)
  auto divide_ieee = [&]() {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 ns = ns4[j];
      q[2 * j] = make_float2(__fadd_rn(__fdiv_rn(a[2 * j].x, -ns.x), 0.0f), __fadd_rn(__fdiv_rn(a[2 * j].y, -ns.y), 0.0f));
      q[2 * j + 1] = make_float2(__fadd_rn(__fdiv_rn(a[2 * j + 1].x, -ns.z), 0.0f), __fadd_rn(__fdiv_rn(a[2 * j + 1].y, -ns.w), 0.0f));
    }
  };
  if (!tile_fdiv) {
    // the same quotients in three packed instructions per pair (qmath::divide_by_constant2)
    const float2 zero = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 ns = ns4[j], r = r4[j];
      q[2 * j] = __fadd2_rn(qmath::divide_by_constant2(a[2 * j], make_float2(ns.x, ns.y), make_float2(r.x, r.y)), zero);
      q[2 * j + 1] = __fadd2_rn(qmath::divide_by_constant2(a[2 * j + 1], make_float2(ns.z, ns.w), make_float2(r.z, r.w)), zero);
    }
  } else {
    divide_ieee();
  }
  uint32_t sb = qmath::group_scale_byte(q);
  if (!tile_fdiv && (sb == 0u || sb >= 0x7Eu)) {
    // Scale byte 0 or 448: a group of tiny or of huge values, where the three-step quotient may have under-
    // or overflowed on the way.  (With a byte in between, the group's largest quotient lies in [2^-10, 2700):
    // every operand that can reach a rounding bound of a code is far from both ends of the range, and the
    // quotients that matter are exact.)
    divide_ieee();
    sb = qmath::group_scale_byte(q);
  }
  uint32_t lo, hi;
  qmath::quantize_group_with(q, sb, lo, hi);
  return make_uint4(lo, hi, sb, 0u);
}

template <int CG, int BN, typename OutT, bool SK = false, bool NEXT = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_w4a4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmLA, const __grid_constant__ CUtensorMap tmLU,
                 const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmSFA,
                 const __grid_constant__ CUtensorMap tmSFB, const __grid_constant__ CUtensorMap tmLAf,
                 const __grid_constant__ CUtensorMap tmLUf, const __grid_constant__ PeerMaps peers, const Params p) {
  using C = Cfg<CG, BN, NEXT>;
  constexpr bool kBf16 = std::is_same<OutT, __nv_bfloat16>::value;

  extern __shared__ uint8_t smem_raw[];
  // 1 KB alignment by pointer arithmetic (not an integer round trip) so that the compiler keeps
  // the shared address space and emits shared-memory loads and stores
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* store_bufs = smem + C::STAGES * C::STAGE_BYTES;        // 1024-aligned: every stage is a multiple of 1 KB
  uint8_t* tail = store_bufs + C::STORE_BYTES;
  float* affine = reinterpret_cast<float*>(tail);                 // [3 or 4][BN] : wcscales, bias, -smooth_next, 1/smooth_next of the current tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail + C::AFFINE_BYTES);
  uint64_t* full = bars;                                          // [STAGES]     A / B (or LoRA) operands landed and scales copied (leader CTA's copy is used)
  uint64_t* empty = bars + C::STAGES;                             // [STAGES]     stage consumed by the MMAs (per CTA)
  uint64_t* full_sf = bars + 2 * C::STAGES;                       // [STAGES]     the stage's scale atoms landed (leader's copy)
  uint64_t* acc_full = bars + 3 * C::STAGES;                      // [ACC_STAGES] accumulator complete (per CTA)
  uint64_t* acc_empty = acc_full + C::ACC_STAGES;                 // [ACC_STAGES] accumulator drained (leader's copy is used)
  uint64_t* sf_empty = acc_empty + C::ACC_STAGES;                 // [SF_BUFS] scale buffer consumed by the MMAs (leader CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_empty + C::SF_BUFS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile uint32_t* sk_ticket = tmem_slot + 2;                   // split-K: the ticket this CTA drew for its tile
  const WaitCtx ctx{abort_flag};
  // bounded wait whose verdict is the same in all lanes of the calling (converged) warp
  auto uwait = [&](uint64_t* bar, uint32_t parity, const WaitCtx& c, unsigned int code, unsigned int tag) -> bool {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, c, code, tag)) != 0;
  };

  // The warp index is taken through a shuffle so that the compiler can prove it warp-uniform: only
  // then do the role branches below count as convergent code, where descriptors and addresses stay
  // in uniform registers.  Single-lane roles also vote on every wait result for the same reason.
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;      // 0 = leader of the pair
  const int pair = blockIdx.x / CG;
  const int num_pairs = gridDim.x / CG;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    // full[s]: the producer's arrival (with the operand bytes) and one arrival per scale copier, made when the
    // stage's scales are in tensor memory (at once for a LoRA slab): the MMA issuer waits once per slab
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1 + SF_WARPS); mbar_init(&empty[s], 1); mbar_init(&full_sf[s], 1); }
    for (int a = 0; a < C::ACC_STAGES; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], EPI_WARPS * CG); }
    for (int b = 0; b < C::SF_BUFS; ++b) mbar_init(&sf_empty[b], 1);
    fence_barrier_init();
  }
  if (warp == EPI_WARPS && lane == 0) {
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmY);
    tma_prefetch_desc(&tmSFA); tma_prefetch_desc(&tmSFB);
    if (p.R > 0) { tma_prefetch_desc(&tmLA); tma_prefetch_desc(&tmLU); }
    if (p.R > 0 && p.la_flags != nullptr) { tma_prefetch_desc(&tmLAf); tma_prefetch_desc(&tmLUf); }
  }
  if (warp == EPI_WARPS + 1) {
    if constexpr (CG == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
    else { tmem_alloc_pair(tmem_slot, C::TMEM_COLS); tmem_relinquish_pair(); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();   // both CTAs' barriers exist before anything remote touches them
  tc_fence_after_sync();
  // Everything above touched only this CTA's shared and tensor memory, so it may overlap the tail of
  // the kernel before this one in the stream; from here on its outputs are read.
  pdl_trigger();
  pdl_wait();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_sf = tmem_base + C::ACC_STAGES * BN;       // SF_BUFS buffers of [SFA 16 | SFB] columns

  const int kt_main = (p.K + BK - 1) / BK;   // the last slab may hold fewer than four 64-element k-blocks
  const int lora_slabs = (p.R + 63) / 64;
  // bf16 output: lora_act comes as hi and lo bf16 planes (two passes over the same lora_up slab) and
  // as an fp16 plane; a tile whose 32-row blocks all carry a zero "does not fit fp16" word takes
  // the fp16 plane and the fp16 copy of lora_up in a single pass.  Every role of both CTAs
  // evaluates this per tile from the same words, so they agree on the number of slabs.
  auto lora_fp16 = [&](int mb) -> bool {
    if (!kBf16 || p.R == 0 || p.la_flags == nullptr) return false;
    constexpr int kWords = CG * BM / 32;
    const uint32_t w = lane < kWords ? __ldg(p.la_flags + mb * kWords + lane) : 0u;
    return __all_sync(0xffffffffu, w == 0u) != 0;
  };
  auto lora_parts = [&](bool fp16_pass) -> int { return (kBf16 && !fp16_pass) ? 2 : 1; };
  const int total_tiles = p.tiles_m * p.tiles_n;
  const int k_groups4 = p.K / 64;            // scale atoms along K
  // Work items: tiles, or (tile, split) pairs numbered tile-major so that the CTAs sharing a tile run
  // at the same time.  Split i of a tile with n slabs (LoRA slabs included, at the end) takes slabs
  // [i n / S, (i + 1) n / S).
  const int S = SK ? p.splits : 1;
  const int total_work = total_tiles * S;
  auto slab_range = [&](int split, int kt_all, int& lo, int& hi) {
    if (SK) { lo = split * kt_all / S; hi = (split + 1) * kt_all / S; } else { lo = 0; hi = kt_all; }
  };
  // Which slab runs at position pos of a tile's kt_all = kt_main + n_lora slabs.  Slab numbers below
  // kt_main are main slabs, the others LoRA slabs.  End-grouped: position = number.  Interleaved (the
  // reference's schedule, cute_kernels/gemm_w4a4/kernel_v2_fa4.py:299-303): LoRA slab j sits at position
  // (j + 1) * stride - 1 with stride = kt_all / n_lora, the main slabs fill the rest in order.  Every
  // role walks the positions with one of these and the same arguments, so all agree.  No division in
  // the per-slab step: the issuing threads have a few hundred cycles per slab for everything.
  struct SlabWalk {
    int kt_main, n_lora, stride, lora_done, next_lora;
    __device__ __forceinline__ void start(int kt_main_, int kt_all, int interleave, int stride_, int first_pos) {
      kt_main = kt_main_;
      n_lora = interleave ? kt_all - kt_main_ : 0;
      stride = stride_;
      lora_done = 0;
      if (n_lora > 0 && first_pos > 0) { lora_done = first_pos / stride; if (lora_done > n_lora) lora_done = n_lora; }
      next_lora = (lora_done + 1) * stride - 1;
    }
    __device__ __forceinline__ int at(int pos) {
      if (lora_done < n_lora && pos == next_lora) { const int kt = kt_main + lora_done; ++lora_done; next_lora += stride; return kt; }
      return pos - lora_done;
    }
  };
  // stride of a tile with one / two LoRA passes (worked out on the host)
  auto lora_stride = [&](bool fp16_pass) -> int { return (kBf16 && !fp16_pass) ? p.stride2 : p.stride1; };
  if (warp == EPI_WARPS) {
    // ------------------------------ producer (both CTAs) ------------------------------
    uint32_t it = 0;
    bool ok = true;
    for (int w = pair; w < total_work && ok; w += num_pairs) {
      const int tile = SK ? w / S : w, split = SK ? w - tile * S : 0;
      const int mb = tile % p.tiles_m, nb = tile / p.tiles_m;
      const int m0 = (mb * CG + rank) * BM;
      const int n0 = nb * BN;
      const int nrow0 = n0 + rank * C::B_ROWS;
      const bool la_fp16 = lora_fp16(mb);
      const int kt_all = kt_main + lora_parts(la_fp16) * lora_slabs;
      int kt_lo, kt_hi;
      slab_range(split, kt_all, kt_lo, kt_hi);
      SlabWalk walk;
      walk.start(kt_main, kt_all, p.interleave, lora_stride(la_fp16), kt_lo);
      for (int pos = kt_lo; pos < kt_hi; ++pos, ++it) {
        const int kt = walk.at(pos);
        const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1;
        if (!uwait(&empty[s], ph ^ 1, ctx, kDevWaitEmpty, it)) { ok = false; break; }
        uint8_t* st = smem + s * C::STAGE_BYTES;
        // Codes past K are zero-filled by TMA.  The scale atoms of a (128-row block, slab) are four
        // consecutive 512-byte rows of the swizzled scale buffer seen as a [blocks * K/64, 512 B] matrix;
        // a short last slab just fetches (and never uses) the rows that follow.  Every byte of a box
        // counts toward the barrier whether it was in bounds or not.
        // Two barriers per stage: the scale atoms (6 KB, requested first) complete on full_sf, the
        // operand tiles on full.  The scale copiers work off full_sf, so a stage's scales are already in
        // tensor memory when its operands land and the MMAs can start at once.  A LoRA slab has no
        // scales; its full_sf is completed by a plain arrival so that both barriers flip once per slab.
        constexpr uint32_t kSfBytes = SFA_BYTES + C::SFB_BYTES, kAbBytes = A_BYTES + C::B_BYTES;
        // the barriers that count this CTA's bytes: its own for CG = 1, the leader's for a pair
        const uint32_t bar = (CG == 2) ? map_to_cta(smem_u32(&full[s]), 0) : smem_u32(&full[s]);
        const uint32_t bar_sf = (CG == 2) ? map_to_cta(smem_u32(&full_sf[s]), 0) : smem_u32(&full_sf[s]);
        if (elect_one()) {
          if (kt < kt_main) {
            if (rank == 0) mbar_arrive_expect_tx(&full_sf[s], kSfBytes * CG);
            tma_load_2d_bar<CG>(st + A_BYTES + C::B_BYTES, &tmSFA, 0, (mb * CG + rank) * k_groups4 + kt * 4, bar_sf);
#pragma unroll
            for (int h = 0; h < BN / 128; ++h)
              tma_load_2d_bar<CG>(st + A_BYTES + C::B_BYTES + SFA_BYTES + h * 2048, &tmSFB, 0,
                                  (nb * (BN / 128) + h) * k_groups4 + kt * 4, bar_sf);
            if (rank == 0) mbar_arrive_expect_tx(&full[s], kAbBytes * CG);
            tma_load_2d_bar<CG>(st, &tmA, kt * 128, m0, bar);
            tma_load_2d_bar<CG>(st + A_BYTES, &tmB, kt * 128, nrow0, bar);
          } else {
            if (rank == 0) { mbar_arrive(&full_sf[s]); mbar_arrive_expect_tx(&full[s], kAbBytes * CG); }
            const int lt = kt - kt_main;
            const int part = lt / lora_slabs, r0 = (lt % lora_slabs) * 64;
            if (la_fp16) {
              tma_load_2d_bar<CG>(st, &tmLAf, r0, m0, bar);
              tma_load_2d_bar<CG>(st + A_BYTES, &tmLUf, r0, nrow0, bar);
            } else {
              tma_load_2d_bar<CG>(st, &tmLA, r0, part * p.M + m0, bar);    // lora_act parts are stacked along rows
              tma_load_2d_bar<CG>(st + A_BYTES, &tmLU, r0, nrow0, bar);
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == EPI_WARPS + 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (rank == 0) {
      constexpr uint64_t kDescAB = smem_desc_base(0, 1024, kSwizzle128B);   // K-major, 8-row groups 1024 B apart
      constexpr uint32_t kIdescMain = idesc_nvfp4(BM * CG, BN);
      constexpr uint32_t kIdescLora = idesc_f16(kBf16, kBf16, BM * CG, BN, false, false);
      constexpr uint32_t kIdescLoraF16 = idesc_f16(false, false, BM * CG, BN, false, false);
      constexpr uint16_t kMask = (CG == 2) ? 3 : 1;
      uint32_t it = 0, tcount = 0, sf_it = 0;
      bool ok = true;
      for (int w = pair; w < total_work && ok; w += num_pairs, ++tcount) {
        const int tile = SK ? w / S : w, split = SK ? w - tile * S : 0;
        const uint32_t as = tcount % C::ACC_STAGES, aph = (tcount / C::ACC_STAGES) & 1;
        if (!uwait(&acc_empty[as], aph ^ 1, ctx, kDevWaitAccFree, tcount)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + as * BN;
        const bool la_fp16 = lora_fp16(tile % p.tiles_m);
        const int kt_all = kt_main + lora_parts(la_fp16) * lora_slabs;
        const uint32_t idesc_lora = la_fp16 ? kIdescLoraF16 : kIdescLora;
        int kt_lo, kt_hi;
        slab_range(split, kt_all, kt_lo, kt_hi);
        SlabWalk walk;
        walk.start(kt_main, kt_all, p.interleave, lora_stride(la_fp16), kt_lo);
        for (int pos = kt_lo; pos < kt_hi; ++pos, ++it) {
          const int kt = walk.at(pos);
          const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1;
          if (!uwait(&full[s], ph, ctx, kDevWaitFull, it)) { ok = false; break; }
          const bool main_slab = kt < kt_main;
          const uint32_t sb = sf_it % C::SF_BUFS;            // its scales are in tensor memory: the copiers arrived on full[s]
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
          const uint32_t tsfa = tmem_sf + sb * C::SF_COLS, tsfb = tsfa + C::SFA_COLS;
          const int nkb = main_slab ? min(4, k_groups4 - kt * 4) : min(4, (p.R - ((kt - kt_main) % lora_slabs) * 64) / 16);
          if (elect_one()) {
            if (main_slab) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (j < nkb)
                  mma_nvfp4<CG>(tmem_acc, smem_desc(kDescAB, a_addr + j * 32), smem_desc(kDescAB, b_addr + j * 32),
                                kIdescMain, tsfa + j * 4, tsfb + j * (BN / 32), ((pos - kt_lo) | j) != 0 ? 1u : 0u);
              tc_commit_local<CG>(&sf_empty[sb]);   // scale buffer reusable once these MMAs are done
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (j < nkb)
                  mma_f16<CG>(tmem_acc, smem_desc(kDescAB, a_addr + j * 32), smem_desc(kDescAB, b_addr + j * 32),
                              idesc_lora, ((pos - kt_lo) | j) != 0 ? 1u : 0u);
            }
            tc_commit_mask<CG>(&empty[s], kMask);          // stage reusable (in both CTAs) once these MMAs have read it
            if (pos == kt_hi - 1) tc_commit_mask<CG>(&acc_full[as], kMask);    // accumulator complete
          }
          __syncwarp();
          if (main_slab) ++sf_it;
        }
      }
    }
  } else if (warp >= EPI_WARPS + 2) {
    // ------------------------------ scale copiers (leader CTA only) ------------------------------
    // Copies the scale atoms of main slab n into scale buffer n % SF_BUFS, up to SF_BUFS - 1 slabs ahead of the MMAs.
    if (rank == 0) {
      constexpr uint64_t kDescSF = smem_desc_base(0, 128, kSwizzleNone);    // 8 x 16 B core matrices, 128 B apart
      const int jlo = (warp - (EPI_WARPS + 2)) * (4 / SF_WARPS);            // this warp's k-blocks: jlo, jlo + 1
      uint32_t it = 0, sf_it = 0;
      bool ok = true;
      for (int w = pair; w < total_work && ok; w += num_pairs) {
        const int tile = SK ? w / S : w, split = SK ? w - tile * S : 0;
        const bool la_fp16 = lora_fp16(tile % p.tiles_m);
        const int kt_all = kt_main + lora_parts(la_fp16) * lora_slabs;
        int kt_lo, kt_hi;
        slab_range(split, kt_all, kt_lo, kt_hi);
        SlabWalk walk;
        walk.start(kt_main, kt_all, p.interleave, lora_stride(la_fp16), kt_lo);
        for (int pos = kt_lo; pos < kt_hi; ++pos, ++it) {
          const int kt = walk.at(pos);
          // Every slab's barrier is waited on in order, LoRA slabs (which carry no scales) included: a
          // waiter that skipped ahead could get two ring revolutions in front of the producer, where the
          // parity of a barrier no longer tells the revolutions apart.
          const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1;
          if (!uwait(&full_sf[s], ph, ctx, kDevWaitFull, 0x20000 + it)) { ok = false; break; }
          if (kt >= kt_main) {                               // no scales: this copier's arrival on the stage's barrier at once
            if (elect_one()) mbar_arrive(&full[s]);
            __syncwarp();
            continue;
          }
          const uint32_t sb = sf_it % C::SF_BUFS;
          if (!uwait(&sf_empty[sb], ((sf_it / C::SF_BUFS) & 1) ^ 1, ctx, kDevWaitMisc, 0x20000 + it)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sfa_addr = smem_u32(smem + s * C::STAGE_BYTES) + A_BYTES + C::B_BYTES;
          const uint32_t sfb_addr = sfa_addr + SFA_BYTES;
          const uint32_t tsfa = tmem_sf + sb * C::SF_COLS, tsfb = tsfa + C::SFA_COLS;
          const int nkb = min(4, k_groups4 - kt * 4);
          if (elect_one()) {
#pragma unroll
            for (int jj = 0; jj < 4 / SF_WARPS; ++jj) {
              const int j = jlo + jj;
              if (j < nkb) {
                tmem_cp_scales<CG>(tsfa + j * 4, smem_desc(kDescSF, sfa_addr + j * 512));
#pragma unroll
                for (int h = 0; h < BN / 128; ++h)
                  tmem_cp_scales<CG>(tsfb + j * (BN / 32) + h * 4, smem_desc(kDescSF, sfb_addr + h * 2048 + j * 512));
              }
            }
            tc_commit_local<CG>(&full[s]);                   // arrives once these copies are done
          }
          __syncwarp();
          ++sf_it;
        }
      }
    }
  } else {
    // ------------------------------ epilogue (warps 0-7, both CTAs) ------------------------------
    // Warp w drains the 32 accumulator rows of lane quarter w % 4 and the column half w / 4.
    const OutT* wc = static_cast<const OutT*>(p.wc);
    const OutT* bias = static_cast<const OutT*>(p.bias);
    const int quarter = warp & 3, chalf = warp >> 2;
    uint8_t* my_bufs = store_bufs + warp * (C::STORE_BUFS * STORE_BUF_BYTES);
    const uint32_t swz = static_cast<uint32_t>(lane & 7);
    uint32_t tcount = 0, nstore = 0;
    bool ok = true;
    for (int w = pair; w < total_work && ok; w += num_pairs, ++tcount) {
      const int tile = SK ? w / S : w, split = SK ? w - tile * S : 0;
      const int mb = tile % p.tiles_m, nb = tile / p.tiles_m;
      const int m0 = (mb * CG + rank) * BM, n0 = nb * BN;
      const uint32_t as = tcount % C::ACC_STAGES, aph = (tcount / C::ACC_STAGES) & 1;
      // stage this tile's per-column affine terms (the previous tile's readers are past the barrier below)
      [[maybe_unused]] bool odd_smooth = false;     // NEXT: some smooth_next of this tile is outside [2^-20, 2^20]
      for (int c = threadIdx.x; c < BN; c += EPI_WARPS * 32) {
        affine[c] = wc != nullptr ? as_f32<OutT>(wc[n0 + c]) : 1.0f;
        affine[BN + c] = bias != nullptr ? as_f32<OutT>(bias[n0 + c]) : 0.0f;
        if constexpr (NEXT) {
          const float sv = as_f32<OutT>(static_cast<const OutT*>(p.smooth_next)[n0 + c]);
          affine[2 * BN + c] = -sv;
          affine[3 * BN + c] = __frcp_rn(sv);
          odd_smooth |= !(sv >= 9.5367431640625e-07f && sv <= 1048576.0f);      // also zero, negative, NaN
        }
      }
      // NEXT: the tile divides with __fdiv_rn if any of its columns asks for it (the same verdict in all warps)
      [[maybe_unused]] bool tile_fdiv = false;
      if constexpr (NEXT) {
        uint32_t any_odd;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\t"
            "bar.red.or.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
            : "=r"(any_odd) : "r"(odd_smooth ? 1u : 0u), "n"(EPI_WARPS * 32) : "memory");
        tile_fdiv = any_odd != 0;
      } else {
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
      }
      if (!mbar_wait(&acc_full[as], aph, ctx, kDevWaitAcc, tcount)) ok = false;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * BN + chalf * (BN / 2);
      // Drain: every column this warp owns goes to registers in one burst, the accumulator is handed
      // back at once, and only then do the affine, the packing and the stores happen.
      uint32_t v[C::GROUPS_PER_WARP][2][32];
      if constexpr (C::GROUPS_PER_WARP == 2) tmem_ld_32x32_x128(taddr, &v[0][0][0]);
      else tmem_ld_32x32_x64(taddr, &v[0][0][0]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CG == 2) mbar_arrive_cluster(&acc_empty[as], 0); else mbar_arrive(&acc_empty[as]);
      }
      bool finish = true;                       // this CTA writes the tile's rows of y
      if constexpr (SK) {
        if (S > 1) {
          // Each thread parks its 16 x GROUPS_PER_WARP float4s at [j][thread] of the CTA's partial tile
          // (consecutive threads, consecutive 16 bytes) and later reads the same places of the other
          // partials, so no thread ever needs another thread's accumulator values.
          constexpr int kVec = C::GROUPS_PER_WARP * 16;
          constexpr int kTileVec = BM * BN / 4;
          const int tid = threadIdx.x;
          float4* mine = p.ws_partials + static_cast<size_t>(tile * S + split) * kTileVec;
          const uint32_t* vf = &v[0][0][0];
#pragma unroll
          for (int j = 0; j < kVec; ++j)
            __stcg(mine + j * (EPI_WARPS * 32) + tid,
                   make_float4(__uint_as_float(vf[4 * j]), __uint_as_float(vf[4 * j + 1]), __uint_as_float(vf[4 * j + 2]),
                               __uint_as_float(vf[4 * j + 3])));
          __threadfence();
          asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
          if (tid == 0) *sk_ticket = atomicAdd(p.ws_tickets + tile, 1u);
          asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
          finish = *sk_ticket == static_cast<uint32_t>(S - 1);
          if (finish) {
            __threadfence();
            // Partial sp is added as a whole before partial sp + 1 is looked at: one round trip to L2
            // per partial with all of a thread's loads in flight together, and the same order of
            // additions whatever order the CTAs finished in.
            const float4* first = p.ws_partials + static_cast<size_t>(tile * S) * kTileVec + tid;
            uint32_t* vw = &v[0][0][0];
#pragma unroll
            for (int j = 0; j < kVec; ++j) {
              const float4 t = __ldcg(first + j * (EPI_WARPS * 32));
              vw[4 * j] = __float_as_uint(t.x); vw[4 * j + 1] = __float_as_uint(t.y);
              vw[4 * j + 2] = __float_as_uint(t.z); vw[4 * j + 3] = __float_as_uint(t.w);
            }
#pragma unroll 1
            for (int sp = 1; sp < S; ++sp) {
              const float4* part = first + static_cast<size_t>(sp) * kTileVec;
#pragma unroll
              for (int h = 0; h < kVec; h += 8) {
                float4 t[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) t[j] = __ldcg(part + (h + j) * (EPI_WARPS * 32));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  vw[4 * (h + j)] = __float_as_uint(__uint_as_float(vw[4 * (h + j)]) + t[j].x);
                  vw[4 * (h + j) + 1] = __float_as_uint(__uint_as_float(vw[4 * (h + j) + 1]) + t[j].y);
                  vw[4 * (h + j) + 2] = __float_as_uint(__uint_as_float(vw[4 * (h + j) + 2]) + t[j].z);
                  vw[4 * (h + j) + 3] = __float_as_uint(__uint_as_float(vw[4 * (h + j) + 3]) + t[j].w);
                }
              }
            }
            if (tid == 0) p.ws_tickets[tile] = 0u;      // every split has drawn its ticket: ready for the next launch
          }
        }
      }
      if (finish) {
#pragma unroll
      for (int g = 0; g < C::GROUPS_PER_WARP; ++g, ++nstore) {
        uint8_t* buf = my_bufs + (nstore % C::STORE_BUFS) * STORE_BUF_BYTES;
        // the TMA store that last read this buffer must be done with it
        if (lane == 0) tma_store_wait_read<C::STORE_BUFS - 1>();
        __syncwarp();
        const int cbase = chalf * (BN / 2) + g * 64;
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          const float4* wc4 = reinterpret_cast<const float4*>(affine + cbase + hc * 32);
          const float4* bs4 = reinterpret_cast<const float4*>(affine + BN + cbase + hc * 32);
          uint32_t o[16];
          [[maybe_unused]] float2 qf[8];      // NEXT: the 16 values of the current column group
          [[maybe_unused]] uint32_t qcodes[4], qscales[2];
          // the four fp32 results of columns 4 i .. 4 i + 3 of this half strip
          auto affine_at = [&](int i, float& a0, float& a1, float& a2, float& a3) {
            a0 = __uint_as_float(v[g][hc][4 * i]); a1 = __uint_as_float(v[g][hc][4 * i + 1]);
            a2 = __uint_as_float(v[g][hc][4 * i + 2]); a3 = __uint_as_float(v[g][hc][4 * i + 3]);
            if (wc != nullptr) {
              const float4 w4 = wc4[i];
              a0 = __fmul_rn(a0, w4.x); a1 = __fmul_rn(a1, w4.y); a2 = __fmul_rn(a2, w4.z); a3 = __fmul_rn(a3, w4.w);
            }
            if (bias != nullptr) {
              const float4 b4 = bs4[i];
              a0 = __fadd_rn(a0, b4.x); a1 = __fadd_rn(a1, b4.y); a2 = __fadd_rn(a2, b4.z); a3 = __fadd_rn(a3, b4.w);
            }
          };
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float a0, a1, a2, a3;
            affine_at(i, a0, a1, a2, a3);
            o[2 * i] = pack2f<OutT>(a0, a1);
            o[2 * i + 1] = pack2f<OutT>(a2, a3);
            if constexpr (NEXT) {
              qf[2 * (i & 3)] = make_float2(a0, a1);
              qf[2 * (i & 3) + 1] = make_float2(a2, a3);
              if ((i & 3) == 3) {
                const int e4 = (cbase + hc * 32) / 4 + (i - 3);      // float4 index of the group's first column
                const uint4 r = next_group_codes(qf[0], qf[1], qf[2], qf[3], qf[4], qf[5], qf[6], qf[7],
                                                 reinterpret_cast<const float4*>(affine + 2 * BN) + e4,
                                                 reinterpret_cast<const float4*>(affine + 3 * BN) + e4, tile_fdiv ? 1 : 0);
                qcodes[2 * (i >> 2)] = r.x; qcodes[2 * (i >> 2) + 1] = r.y; qscales[i >> 2] = r.z;
              }
            }
          }
          if constexpr (NEXT) {
            if (ok) {
              // this thread's row: 32 columns = 16 code bytes and two scale bytes
              const uint32_t row = static_cast<uint32_t>(m0 + quarter * 32 + lane);
              const uint32_t col = static_cast<uint32_t>(n0 + cbase + hc * 32);
              *reinterpret_cast<uint4*>(p.qout + static_cast<size_t>(row) * (p.N >> 1) + (col >> 1)) =
                  make_uint4(qcodes[0], qcodes[1], qcodes[2], qcodes[3]);
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const uint32_t gcol = (col >> 4) + h;
                p.oscales[static_cast<size_t>(gcol) * p.M + row] = static_cast<uint8_t>(qscales[h]);
                if (p.oscales_swz != nullptr) p.oscales_swz[sf_swizzled_offset(row, gcol, p.N >> 4)] = static_cast<uint8_t>(qscales[h]);
              }
            }
          }
          // row `lane` of the strip: 16-byte chunks hc*4 .. hc*4+3, XOR-swizzled like the TMA box
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t chunk = static_cast<uint32_t>(hc * 4 + i) ^ swz;
            *reinterpret_cast<uint4*>(buf + lane * 128 + chunk * 16) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmY, buf, p.col0 + n0 + cbase, m0 + quarter * 32);
          // the same strip into every peer's matrix: the copy engine sends it over NVLink while the warp goes on
          for (int d = 0; d < p.n_peers; ++d) tma_store_2d(&peers.m[d], buf, p.col0 + n0 + cbase, m0 + quarter * 32);
          tma_store_commit();
        }
      }
      }
      // affine[] may be overwritten after this barrier; it also makes the eight warps agree on whether to go on
      uint32_t any_failed;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\tsetp.eq.u32 p, %1, 0;\n\t"
          "bar.red.or.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
          : "=r"(any_failed) : "r"(ok ? 1u : 0u), "n"(EPI_WARPS * 32) : "memory");
      ok = any_failed == 0;
    }
    if (lane == 0) tma_store_wait_all<0>();   // global writes of this warp are complete before the CTA ends
    __syncwarp();
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
  if constexpr (CG == 2) cluster_sync_all();   // the partner may still read this CTA's shared memory / signal its barriers
  if (warp == EPI_WARPS + 1) {
    tc_fence_after_sync();
    if constexpr (CG == 1) tmem_dealloc(tmem_base, C::TMEM_COLS); else tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace gemm

bool gemm_supported(int M, int N, int K, int R) {
  return M > 0 && N > 0 && K > 0 && M % 128 == 0 && N % 128 == 0 && K % 64 == 0 && R >= 0 && R % 16 == 0;
}

template <int CG, int BN, typename OutT, bool SK = false, bool NEXT = false>
static int launch_gemm_t(const void* act, const void* wgt, const void* sfa, const void* sfb, const void* la,
                         const void* lu, const void* lu_f16, const void* wc, const void* bias, void* y, int M, int N,
                         int K, int R, const GemmTp& tp, cudaStream_t stream, int splits = 1) {
  using C = gemm::Cfg<CG, BN, NEXT>;
  constexpr bool kBf16 = std::is_same<OutT, __nv_bfloat16>::value;
  CUtensorMap tmA, tmB, tmLA, tmLU, tmY, tmSFA, tmSFB, tmLAf, tmLUf;
  int rc;
  const uint64_t atoms_k = K / 64;
  if ((rc = make_tmap_2d(&tmSFA, sfa, 4, (M / 128) * atoms_k, 128, 512, 4, 128, kTmapSwizzleNone)) != SVDQ_OK) return rc;
  if ((rc = make_tmap_2d(&tmSFB, sfb, 4, (N / 128) * atoms_k, 128, 512, 4, 128, kTmapSwizzleNone)) != SVDQ_OK) return rc;
  if ((rc = make_tmap_2d(&tmA, act, 1, M, K / 2, K / 2, gemm::BM, 128, kTmapSwizzle128)) != SVDQ_OK) return rc;
  if ((rc = make_tmap_2d(&tmB, wgt, 1, N, K / 2, K / 2, C::B_ROWS, 128, kTmapSwizzle128)) != SVDQ_OK) return rc;
  const int y_ld = tp.y_ld > 0 ? tp.y_ld : N;      // y may be the [M, y_ld] matrix this launch fills N columns of
  if ((rc = make_tmap_2d(&tmY, y, 2, M, y_ld, static_cast<uint64_t>(y_ld) * 2, 32, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
  if (R > 0) {
    const uint64_t la_rows = static_cast<uint64_t>(M) * (std::is_same<OutT, __nv_bfloat16>::value ? 2 : 1);
    if ((rc = make_tmap_2d(&tmLA, la, 2, la_rows, R, static_cast<uint64_t>(R) * 2, gemm::BM, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
    if ((rc = make_tmap_2d(&tmLU, lu, 2, N, R, static_cast<uint64_t>(R) * 2, C::B_ROWS, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
  } else {
    tmLA = tmA; tmLU = tmB;
  }
  gemm::Params p;
  p.la_flags = nullptr;
  tmLAf = tmLA; tmLUf = tmLU;
  if (kBf16 && R > 0 && lu_f16 != nullptr) {
    // bf16 form of lora_act: planes hi, lo, fp16, then the per-32-row flag words
    const size_t plane = static_cast<size_t>(M) * R;
    const void* la_f16 = static_cast<const uint16_t*>(la) + 2 * plane;
    if ((rc = make_tmap_2d(&tmLAf, la_f16, 2, M, R, static_cast<uint64_t>(R) * 2, gemm::BM, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
    if ((rc = make_tmap_2d(&tmLUf, lu_f16, 2, N, R, static_cast<uint64_t>(R) * 2, C::B_ROWS, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
    p.la_flags = lora16_flags(la, plane);
  }
  p.wc = wc; p.bias = bias;
  p.M = M; p.N = N; p.K = K; p.R = R;
  p.tiles_m = M / (gemm::BM * CG); p.tiles_n = N / BN;
  p.col0 = tp.y_ld > 0 ? tp.col0 : 0; p.y_ld = y_ld; p.n_peers = tp.n_peers;
  gemm::PeerMaps peers;
  for (int d = 0; d < 7; ++d) peers.m[d] = tmY;
  for (int d = 0; d < tp.n_peers; ++d)
    if ((rc = make_tmap_2d(&peers.m[d], tp.y_peer[d], 2, M, y_ld, static_cast<uint64_t>(y_ld) * 2, 32, 64, kTmapSwizzle128)) != SVDQ_OK) return rc;
  p.splits = SK ? splits : 1;
  p.interleave = tp.interleave;
  {
    const int kt_main = (K + gemm::BK - 1) / gemm::BK, ls = (R + 63) / 64;
    p.stride1 = ls > 0 ? (kt_main + ls) / ls : 1;
    p.stride2 = ls > 0 ? (kt_main + 2 * ls) / (2 * ls) : 1;
  }
  p.ws_tickets = static_cast<unsigned int*>(tp.ws);
  p.ws_partials = tp.ws != nullptr ? reinterpret_cast<float4*>(static_cast<uint8_t*>(tp.ws) + kSplitTicketBytes) : nullptr;
  p.smooth_next = tp.smooth_next;
  p.qout = static_cast<uint8_t*>(tp.qout);
  p.oscales = static_cast<uint8_t*>(tp.oscales);
  p.oscales_swz = static_cast<uint8_t*>(tp.oscales_swz);
  auto kern = gemm::gemm_w4a4_kernel<CG, BN, OutT, SK, NEXT>;
  // the attribute is per device: remember which devices of this process have it
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SVDQ_ERR_CUDA;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) return SVDQ_ERR_LAUNCH;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int tiles = p.tiles_m * p.tiles_n * p.splits;
  const int max_pairs = sm_count() / CG;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pairs * CG, 1, 1);
  cfg.blockDim = dim3(gemm::NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmLA, tmLU, tmY, tmSFA, tmSFB, tmLAf, tmLUf, peers, p) != cudaSuccess) return SVDQ_ERR_LAUNCH;
  return SVDQ_OK;
}

template <typename OutT, bool NEXT>
static int launch_gemm_dt(int cg, int bn, const void* act, const void* wgt, const void* sfa, const void* sfb,
                          const void* la, const void* lu, const void* lu_f16, const void* wc, const void* bias, void* y,
                          int M, int N, int K, int R, const GemmTp& tp, cudaStream_t stream) {
  if (cg == 2 && bn == 256) return launch_gemm_t<2, 256, OutT, false, NEXT>(act, wgt, sfa, sfb, la, lu, lu_f16, wc, bias, y, M, N, K, R, tp, stream);
  if (cg == 2 && bn == 128) return launch_gemm_t<2, 128, OutT, false, NEXT>(act, wgt, sfa, sfb, la, lu, lu_f16, wc, bias, y, M, N, K, R, tp, stream);
  if (cg == 1 && bn == 256) return launch_gemm_t<1, 256, OutT, false, NEXT>(act, wgt, sfa, sfb, la, lu, lu_f16, wc, bias, y, M, N, K, R, tp, stream);
  return launch_gemm_t<1, 128, OutT, false, NEXT>(act, wgt, sfa, sfb, la, lu, lu_f16, wc, bias, y, M, N, K, R, tp, stream);
}

// Split-K plan for a problem with few tiles: 128 x 128 tiles, each tile's slabs shared by S CTAs that
// all run at once (tiles * S <= SMs).  One CTA streams a tile's slabs at about 0.3 us each however
// few tiles there are (32 KB per slab through one SM's load path), so with a few dozen tiles most
// SMs idle and the run time is one tile's K loop.  Splitting costs about 3.3 us (partials to L2, a
// fence, the ticket, one read per partial), which the shorter loops repay from about 24 slabs on
// (measured, 256 rows x 3072 columns: K = 3840 9.1 -> 10.0 us, K = 10240 16.1 -> 12.7 us,
// K = 15360 22.6 -> 17.7 us).  Returns S (1 = no split).
int gemm_split_plan(int M, int N, int K, int R) {
  if (!gemm_supported(M, N, K, R)) return 1;
  const long long tiles = static_cast<long long>(M / 128) * (N / 128);
  const int slabs = (K + gemm::BK - 1) / gemm::BK;
  const int sms = sm_count();
  if (tiles * 2 > sms || tiles > kSplitMaxTiles || slabs < 24) return 1;
  int s = static_cast<int>(sms / tiles);
  if (s > 4) s = 4;
  if (s > slabs / 6) s = slabs / 6;               // at least six slabs per split
  return s < 2 ? 1 : s;
}

size_t gemm_split_workspace_bytes(int M, int N, int K, int R) {
  const int s = gemm_split_plan(M, N, K, R);
  if (s < 2) return 0;
  return kSplitTicketBytes + static_cast<size_t>(M / 128) * (N / 128) * s * (128 * 128 * 4);
}

// Default LoRA schedule: after the main slabs.  Same-box A/B on the four benchmark shapes: interleaved
// 27.1 / 121.0 / 102.4 / 55.0 us against 27.4 / 120.5 / 102.6 / 55.0 us at the end (within run-to-run noise; the
// reference measured +0.5 % for its interleave, docs/gotchas/cute_dsl.md:368-377).
constexpr int kLoraInterleaveDefault = 0;

// variant: 0 = choose; 128 / 256 = one CTA per tile with that N tile; 2128 / 2256 = CTA pairs (256-row tiles);
// 10000 * S + 128 = split-K with S CTAs per 128 x 128 tile (needs the workspace)
int launch_gemm_w4a4(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                     const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales,
                     const void* bias, void* y, int M, int N, int K, int R, int dtype, int variant,
                     const GemmTp& tp_in, cudaStream_t stream) {
  if (!gemm_supported(M, N, K, R)) return SVDQ_ERR_SHAPE;
  // LoRA schedule bits of `variant`: interleaved, end-grouped, or (neither) the library's default
  GemmTp tp = tp_in;
  if (variant & SVDQ_GEMM_LORA_INTERLEAVE) tp.interleave = 1;
  else if (variant & SVDQ_GEMM_LORA_AT_END) tp.interleave = 0;
  else tp.interleave = kLoraInterleaveDefault;
  variant &= ~(SVDQ_GEMM_LORA_INTERLEAVE | SVDQ_GEMM_LORA_AT_END);
  if (tp.n_peers < 0 || tp.n_peers > 7) return SVDQ_ERR_SHAPE;
  if (tp.y_ld > 0 && (tp.col0 < 0 || tp.col0 % 64 != 0 || tp.col0 + N > tp.y_ld || tp.y_ld % 8 != 0)) return SVDQ_ERR_SHAPE;
  if (tp.y_ld <= 0 && tp.n_peers > 0) return SVDQ_ERR_SHAPE;
  const bool next = tp.smooth_next != nullptr;
  if (next && (tp.qout == nullptr || tp.oscales == nullptr || tp.y_ld > 0 || variant >= 10000)) return SVDQ_ERR_UNSUPPORTED;
  int cg, bn;
  if (!next && (variant == 0 || variant >= 10000)) {
    // split-K: planned (variant 0, plain form, workspace large enough) or forced by the caller
    int s = 1;
    if (variant == 0 && tp.y_ld <= 0 && tp.ws != nullptr) {
      s = gemm_split_plan(M, N, K, R);
      if (s >= 2 && tp.ws_bytes < gemm_split_workspace_bytes(M, N, K, R)) s = 1;
    } else if (variant >= 10000) {
      s = variant / 10000;
      const long long tiles = static_cast<long long>(M / 128) * (N / 128);
      if (variant % 10000 != 128 || s < 2 || s > kSplitMax || tiles > kSplitMaxTiles || tp.ws == nullptr || tp.y_ld > 0 ||
          s > (K + gemm::BK - 1) / gemm::BK || tiles * s > sm_count() ||
          tp.ws_bytes < kSplitTicketBytes + static_cast<size_t>(tiles) * s * (128 * 128 * 4))
        return SVDQ_ERR_UNSUPPORTED;
    }
    if (s >= 2) {
      if (dtype == SVDQ_DTYPE_F16)
        return launch_gemm_t<1, 128, __half, true>(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, nullptr, wcscales, bias, y, M, N, K, R, tp, stream, s);
      if (dtype == SVDQ_DTYPE_BF16)
        return launch_gemm_t<1, 128, __nv_bfloat16, true>(act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, lora_up_f16, wcscales, bias, y, M, N, K, R, tp, stream, s);
      return SVDQ_ERR_DTYPE;
    }
  }
  if (variant == 0) {
    // Pick the tile shape with the least estimated time: waves of tiles over the SMs (or SM pairs)
    // times the measured relative time of one tile (a 128-column tile takes 0.72 of a 256-column
    // one, not half: it moves more operand bytes per flop; a single CTA per tile takes 1.12 of a
    // pair's time for loading all of B itself).  Large problems end on 256 x 256 pair tiles, a few
    // hundred rows on narrower tiles that put more SMs to work.
    const int sms = sm_count();
    double best = 1e30;
    cg = 1; bn = 128;
    for (int c : {2, 1})
      for (int b : {256, 128}) {
        if (M % (128 * c) != 0 || N % b != 0) continue;
        const long long tiles = static_cast<long long>(M / (128 * c)) * (N / b);
        const long long units = sms / c;
        const double cost = static_cast<double>((tiles + units - 1) / units) * (b == 256 ? 1.0 : 0.72) * (c == 2 ? 1.0 : 1.12);
        if (cost < best) { best = cost; cg = c; bn = b; }
      }
  } else if (variant == 128 || variant == 256) {
    cg = 1; bn = variant;
  } else {
    cg = variant / 1000; bn = variant % 1000;
  }
  if ((cg != 1 && cg != 2) || (bn != 128 && bn != 256)) return SVDQ_ERR_UNSUPPORTED;
  if (M % (128 * cg) != 0 || N % bn != 0) return SVDQ_ERR_SHAPE;
  if (dtype == SVDQ_DTYPE_F16)
    return next ? launch_gemm_dt<__half, true>(cg, bn, act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, nullptr, wcscales, bias, y, M, N, K, R, tp, stream)
                : launch_gemm_dt<__half, false>(cg, bn, act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, nullptr, wcscales, bias, y, M, N, K, R, tp, stream);
  if (dtype == SVDQ_DTYPE_BF16)
    return next ? launch_gemm_dt<__nv_bfloat16, true>(cg, bn, act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, lora_up_f16, wcscales, bias, y, M, N, K, R, tp, stream)
                : launch_gemm_dt<__nv_bfloat16, false>(cg, bn, act, wgt, ascales_swz, wscales_swz, lora_act16, lora_up, lora_up_f16, wcscales, bias, y, M, N, K, R, tp, stream);
  return SVDQ_ERR_DTYPE;
}

}  // namespace svdq
