/*
 * svdq_b200 — C ABI of the B200 (sm_100a) SVDQuant W4A4 linear.
 *
 * Plain pointers and sizes only; no C++ or framework types cross this line.
 * Every function returns an SVDQ_* status, never throws, never allocates
 * unless stated, and (except the *_host calls and svdq_device_status) never
 * synchronises: kernels are queued on the `stream` argument (a cudaStream_t
 * passed as void*; NULL = the default stream).  The caller owns every buffer.
 *
 * Each entry point names the reference interface it stands in for, by that
 * project's own paths.
 */
#ifndef SVDQ_B200_H_
#define SVDQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of 16-bit (and, for the weight packer, 32-bit) tensors */
enum { SVDQ_DTYPE_F16 = 0, SVDQ_DTYPE_BF16 = 1, SVDQ_DTYPE_F32 = 2 };

/* status codes */
enum {
  SVDQ_OK = 0,
  SVDQ_ERR_NULL = 1,      /* a required pointer is NULL */
  SVDQ_ERR_SHAPE = 2,     /* a size breaks the op's contract (see each function) */
  SVDQ_ERR_DTYPE = 3,
  SVDQ_ERR_ALIGN = 4,     /* a pointer is not 16-byte aligned */
  SVDQ_ERR_LAUNCH = 5,    /* the CUDA runtime refused a launch / descriptor */
  SVDQ_ERR_DEVICE = 6,    /* a kernel gave up on a bounded wait; see svdq_device_status */
  SVDQ_ERR_UNSUPPORTED = 7,
  SVDQ_ERR_CUDA = 8       /* other CUDA runtime failure (copy, allocation in plan/host calls) */
};

/* flags for svdq_quantize_w4a4_act_fuse_lora */
enum {
  SVDQ_QUANT_AUTO = 0,        /* fused tensor-core kernel when the shape allows, else the generic kernels */
  SVDQ_QUANT_FORCE_GENERIC = 1,
  SVDQ_QUANT_FORCE_FUSED = 2, /* the cluster form of the fused kernel; error instead of falling back */
  /* the streaming form of the fused kernel (tall activations); error if it does not apply.  Tile height
   * and K split may be forced too: SVDQ_QUANT_FORCE_STREAM | (tile_rows << 8) | (k_split << 4), tile_rows
   * 128 or 256 (0 = planned), k_split 1, 2, 4 or 8 (0 = planned) */
  SVDQ_QUANT_FORCE_STREAM = 0x100000
};

/* bits that may be OR-ed into the `variant` argument of the GEMM entry points */
enum {
  SVDQ_GEMM_LORA_INTERLEAVE = 1 << 24,  /* a tile's LoRA-up slabs spread evenly among its main K slabs */
  SVDQ_GEMM_LORA_AT_END = 1 << 25       /* ... after them */
};

const char* svdq_status_string(int status);
int svdq_version(void);

/*
 * One-time preparation of a smoothing vector: writes {smooth[k], 1/smooth[k]} as K float pairs
 * followed by one 8-byte flag word (so smooth_table holds 8*K + 8 bytes, 16-byte aligned).
 * smooth is a per-layer constant, so callers build the table once and pass it with every
 * quantizer call.  No counterpart in the reference, which divides inside its kernel
 * (triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:153-158).
 */
int svdq_prepare_smooth(const void* smooth, void* smooth_table, int K, int dtype, void* stream);

/*
 * Fused activation quantizer + LoRA-down.
 * Stands in for quantize_w4a4_act_fuse_lora(input, lora_down, smooth, fp4=True, pad_size)
 *   (triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:289-400; oracle
 *    baseline/kernels/quantize_w4a4_act_fuse_lora/ref.py:19-50).
 *
 *   x          [M, K]        f16/bf16, row-major, K % 16 == 0
 *   lora_down  [K, R]        same type (R may be 0, then lora_down may be NULL)
 *   smooth     [K] or NULL   same type
 *   smooth_table  from svdq_prepare_smooth(smooth), or NULL; without it a smoothed call takes the
 *                 generic (slower, CUDA-core) kernels
 *   act        [M_pad, K/2]  u8   two E2M1 codes per byte, even k in the low nibble
 *   ascales    [K/16, M_pad] u8   E4M3 bit patterns (the reference's transposed layout)
 *   lora_act   [M_pad, R]    f32  rows >= M are zero
 *   ascales_swz  optional, M_pad*K/16 bytes: the same scales in the 128-row x 4-group
 *                atom order the tensor core reads (needs M_pad % 128 == 0, K % 64 == 0)
 *   lora_act16   optional: lora_act in the 16-bit form svdq_gemm_w4a4 consumes;
 *                svdq_lora_act16_elems(M_pad, R, dtype) 16-bit elements.  dtype f16: [M_pad, R]
 *                fp16, rounded once, magnitudes beyond 65504 clamped.  dtype bf16: three
 *                [M_pad, R] planes - hi = bf16(v), lo = bf16(v - hi), and v as fp16 (clamped) -
 *                followed by one 32-bit word per 32 rows that is non-zero when some value of
 *                those rows does not fit fp16
 *   M_pad      rows of the outputs, >= M (the reference pads M up to a multiple of 256)
 * Rows M..M_pad-1 of act / ascales are written as zero bytes, as the oracle does.
 */
int svdq_quantize_w4a4_act_fuse_lora(const void* x, const void* lora_down, const void* smooth,
                                     const void* smooth_table,
                                     void* act, void* ascales, float* lora_act,
                                     void* ascales_swz, void* lora_act16,
                                     int M, int K, int R, int M_pad, int dtype, int flags, void* stream);

/*
 * svdq_quantize_w4a4_act_fuse_lora with a caller-owned workspace in device memory, needed by the
 * streaming form of the fused kernel (flags = SVDQ_QUANT_FORCE_STREAM ...): CTAs own 128 or 256 rows
 * and a share of K, and the partial LoRA sums of a row tile meet in the workspace (fp32, added in a
 * fixed order: results do not depend on timing).  svdq_quantize_workspace_bytes returns the size
 * the planned tile height and K split of this problem need (0: none); a forced split of k ranks needs
 * 2048 + k * M_pad * 512 bytes.  With other flags the workspace is ignored and the call is
 * svdq_quantize_w4a4_act_fuse_lora.  Outputs are identical in codes and scales; lora_act differs
 * from the other forms only by fp32 summation order.  The library does not choose this form by
 * itself: on the benchmark shapes it measured a few per cent slower than the cluster form.
 * The first 2048 bytes of the workspace are counters: zero them once before the first call; every
 * completed call leaves them zero.  Calls that share a workspace must not overlap in time (same
 * stream, or ordered by events); after a call whose bounded wait expired (svdq_device_status != 0)
 * zero them again.  No counterpart in the reference (its Triton kernel adds the partial sums with
 * atomics into a zero-filled lora_act, triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:204-286).
 */
unsigned long long svdq_quantize_workspace_bytes(int M, int K, int R, int M_pad);
int svdq_quantize_w4a4_act_fuse_lora_ws(const void* x, const void* lora_down, const void* smooth,
                                        const void* smooth_table, void* act, void* ascales, float* lora_act,
                                        void* ascales_swz, void* lora_act16, int M, int K, int R, int M_pad,
                                        int dtype, int flags, void* workspace, unsigned long long workspace_bytes,
                                        void* stream);

/*
 * How many clusters of `k_split` CTAs (1, 2, 4 or 8) of the fused quantizer the current device can
 * keep resident at once for LoRA rank R; -1 on error.  Introspection for tuning; the reference
 * has no counterpart (its Triton launch picks k_splits from a table,
 * triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:344-378).
 */
int svdq_quantizer_max_active_clusters(int R, int k_split, int dtype);

/*
 * NVFP4 row packer (weights: pad 1).
 * Stands in for quantize_nvfp4_rows(x, pad_size) (baseline/kernels/_nvfp4.py:60-95).
 *   x [rows, K] f16/bf16/f32 -> codes [rows_pad, K/2], scales [K/16, rows_pad],
 *   optional scales_swz as above.
 */
int svdq_quantize_nvfp4_rows(const void* x, void* codes, void* scales, void* scales_swz,
                             int rows, int rows_pad, int K, int dtype, void* stream);

/*
 * Canonical [K/16, rows] scale bytes -> tensor-core atom order.
 * Stands in for _repack_scales_cutlass_atom (cute_kernels/gemm_w4a4/kernel.py:194-225).
 * rows % 128 == 0 and (K/16) % 4 == 0.
 */
int svdq_swizzle_scales(const void* scales, void* scales_swz, int k_groups, int rows, void* stream);

/* 16-bit elements of the lora_act16 form of a [rows, R] lora_act for dtype (-1 on bad arguments). */
long long svdq_lora_act16_elems(int rows, int R, int dtype);

/* f32 lora_act [rows, R] -> its 16-bit form of type dtype, as described for lora_act16 above (stands
 * in for the cast launch_v2 does at cute_kernels/gemm_w4a4/kernel_v2_fa4.py:176-184).  For bf16 this
 * route marks every row block "does not fit fp16" without looking, so the GEMM takes two passes. */
int svdq_cast_lora_act(const float* src, void* dst, int rows, int R, int dtype, void* stream);

/* HOST helper: bf16 lora_up [count values] -> fp16, for svdq_gemm_w4a4's lora_up_f16.  Returns
 * SVDQ_ERR_UNSUPPORTED (and an unusable output) if a value is NaN or beyond fp16's range; values
 * below 2^-14 lose bits, as they would in any fp16 LoRA.  No counterpart in the reference, which
 * multiplies bf16 lora_act by bf16 lora_up in one pass and accepts the 7e-3 error of that. */
int svdq_lora_up_to_f16(const void* lora_up_bf16_host, void* out_f16_host, long long count);

/*
 * W4A4 GEMM + LoRA-up + per-column affine.
 * Stands in for launch_v2(act, wgt, ascales, wscales, lora_act_in, lora_up, wcscales, bias, out_dtype)
 *   (cute_kernels/gemm_w4a4/kernel_v2_fa4.py:113-225; oracle baseline/kernels/gemm_w4a4/ref.py:33-78).
 *
 *   act         [M, K/2] u8        wgt        [N, K/2] u8
 *   ascales_swz  M*K/16 bytes      wscales_swz N*K/16 bytes   (atom order, see above)
 *   lora_act16  16-bit form of lora_act for dtype (see above) or NULL
 *   lora_up     [N, R] of type dtype or NULL (both or neither)
 *   lora_up_f16 dtype bf16 only, optional: lora_up as fp16 [N, R] on the device.  With it, output
 *               tiles whose rows of lora_act all fit fp16 (the words behind lora_act16) take one
 *               fp16 LoRA pass instead of the hi + lo bf16 passes; other tiles are unaffected.
 *   wcscales    [N] or NULL        bias       [N] or NULL     (type = dtype)
 *   y           [M, N] dtype
 * Contract: M % 128 == 0, N % 128 == 0, K % 64 == 0, R % 16 == 0 (svdq_gemm_w4a4_supported).
 * variant: 0 = let the library pick; 128 / 256 = one CTA per 128 x variant tile;
 *          2128 / 2256 = CTA pairs on 256 x 128 / 256 x 256 tiles (needs M % 256 == 0).
 *          OR-ed with SVDQ_GEMM_LORA_INTERLEAVE or SVDQ_GEMM_LORA_AT_END it also fixes where a tile's
 *          LoRA-up slabs run: spread evenly among its main K slabs (launch_v2's lora_schedule =
 *          "interleave", cute_kernels/gemm_w4a4/kernel_v2_fa4.py:126, :299-303) or after them; with
 *          neither bit the library takes the one it measured faster.  The result is the same sum in a
 *          different order (within the GEMM tolerance of each other, not bit-identical).
 *   y = cast( (deq(act) deq(wgt)^T + lora_act16 lora_up^T) * wcscales + bias )
 */
int svdq_gemm_w4a4(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                   const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales, const void* bias,
                   void* y, int M, int N, int K, int R, int dtype, int variant, void* stream);

/*
 * svdq_gemm_w4a4 that also quantises its result for the next W4A4 linear, in the same epilogue:
 * the optional smooth_next -> (qout, oscales) outputs of gemm_w4a4_ref
 * (baseline/kernels/gemm_w4a4/ref.py:80-87; the reference's own GPU kernels dropped them,
 * docs/architecture.md:78-99).  The fp32 result (after wcscales and bias, BEFORE the cast to the
 * output type) is divided by smooth_next and packed with quantize_nvfp4_rows(pad_size = 1):
 *   smooth_next [N]       f16/bf16 (the output type)
 *   qout        [M, N/2]  u8, two E2M1 codes per byte
 *   oscales     [N/16, M] u8, E4M3 bit patterns
 *   oscales_swz optional, M*N/16 bytes: oscales in the tensor-core atom order (needs N % 64 == 0),
 *               so that a following svdq_gemm_w4a4 can take (qout, oscales_swz) as its act / ascales_swz
 * y is written as by svdq_gemm_w4a4.  Codes and scales equal the oracle's wherever the kernel's
 * fp32 y equals the oracle's (both add the same products, in different orders).
 * Plain tiles only: variants 0, 128, 256, 2128, 2256.
 */
int svdq_gemm_w4a4_next(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                        const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales,
                        const void* bias, void* y, const void* smooth_next, void* qout, void* oscales, void* oscales_swz,
                        int M, int N, int K, int R, int dtype, int variant, void* stream);

/*
 * svdq_gemm_w4a4 with a caller-owned workspace in device memory, for problems with few output tiles
 * (a few hundred rows: the small-M shapes of GEMM_SHAPES in
 * cute_kernels/gemm_w4a4/harness.py:17-24, where the reference's kernels leave most SMs idle).
 * With variant 0 and a workspace of at least svdq_gemm_w4a4_workspace_bytes(M, N, K, R) bytes the
 * library shares each 128 x 128 tile's K loop among several CTAs (split-K): each adds its part in
 * fp32, parks it in the workspace, and the CTA that arrives last sums the parts in a fixed order
 * and writes y, so results do not depend on timing.  variant 10000 * S + 128 forces S CTAs per tile.
 * svdq_gemm_w4a4_workspace_bytes returns 0 where splitting does not apply; then (or with a NULL or
 * smaller workspace) the call is svdq_gemm_w4a4.
 * The first 1024 bytes of the workspace are ticket counters: zero them once before the first call;
 * every call leaves them zero.  Calls that share a workspace must not overlap in time (same stream,
 * or ordered by events); after a call whose bounded wait expired (svdq_device_status != 0) zero it again.
 */
unsigned long long svdq_gemm_w4a4_workspace_bytes(int M, int N, int K, int R);
int svdq_gemm_w4a4_ws(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                      const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales, const void* bias,
                      void* y, int M, int N, int K, int R, int dtype, int variant, void* workspace,
                      unsigned long long workspace_bytes, void* stream);

/*
 * svdq_gemm_w4a4_ws on a workspace that is part of the library image: no counterpart in the reference.
 * For callers that must not allocate device memory around the call: a serving loop that has handed
 * the whole device to its own pool and runs with allocation closed once it is warm; a binding
 * from another language (cgo, JNI) that has no owner for a device buffer that must outlive the
 * call; a latency-bound loop that cannot afford the device-wide synchronisation an allocation or
 * a release may bring.  The function itself allocates and frees nothing, on the host or the device.
 * The workspace is a static array in device memory of 1024 + 148 * 65536 bytes (9.25 MiB, taken on
 * every device that loads the library); a call whose split plan (or forced split count, variant
 * 10000 * S + 128) needs more returns SVDQ_ERR_UNSUPPORTED and launches nothing.  Otherwise the
 * result is that of svdq_gemm_w4a4_ws with a large enough workspace, bit for bit.
 * The first call on each device looks the array's address up through the runtime, which may load
 * the module: make that call before any stream capture is begun on that device.
 * One array per device and process, shared by every caller: calls on the same device must not
 * overlap in time (one stream, or ordered by events); two overlapping calls would mix their partial
 * tiles and tickets.  The ticket counters are zero when the library is loaded and every completed
 * call leaves them zero, so nothing needs zeroing between calls; after a call whose bounded wait
 * expired they may be left non-zero: svdq_device_status, when it reports such a failure, also puts
 * the counters of the current device's array back to zero (a memset, nothing is allocated), so
 * read the status on that device before the next call of this entry point.
 */
int svdq_gemm_w4a4_static_ws(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                             const void* lora_act16, const void* lora_up, const void* lora_up_f16, const void* wcscales,
                             const void* bias, void* y, int M, int N, int K, int R, int dtype, int variant, void* stream);

/*
 * Column-sharded (tensor-parallel) form of svdq_gemm_w4a4, one call per GPU: this GPU holds rows
 * [col0, col0 + N) of wgt / wscales / lora_up / wcscales / bias and computes those columns of the
 * [M, N_total] result.  Every finished 32 x 64 strip is written into y_full (this GPU's copy of the
 * whole result) and, as one TMA store per peer over NVLink, into the same place of y_full_peers[0 ..
 * n_peers-1] (device pointers to the other GPUs' copies, mapped into this process: symmetric
 * memory, CUDA IPC or cuMemMap), so the all-gather the sharding needs rides on the GEMM's epilogue
 * instead of following it.  The caller orders the ranks around the call: nobody may still read its
 * y_full when a peer starts, and a rank reads its y_full only after every peer's launch has
 * completed (a stream barrier over the ranks on either side).  col0 % 64 == 0, N_total % 8 == 0,
 * n_peers <= 7.  No counterpart in the reference, which has no multi-GPU code.
 */
int svdq_gemm_w4a4_columns(const void* act, const void* wgt, const void* ascales_swz, const void* wscales_swz,
                           const void* lora_act16, const void* lora_up, const void* lora_up_f16,
                           const void* wcscales, const void* bias, void* y_full, void* const* y_full_peers,
                           int n_peers, int N_total, int col0, int M, int N, int K, int R, int dtype,
                           int variant, void* stream);

/* 1 if (M, N, K, R) is inside the GEMM contract, else 0. */
int svdq_gemm_w4a4_supported(int M, int N, int K, int R);

/*
 * Reads (and clears) the device status word that kernels write when a bounded
 * wait expires.  Synchronises the device.  out[0]=code (0 = clean), out[1]=block,
 * out[2]=tag, out[3]=how many waits gave up.  When it reports a failure it also
 * zeroes the ticket counters of the library's static split-K workspace on the
 * current device (see svdq_gemm_w4a4_static_ws).
 */
int svdq_device_status(unsigned int out[4]);

/*
 * Self-test of the bounded waits every kernel of this library uses: launches one warp that waits,
 * with the library's own wait routine, on a barrier nothing arrives on.  After limit_ns (at most
 * 1e8) the wait gives up, records code 6 with tag 0x5E1F in the status word and the kernel ends
 * normally; svdq_device_status then returns SVDQ_ERR_DEVICE once and the device stays usable.
 * seen_device (optional, 4 bytes of device memory) receives bit 0 = first wait succeeded, bit 1 =
 * second wait succeeded, bit 2 = the CTA's abort flag was raised; expected value 4.
 * No counterpart in the reference (its kernels have unbounded waits).
 */
int svdq_selftest_wait_expiry(unsigned long long limit_ns, unsigned int* seen_device, void* stream);

/*
 * Self-test of the division svdq_gemm_w4a4_next uses for y / smooth_next: for every fp32 significand of
 * the dividend (2^23) and every 11-bit significand of the divisor (2^10, which covers fp16 and bf16) it
 * compares the three-step quotient through the correctly rounded reciprocal with the IEEE quotient and
 * counts the pairs that differ into *mismatches_device (8 bytes of device memory; expected 0).  About
 * 10 ms of GPU time.  No counterpart in the reference (which divides in PyTorch).
 */
int svdq_selftest_divide(unsigned long long* mismatches_device, void* stream);

/*
 * Whole linear from HOST buffers: copies x to the device, runs quantizer and
 * GEMM on weights already resident in the plan, copies y back and waits.
 * A plan owns its device buffers (allocated once in svdq_linear_plan_create).
 * There is no counterpart in the reference, whose ops take device tensors; this
 * is the host-buffer form of calling its two ops back to back.
 */
typedef struct svdq_linear_plan svdq_linear_plan;
int svdq_linear_plan_create(svdq_linear_plan** plan, int max_M, int K, int N, int R, int dtype,
                            const void* wgt_host, const void* wscales_host, const void* lora_down_host,
                            const void* lora_up_host, const void* smooth_host, const void* wcscales_host,
                            const void* bias_host);
int svdq_linear_plan_forward_host(svdq_linear_plan* plan, const void* x_host, void* y_host, int M);
/*
 * Pipelined form of the same call.  svdq_linear_plan_submit queues x copy -> quantizer -> GEMM ->
 * y copy for one batch and returns; up to two batches are in flight on three streams (copy in,
 * kernels, copy out), so the PCIe transfers of neighbouring batches overlap the kernels and each
 * other.  A third submit first waits for the oldest batch.  svdq_linear_plan_wait returns when
 * every submitted batch has its y on the host.  x_host / y_host of a batch must stay valid (and y
 * unread) until a wait, or the second-next submit, has returned.  Page-locked buffers are copied
 * from and to directly; pageable ones pass through staging buffers of the plan.
 * svdq_linear_plan_forward_host(...) is submit followed by wait.
 */
int svdq_linear_plan_submit(svdq_linear_plan* plan, const void* x_host, void* y_host, int M);
int svdq_linear_plan_wait(svdq_linear_plan* plan);
void svdq_linear_plan_destroy(svdq_linear_plan* plan);

#ifdef __cplusplus
}
#endif
#endif /* SVDQ_B200_H_ */
