"""Operator API of the W4A4 linear, drop-in for the reference's two entry points.

    quantize_w4a4_act_fuse_lora(input, lora_down, smooth, *, fp4=True, pad_size=256)
        -> (act u8 [M_pad, K/2], ascales e4m3 [K/16, M_pad], lora_act f32 [M_pad, R])
        mirrors triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:289-400
    gemm_w4a4(act, wgt, ascales, wscales, lora_act_in, lora_up, wcscales, bias, out_dtype=...)
        -> y [M_pad, N]
        mirrors launch_v2 at cute_kernels/gemm_w4a4/kernel_v2_fa4.py:113-225
        (same argument meaning, AssertionError on contract violations as
        cute_kernels/gemm_w4a4/kernel.py:116-171 raises them)
    quantize_nvfp4_rows(x, pad_size=1) -> (packed, scales)
        mirrors baseline/kernels/_nvfp4.py:60-95 (the offline weight packer), on the GPU

Tensors stay torch tensors on the CUDA device; all arithmetic happens in
libsvdq_b200.so through its C ABI on torch's current stream, asynchronously.

Two layout seams are hidden here.  The tensor core reads block scales in a
128-row x 4-group atom order and reads the LoRA activations as 16-bit values,
while the API tensors are the reference's canonical `[K/16, rows]` scales and an
fp32 `lora_act`.  The quantizer therefore also writes both twins and attaches
them to the tensors it returns (the 16-bit twin is one fp16 plane, or for bf16 a
hi plane and a lo plane whose sum carries 16 significant bits, because the dense
MMA needs lora_act in lora_up's format and a single bf16 copy is too coarse);
`gemm_w4a4` picks them up when the tensors
arrive unmodified, and otherwise (tensors from elsewhere, e.g. weight scales)
derives them once with two small kernels of the same library and caches them
on the tensor object.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

_DT = {torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32}
_TWIN = "_svdq_twins"  # attribute of the owner's storage object: {(offset, numel): (twin, owner version)}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _attach(owner: torch.Tensor, twin: torch.Tensor) -> None:
    """Remember `twin` as the derived form of `owner`'s current contents.

    The record hangs on the owner's storage object, not on the tensor wrapper: a tensor that went
    through the dispatcher (torch.ops.*), a view or a detach() is a new wrapper around the same
    storage, and the storage object lives exactly as long as the memory does, so a record can
    neither be lost on the way nor outlive its data and be found by a later tensor at the same
    address.  The owner's version counter (bumped by every in-place torch op) guards against
    edits after the fact."""
    st = owner.untyped_storage()
    recs = getattr(st, _TWIN, None)
    if recs is None:
        recs = {}
        setattr(st, _TWIN, recs)
    recs[(owner.storage_offset(), owner.numel())] = (twin, owner._version)


def _attached(owner: torch.Tensor, any_version: bool = False) -> Optional[torch.Tensor]:
    recs = getattr(owner.untyped_storage(), _TWIN, None)
    if recs is None:
        return None
    rec = recs.get((owner.storage_offset(), owner.numel()))
    if rec is None or (rec[1] != owner._version and not any_version):
        return None
    return rec[0]


class _on_device:
    """`with torch.cuda.device(dev)` only when `dev` is not already current (the switch costs
    several microseconds of host time per call, more than the launch itself)."""
    __slots__ = ("ctx",)

    def __init__(self, dev: torch.device):
        idx = dev.index
        self.ctx = None if idx is None or idx == torch.cuda.current_device() else torch.cuda.device(idx)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)
        return False


def _smooth_table(smooth: torch.Tensor) -> torch.Tensor:
    """{smooth, 1/smooth} pairs + flag word for the fused kernel; built once per smooth tensor."""
    twin = _attached(smooth)
    if twin is not None:
        return twin
    K = smooth.shape[0]
    lib = _lib.load()
    table = torch.empty(2 * K + 4, dtype=torch.float32, device=smooth.device)
    with _on_device(smooth.device):
        rc = lib.svdq_prepare_smooth(_ptr(smooth), _ptr(table), K, _DT[smooth.dtype], _stream(smooth.device))
    _lib.check(rc, "prepare_smooth")
    _attach(smooth, table)
    return table


def quantize_w4a4_act_fuse_lora(
    input: torch.Tensor,
    lora_down: torch.Tensor,
    smooth: Optional[torch.Tensor],
    *,
    fp4: bool = True,
    pad_size: int = 256,
    block_m: int = 64,          # accepted for call-site compatibility; the kernel picks its own tiling
    block_n: int = 64,
    k_splits: Optional[int] = None,
    out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
    _force: int = _lib.QUANT_AUTO,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """`out = (act, ascales, lora_act)` writes into tensors of a previous call (same shapes) instead
    of allocating; their layout twins are reused as well, so a steady-state call allocates nothing."""
    assert input.dim() == 2 and lora_down.dim() == 2
    assert input.is_cuda and lora_down.is_cuda
    assert input.dtype == lora_down.dtype
    assert input.dtype in (torch.float16, torch.bfloat16)
    M, K = input.shape
    K2, R = lora_down.shape
    assert K == K2, f"K mismatch: input K={K}, lora_down K={K2}"
    assert K % 16 == 0, "NVFP4 group size is 16; K must be divisible by 16"
    if smooth is not None:
        assert smooth.is_cuda and smooth.dtype == input.dtype
        assert smooth.shape == (K,)
    if not fp4:
        raise NotImplementedError("INT4 branch pending; for now only fp4=True.")
    assert pad_size >= 1

    lib = _lib.load()
    dev = input.device
    M_pad = ((M + pad_size - 1) // pad_size) * pad_size
    x = input.contiguous()
    ld = lora_down.contiguous()
    sm = None if smooth is None else smooth.contiguous()
    table = None
    if sm is not None and _force != _lib.QUANT_FORCE_GENERIC:
        table = _smooth_table(sm)
    want_swz = M_pad % 128 == 0 and K % 64 == 0 and M_pad > 0
    swz = la16 = None
    if out is not None:
        act, ascales, lora_act = out
        assert act.shape == (M_pad, K // 2) and act.dtype == torch.uint8 and act.is_contiguous() and act.device == dev
        assert ascales.shape == (K // 16, M_pad) and ascales.dtype == torch.float8_e4m3fn and ascales.is_contiguous()
        assert lora_act.shape == (M_pad, R) and lora_act.dtype == torch.float32 and lora_act.is_contiguous()
        swz = _attached(ascales, any_version=True)
        la16 = _attached(lora_act, any_version=True)
        if la16 is not None and la16.dtype != input.dtype:
            la16 = None
    else:
        act = torch.empty((M_pad, K // 2), dtype=torch.uint8, device=dev)
        ascales = torch.empty((K // 16, M_pad), dtype=torch.float8_e4m3fn, device=dev)
        lora_act = torch.empty((M_pad, R), dtype=torch.float32, device=dev)
    if want_swz and swz is None:
        swz = torch.empty(M_pad * (K // 16), dtype=torch.uint8, device=dev)
    # 16-bit form of lora_act for the GEMM: one fp16 plane; or bf16 hi and lo planes, an fp16 plane
    # and the per-32-row "fits fp16" words (a flat buffer, see include/svdq_b200.h)
    if R > 0 and la16 is None:
        la16 = torch.empty(_la16_elems(M_pad, R, input.dtype), dtype=input.dtype, device=dev)
    # the streaming form (on request) lets its K ranks meet in a workspace, cached per device and stream
    ws = None
    if _force >= _lib.QUANT_FORCE_STREAM:
        ws = _workspace(_QUANT_WS, dev, _QUANT_WS_FORCED, 2048)
    with _on_device(dev):
        if ws is not None:
            rc = lib.svdq_quantize_w4a4_act_fuse_lora_ws(
                _ptr(x), _ptr(ld), _ptr(sm), _ptr(table), _ptr(act), _ptr(ascales), _ptr(lora_act), _ptr(swz), _ptr(la16),
                M, K, R, M_pad, _DT[input.dtype], _force, _ptr(ws), ws.numel(), _stream(dev))
        else:
            rc = lib.svdq_quantize_w4a4_act_fuse_lora(
                _ptr(x), _ptr(ld), _ptr(sm), _ptr(table), _ptr(act), _ptr(ascales), _ptr(lora_act), _ptr(swz), _ptr(la16),
                M, K, R, M_pad, _DT[input.dtype], _force, _stream(dev))
    _lib.check(rc, "quantize_w4a4_act_fuse_lora")
    if swz is not None:
        _attach(ascales, swz)
    if la16 is not None:
        _attach(lora_act, la16)
    return act, ascales, lora_act


_LA16_ELEMS: dict = {}


def _la16_elems(rows: int, R: int, dtype: torch.dtype) -> int:
    key = (rows, R, dtype)
    n = _LA16_ELEMS.get(key)
    if n is None:
        n = _LA16_ELEMS[key] = int(_lib.load().svdq_lora_act16_elems(rows, R, _DT[dtype]))
    return n


def quantize_nvfp4_rows(x: torch.Tensor, *, pad_size: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """GPU row packer: `[rows, K]` f16/bf16/f32 -> (`[rows_pad, K/2]` u8, `[K/16, rows_pad]` e4m3)."""
    assert x.dim() == 2 and x.is_cuda
    assert x.dtype in _DT
    rows, K = x.shape
    assert K % 16 == 0, "NVFP4 group size is 16"
    lib = _lib.load()
    dev = x.device
    rows_pad = ((rows + pad_size - 1) // pad_size) * pad_size
    xc = x.contiguous()
    packed = torch.empty((rows_pad, K // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((K // 16, rows_pad), dtype=torch.float8_e4m3fn, device=dev)
    want_swz = rows_pad % 128 == 0 and K % 64 == 0 and rows_pad > 0
    swz = torch.empty(rows_pad * (K // 16), dtype=torch.uint8, device=dev) if want_swz else None
    with _on_device(dev):
        rc = lib.svdq_quantize_nvfp4_rows(_ptr(xc), _ptr(packed), _ptr(scales), _ptr(swz), rows, rows_pad, K,
                                          _DT[x.dtype], _stream(dev))
    _lib.check(rc, "quantize_nvfp4_rows")
    if swz is not None:
        _attach(scales, swz)
    return packed, scales


def swizzle_scales(scales: torch.Tensor) -> torch.Tensor:
    """Canonical `[K/16, rows]` e4m3 scales -> flat uint8 in tensor-core atom order (cached on the tensor)."""
    twin = _attached(scales)
    if twin is not None:
        return twin
    G, rows = scales.shape
    assert rows % 128 == 0, f"CUTLASS SF atom: M ({rows}) must be a multiple of 128"
    assert G % 4 == 0, f"CUTLASS SF atom: K/16 ({G}) must be a multiple of 4"
    lib = _lib.load()
    src = scales.contiguous()
    out = torch.empty(G * rows, dtype=torch.uint8, device=scales.device)
    with _on_device(scales.device):
        rc = lib.svdq_swizzle_scales(_ptr(src), _ptr(out), G, rows, _stream(scales.device))
    _lib.check(rc, "swizzle_scales")
    _attach(scales, out)
    return out


def _lora_act_16(lora_act_in: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """lora_act in the 16-bit form the GEMM consumes (flat; layout in include/svdq_b200.h)."""
    twin = _attached(lora_act_in)
    if twin is not None and twin.dtype == out_dtype:
        return twin
    if lora_act_in.dtype == torch.float16 and out_dtype == torch.float16:
        return lora_act_in.contiguous()
    src = lora_act_in if lora_act_in.dtype == torch.float32 else lora_act_in.float()
    lib = _lib.load()
    src = src.contiguous()
    rows, R = src.shape
    out = torch.empty(_la16_elems(rows, R, out_dtype), dtype=out_dtype, device=src.device)
    with _on_device(src.device):
        rc = lib.svdq_cast_lora_act(_ptr(src), _ptr(out), rows, R, _DT[out_dtype], _stream(src.device))
    _lib.check(rc, "cast_lora_act")
    return out


def _lora_up_f16(lora_up: torch.Tensor) -> Optional[torch.Tensor]:
    """fp16 copy of a bf16 lora_up (cached on the tensor) for the single-pass LoRA route of the GEMM;
    None if a value does not fit fp16."""
    twin = _attached(lora_up)
    if twin is not None:
        return twin if twin.numel() else None
    host = lora_up.detach().cpu().contiguous()
    out = torch.empty(host.shape, dtype=torch.float16)
    rc = _lib.load().svdq_lora_up_to_f16(_ptr(host), _ptr(out), host.numel())
    dev_copy = out.to(lora_up.device) if rc == _lib.OK else torch.empty(0, dtype=torch.float16, device=lora_up.device)
    _attach(lora_up, dev_copy)
    return dev_copy if dev_copy.numel() else None


def gemm_w4a4(
    act: torch.Tensor,
    wgt: torch.Tensor,
    ascales: torch.Tensor,
    wscales: torch.Tensor,
    lora_act_in: Optional[torch.Tensor] = None,
    lora_up: Optional[torch.Tensor] = None,
    wcscales: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
    *,
    use_2cta: bool = False,                 # accepted for call-site compatibility
    tiler_mn: Optional[Tuple[int, int]] = None,
    lora_schedule: str = "interleave",
    smooth_next: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    _columns: Optional[Tuple[torch.Tensor, list, int]] = None,
    _splits: Optional[int] = None,
) -> torch.Tensor:
    """`smooth_next [N]` (the optional argument of the reference's gemm_w4a4_ref,
    baseline/kernels/gemm_w4a4/ref.py:80-87): the call returns `(y, qout, oscales)`, where qout
    `[M, N/2]` / oscales `[N/16, M]` are the NVFP4 codes and scales of the fp32 result (before its
    cast) divided by smooth_next - the `act` / `ascales` of a following W4A4 linear, made in this
    GEMM's epilogue instead of by a quantizer pass over y.

    Problems with few output tiles (a few hundred rows) take the split-K form (svdq_gemm_w4a4_ws) with
    a workspace cached per device and stream; `_splits = S` forces S CTAs per 128 x 128 tile, `_splits = 1`
    forbids splitting.

    `_columns = (y_full, peer_ptrs, col0)` selects the column-sharded form (svdq_gemm_w4a4_columns):
    the `[M, N]` result of this call goes into columns `[col0, col0 + N)` of the local `[M, N_total]`
    tensor `y_full` and of the peers' copies at the raw device pointers `peer_ptrs`; `y_full` is
    returned.  See `sharding.linear_columns_fused` for the ordering the caller owes."""
    if out_dtype is None:
        out_dtype = lora_up.dtype if lora_up is not None else torch.float16
    assert act.is_cuda and wgt.is_cuda and ascales.is_cuda and wscales.is_cuda, "all inputs must live on CUDA"
    assert act.dtype == torch.uint8 and wgt.dtype == torch.uint8, \
        f"act/wgt must be uint8 NVFP4-packed; got {act.dtype}/{wgt.dtype}"
    assert ascales.dtype == torch.float8_e4m3fn and wscales.dtype == torch.float8_e4m3fn, \
        f"scales must be fp8_e4m3fn; got {ascales.dtype}/{wscales.dtype}"
    assert out_dtype in (torch.float16, torch.bfloat16), f"out_dtype must be fp16 or bf16; got {out_dtype}"
    M, K_half = act.shape
    N, K_half_w = wgt.shape
    assert K_half == K_half_w, f"act/wgt K disagree: {K_half} vs {K_half_w}"
    K = K_half * 2
    assert K % 16 == 0, f"K ({K}) must be a multiple of 16"
    G = K // 16
    assert ascales.shape == (G, M), f"ascales shape {tuple(ascales.shape)} != ({G}, {M})"
    assert wscales.shape == (G, N), f"wscales shape {tuple(wscales.shape)} != ({G}, {N})"
    assert (lora_act_in is None) == (lora_up is None), "lora_act_in and lora_up must both be provided or both None"
    R = 0
    if lora_act_in is not None:
        assert lora_act_in.is_cuda and lora_up.is_cuda, "LoRA inputs must live on CUDA"
        assert lora_act_in.shape[0] == M, f"lora_act_in shape {tuple(lora_act_in.shape)} row != M ({M})"
        assert lora_up.shape[0] == N, f"lora_up shape {tuple(lora_up.shape)} row != N ({N})"
        R = lora_act_in.shape[1]
        assert lora_up.shape[1] == R, f"lora_act_in/lora_up R disagree: {lora_act_in.shape[1]} vs {lora_up.shape[1]}"
        assert R % 16 == 0, f"R ({R}) must be a multiple of LoRA atom K (16)"
        assert lora_up.dtype == out_dtype, f"lora_up dtype {lora_up.dtype} must match out_dtype {out_dtype}"
    if wcscales is not None:
        assert wcscales.shape == (N,), f"wcscales must be [N]; got {tuple(wcscales.shape)}"
    if bias is not None:
        assert bias.shape == (N,), f"bias must be [N]; got {tuple(bias.shape)}"
    assert M % 128 == 0, f"M ({M}) must be a multiple of 128"
    assert N % 128 == 0, f"N ({N}) must be a multiple of 128"
    assert K % 64 == 0, f"K ({K}) must be a multiple of 64 for NVFP4 scale atoms"
    variant = 0
    if tiler_mn is not None:
        assert tiler_mn[0] in (128, 256) and tiler_mn[1] in (128, 256)
        assert M % tiler_mn[0] == 0 and N % tiler_mn[1] == 0
        variant = (2000 if tiler_mn[0] == 256 else 0) + tiler_mn[1]
    # where a tile's LoRA-up slabs run: "interleave" (launch_v2's default spelling) leaves the choice to
    # the library, "interleaved" / "at_end" fix it
    assert lora_schedule in ("interleave", "interleaved", "at_end", "end"), f"unknown lora_schedule {lora_schedule!r}"
    sched = _lib.GEMM_LORA_INTERLEAVE if lora_schedule == "interleaved" else \
        (_lib.GEMM_LORA_AT_END if lora_schedule in ("at_end", "end") else 0)

    lib = _lib.load()
    dev = act.device
    a = act.contiguous()
    w = wgt.contiguous()
    sa = swizzle_scales(ascales)
    sw = swizzle_scales(wscales)
    la = lu = lu16 = None
    if R > 0:
        la = _lora_act_16(lora_act_in, out_dtype)
        lu = lora_up.contiguous()
        if out_dtype == torch.bfloat16:
            lu16 = _lora_up_f16(lu)
    wc = None if wcscales is None else wcscales.to(out_dtype).contiguous()
    b = None if bias is None else bias.to(out_dtype).contiguous()
    if _columns is not None:
        import ctypes
        y_full, peer_ptrs, col0 = _columns
        assert y_full.is_cuda and y_full.is_contiguous() and y_full.dtype == out_dtype and y_full.shape[0] == M
        n_total = y_full.shape[1]
        assert 0 <= col0 and col0 + N <= n_total and col0 % 64 == 0 and len(peer_ptrs) <= 7
        arr = (ctypes.c_void_p * max(1, len(peer_ptrs)))(*peer_ptrs)
        with _on_device(dev):
            rc = lib.svdq_gemm_w4a4_columns(_ptr(a), _ptr(w), _ptr(sa), _ptr(sw), _ptr(la), _ptr(lu), _ptr(lu16), _ptr(wc),
                                            _ptr(b), _ptr(y_full), arr, len(peer_ptrs), n_total, col0, M, N, K, R,
                                            _DT[out_dtype], variant | sched, _stream(dev))
        _lib.check(rc, "gemm_w4a4_columns")
        return y_full
    if out is not None:
        assert out.shape == (M, N) and out.dtype == out_dtype and out.is_contiguous() and out.device == dev
        y = out
    else:
        y = torch.empty((M, N), dtype=out_dtype, device=dev)
    if smooth_next is not None:
        assert smooth_next.is_cuda and smooth_next.shape == (N,), f"smooth_next must be [N]; got {tuple(smooth_next.shape)}"
        assert _splits is None or _splits == 1
        sn = smooth_next.to(out_dtype).contiguous()
        qout = torch.empty((M, N // 2), dtype=torch.uint8, device=dev)
        oscales = torch.empty((N // 16, M), dtype=torch.float8_e4m3fn, device=dev)
        oswz = torch.empty(M * (N // 16), dtype=torch.uint8, device=dev) if N % 64 == 0 else None
        with _on_device(dev):
            rc = lib.svdq_gemm_w4a4_next(_ptr(a), _ptr(w), _ptr(sa), _ptr(sw), _ptr(la), _ptr(lu), _ptr(lu16), _ptr(wc), _ptr(b),
                                         _ptr(y), _ptr(sn), _ptr(qout), _ptr(oscales), _ptr(oswz), M, N, K, R,
                                         _DT[out_dtype], variant | sched, _stream(dev))
        _lib.check(rc, "gemm_w4a4_next")
        if oswz is not None:
            _attach(oscales, oswz)
        return y, qout, oscales
    ws = None
    if _splits is not None and _splits > 1:
        variant = 10000 * _splits + 128
        ws = _split_workspace(dev, 1024 + (M // 128) * (N // 128) * _splits * 65536)
    elif variant == 0 and _splits is None:
        need = int(lib.svdq_gemm_w4a4_workspace_bytes(M, N, K, R))
        if need > 0:
            ws = _split_workspace(dev, need)
    with _on_device(dev):
        if ws is not None:
            rc = lib.svdq_gemm_w4a4_ws(_ptr(a), _ptr(w), _ptr(sa), _ptr(sw), _ptr(la), _ptr(lu), _ptr(lu16), _ptr(wc), _ptr(b),
                                       _ptr(y), M, N, K, R, _DT[out_dtype], variant | sched, _ptr(ws), ws.numel(), _stream(dev))
        else:
            rc = lib.svdq_gemm_w4a4(_ptr(a), _ptr(w), _ptr(sa), _ptr(sw), _ptr(la), _ptr(lu), _ptr(lu16), _ptr(wc), _ptr(b),
                                    _ptr(y), M, N, K, R, _DT[out_dtype], variant | sched, _stream(dev))
    _lib.check(rc, "gemm_w4a4")
    return y


_SPLIT_WS: dict = {}     # GEMM split-K workspaces
_QUANT_WS: dict = {}     # quantizer (streaming form) workspaces
_QUANT_WS_BYTES: dict = {}
_QUANT_WS_FORCED = 2048 + 8 * 8192 * 512     # room for any forced split of up to 8192 padded rows


def _workspace(table: dict, dev: torch.device, nbytes: int, head: int) -> torch.Tensor:
    """Workspace of the current stream of `dev` (its first `head` bytes are counters, zeroed when it is
    made; every completed call leaves them zero).  One per stream, because calls that share a
    workspace must not overlap."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream(dev))
    ws = table.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 10 << 20), dtype=torch.uint8, device=dev)
        ws[:head].zero_()                      # the counters; the partial sums need no initial value
        table[key] = ws
    return ws


def _split_workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    return _workspace(_SPLIT_WS, dev, nbytes, 1024)


def _quant_ws_bytes(M: int, K: int, R: int, M_pad: int) -> int:
    key = (M, K, R, M_pad)
    n = _QUANT_WS_BYTES.get(key)
    if n is None:
        n = _QUANT_WS_BYTES[key] = int(_lib.load().svdq_quantize_workspace_bytes(M, K, R, M_pad))
    return n


def reset_workspaces() -> None:
    """Forget the cached workspaces (new ones are made, with zeroed counters, on the next calls).  Call
    this after `_lib.device_status()` reported a failure: a kernel that gave up on a bounded wait may
    have left counters non-zero."""
    _SPLIT_WS.clear()
    _QUANT_WS.clear()


launch_v2 = gemm_w4a4   # the reference's name for the same entry point


class LinearPlan:
    """Host-buffer form of the whole linear (x on the host in, y on the host out).

    Weights are uploaded once; `forward_host` copies x to the device, runs the
    quantizer and the GEMM, copies y back and waits.  Thin wrapper over
    svdq_linear_plan_* of the C ABI.
    """

    def __init__(self, max_M: int, K: int, N: int, R: int, dtype: torch.dtype, *, wgt, wscales, lora_down=None,
                 lora_up=None, smooth=None, wcscales=None, bias=None, device: Optional[int] = None):
        import ctypes
        self._lib = _lib.load()
        self._handle = ctypes.c_void_p()
        self.max_M, self.K, self.N, self.R, self.dtype = max_M, K, N, R, dtype
        self.device = torch.cuda.current_device() if device is None else device

        def host(t):
            return None if t is None else t.detach().cpu().contiguous()

        keep = [host(t) for t in (wgt, wscales, lora_down, lora_up, smooth, wcscales, bias)]
        with torch.cuda.device(self.device):
            rc = self._lib.svdq_linear_plan_create(ctypes.byref(self._handle), max_M, K, N, R, _DT[dtype],
                                                   *[_ptr(t) for t in keep])
        _lib.check(rc, "linear_plan_create")

    def forward_host(self, x_host: torch.Tensor, y_host: torch.Tensor) -> torch.Tensor:
        assert not x_host.is_cuda and not y_host.is_cuda
        assert x_host.is_contiguous() and y_host.is_contiguous()
        M = x_host.shape[0]
        assert x_host.shape == (M, self.K) and y_host.shape == (M, self.N)
        assert x_host.dtype == self.dtype and y_host.dtype == self.dtype
        with torch.cuda.device(self.device):
            rc = self._lib.svdq_linear_plan_forward_host(self._handle, _ptr(x_host), _ptr(y_host), M)
        _lib.check(rc, "linear_plan_forward_host")
        return y_host

    def submit(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        """Queue one batch (x copy, kernels, y copy) and return; at most two are in flight.

        Keep both tensors alive and leave `y_host` unread until `wait()` (or the second-next
        `submit`) has returned."""
        assert not x_host.is_cuda and not y_host.is_cuda
        assert x_host.is_contiguous() and y_host.is_contiguous()
        M = x_host.shape[0]
        assert x_host.shape == (M, self.K) and y_host.shape == (M, self.N)
        assert x_host.dtype == self.dtype and y_host.dtype == self.dtype
        with torch.cuda.device(self.device):
            rc = self._lib.svdq_linear_plan_submit(self._handle, _ptr(x_host), _ptr(y_host), M)
        _lib.check(rc, "linear_plan_submit")

    def wait(self) -> None:
        """Return once every submitted batch has its y on the host."""
        with torch.cuda.device(self.device):
            rc = self._lib.svdq_linear_plan_wait(self._handle)
        _lib.check(rc, "linear_plan_wait")

    def close(self) -> None:
        if self._handle:
            self._lib.svdq_linear_plan_destroy(self._handle)
            self._handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass
