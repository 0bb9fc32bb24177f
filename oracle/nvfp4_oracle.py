"""CPU oracle for the SVDQuant W4A4 linear (NVFP4) — TEST INFRASTRUCTURE ONLY.

This module is a numpy restatement of the reference's PyTorch ground truth
for the two-op hot path.  It exists to check the CUDA kernels; nothing in the
shipped package may import it.  Only the test suite, the smoke entry and the
CPU-baseline / reference arms of the benchmark are allowed to call it.

Parity is pinned: every function here is compared bit-for-bit (codes, scales)
or to fp32 round-off (matmul outputs) against fixtures that were produced by
executing the reference's own modules (see tests/golden/make_golden.py), and
against the reference itself whenever its checkout is importable.

What each function follows in the reference project:

  e4m3 encode/decode      torch.float8_e4m3fn casts used at
                          baseline/kernels/_nvfp4.py:84-85 (round-to-nearest-even,
                          subnormals kept, inputs pre-clamped to [1e-12, 448])
  e2m1_codes              baseline/kernels/_nvfp4.py:27-41  (_quantize_e2m1)
  pack/unpack nibbles     baseline/kernels/_nvfp4.py:44-57
  quantize_nvfp4_rows     baseline/kernels/_nvfp4.py:60-95
  dequantize_nvfp4_rows   baseline/kernels/_nvfp4.py:98-114
  quantize_w4a4_act_fuse_lora
                          baseline/kernels/quantize_w4a4_act_fuse_lora/ref.py:19-50
  gemm_w4a4               baseline/kernels/gemm_w4a4/ref.py:33-78 (the optional
                          next-layer quantize at :80-87 is also restated)
  swizzle_scales          cute_kernels/gemm_w4a4/kernel.py:194-225
                          (_repack_scales_cutlass_atom; the 128x4 scale atom)

Conventions: 16-bit tensors travel as numpy uint16 bit patterns together with
a dtype tag ("fp16" | "bf16"); fp8 scales travel as uint8 bit patterns.
"""
from __future__ import annotations

import numpy as np

FP4_MAX = np.float32(6.0)
E4M3_MAX = np.float32(448.0)
GROUP = 16

# ---------------------------------------------------------------------------
# 16-bit helpers
# ---------------------------------------------------------------------------

def bits_to_f32(bits: np.ndarray, dtype: str) -> np.ndarray:
    """uint16 bit patterns of fp16 / bf16 values -> float32 (exact)."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    if dtype == "fp16":
        return bits.view(np.float16).astype(np.float32)
    if dtype == "bf16":
        return (bits.astype(np.uint32) << 16).view(np.float32)
    raise ValueError(f"dtype must be 'fp16' or 'bf16', got {dtype!r}")


def f32_to_bits(x: np.ndarray, dtype: str) -> np.ndarray:
    """float32 -> uint16 bit patterns, round-to-nearest-even (what a torch
    `.to(float16/bfloat16)` does, baseline/kernels/gemm_w4a4/ref.py:77-78)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == "fp16":
        with np.errstate(over="ignore"):
            return x.astype(np.float16).view(np.uint16)
    if dtype == "bf16":
        u = x.view(np.uint32)
        nan = np.isnan(x)
        lsb = (u >> 16) & np.uint32(1)
        r = ((u + np.uint32(0x7FFF) + lsb) >> 16).astype(np.uint16)
        r[nan] = np.uint16(0x7FC0)
        return r
    raise ValueError(f"dtype must be 'fp16' or 'bf16', got {dtype!r}")


# ---------------------------------------------------------------------------
# FP8 E4M3 (the "fn" flavour: no inf, max 448)
# ---------------------------------------------------------------------------

def _e4m3_positive_table() -> np.ndarray:
    vals = np.empty(127, dtype=np.float32)
    for code in range(127):
        e, m = code >> 3, code & 7
        vals[code] = (m / 8.0) * 2.0 ** -6 if e == 0 else (1.0 + m / 8.0) * 2.0 ** (e - 7)
    return vals


_E4M3_POS = _e4m3_positive_table()                      # codes 0x00..0x7E, ascending
_E4M3_MID = ((_E4M3_POS[:-1].astype(np.float64) + _E4M3_POS[1:].astype(np.float64)) / 2.0)
_E4M3_DECODE = np.concatenate([_E4M3_POS, [np.float32(np.nan)], -_E4M3_POS, [np.float32(np.nan)]]).astype(np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 in [0, 448] -> e4m3fn bit pattern (uint8), nearest, ties to the
    even code.  Matches the torch cast the reference applies to the clamped
    scale (baseline/kernels/_nvfp4.py:83-84)."""
    x = np.asarray(x, dtype=np.float32)
    if x.size and (np.any(x < 0) or np.any(x > E4M3_MAX) or np.any(np.isnan(x))):
        raise ValueError("e4m3_encode expects values pre-clamped to [0, 448]")
    xd = x.astype(np.float64)
    below = np.searchsorted(_E4M3_MID, xd, side="left")          # mids strictly below x
    upto = np.searchsorted(_E4M3_MID, xd, side="right")          # mids <= x
    code = below.astype(np.int64)
    tie = upto != below                                          # x sits exactly on a midpoint
    # on a tie the candidates are codes `below` and `below+1`; keep the even one
    code = np.where(tie & ((code & 1) == 1), code + 1, code)
    return code.astype(np.uint8)


def e4m3_decode(bits: np.ndarray) -> np.ndarray:
    return _E4M3_DECODE[np.asarray(bits, dtype=np.uint8)]


# ---------------------------------------------------------------------------
# E2M1 codes and nibble packing
# ---------------------------------------------------------------------------

_E2M1_BOUNDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
_E2M1_LEVELS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def e2m1_codes(v: np.ndarray) -> np.ndarray:
    """fp32 -> 4-bit code.  Magnitude = how many of the seven bounds are <= |v|
    (so a value exactly on a bound rounds AWAY from zero), |v| saturates at 6,
    bit 3 = (v < 0).  NaN compares false everywhere -> code 0.  +-inf -> 7|sign.
    Follows baseline/kernels/_nvfp4.py:27-41."""
    v = np.asarray(v, dtype=np.float32)
    with np.errstate(invalid="ignore"):
        mag = np.minimum(np.abs(v), FP4_MAX)
        idx = np.zeros(v.shape, dtype=np.uint8)
        for b in _E2M1_BOUNDS:
            idx += (mag >= b)
        sign = (v < 0).astype(np.uint8) << 3
    return idx | sign


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """[..., K] codes -> [..., K/2] bytes; even k in the low nibble."""
    assert codes.shape[-1] % 2 == 0
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0x0F
    out[..., 1::2] = packed >> 4
    return out


# ---------------------------------------------------------------------------
# Row quantiser / dequantiser
# ---------------------------------------------------------------------------

def quantize_nvfp4_rows(x: np.ndarray, pad_size: int = 1):
    """fp32 [rows, K] -> (packed u8 [rows_pad, K/2], scales u8(e4m3) [K/16, rows_pad]).

    scale = e4m3( clamp(amax16 / 6, 1e-12, 448) ); codes = e2m1( x / float(scale) ).
    Rows added by padding are all-zero inputs: scale byte 0x00, and 0/0 = NaN
    encodes as code 0, so those rows are 0x00 throughout.
    """
    x = np.asarray(x, dtype=np.float32)
    assert x.ndim == 2
    rows, K = x.shape
    assert K % GROUP == 0, "NVFP4 group size is 16"
    rows_pad = -(-rows // pad_size) * pad_size
    xp = np.zeros((rows_pad, K), dtype=np.float32)
    xp[:rows] = x
    blk = xp.reshape(rows_pad, K // GROUP, GROUP)
    amax = np.abs(blk).max(axis=-1)
    s = np.clip(amax / FP4_MAX, np.float32(1e-12), E4M3_MAX).astype(np.float32)
    s_bits = e4m3_encode(s)
    s_back = e4m3_decode(s_bits)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = blk / s_back[..., None]
    codes = e2m1_codes(q).reshape(rows_pad, K)
    return pack_nibbles(codes), np.ascontiguousarray(s_bits.T)


def dequantize_nvfp4_rows(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    rows, k2 = packed.shape
    K = 2 * k2
    assert scales.shape == (K // GROUP, rows)
    codes = unpack_nibbles(packed)
    vals = _E2M1_LEVELS[codes & 7] * (1.0 - 2.0 * ((codes >> 3) & 1).astype(np.float32))
    s = e4m3_decode(scales).T                                   # [rows, K/16]
    return (vals.reshape(rows, K // GROUP, GROUP) * s[..., None]).reshape(rows, K).astype(np.float32)


# ---------------------------------------------------------------------------
# The two operators
# ---------------------------------------------------------------------------

def quantize_w4a4_act_fuse_lora(x_bits, lora_down_bits, smooth_bits, dtype: str, pad_size: int = 256):
    """Returns (act u8 [M_pad,K/2], ascales u8 [K/16,M_pad], lora_act f32 [M_pad,R]).

    LoRA-down takes the RAW activations; only the quantised branch sees
    x / smooth (baseline/kernels/quantize_w4a4_act_fuse_lora/ref.py:36-48).
    """
    x = bits_to_f32(x_bits, dtype)
    ld = bits_to_f32(lora_down_bits, dtype)
    M, K = x.shape
    assert ld.shape[0] == K
    R = ld.shape[1]
    M_pad = -(-M // pad_size) * pad_size
    lora = np.zeros((M_pad, R), dtype=np.float32)
    if R:
        lora[:M] = x @ ld
    xs = x if smooth_bits is None else x / bits_to_f32(smooth_bits, dtype)[None, :]
    act, ascales = quantize_nvfp4_rows(xs, pad_size=pad_size)
    return act, ascales, lora


def gemm_w4a4(act, wgt, ascales, wscales, lora_act_in, lora_up_bits, wcscales_bits, bias_bits,
              dtype: str, smooth_next_bits=None):
    """y = cast( ((deq(act) @ deq(wgt)^T) + lora_act_in @ lora_up^T) * wcscales + bias ).

    LoRA is added BEFORE the per-column affine (baseline/kernels/gemm_w4a4/ref.py:64-75).
    Returns (y_bits u16 [M_pad,N], y_f32, qout, oscales); the last two are None
    unless `smooth_next_bits` is given (ref.py:80-87).
    """
    a = dequantize_nvfp4_rows(act, ascales)
    w = dequantize_nvfp4_rows(wgt, wscales)
    y = a @ w.T
    if lora_act_in is not None:
        lu = bits_to_f32(lora_up_bits, dtype)
        y = y + np.asarray(lora_act_in, dtype=np.float32) @ lu.T
    if wcscales_bits is not None:
        y = y * bits_to_f32(wcscales_bits, dtype)[None, :]
    if bias_bits is not None:
        y = y + bits_to_f32(bias_bits, dtype)[None, :]
    y = y.astype(np.float32)
    qout = oscales = None
    if smooth_next_bits is not None:
        qout, oscales = quantize_nvfp4_rows(y / bits_to_f32(smooth_next_bits, dtype)[None, :], pad_size=1)
    return f32_to_bits(y, dtype), y, qout, oscales


# ---------------------------------------------------------------------------
# Scale-factor atom layout consumed by the tensor core
# ---------------------------------------------------------------------------

def swizzle_scales(scales: np.ndarray) -> np.ndarray:
    """[K/16, rows] canonical -> flat bytes in the 128-row x 4-group atom order.

    Byte address of (row m, group g):
        ((m // 128) * (G // 4) + g // 4) * 512 + (m % 32) * 16 + ((m // 32) % 4) * 4 + g % 4
    """
    G, rows = scales.shape
    assert rows % 128 == 0 and G % 4 == 0
    t = np.ascontiguousarray(scales.T).reshape(rows // 128, 4, 32, G // 4, 4)
    return np.ascontiguousarray(t.transpose(0, 3, 2, 1, 4)).reshape(-1)


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))
