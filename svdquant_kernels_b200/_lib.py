"""ctypes binding of libsvdq_b200.so (the C ABI in include/svdq_b200.h).

The library is built in-tree by `svdquant_kernels_b200.build`.  There is no
fallback: if the shared object is missing or a symbol cannot be resolved the
import of the operators fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_longlong, c_ulonglong, c_void_p, POINTER, c_float, c_uint

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libsvdq_b200.so")

DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 0, 1, 2
QUANT_AUTO, QUANT_FORCE_GENERIC, QUANT_FORCE_FUSED, QUANT_FORCE_STREAM = 0, 1, 2, 0x100000
OK = 0
GEMM_LORA_INTERLEAVE, GEMM_LORA_AT_END = 1 << 24, 1 << 25

# name -> (restype, argtypes); kept in the order of include/svdq_b200.h
SIGNATURES = {
    "svdq_status_string": (c_char_p, [c_int]),
    "svdq_version": (c_int, []),
    "svdq_prepare_smooth": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "svdq_quantize_w4a4_act_fuse_lora": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "svdq_quantize_workspace_bytes": (c_ulonglong, [c_int, c_int, c_int, c_int]),
    "svdq_quantize_w4a4_act_fuse_lora_ws": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                    c_ulonglong, c_void_p]),
    "svdq_quantizer_max_active_clusters": (c_int, [c_int, c_int, c_int]),
    "svdq_quantize_nvfp4_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "svdq_swizzle_scales": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "svdq_lora_act16_elems": (c_longlong, [c_int, c_int, c_int]),
    "svdq_cast_lora_act": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "svdq_lora_up_to_f16": (c_int, [c_void_p, c_void_p, c_longlong]),
    "svdq_gemm_w4a4": (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_void_p]),
    "svdq_gemm_w4a4_next": (c_int, [c_void_p] * 14 + [c_int] * 6 + [c_void_p]),
    "svdq_gemm_w4a4_workspace_bytes": (c_ulonglong, [c_int, c_int, c_int, c_int]),
    "svdq_gemm_w4a4_ws": (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_void_p, c_ulonglong, c_void_p]),
    "svdq_gemm_w4a4_static_ws": (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_void_p]),
    "svdq_gemm_w4a4_columns": (c_int, [c_void_p] * 10 + [POINTER(c_void_p)] + [c_int] * 9 + [c_void_p]),
    "svdq_gemm_w4a4_supported": (c_int, [c_int, c_int, c_int, c_int]),
    "svdq_device_status": (c_int, [POINTER(c_uint)]),
    "svdq_selftest_wait_expiry": (c_int, [c_ulonglong, c_void_p, c_void_p]),
    "svdq_selftest_divide": (c_int, [c_void_p, c_void_p]),
    "svdq_linear_plan_create": (c_int, [POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int] + [c_void_p] * 7),
    "svdq_linear_plan_forward_host": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "svdq_linear_plan_submit": (c_int, [c_void_p, c_void_p, c_void_p, c_int]),
    "svdq_linear_plan_wait": (c_int, [c_void_p]),
    "svdq_linear_plan_destroy": (None, [c_void_p]),
}

_lib = None


class SvdqLibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load (once) and type the shared library; raise if it is not there."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise SvdqLibraryError(
            f"{LIB_PATH} is missing. Build it with `python -m svdquant_kernels_b200.build` "
            "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # pragma: no cover - stale build
            raise SvdqLibraryError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_string(code: int) -> str:
    return load().svdq_status_string(code).decode()


def check(code: int, what: str) -> None:
    if code != OK:
        raise RuntimeError(f"{what}: svdq status {code} ({status_string(code)})")


def device_status() -> tuple[int, list[int]]:
    """(status, [code, block, tag, count]) — synchronises the device."""
    buf = (c_uint * 4)()
    rc = load().svdq_device_status(buf)
    return rc, list(buf)
