"""The C ABI without a GPU: the library loads, exports exactly what the header
declares, and rejects bad arguments before touching CUDA."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "svdq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(svdq_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_table_agree():
    from svdquant_kernels_b200 import _lib
    assert _declared_functions() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    for name in _declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/svdq_b200.h but not exported"


def test_status_strings(lib_path):
    from svdquant_kernels_b200 import _lib
    assert _lib.status_string(0) == "ok"
    assert "contract" in _lib.status_string(2)
    assert _lib.load().svdq_version() >= 100


def test_argument_validation_needs_no_device(lib_path):
    from svdquant_kernels_b200 import _lib
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p = (p + 15) & ~15
    # K not a multiple of 16
    assert lib.svdq_quantize_w4a4_act_fuse_lora(p, p, None, None, p, p, p, None, None, 4, 24, 0, 4, 0, 0, None) == 2
    # unsupported dtype
    assert lib.svdq_quantize_w4a4_act_fuse_lora(p, p, None, None, p, p, p, None, None, 4, 32, 0, 4, 2, 0, None) == 3
    # missing output
    assert lib.svdq_quantize_w4a4_act_fuse_lora(p, p, None, None, None, p, p, None, None, 4, 32, 0, 4, 0, 0, None) == 1
    # misaligned input
    assert lib.svdq_quantize_w4a4_act_fuse_lora(p + 2, p, None, None, p, p, p, None, None, 4, 32, 0, 4, 0, 0, None) == 4
    # empty problem is a no-op
    assert lib.svdq_quantize_w4a4_act_fuse_lora(None, None, None, None, None, None, None, None, None, 0, 32, 0, 0, 0, 0, None) == 0
    # GEMM contract
    assert lib.svdq_gemm_w4a4_supported(256, 128, 128, 16) == 1
    assert lib.svdq_gemm_w4a4_supported(4352, 15360, 3840, 128) == 1
    assert lib.svdq_gemm_w4a4_supported(100, 128, 128, 16) == 0
    assert lib.svdq_gemm_w4a4_supported(256, 128, 96, 16) == 0
    assert lib.svdq_gemm_w4a4_supported(256, 128, 128, 8) == 0
    assert lib.svdq_gemm_w4a4(p, p, p, p, None, None, None, None, None, p, 100, 128, 128, 0, 0, 0, None) == 2
    assert lib.svdq_gemm_w4a4(p, p, p, p, p, None, None, None, None, p, 128, 128, 128, 16, 0, 0, None) == 1
    assert lib.svdq_gemm_w4a4(p, p, p, p, None, None, None, None, None, p, 128, 128, 128, 0, 5, 0, None) == 3
    assert lib.svdq_swizzle_scales(p, p, 6, 128, None) == 2
    # sizes of the 16-bit lora_act form: one plane for fp16; three planes + a word per 32 rows for bf16
    assert lib.svdq_lora_act16_elems(256, 32, 0) == 256 * 32
    assert lib.svdq_lora_act16_elems(256, 32, 1) == 3 * 256 * 32 + 2 * 8
    assert lib.svdq_lora_act16_elems(-1, 32, 1) == -1
    # host-side bf16 -> fp16 copy of lora_up: exact for ordinary values, refused beyond fp16's range
    import numpy as np
    src = np.array([0x3F80, 0xBC00, 0x0000, 0x4000], dtype=np.uint16)          # 1.0, -0.0078125, 0, 2.0 as bf16
    dst = np.zeros(4, dtype=np.float16)
    assert lib.svdq_lora_up_to_f16(src.ctypes.data, dst.ctypes.data, 4) == 0
    assert dst.tolist() == [1.0, -0.0078125, 0.0, 2.0]
    big = np.array([0x4800], dtype=np.uint16)                                   # 131072 as bf16
    assert lib.svdq_lora_up_to_f16(big.ctypes.data, dst.ctypes.data, 1) == 7
    # split-K workspace: only for few tiles and a long K; ticket block + tiles x splits partial tiles of 64 KB
    assert lib.svdq_gemm_w4a4_workspace_bytes(256, 3072, 10240, 32) == 1024 + 48 * 3 * 65536
    assert lib.svdq_gemm_w4a4_workspace_bytes(256, 3840, 15360, 128) == 1024 + 60 * 2 * 65536
    assert lib.svdq_gemm_w4a4_workspace_bytes(256, 3072, 3840, 128) == 0          # K too short to repay the split
    assert lib.svdq_gemm_w4a4_workspace_bytes(4352, 3072, 10240, 32) == 0         # plenty of tiles
    assert lib.svdq_gemm_w4a4_workspace_bytes(100, 3072, 10240, 32) == 0          # not a supported shape
    # the workspace forms check their arguments like the plain call, before anything is launched
    assert lib.svdq_gemm_w4a4_ws(p, p, p, p, None, None, None, None, None, p, 100, 128, 128, 0, 0, 0, p, 4096, None) == 2
    assert lib.svdq_gemm_w4a4_ws(p, p, p, p, None, None, None, None, None, p, 128, 128, 128, 0, 0, 0, p + 4, 4096, None) == 4
    assert lib.svdq_gemm_w4a4_static_ws(p, p, p, p, None, None, None, None, None, p, 100, 128, 128, 0, 0, 0, None) == 2
    assert lib.svdq_gemm_w4a4_static_ws(p, p, p, p, None, None, None, None, None, p, 256, 3072, 10240, 0, 0, 40128, None) == 7


def test_operator_asserts_mirror_the_reference(lib_path):
    """Contract violations raise AssertionError / NotImplementedError like the reference's host code."""
    import torch
    from svdquant_kernels_b200 import ops
    x = torch.zeros(4, 32, dtype=torch.float16)
    with pytest.raises(AssertionError):
        ops.quantize_w4a4_act_fuse_lora(x, torch.zeros(32, 16, dtype=torch.float16), None)   # not on CUDA
    with pytest.raises(AssertionError):
        ops.gemm_w4a4(torch.zeros(128, 64, dtype=torch.uint8), torch.zeros(128, 64, dtype=torch.uint8),
                      torch.zeros(8, 128), torch.zeros(8, 128))


def test_header_is_plain_c_and_links(lib_path, tmp_path):
    """include/svdq_b200.h must compile as C99 (it is the contract for cgo / JNI / FFI bindings) and a C
    program must link against the library and call it without Python or PyTorch in the picture."""
    import os
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler here")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "use_abi.c"
    src.write_text(
        '#include <string.h>\n#include "svdq_b200.h"\n'
        "int main(void) {\n"
        "  if (svdq_version() < 100) return 1;\n"
        '  if (strcmp(svdq_status_string(SVDQ_OK), "ok") != 0) return 2;\n'
        "  if (svdq_gemm_w4a4_supported(256, 128, 128, 16) != 1) return 3;\n"
        "  if (svdq_lora_act16_elems(256, 32, SVDQ_DTYPE_BF16) != 3 * 256 * 32 + 16) return 4;\n"
        "  return 0;\n}\n")
    exe = tmp_path / "use_abi"
    libdir = os.path.dirname(lib_path)
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(root, "include"),
                    str(src), "-o", str(exe), "-L", libdir, "-l:" + os.path.basename(lib_path),
                    "-Wl,-rpath," + libdir], check=True)
    assert subprocess.run([str(exe)]).returncode == 0
