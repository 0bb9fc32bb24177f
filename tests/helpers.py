"""Shared helpers of the GPU parity tests: torch <-> oracle conversions."""
import numpy as np
import torch

from oracle import nvfp4_oracle as O

DT_NAME = {torch.float16: "fp16", torch.bfloat16: "bf16"}
NAME_DT = {"fp16": torch.float16, "bf16": torch.bfloat16}


def bits(t: torch.Tensor) -> np.ndarray:
    """16-bit torch tensor (any device) -> uint16 bit patterns."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bits(a: np.ndarray, dtype: torch.dtype, device="cuda") -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(dtype).to(device)


def u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def oracle_quantize(x, lora_down, smooth, pad_size=256):
    name = DT_NAME[x.dtype]
    return O.quantize_w4a4_act_fuse_lora(bits(x), bits(lora_down), None if smooth is None else bits(smooth), name, pad_size)


def oracle_gemm(act, wgt, ascales, wscales, lora_act, lora_up, wc, bias, dtype):
    name = DT_NAME[dtype]
    y_bits, y32, _, _ = O.gemm_w4a4(act, wgt, ascales, wscales, lora_act, None if lora_up is None else bits(lora_up),
                                    None if wc is None else bits(wc), None if bias is None else bits(bias), name)
    return y_bits, y32


def rel_l2_vs_bits(y: torch.Tensor, y_bits: np.ndarray) -> float:
    name = DT_NAME[y.dtype]
    return O.rel_l2(O.bits_to_f32(bits(y), name), O.bits_to_f32(y_bits, name))


def assert_device_clean():
    from svdquant_kernels_b200 import _lib
    rc, words = _lib.device_status()
    assert rc == 0, f"device status {words}: a kernel gave up on a bounded wait"
