"""torch.library registration of the two operators, for callers that want dispatcher-visible ops
(`torch.ops.svdq_b200.*`): tracing / torch.compile graphs, CUDA-graph capture through the dispatcher,
serving stacks that resolve kernels by qualified name.

The reference registers nothing on CUDA and keeps its pod-side registration as a pattern only
(csrc/python/svdquant_w4a4_op.cpp:127-136, docs/architecture.md:18-22); the schemas below follow its
Python signatures (triton_kernels/quantize_w4a4_act_fuse_lora/kernel.py:289-400,
cute_kernels/gemm_w4a4/kernel_v2_fa4.py:113-225).

The layout twins `ops` makes next to its outputs (tensor-core scale order, 16-bit lora_act) are
recorded on the outputs' storage objects, which the dispatcher hands through unchanged, so a
`torch.ops.svdq_b200.gemm_w4a4` call on the quantizer op's outputs finds them and runs the same
kernels as the plain Python path; both ops can be captured in a CUDA graph.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops

__all__ = ["quantize_w4a4_act_fuse_lora", "gemm_w4a4"]


@torch.library.custom_op("svdq_b200::quantize_w4a4_act_fuse_lora", mutates_args=(), device_types="cuda")
def quantize_w4a4_act_fuse_lora(input: torch.Tensor, lora_down: torch.Tensor, smooth: Optional[torch.Tensor] = None,
                                pad_size: int = 256) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    act, ascales, lora_act = ops.quantize_w4a4_act_fuse_lora(input, lora_down, smooth, fp4=True, pad_size=pad_size)
    return act, ascales, lora_act


@quantize_w4a4_act_fuse_lora.register_fake
def _(input, lora_down, smooth=None, pad_size=256):
    M, K = input.shape
    R = lora_down.shape[1]
    torch._check(K % 16 == 0, lambda: "NVFP4 group size is 16; K must be divisible by 16")
    M_pad = (M + pad_size - 1) // pad_size * pad_size
    return (input.new_empty((M_pad, K // 2), dtype=torch.uint8),
            input.new_empty((K // 16, M_pad), dtype=torch.float8_e4m3fn),
            input.new_empty((M_pad, R), dtype=torch.float32))


@torch.library.custom_op("svdq_b200::gemm_w4a4", mutates_args=(), device_types="cuda")
def gemm_w4a4(act: torch.Tensor, wgt: torch.Tensor, ascales: torch.Tensor, wscales: torch.Tensor,
              lora_act_in: Optional[torch.Tensor] = None, lora_up: Optional[torch.Tensor] = None,
              wcscales: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
              out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    return ops.gemm_w4a4(act, wgt, ascales, wscales, lora_act_in, lora_up, wcscales, bias, out_dtype)


@gemm_w4a4.register_fake
def _(act, wgt, ascales, wscales, lora_act_in=None, lora_up=None, wcscales=None, bias=None, out_dtype=None):
    if out_dtype is None:
        out_dtype = lora_up.dtype if lora_up is not None else torch.float16
    return act.new_empty((act.shape[0], wgt.shape[0]), dtype=out_dtype)
