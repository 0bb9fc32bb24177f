"""Seeded synthetic W4A4-linear workloads (shapes and value distributions of
the five benchmark configurations).

No dataset is involved anywhere on this path: the reference draws its smoke
and bench inputs from a CPU generator as well
(baseline/kernels/gemm_w4a4/harness.py:42-84), so that every machine sees the
same bits.  These generators follow the same idea with the distributions the
benchmark configurations name: Gaussian activations with a few outlier
channels scaled x20, smooth = sqrt(column amax) clamped at 1e-2, weights
N(0, 0.02) divided by smooth, LoRA factors N(0, 1/sqrt(K)) and N(0, 0.01),
bias N(0, 0.01), per-channel scales 1 or U(0.5, 1.5).

Everything is drawn in fp32 on the CPU and cast once; weights are returned
unquantised (fp32) so that the caller chooses the packer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class LinearShape:
    name: str
    M: int
    K: int
    N: int
    R: int
    dtype: torch.dtype
    act: str = "gauss"          # "gauss" | "gelu"
    outlier_cols: int = 4
    unit_wcscales: bool = False


CONFIGS: dict[str, LinearShape] = {
    "c0": LinearShape("c0", 64, 128, 128, 16, torch.float16, unit_wcscales=True),
    "c1": LinearShape("c1", 4352, 3840, 3072, 128, torch.float16),
    "c2": LinearShape("c2", 4352, 3840, 15360, 128, torch.bfloat16),   # 0.1 % of K = 4 outlier columns
    "c3": LinearShape("c3", 4352, 15360, 3840, 128, torch.bfloat16, act="gelu"),
    "c4": LinearShape("c4", 4352, 10240, 3072, 32, torch.float16),
}
# A few hundred rows (the small-M shapes of the reference's GEMM_SHAPES, cute_kernels/gemm_w4a4/harness.py:17-24,
# and their long-K relatives): not benchmark configurations, but `bench.py --config s0..s2` times them too.
SMALL_M: dict[str, LinearShape] = {
    "s0": LinearShape("s0", 256, 3840, 3072, 128, torch.float16),
    "s1": LinearShape("s1", 256, 10240, 3072, 32, torch.float16),
    "s2": LinearShape("s2", 256, 15360, 3840, 128, torch.bfloat16, act="gelu"),
}
_SEED_BASE = 1234


@dataclass
class LinearInputs:
    shape: LinearShape
    x: torch.Tensor              # [M, K]  16-bit
    smooth: torch.Tensor         # [K]     16-bit
    w: torch.Tensor              # [N, K]  fp32, already divided by smooth; quantise with pad_size=1
    lora_down: torch.Tensor      # [K, R]  16-bit
    lora_up: torch.Tensor        # [N, R]  16-bit
    wcscales: torch.Tensor       # [N]     16-bit
    bias: torch.Tensor           # [N]     16-bit


def make_inputs(shape: LinearShape, *, seed: Optional[int] = None, m_rows: Optional[int] = None,
                row_offset: int = 0) -> LinearInputs:
    """Draw one configuration on the CPU.

    `m_rows` / `row_offset` select a slab of a taller activation matrix (used
    when the rows are sharded over several GPUs: every rank draws the same
    weights and its own rows).
    """
    idx = list(CONFIGS).index(shape.name) if shape.name in CONFIGS else 99
    base = _SEED_BASE + idx if seed is None else seed
    M = shape.M if m_rows is None else m_rows
    K, N, R = shape.K, shape.N, shape.R

    def gen(offset: int) -> torch.Generator:
        return torch.Generator().manual_seed(base * 1000 + offset)

    x = torch.randn(M, K, generator=gen(10 + row_offset), dtype=torch.float32)
    if shape.act == "gelu":
        x = torch.nn.functional.gelu(x)
    cols = torch.randperm(K, generator=gen(1))[: shape.outlier_cols]
    x[:, cols] *= 20.0
    # smooth comes from a fixed calibration slab so that it does not depend on the shard
    calib = torch.randn(256, K, generator=gen(2), dtype=torch.float32)
    if shape.act == "gelu":
        calib = torch.nn.functional.gelu(calib)
    calib[:, cols] *= 20.0
    smooth = calib.abs().amax(0).pow(0.5).clamp_min(1e-2)
    w = torch.randn(N, K, generator=gen(3), dtype=torch.float32) * 0.02
    w = w / smooth[None, :]
    lora_down = torch.randn(K, R, generator=gen(4), dtype=torch.float32) / (K ** 0.5)
    lora_up = torch.randn(N, R, generator=gen(5), dtype=torch.float32) * 0.01
    bias = torch.randn(N, generator=gen(6), dtype=torch.float32) * 0.01
    if shape.unit_wcscales:
        wc = torch.ones(N, dtype=torch.float32)
    else:
        wc = torch.rand(N, generator=gen(7), dtype=torch.float32) + 0.5
    dt = shape.dtype
    return LinearInputs(shape, x.to(dt), smooth.to(dt), w, lora_down.to(dt), lora_up.to(dt), wc.to(dt), bias.to(dt))


def quantizer_bytes(M: int, K: int, R: int, pad: int = 256) -> int:
    """Algorithmic HBM bytes of one quantizer pass: read x, lora_down, smooth;
    write codes, scales, lora_act."""
    M_pad = -(-M // pad) * pad
    return M * K * 2 + K * R * 2 + K * 2 + M_pad * K // 2 + M_pad * K // 16 + M_pad * R * 4


def gemm_flops(M: int, N: int, K: int) -> int:
    """Algorithmic FLOPs of the main product (the LoRA product is reported apart)."""
    return 2 * M * N * K
