"""Generates tests/golden/*.npz by EXECUTING the reference's own PyTorch code.

Run in a checkout that has the reference mounted:

    python tests/golden/make_golden.py /path/to/reference

Every fixture stores the exact input bits and what the reference returned:
  quantize_w4a4_act_fuse_lora_ref  (baseline/kernels/quantize_w4a4_act_fuse_lora/ref.py:19)
  quantize_nvfp4_rows / dequantize (baseline/kernels/_nvfp4.py:60, :98)
  gemm_w4a4_ref                    (baseline/kernels/gemm_w4a4/ref.py:33)
  _repack_scales_cutlass_atom      (cute_kernels/gemm_w4a4/kernel.py:194, restated as the
                                    same transpose/reshape/permute on the CPU tensor)
The fixtures are small (tens of KB) and are what pins the oracle under oracle/.
"""
import os
import sys

import numpy as np
import torch


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def u8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy().copy()


def build_case(name, M, K, N, R, dtype, seed, with_smooth=True, edge=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    cols = torch.randperm(K, generator=g)[:4]
    x[:, cols] *= 20.0
    if edge:
        # exact rounding ties, saturating values, an all-zero group, a tiny group whose
        # scale underflows to 0x00 (non-zero elements then saturate), signed zeros
        x[0, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0,
                                  -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
        x[1, 16:32] = 0.0
        x[2, 32:48] = 1e-4
        x[2, 33] = -1e-4
        x[2, 34] = 0.0
        x[3, 48:64] = 0.0
        x[3, 49] = -0.0
        x[4, :16] = 3e-3          # scale lands in the e4m3 subnormal range
        x[5, :16] = 440.0 * 6     # scale clamps near 448
        x[6, :16] = 1e4
    x = x.to(dtype)
    smooth = None
    if with_smooth:
        smooth = x.float().abs().amax(0).pow(0.5).clamp_min(1e-2).to(dtype)
        if edge:
            smooth[:64] = 1.0
            smooth = smooth.to(dtype)
    w = torch.randn(N, K, generator=g) * 0.02
    if smooth is not None:
        w = w / smooth.float()[None, :]
    lora_down = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype)
    lora_up = (torch.randn(N, R, generator=g) * 0.01).to(dtype)
    bias = (torch.randn(N, generator=g) * 0.01).to(dtype)
    wc = (torch.rand(N, generator=g) + 0.5).to(dtype)

    act, ascales, lora_act = quantize_w4a4_act_fuse_lora_ref(x, lora_down, smooth)
    wgt, wscales = quantize_nvfp4_rows(w, pad_size=1)
    y, _, _ = gemm_w4a4_ref(act, wgt, ascales, wscales, lora_act, lora_up, bias=bias, wcscales=wc)
    y_plain, _, _ = gemm_w4a4_ref(act, wgt, ascales, wscales, lora_act, lora_up)
    deq = dequantize_nvfp4_rows(act, ascales)
    out = dict(
        M=M, K=K, N=N, R=R, dtype="fp16" if dtype == torch.float16 else "bf16",
        x=bits16(x), lora_down=bits16(lora_down), lora_up=bits16(lora_up), bias=bits16(bias), wcscales=bits16(wc),
        w=w.numpy().copy(),
        act=u8(act), ascales=u8(ascales), lora_act=lora_act.numpy().copy(),
        wgt=u8(wgt), wscales=u8(wscales),
        y=bits16(y), y_plain=bits16(y_plain),
    )
    if M * K <= 8192:
        out["act_dequant"] = deq.numpy().copy()
    if smooth is not None:
        out["smooth"] = bits16(smooth)
    M_pad = act.shape[0]
    if M_pad % 128 == 0 and (K // 16) % 4 == 0:
        mk = ascales.view(torch.uint8).T.contiguous().reshape(M_pad // 128, 4, 32, K // 64, 4)
        out["ascales_atom"] = mk.permute(0, 3, 2, 1, 4).contiguous().reshape(-1).numpy().copy()
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), name + ".npz"), **out)
    print(name, "written; act bytes", act.numel())


def build_next_case(name, M, K, N, R, dtype, seed, exact):
    """gemm_w4a4_ref with smooth_next: the next layer's NVFP4 codes and scales of the fp32 result
    (baseline/kernels/gemm_w4a4/ref.py:80-87).  exact=True zeroes lora_up, so that y is a sum of
    fp4 x fp4 products with e4m3 scales that fp32 adds without rounding in any order at this size:
    such a fixture pins codes and scales bit for bit whatever the summation order of the matmul."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[:4]] *= 20.0
    x = x.to(dtype)
    smooth = x.float().abs().amax(0).pow(0.5).clamp_min(1e-2).to(dtype)
    w = torch.randn(N, K, generator=g) * 0.02 / smooth.float()[None, :]
    lora_down = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype)
    lora_up = (torch.randn(N, R, generator=g) * 0.01).to(dtype)
    if exact:
        lora_up.zero_()
    bias = (torch.randn(N, generator=g) * 0.01).to(dtype)
    wc = (torch.rand(N, generator=g) + 0.5).to(dtype)
    smooth_next = (torch.rand(N, generator=g) * 1.5 + 0.25).to(dtype)
    act, ascales, lora_act = quantize_w4a4_act_fuse_lora_ref(x, lora_down, smooth)
    wgt, wscales = quantize_nvfp4_rows(w, pad_size=1)
    y, qout, oscales = gemm_w4a4_ref(act, wgt, ascales, wscales, lora_act, lora_up, bias=bias, wcscales=wc,
                                     smooth_next=smooth_next)
    out = dict(
        M=M, K=K, N=N, R=R, dtype="fp16" if dtype == torch.float16 else "bf16", exact=int(exact),
        act=u8(act), ascales=u8(ascales), lora_act=lora_act.numpy().copy(), wgt=u8(wgt), wscales=u8(wscales),
        lora_up=bits16(lora_up), bias=bits16(bias), wcscales=bits16(wc), smooth_next=bits16(smooth_next),
        y=bits16(y), qout=u8(qout), oscales=u8(oscales),
    )
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), name + ".npz"), **out)
    print(name, "written; qout bytes", qout.numel())


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference> [linear|next]")
    ref = sys.argv[1]
    which = sys.argv[2] if len(sys.argv) > 2 else "all"
    sys.path.insert(0, ref)
    from baseline.kernels._nvfp4 import dequantize_nvfp4_rows, quantize_nvfp4_rows
    from baseline.kernels.gemm_w4a4.ref import gemm_w4a4_ref
    from baseline.kernels.quantize_w4a4_act_fuse_lora.ref import quantize_w4a4_act_fuse_lora_ref

    torch.manual_seed(0)
    if which in ("all", "linear"):
        build_case("c0_fp16", 64, 128, 128, 16, torch.float16, 1234)
        build_case("edge_fp16", 40, 128, 128, 16, torch.float16, 11, edge=True)
        build_case("edge_bf16", 40, 128, 128, 32, torch.bfloat16, 12, edge=True)
        build_case("nosmooth_bf16", 130, 192, 256, 48, torch.bfloat16, 13, with_smooth=False)
        build_case("tail_fp16", 200, 320, 256, 64, torch.float16, 14)
    if which in ("all", "next"):
        # file names start with "next_": the linear-layer tests skip them, test_next_layer_* take them
        build_next_case("next_exact_fp16", 100, 256, 128, 16, torch.float16, 21, exact=True)
        build_next_case("next_lora_bf16", 130, 192, 256, 32, torch.bfloat16, 22, exact=False)
