"""Seeded sweep over odd shapes and option mixes: whatever path the dispatch picks (fused or CUDA-core
quantizer, any GEMM tile shape, either bf16 LoRA route), codes and scales must be bit-exact and
lora_act / y within rel-L2 1e-3 of the oracle."""
import random

import pytest
import torch

from helpers import assert_device_clean, oracle_gemm, oracle_quantize, rel_l2_vs_bits, u8
from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_shapes(seed):
    from svdquant_kernels_b200 import ops
    rnd = random.Random(seed)
    for it in range(14):
        dtype = rnd.choice([torch.float16, torch.bfloat16])
        M = rnd.choice([1, 37, 64, 100, 128, 200, 256, 300, 511, 512, 640, 1000])
        K = 64 * rnd.randint(1, 40)
        N = 128 * rnd.randint(1, 8)
        R = rnd.choice([0, 16, 32, 48, 64, 96, 128, 160, 256])
        pad = rnd.choice([256, 256, 128])
        g = torch.Generator().manual_seed(seed * 1000 + it)
        x = torch.randn(M, K, generator=g) * rnd.choice([1.0, 0.01, 30.0])
        x[:, torch.randperm(K, generator=g)[:3]] *= 25
        if rnd.random() < 0.3:
            x[torch.rand(M, K, generator=g) < 0.1] = 0
        x = x.to(dtype)
        sm = None if rnd.random() < 0.2 else (torch.rand(K, generator=g) * 3 + 0.05).to(dtype)
        ld = (torch.randn(K, max(R, 1), generator=g) / K ** 0.5).to(dtype)[:, :R].contiguous()
        lu = (torch.randn(N, max(R, 1), generator=g) * 0.01).to(dtype)[:, :R].contiguous()
        w = torch.randn(N, K, generator=g) * 0.02
        wc = None if rnd.random() < 0.5 else (torch.rand(N, generator=g) + 0.5).to(dtype)
        b = None if rnd.random() < 0.5 else (torch.randn(N, generator=g) * 0.01).to(dtype)
        what = f"seed {seed} case {it}: {dtype} M={M} K={K} N={N} R={R} pad={pad} smooth={sm is not None}"
        act, asc, la = ops.quantize_w4a4_act_fuse_lora(x.cuda(), ld.cuda(), None if sm is None else sm.cuda(), pad_size=pad)
        torch.cuda.synchronize()
        o_act, o_sc, o_la = oracle_quantize(x, ld, sm, pad)
        assert int((u8(act) != o_act).sum()) == 0, what
        assert int((u8(asc) != o_sc).sum()) == 0, what
        if R:
            assert O.rel_l2(la.cpu().numpy(), o_la) <= 1e-3, what
        wgt, wsc = ops.quantize_nvfp4_rows(w.cuda(), pad_size=1)
        y = ops.gemm_w4a4(act, wgt, asc, wsc, la if R else None, lu.cuda() if R else None,
                          None if wc is None else wc.cuda(), None if b is None else b.cuda(), dtype)
        torch.cuda.synchronize()
        y_bits, _ = oracle_gemm(u8(act), u8(wgt), u8(asc), u8(wsc), la.cpu().numpy() if R else None, lu if R else None, wc, b, dtype)
        assert rel_l2_vs_bits(y, y_bits) <= 1e-3, what
    assert_device_clean()
