"""Dispatcher registration (torch.ops.svdq_b200.*): shape inference without a device, and on the GPU
the registered ops must return exactly what the plain Python operators return."""
import pytest
import torch


def test_fake_kernels_infer_shapes_and_dtypes(lib_path):
    from torch._subclasses.fake_tensor import FakeTensorMode
    from svdquant_kernels_b200 import torch_ops  # noqa: F401  (registers the ops)
    with FakeTensorMode():
        x = torch.empty(300, 256, dtype=torch.bfloat16, device="cuda")
        ld = torch.empty(256, 32, dtype=torch.bfloat16, device="cuda")
        sm = torch.empty(256, dtype=torch.bfloat16, device="cuda")
        act, asc, la = torch.ops.svdq_b200.quantize_w4a4_act_fuse_lora(x, ld, sm)
        assert act.shape == (512, 128) and act.dtype == torch.uint8
        assert asc.shape == (16, 512) and asc.dtype == torch.float8_e4m3fn
        assert la.shape == (512, 32) and la.dtype == torch.float32
        act64, _, _ = torch.ops.svdq_b200.quantize_w4a4_act_fuse_lora(x, ld, None, 64)
        assert act64.shape == (320, 128)
        wgt = torch.empty(384, 128, dtype=torch.uint8, device="cuda")
        wsc = torch.empty(16, 384, dtype=torch.float8_e4m3fn, device="cuda")
        lu = torch.empty(384, 32, dtype=torch.bfloat16, device="cuda")
        y = torch.ops.svdq_b200.gemm_w4a4(act, wgt, asc, wsc, la, lu)
        assert y.shape == (512, 384) and y.dtype == torch.bfloat16
        y16 = torch.ops.svdq_b200.gemm_w4a4(act, wgt, asc, wsc)
        assert y16.dtype == torch.float16


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_registered_ops_equal_the_python_operators(dtype):
    from svdquant_kernels_b200 import ops, torch_ops  # noqa: F401
    from helpers import assert_device_clean
    g = torch.Generator().manual_seed(4)
    M, K, N, R = 300, 512, 384, 32
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    sm = (torch.rand(K, generator=g) + 0.5).to(dtype).cuda()
    ld = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype).cuda()
    lu = (torch.randn(N, R, generator=g) * 0.01).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) * 0.02).cuda()
    wgt, wsc = ops.quantize_nvfp4_rows(w, pad_size=1)
    a0, s0, l0 = ops.quantize_w4a4_act_fuse_lora(x, ld, sm)
    a1, s1, l1 = torch.ops.svdq_b200.quantize_w4a4_act_fuse_lora(x, ld, sm)
    assert torch.equal(a0, a1) and torch.equal(s0.view(torch.uint8), s1.view(torch.uint8)) and torch.equal(l0, l1)
    y0 = ops.gemm_w4a4(a0, wgt, s0, wsc, l0, lu, None, None, dtype)
    y1 = torch.ops.svdq_b200.gemm_w4a4(a1, wgt, s1, wsc, l1, lu, None, None, dtype)
    torch.cuda.synchronize()
    assert_device_clean()
    # fp16: identical (the 16-bit lora_act is the same rounding either way); bf16: the dispatcher copy has
    # lost its twins, so the GEMM takes the two-pass bf16 LoRA route instead of the fp16 one
    if dtype == torch.float16:
        assert torch.equal(y0, y1)
    else:
        rel = ((y0.float() - y1.float()).norm() / y0.float().norm()).item()
        assert rel <= 1e-3
