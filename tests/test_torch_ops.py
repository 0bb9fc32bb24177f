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
    # the layout twins ride on the storage, so the dispatcher path runs the very same kernels
    assert torch.equal(y0, y1)
    assert ops._attached(s1) is not None and ops._attached(l1) is not None


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_cuda_graph_through_the_dispatcher_matches_the_oracle(dtype):
    """Quantizer + GEMM captured through torch.ops in one CUDA graph; the replay on fresh input must
    give codes and scales equal to the oracle's bit for bit, y within the GEMM tolerance, and the
    same y as the plain Python operators."""
    from svdquant_kernels_b200 import ops, torch_ops  # noqa: F401
    from helpers import assert_device_clean, oracle_gemm, oracle_quantize, rel_l2_vs_bits, u8
    g = torch.Generator().manual_seed(14)
    M, K, N, R = 512, 1024, 512, 64
    sm = (torch.rand(K, generator=g) + 0.5).to(dtype)
    ld = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype)
    lu = (torch.randn(N, R, generator=g) * 0.01).to(dtype)
    c = (torch.rand(N, generator=g) + 0.5).to(dtype)
    b = (torch.randn(N, generator=g) * 0.01).to(dtype)
    w = torch.randn(N, K, generator=g) * 0.02
    wgt, wsc = ops.quantize_nvfp4_rows(w.cuda(), pad_size=1)
    x_static = torch.randn(M, K, generator=g).to(dtype).cuda()
    sm_d, ld_d, lu_d, c_d, b_d = sm.cuda(), ld.cuda(), lu.cuda(), c.cuda(), b.cuda()

    def step():
        a, s, l = torch.ops.svdq_b200.quantize_w4a4_act_fuse_lora(x_static, ld_d, sm_d)
        return a, s, l, torch.ops.svdq_b200.gemm_w4a4(a, wgt, s, wsc, l, lu_d, c_d, b_d, dtype)

    step()                                             # warm: weight-side twins and the smooth table exist
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        a, s, l, y = step()
    x_new = torch.randn(M, K, generator=g).to(dtype)
    x_static.copy_(x_new.cuda())
    graph.replay()
    torch.cuda.synchronize()
    assert_device_clean()
    o_act, o_sc, o_la = oracle_quantize(x_new, ld, sm)
    assert (u8(a) == o_act).all() and (u8(s) == o_sc).all()
    y_bits, _ = oracle_gemm(o_act, u8(wgt), o_sc, u8(wsc), o_la, lu, c, b, dtype)
    assert rel_l2_vs_bits(y, y_bits) <= 1e-3
    a2, s2, l2 = ops.quantize_w4a4_act_fuse_lora(x_static, ld_d, sm_d)
    y2 = ops.gemm_w4a4(a2, wgt, s2, wsc, l2, lu_d, c_d, b_d, dtype)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
