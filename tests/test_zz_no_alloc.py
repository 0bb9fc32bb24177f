"""svdq_gemm_w4a4_static_ws (split-K on the workspace inside the library image) against
svdq_gemm_w4a4_ws (caller-owned workspace) on the same inputs: two calls in a row, both bit-identical
to the existing entry point, and a split count the static array has no room for is refused.
Collected last: the entry point under test keeps its state in the library image for the rest of the
process."""
import pytest
import torch

from helpers import assert_device_clean

pytestmark = pytest.mark.gpu


def _inputs(M, K, N, R, dtype, seed):
    from svdquant_kernels_b200 import ops
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    sm = (torch.rand(K, generator=g) + 0.5).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) * 0.02).cuda()
    ld = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype).cuda()
    lu = (torch.randn(N, R, generator=g) * 0.01).to(dtype).cuda()
    c = (torch.rand(N, generator=g) + 0.5).to(dtype).cuda()
    b = (torch.randn(N, generator=g) * 0.01).to(dtype).cuda()
    act, asc, la = ops.quantize_w4a4_act_fuse_lora(x, ld, sm)
    wgt, wsc = ops.quantize_nvfp4_rows(w, pad_size=1)
    return act, wgt, asc, wsc, la, lu, c, b


def _static_call(args, dtype, variant=0):
    """The new entry point through ctypes, on torch's current stream; returns (status, y)."""
    from svdquant_kernels_b200 import ops, _lib
    act, wgt, asc, wsc, la, lu, c, b = args
    lib = _lib.load()
    M, N, K, R = act.shape[0], wgt.shape[0], act.shape[1] * 2, lu.shape[1]
    sa, sw = ops.swizzle_scales(asc), ops.swizzle_scales(wsc)
    la16 = ops._lora_act_16(la, dtype)
    lu16 = ops._lora_up_f16(lu) if dtype == torch.bfloat16 else None
    y = torch.empty((M, N), dtype=dtype, device=act.device)
    p = ops._ptr
    rc = lib.svdq_gemm_w4a4_static_ws(p(act), p(wgt), p(sa), p(sw), p(la16), p(lu), p(lu16), p(c), p(b), p(y), M, N, K, R,
                                      ops._DT[dtype], variant, ops._stream(act.device))
    return rc, y


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_static_workspace_matches_caller_owned_workspace(dtype):
    from svdquant_kernels_b200 import ops, _lib
    M, K, N, R = 256, 10240, 3072, 32
    assert int(_lib.load().svdq_gemm_w4a4_workspace_bytes(M, N, K, R)) > 0      # this shape takes the split-K form
    args = _inputs(M, K, N, R, dtype, 21)
    act, wgt, asc, wsc, la, lu, c, b = args
    want = ops.gemm_w4a4(act, wgt, asc, wsc, la, lu, c, b, dtype)              # svdq_gemm_w4a4_ws
    for call in range(2):
        rc, y = _static_call(args, dtype)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.equal(y, want), f"call {call}"
    # a forced split count, and a problem that does not split at all (plain tiles, no workspace use)
    rc, y = _static_call(args, dtype, variant=20128)
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(y, ops.gemm_w4a4(act, wgt, asc, wsc, la, lu, c, b, dtype, _splits=2))
    small = _inputs(512, 512, 512, 32, dtype, 22)
    rc, y = _static_call(small, dtype)
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(y, ops.gemm_w4a4(*small, dtype))
    assert_device_clean()


def test_static_workspace_refuses_what_does_not_fit():
    from svdquant_kernels_b200 import _lib
    args = _inputs(256, 10240, 3072, 32, torch.float16, 23)
    rc, _ = _static_call(args, torch.float16, variant=40128)      # 48 tiles x 4 splits = 192 partial tiles > 148
    assert rc == 7, _lib.status_string(rc)
    torch.cuda.synchronize()
    assert_device_clean()


def test_static_workspace_calls_allocate_nothing_and_chain_without_host_syncs():
    """The point of the entry point: once it has been called on a device, further calls take no device
    memory from anywhere (free memory as the driver reports it does not move), and calls queued back to
    back on one stream with no host synchronisation in between - each starts its set-up while the one
    before it is still running - all return the result of the caller-workspace form."""
    from svdquant_kernels_b200 import ops
    dtype = torch.float16
    args = _inputs(256, 10240, 3072, 32, dtype, 24)
    act, wgt, asc, wsc, la, lu, c, b = args
    want = ops.gemm_w4a4(act, wgt, asc, wsc, la, lu, c, b, dtype)
    rc, y = _static_call(args, dtype)                 # first call on this device may look the array's address up
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(y, want)
    lib = __import__("svdquant_kernels_b200._lib", fromlist=["load"]).load()
    sa, sw = ops.swizzle_scales(asc), ops.swizzle_scales(wsc)
    la16 = ops._lora_act_16(la, dtype)
    M, N, K, R = act.shape[0], wgt.shape[0], act.shape[1] * 2, lu.shape[1]
    ys = [torch.empty((M, N), dtype=dtype, device=act.device) for _ in range(10)]
    p, stream = ops._ptr, ops._stream(act.device)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for y_i in ys:                                     # ten calls queued, nothing waited for
        rc = lib.svdq_gemm_w4a4_static_ws(p(act), p(wgt), p(sa), p(sw), p(la16), p(lu), None, p(c), p(b), p(y_i), M, N, K, R,
                                          ops._DT[dtype], 0, stream)
        assert rc == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "a call of the allocation-free entry point changed the device's free memory"
    for i, y_i in enumerate(ys):
        assert torch.equal(y_i, want), f"queued call {i}"
    assert_device_clean()
