"""Host-buffer plan (svdq_linear_plan_*): the one-call form and the pipelined submit / wait form
must return bit for bit what the two device ops return on the same inputs, whatever mix of
page-locked and pageable caller buffers they are given, and the device path itself is checked
against the oracle in test_quantize_gpu.py / test_gemm_gpu.py."""
import pytest
import torch

from helpers import assert_device_clean

pytestmark = pytest.mark.gpu


def _setup(M, K, N, R, dtype, seed):
    from svdquant_kernels_b200 import ops
    g = torch.Generator().manual_seed(seed)
    sm = (torch.rand(K, generator=g) + 0.5).to(dtype)
    w = torch.randn(N, K, generator=g) * 0.02 / sm.float()[None, :]
    ld = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype)
    lu = (torch.randn(N, R, generator=g) * 0.01).to(dtype)
    b = (torch.randn(N, generator=g) * 0.01).to(dtype)
    c = (torch.rand(N, generator=g) + 0.5).to(dtype)
    wgt, wsc = ops.quantize_nvfp4_rows(w.cuda(), pad_size=1)
    plan = ops.LinearPlan(M, K, N, R, dtype, wgt=wgt.cpu(), wscales=wsc.view(torch.uint8).cpu(), lora_down=ld,
                          lora_up=lu, smooth=sm, wcscales=c, bias=b)

    def device_path(x):
        act, asc, la = ops.quantize_w4a4_act_fuse_lora(x.cuda(), ld.cuda(), sm.cuda())
        y = ops.gemm_w4a4(act, wgt, asc, wsc, la, lu.cuda(), c.cuda(), b.cuda(), dtype)
        torch.cuda.synchronize()
        return y[: x.shape[0]].cpu()

    return plan, device_path, g


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_forward_host_matches_device_ops(dtype):
    M, K, N, R = 300, 256, 256, 32
    plan, device_path, g = _setup(M, K, N, R, dtype, 5)
    try:
        for rows, pinned in ((300, True), (300, False), (77, False), (256, True)):
            x = torch.randn(rows, K, generator=g).to(dtype)
            y = torch.empty(rows, N, dtype=dtype)
            if pinned:
                x, y = x.pin_memory(), y.pin_memory()
            plan.forward_host(x, y)
            assert torch.equal(y, device_path(x)), (rows, pinned)
    finally:
        plan.close()
    assert_device_clean()


def test_pipelined_batches_keep_their_identity():
    """Seven different batches through submit/wait with two in flight: every y belongs to its own x."""
    M, K, N, R, dtype = 512, 512, 384, 64, torch.float16
    plan, device_path, g = _setup(M, K, N, R, dtype, 9)
    try:
        xs = [torch.randn(M - 13 * i, K, generator=g).to(dtype) for i in range(7)]
        xs = [x.pin_memory() if i % 2 == 0 else x for i, x in enumerate(xs)]          # mixed pinned / pageable
        ys = [torch.empty(x.shape[0], N, dtype=dtype) for x in xs]
        ys = [y.pin_memory() if i % 3 == 0 else y for i, y in enumerate(ys)]
        for x, y in zip(xs, ys):
            plan.submit(x, y)
        plan.wait()
        for i, (x, y) in enumerate(zip(xs, ys)):
            assert torch.equal(y, device_path(x)), f"batch {i}"
        # a wait with nothing in flight, then the plan is still usable
        plan.wait()
        plan.forward_host(xs[0], ys[0])
        assert torch.equal(ys[0], device_path(xs[0]))
    finally:
        plan.close()
    assert_device_clean()


def test_plan_rejects_bad_calls():
    M, K, N, R, dtype = 256, 256, 256, 32, torch.float16
    plan, _, g = _setup(M, K, N, R, dtype, 3)
    try:
        x = torch.zeros(M + 1, K, dtype=dtype)
        y = torch.zeros(M + 1, N, dtype=dtype)
        with pytest.raises(RuntimeError):
            plan.forward_host(x, y)          # more rows than the plan was made for
    finally:
        plan.close()


def test_few_rows_long_k():
    """A plan whose calls have few rows and a long K: its GEMM takes the split-K form with the plan's own
    workspace, and the result is still the device operators' result bit for bit."""
    M, K, N, R, dtype = 200, 6144, 512, 32, torch.float16
    plan, device_path, g = _setup(M, K, N, R, dtype, 11)
    try:
        for rows in (200, 200, 64):
            x = torch.randn(rows, K, generator=g).to(dtype).pin_memory()
            y = torch.empty(rows, N, dtype=dtype).pin_memory()
            plan.forward_host(x, y)
            assert torch.equal(y, device_path(x)), rows
    finally:
        plan.close()
    assert_device_clean()
