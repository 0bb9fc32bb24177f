"""The bounded wait every kernel of the library relies on, made to run out on purpose in the one
harmless way there is: a single warp waits on a barrier that nothing arrives on, gives up after a
millisecond, records its code and ends normally.  Nothing faults, traps or waits forever; the
context stays usable, which the test checks by running an ordinary operator right after."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_is_reported_and_leaves_the_device_usable():
    from svdquant_kernels_b200 import _lib, ops
    lib = _lib.load()
    torch.cuda.synchronize()
    rc, words = _lib.device_status()
    assert rc == 0, words
    seen = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.svdq_selftest_wait_expiry(1_000_000, seen.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    # first wait gave up (bit 0 clear), the second returned at once without success (bit 1 clear), abort flag raised
    assert int(seen.item()) == 4
    rc, words = _lib.device_status()
    assert rc == 6, (rc, words)                               # SVDQ_ERR_DEVICE
    assert words[0] == 6 and words[2] == 0x5E1F and words[3] >= 1, words     # kDevWaitMisc, the self-test's tag
    assert "bounded wait" in _lib.status_string(rc)
    # the word is cleared by the read, and an ordinary launch afterwards is clean and correct
    rc, words = _lib.device_status()
    assert rc == 0 and words == [0, 0, 0, 0]
    x = torch.randn(256, 256, generator=torch.Generator().manual_seed(1)).half().cuda()
    ld = torch.zeros(256, 16, dtype=torch.float16, device="cuda")
    act, asc, la = ops.quantize_w4a4_act_fuse_lora(x, ld, None)
    act2, asc2, _ = ops.quantize_w4a4_act_fuse_lora(x, ld, None, _force=_lib.QUANT_FORCE_GENERIC)
    torch.cuda.synchronize()
    assert torch.equal(act, act2) and torch.equal(asc.view(torch.uint8), asc2.view(torch.uint8))
    rc, words = _lib.device_status()
    assert rc == 0, words


def test_selftest_refuses_long_limits():
    from svdquant_kernels_b200 import _lib
    assert _lib.load().svdq_selftest_wait_expiry(10_000_000_000, None, None) == 2
    assert _lib.load().svdq_selftest_wait_expiry(0, None, None) == 2
