"""Quantizer parity on the GPU, through the C ABI: codes and scales bit-exact
against the oracle and the reference-generated fixtures, lora_act within
rel-L2 1e-3 (it is observed near 1e-7: fp32 accumulation of exact products)."""
import numpy as np
import pytest
import torch

from conftest import golden_names, load_golden
from helpers import NAME_DT, assert_device_clean, bits, from_bits, oracle_quantize, u8
from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu
LORA_TOL = 1e-3
GENERIC, FUSED, STREAM = 1, 2, 0x100000


def _ops():
    from svdquant_kernels_b200 import ops
    return ops


def _check(x, ld, sm, force, pad=256):
    ops = _ops()
    act, ascales, lora = ops.quantize_w4a4_act_fuse_lora(x, ld, sm, fp4=True, pad_size=pad, _force=force)
    torch.cuda.synchronize()
    assert_device_clean()
    o_act, o_sc, o_lora = oracle_quantize(x, ld, sm, pad)
    assert act.dtype == torch.uint8 and ascales.dtype == torch.float8_e4m3fn and lora.dtype == torch.float32
    assert tuple(act.shape) == o_act.shape and tuple(ascales.shape) == o_sc.shape and tuple(lora.shape) == o_lora.shape
    assert int((u8(ascales) != o_sc).sum()) == 0, "scale bytes differ"
    assert int((u8(act) != o_act).sum()) == 0, "code bytes differ"
    if ld.shape[1] > 0:
        assert O.rel_l2(lora.cpu().numpy(), o_lora) <= LORA_TOL
    M = x.shape[0]
    assert (lora[M:] == 0).all()
    # the twins the GEMM consumes
    twin = ops._attached(ascales)
    if act.shape[0] % 128 == 0 and (2 * act.shape[1]) % 64 == 0:
        assert twin is not None, "the quantizer did not leave the tensor-core twin of the scales"
        assert (twin.cpu().numpy() == O.swizzle_scales(o_sc)).all(), "swizzled scales differ"
    twin16 = ops._attached(lora)
    if ld.shape[1] > 0:
        assert twin16 is not None, "the quantizer did not leave the 16-bit twin of lora_act"
        twin16 = (twin16,)
        la = lora.cpu().numpy()
        want16 = O.f32_to_bits(np.clip(la, -65504.0, 65504.0), "fp16")
        if x.dtype == torch.float16:
            assert (bits(twin16[0]).reshape(la.shape) == want16).all(), "fp16 lora_act is not the rounded fp32 one"
        else:
            # flat: hi plane, lo plane, fp16 plane, then one 32-bit word per 32 rows (0 = fits fp16)
            hi = O.f32_to_bits(la, "bf16")
            lo = O.f32_to_bits(la - O.bits_to_f32(hi, "bf16"), "bf16")
            got = bits(twin16[0])
            n = la.size
            assert (got[:n].reshape(la.shape) == hi).all() and (got[n:2 * n].reshape(la.shape) == lo).all(), \
                "bf16 hi/lo planes of lora_act differ"
            assert (got[2 * n:3 * n].reshape(la.shape) == want16).all(), "fp16 plane of lora_act differs"
            flags = got[3 * n:].astype(np.uint32)
            flags = flags[0::2] | (flags[1::2] << 16)
            blocks = -(-la.shape[0] // 32)
            unfit = np.array([not (np.abs(la[32 * b:32 * b + 32]) <= 65504.0).all() for b in range(blocks)])
            if force >= STREAM or force == FUSED:
                # a zero word promises that the 32 rows fit fp16: exact in both fused forms, for every K split
                assert ((flags[:blocks] != 0) == unfit).all(), "fits-fp16 words of lora_act differ"
            else:
                assert (flags[:blocks] != 0).all(), "the CUDA-core path must mark every row block"
    return act, ascales, lora


def _inputs(M, K, R, dtype, seed, smooth=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[:4]] *= 20
    x = x.to(dtype)
    sm = x.float().abs().amax(0).pow(0.5).clamp_min(1e-2).to(dtype) if smooth else None
    ld = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype)
    return x.cuda(), ld.cuda(), None if sm is None else sm.cuda()


@pytest.mark.parametrize("force", [GENERIC, FUSED])
@pytest.mark.parametrize("name", golden_names())
def test_against_reference_fixtures(name, force):
    g = load_golden(name)
    dt = NAME_DT[g["dtype"]]
    if force == FUSED and g["K"] % 64 != 0:
        pytest.skip("fused kernel takes K % 64 == 0")
    x = from_bits(g["x"], dt)
    ld = from_bits(g["lora_down"], dt)
    sm = from_bits(g["smooth"], dt) if "smooth" in g else None
    act, ascales, lora = _ops().quantize_w4a4_act_fuse_lora(x, ld, sm, _force=force)
    torch.cuda.synchronize()
    assert_device_clean()
    assert (u8(act) == g["act"]).all() and (u8(ascales) == g["ascales"]).all()
    assert O.rel_l2(lora.cpu().numpy(), g["lora_act"]) <= LORA_TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,R", [(64, 128, 16), (1, 64, 32), (300, 256, 32), (257, 1024, 128), (512, 3840, 128),
                                   (700, 2560, 64), (130, 640, 256), (256, 192, 0),
                                   # long K: every ring depth (it depends on R) goes through many revolutions
                                   (256, 2560, 256), (200, 7680, 256), (192, 15360, 64), (128, 10240, 32)])
def test_fused_matches_oracle(M, K, R, dtype):
    x, ld, sm = _inputs(M, K, R, dtype, 100 + M + K)
    _check(x, ld, sm, FUSED)
    _check(x, ld, None, FUSED)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("R", [8, 40, 96, 136, 256])
def test_two_rank_exchange_at_every_rank_width(R, dtype):
    """37 to 74 row tiles run as clusters of two K ranks, which hand each other the partial LoRA sums of 32
    rows through the copy engine; ranks that do not fill the accumulator's width, and the widest one."""
    x, ld, sm = _inputs(2400, 640, R, dtype, 17 + R)
    _check(x, ld, sm, FUSED, 256)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,R,tm,ks", [(512, 512, 32, 128, 4), (512, 1024, 128, 256, 2), (1024, 1024, 64, 256, 8),
                                         (300, 640, 16, 128, 2), (256, 256, 0, 128, 1), (700, 2560, 128, 256, 1),
                                         (2000, 1536, 128, 128, 4), (2304, 960, 104, 256, 8), (256, 15360, 128, 256, 8),
                                         (128, 7680, 8, 128, 4)])
def test_stream_form_matches_oracle(M, K, R, tm, ks, dtype):
    """The form for tall activations, with tile height and K split forced so that every combination runs
    on small inputs: codes, scales and twins as in the cluster form, the K ranks' partial LoRA sums
    met in the workspace (twice in a row: the counters must return to zero)."""
    x, ld, sm = _inputs(M, K, R, dtype, 300 + M + K)
    force = STREAM | (tm << 8) | (ks << 4)
    _check(x, ld, sm, force)
    _check(x, ld, None, force)
    a, s, l = _check(x, ld, sm, force)
    a2, s2, l2 = _ops().quantize_w4a4_act_fuse_lora(x, ld, sm)       # whatever form the library picks
    torch.cuda.synchronize()
    assert torch.equal(a, a2) and torch.equal(s.view(torch.uint8), s2.view(torch.uint8))
    if R > 0:
        assert O.rel_l2(l.cpu().numpy(), l2.cpu().numpy()) <= 1e-5


def test_stream_form_full_size_and_deterministic():
    """The benchmark shape in the planned streaming form (4352 x 3840, R = 128: 34 tiles x 4 or 17 x 8
    CTAs) against the oracle, and ten runs of it give one lora_act: the K ranks are added in rank
    order whatever order they arrive in."""
    from svdquant_kernels_b200.workloads import CONFIGS, make_inputs
    inp = make_inputs(CONFIGS["c1"])
    x, ld, sm = inp.x.cuda(), inp.lora_down.cuda(), inp.smooth.cuda()
    for force in (STREAM, STREAM | (256 << 8) | (8 << 4), STREAM | (128 << 8) | (4 << 4)):
        _, _, first = _check(x, ld, sm, force)
        for _ in range(9):
            _, _, l = _ops().quantize_w4a4_act_fuse_lora(x, ld, sm, _force=force)
            assert torch.equal(first, l)
    torch.cuda.synchronize()
    assert_device_clean()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,R,pad", [(64, 128, 16, 256), (33, 48, 5, 1), (100, 80, 24, 16), (260, 528, 40, 256)])
def test_generic_matches_oracle(M, K, R, pad, dtype):
    x, ld, sm = _inputs(M, K, R, dtype, 7 + M)
    _check(x, ld, sm, GENERIC, pad)


@pytest.mark.parametrize("force", [GENERIC, FUSED])
def test_edge_values(force):
    """Exact ties, saturation, zero and sub-threshold groups, signed zeros, e4m3 subnormal and clamped scales."""
    dtype = torch.float16
    M, K, R = 128, 256, 16
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=g)
    x[0, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x[1, 16:32] = 0
    x[2, 32:48] = 1e-4; x[2, 33] = -1e-4; x[2, 34] = 0
    x[3, 48:64] = 0; x[3, 49] = -0.0
    x[4, :16] = 3e-3
    x[5, :16] = 2640.0
    x[6, :16] = 6e4
    x[7, :] = 0
    for i in range(8, 40):           # a sweep of magnitudes so every e4m3 scale exponent shows up
        x[i] *= 2.0 ** (i - 24)
    x = x.clamp(-6e4, 6e4).to(dtype).cuda()      # finite inputs only
    ld = (torch.randn(K, R, generator=g) / 16).to(dtype).cuda()
    sm = torch.ones(K, dtype=dtype).cuda()
    sm[64:] = (torch.rand(K - 64, generator=g) * 3 + 0.05).to(dtype).cuda()
    _check(x, ld, sm, force)
    _check(x, ld, None, force)


def test_full_size_config_is_bit_exact():
    """The benchmark shape (4352 x 3840, R = 128, fp16) against the oracle."""
    from svdquant_kernels_b200.workloads import CONFIGS, make_inputs
    inp = make_inputs(CONFIGS["c1"])
    x, ld, sm = inp.x.cuda(), inp.lora_down.cuda(), inp.smooth.cuda()
    _check(x, ld, sm, FUSED)


def test_weight_packer_matches_oracle():
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    w = torch.randn(384, 640, generator=g) * 0.02
    packed, scales = ops.quantize_nvfp4_rows(w.cuda(), pad_size=1)
    o_p, o_s = O.quantize_nvfp4_rows(w.numpy(), 1)
    assert (u8(packed) == o_p).all() and (u8(scales) == o_s).all()
    for dt in (torch.float16, torch.bfloat16):
        wd = w.to(dt)
        packed, scales = ops.quantize_nvfp4_rows(wd.cuda(), pad_size=1)
        o_p, o_s = O.quantize_nvfp4_rows(wd.float().numpy(), 1)
        assert (u8(packed) == o_p).all() and (u8(scales) == o_s).all()


def test_row_permutation_property_full_size():
    """Size-independent property at the largest K: rows are quantised independently, so permuting the
    rows of x permutes codes, scales and lora_act the same way; a sample of rows is checked against
    the oracle."""
    ops = _ops()
    g = torch.Generator().manual_seed(9)
    M, K, R = 4352, 15360, 128
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ld = (torch.randn(K, R, generator=g) / K ** 0.5).to(torch.bfloat16)
    sm = (torch.rand(K, generator=g) * 2 + 0.25).to(torch.bfloat16)
    perm = torch.randperm(M, generator=g)
    xd, ldd, smd = x.cuda(), ld.cuda(), sm.cuda()
    a1, s1, l1 = ops.quantize_w4a4_act_fuse_lora(xd, ldd, smd)
    a2, s2, l2 = ops.quantize_w4a4_act_fuse_lora(xd[perm.cuda()].contiguous(), ldd, smd)
    torch.cuda.synchronize()
    assert_device_clean()
    pc = perm.cuda()
    assert torch.equal(a1[:M][pc], a2[:M])
    assert torch.equal(s1.view(torch.uint8)[:, :M][:, pc], s2.view(torch.uint8)[:, :M])
    assert torch.equal(l1[:M][pc], l2[:M])      # same tile-local arithmetic order for every row
    rows = torch.arange(0, M, 97)
    o_act, o_sc, o_lora = oracle_quantize(x[rows], ld, sm, pad_size=1)
    assert (u8(a1)[rows.numpy()] == o_act).all()
    assert (u8(s1)[:, rows.numpy()] == o_sc).all()
    assert O.rel_l2(l1.cpu().numpy()[rows.numpy()], o_lora) <= LORA_TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("smooth_kind", ["positive", "none", "some_negative"])
def test_signed_zeros_and_negative_smooth(dtype, smooth_kind):
    """-0.0 inputs must come out with code 0 (the reference sets the sign bit only for values < 0), also
    next to tiny negative values (code 8) in the same group, and a smooth vector with negative entries
    (outside the fast divide's domain) must still be bit-exact."""
    M, K, R = 128, 256, 16
    g = torch.Generator().manual_seed(21)
    x = torch.randn(M, K, generator=g)
    x[:, 0:16] = 0.0
    x[::2, 0:16] = -0.0
    x[:, 16:32] = -0.0
    x[:, 16] = 3.0                      # a group of -0 with one real value: non-zero scale
    x[:, 32:48] *= 1e-4
    x[1::3, 40] = -0.0
    x = x.to(dtype)
    ld = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype)
    if smooth_kind == "none":
        sm = None
    else:
        sm = (torch.rand(K, generator=g) + 0.5)
        if smooth_kind == "some_negative":
            sm[5] = -sm[5]
            sm[17] = -sm[17]
            sm[200] = -sm[200]
        sm = sm.to(dtype).cuda()
    _check(x.cuda(), ld.cuda(), sm, FUSED)
    _check(x.cuda(), ld.cuda(), sm, GENERIC)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_no_rows_and_strided_input(dtype):
    """An input without rows gives empty outputs of the right shapes and types and launches nothing
    that fails; a non-contiguous view of x is quantised like its contiguous copy."""
    ops = _ops()
    K, R = 128, 16
    ld = torch.zeros(K, R, dtype=dtype).cuda()
    sm = torch.ones(K, dtype=dtype).cuda()
    act, ascales, lora = ops.quantize_w4a4_act_fuse_lora(torch.empty(0, K, dtype=dtype).cuda(), ld, sm, fp4=True)
    torch.cuda.synchronize()
    assert_device_clean()
    assert tuple(act.shape) == (0, K // 2) and tuple(ascales.shape) == (K // 16, 0) and tuple(lora.shape) == (0, R)
    assert act.dtype == torch.uint8 and ascales.dtype == torch.float8_e4m3fn and lora.dtype == torch.float32

    x, ld, sm = _inputs(300, 512, 32, dtype, 77)
    wide = torch.zeros(300, 1024, dtype=dtype).cuda()
    wide[:, ::2] = x
    a1, s1, l1 = ops.quantize_w4a4_act_fuse_lora(wide[:, ::2], ld, sm, fp4=True)
    a2, s2, l2 = ops.quantize_w4a4_act_fuse_lora(x, ld, sm, fp4=True)
    torch.cuda.synchronize()
    assert_device_clean()
    assert torch.equal(a1, a2) and torch.equal(s1.view(torch.uint8), s2.view(torch.uint8)) and torch.equal(l1, l2)


def test_out_argument_reuses_buffers_and_twins():
    """`out=` writes into the tensors of an earlier call; the layout twins move with them, so a second
    call allocates nothing and the GEMM sees the new contents."""
    from svdquant_kernels_b200 import ops
    g = torch.Generator().manual_seed(31)
    M, K, R, N, dtype = 512, 512, 32, 256, torch.float16
    ld = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype).cuda()
    sm = (torch.rand(K, generator=g) + 0.5).to(dtype).cuda()
    lu = (torch.randn(N, R, generator=g) * 0.01).to(dtype).cuda()
    wgt, wsc = ops.quantize_nvfp4_rows((torch.randn(N, K, generator=g) * 0.02).cuda(), pad_size=1)
    x1 = torch.randn(M, K, generator=g).to(dtype).cuda()
    x2 = torch.randn(M, K, generator=g).to(dtype).cuda()
    q = ops.quantize_w4a4_act_fuse_lora(x1, ld, sm)
    y = ops.gemm_w4a4(q[0], wgt, q[1], wsc, q[2], lu, None, None, dtype)
    swz_ptr = ops._attached(q[1]).data_ptr()
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    q_again = ops.quantize_w4a4_act_fuse_lora(x2, ld, sm, out=q)
    y_again = ops.gemm_w4a4(q[0], wgt, q[1], wsc, q[2], lu, None, None, dtype, out=y)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert q_again[0] is q[0] and y_again is y and ops._attached(q[1]).data_ptr() == swz_ptr
    fresh = ops.quantize_w4a4_act_fuse_lora(x2, ld, sm)
    y_fresh = ops.gemm_w4a4(fresh[0], wgt, fresh[1], wsc, fresh[2], lu, None, None, dtype)
    torch.cuda.synchronize()
    assert torch.equal(q[0], fresh[0]) and torch.equal(q[2], fresh[2]) and torch.equal(y, y_fresh)
    assert_device_clean()


def test_cluster_capacity_query():
    """How many clusters of 1, 2, 4 and 8 CTAs of the fused kernel the device holds at once: the query
    answers for every split the kernel can be launched with."""
    from svdquant_kernels_b200 import _lib
    lib = _lib.load()
    caps = {ks: lib.svdq_quantizer_max_active_clusters(128, ks, _lib.DTYPE_F16) for ks in (1, 2, 4, 8)}
    assert all(v > 0 for v in caps.values()), caps
    assert caps[1] >= caps[2] >= caps[4] >= caps[8]
    assert lib.svdq_quantizer_max_active_clusters(128, 3, _lib.DTYPE_F16) == -1


@pytest.mark.parametrize("M,K", [(256, 3840), (1024, 2560), (2304, 1024)])
def test_fits_fp16_words_are_exact_for_every_split(M, K):
    """bf16: the word per 32 rows that tells the GEMM whether lora_act fits fp16 there.  Few rows run with
    four or eight CTAs per row tile, whose verdicts on a shared 32-row block are gathered through
    distributed shared memory; many rows with two.  Rows 40-49 and the last 20 rows are blown up past
    65504, everything else fits: exactly those blocks must be marked."""
    dtype, R = torch.bfloat16, 64
    g = torch.Generator().manual_seed(77 + M)
    x = torch.randn(M, K, generator=g)
    x[40:50] *= 3000.0
    x[M - 20:] *= 3000.0
    ld = torch.randn(K, R, generator=g)                      # large on purpose: |lora_act| ~ 3000 * sqrt(K)
    _, _, la = _check(x.to(dtype).cuda(), ld.to(dtype).cuda(), None, FUSED)
    blocks = la.abs().reshape(M // 32, -1).amax(1).cpu()
    big = blocks > 65504
    assert big[1] and big[-1] and int(big.sum()) == 2, "the test's inputs do not overflow where they should"
