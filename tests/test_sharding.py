"""Partition logic and the two multi-GPU forms on CPU: world size 2 under gloo, the oracle as compute."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_golden
from oracle import nvfp4_oracle as O
from svdquant_kernels_b200 import sharding


def test_row_slabs_cover_without_overlap():
    for M, world in ((4352 * 8, 8), (4352, 2), (1000, 4), (256, 8), (0, 2)):
        seen = 0
        for r in range(world):
            start, n = sharding.row_slab(M, world, r)
            assert start == seen and n >= 0
            if n and start + n < M:
                assert n % 256 == 0
            seen += n
        assert seen == M
    assert sharding.row_slab(4352 * 4, 4, 2) == (4352 * 2, 4352)


def test_column_slabs():
    assert sharding.column_slab(3072, 8, 3) == (3 * 384, 384)
    with pytest.raises(AssertionError):
        sharding.column_slab(3072, 5, 0)
    with pytest.raises(AssertionError):
        sharding.column_slab(3072, 16, 0)     # 192 is not a multiple of the 128-column tile


def _bits_t(a):
    # gloo has no 16-bit integer collectives: carry the bit patterns as int32
    return torch.from_numpy(a.astype(np.int32))


def _bits_n(t):
    return t.numpy().astype(np.uint16)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = load_golden("tail_fp16")       # M=200 K=320 N=256 R=64
        dt = g["dtype"]

        def whole_linear(x_bits, rows_n0=0, n_cols=None):
            act, asc, la = O.quantize_w4a4_act_fuse_lora(x_bits, g["lora_down"], g["smooth"], dt, pad_size=1)
            n0, n1 = rows_n0, rows_n0 + (n_cols or g["N"])
            y, _, _, _ = O.gemm_w4a4(act, g["wgt"][n0:n1], asc, g["wscales"][:, n0:n1], la, g["lora_up"][n0:n1],
                                     g["wcscales"][n0:n1], g["bias"][n0:n1], dt)
            return y

        full = whole_linear(g["x"])
        # rows: every rank its slab, no collective; rank 0 collects only to compare
        start, n = sharding.row_slab(g["M"], world, rank, multiple=64)
        y_rows = sharding.linear_rows(_bits_t(g["x"][start:start + n]),
                                      lambda xb: _bits_t(whole_linear(_bits_n(xb))))
        # the CPU BLAS picks its summation order by matrix shape, so slabs match to fp32 round-off, not bit for bit
        def close(a_bits, b_bits):
            return O.rel_l2(O.bits_to_f32(a_bits, dt), O.bits_to_f32(b_bits, dt)) <= 1e-4
        ok_rows = bool(close(_bits_n(y_rows), full[start:start + n]))
        # columns: all-gather of the slabs
        n0, ncols = sharding.column_slab(g["N"], world, rank)
        y_cols = sharding.linear_columns(_bits_t(g["x"]),
                                         lambda xb: _bits_t(whole_linear(_bits_n(xb), n0, ncols)), g["N"])
        ok_cols = bool(close(_bits_n(y_cols), full))
        q.put((rank, ok_rows, ok_cols, tuple(y_cols.shape)))
    except Exception as e:      # report instead of leaving the parent waiting on the queue
        q.put((rank, False, False, repr(e)))
    finally:
        dist.destroy_process_group()


def test_row_and_column_sharding_world2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_rows, ok_cols, shape in results:
        assert ok_rows, f"rank {rank}: row-sharded slab differs from the unsharded result ({shape})"
        assert ok_cols, f"rank {rank}: gathered column slabs differ from the unsharded result"
        assert shape == (200, 256)
