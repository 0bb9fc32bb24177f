"""Column-sharded linear with the all-gather fused into the GEMM epilogue, on 2, 4 and 8 GPUs (each
skipped on a machine with fewer): every rank's copy of the result must equal, bit for bit, what one GPU computes alone, and
the NCCL all-gather form of the same sharding must agree too."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, dtype_name, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from svdquant_kernels_b200 import ops, sharding, _lib
        dtype = getattr(torch, dtype_name)
        M, K, N, R = 512, 512, 1024, 64
        g = torch.Generator().manual_seed(123)
        x = torch.randn(M, K, generator=g).to(dtype)
        sm = (torch.rand(K, generator=g) + 0.5).to(dtype)
        w = torch.randn(N, K, generator=g) * 0.02 / sm.float()[None, :]
        ld = (torch.randn(K, R, generator=g) / K ** 0.5).to(dtype)
        lu = (torch.randn(N, R, generator=g) * 0.01).to(dtype)
        b = (torch.randn(N, generator=g) * 0.01).to(dtype)
        c = (torch.rand(N, generator=g) + 0.5).to(dtype)
        act, asc, la = ops.quantize_w4a4_act_fuse_lora(x.to(dev), ld.to(dev), sm.to(dev))
        wgt, wsc = ops.quantize_nvfp4_rows(w.to(dev), pad_size=1)
        y_one = ops.gemm_w4a4(act, wgt, asc, wsc, la, lu.to(dev), c.to(dev), b.to(dev), dtype)

        col0, n = sharding.column_slab(N, world, rank, multiple=128)
        sl = slice(col0, col0 + n)
        lin = sharding.ColumnShardedLinear(M, N, dtype, wgt=wgt[sl].contiguous(), wscales=wsc[:, sl].contiguous(),
                                           lora_up=lu[sl].to(dev).contiguous(), wcscales=c[sl].to(dev).contiguous(),
                                           bias=b[sl].to(dev).contiguous())
        ok = True
        for it in range(3):                       # reuse of the symmetric buffer across calls
            y_tp = lin.forward(act, asc, la)
            torch.cuda.synchronize()
            ok = ok and torch.equal(y_tp, y_one)
            lin.y.zero_()
            torch.cuda.synchronize()
            dist.barrier()

        def slab(_x):
            return ops.gemm_w4a4(act, wgt[sl].contiguous(), asc, wsc[:, sl].contiguous(), la, lu[sl].to(dev).contiguous(),
                                 c[sl].to(dev).contiguous(), b[sl].to(dev).contiguous(), dtype)

        y_nccl = sharding.linear_columns(x, slab, N)
        torch.cuda.synchronize()
        ok_nccl = torch.equal(y_nccl, y_one)
        rc, words = _lib.device_status()
        q.put((rank, bool(ok), bool(ok_nccl), rc))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype_name", ["float16", "bfloat16"])
def test_fused_all_gather_matches_single_gpu(dtype_name, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 300)
    procs = [ctx.Process(target=_worker, args=(r, world, port, dtype_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    results = [q.get(timeout=10) for _ in range(world)]
    for p in procs:
        assert p.exitcode == 0
    for rank, ok, ok_nccl, rc in results:
        assert ok, f"rank {rank}: fused result differs from the single-GPU result"
        assert ok_nccl, f"rank {rank}: NCCL all-gather result differs from the single-GPU result"
        assert rc == 0
