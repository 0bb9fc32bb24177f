"""Multi-GPU forms of the W4A4 linear: one process per GPU, torch.distributed for the plumbing.

Rows of x / act / y are independent in both kernels (quantisation groups run along K inside a
row, GEMM rows never mix), so the natural sharding is by rows with replicated weights and NO
collective on the data path (`row_slab`, `linear_rows`).  The tensor-parallel option shards the
weight rows (columns of y): every rank quantises the full x, multiplies by its slab of
`wgt / wscales / lora_up / wcscales / bias`, and the column slabs of y are all-gathered
(`column_slab`, `linear_columns`).  The reference has no multi-GPU code at all; its operators are
the per-rank building blocks here.

The compute step is passed in as a callable so that the same partition / gather logic runs under
the gloo backend on CPU in the tests (with the oracle as the compute) and under NCCL on GPUs
(with `ops`).

`ColumnShardedLinear` is the B200-native form of the tensor-parallel option: the result lives in
symmetric memory on every GPU and each rank's GEMM writes its finished tiles straight into every
peer's copy over NVLink from its epilogue, so there is no all-gather kernel after the GEMM at all,
only a barrier over the ranks.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def row_slab(M: int, world: int, rank: int, multiple: int = 256) -> Tuple[int, int]:
    """(first row, row count) of `rank`: contiguous slabs, sizes multiples of `multiple` except
    possibly the last non-empty one; ranks beyond the data get (M, 0)."""
    assert 0 <= rank < world and M >= 0 and multiple >= 1
    units = -(-M // multiple)
    base, rem = divmod(units, world)
    first_unit = rank * base + min(rank, rem)
    n_units = base + (1 if rank < rem else 0)
    start = min(first_unit * multiple, M)
    stop = min((first_unit + n_units) * multiple, M)
    return start, stop - start


def column_slab(N: int, world: int, rank: int, multiple: int = 128) -> Tuple[int, int]:
    """(first column, column count) of `rank`; N must split into equal slabs of a multiple of
    `multiple` columns (the GEMM's N-tile), e.g. 3072 / 8 = 384 = 3 x 128."""
    assert N % world == 0, f"N ({N}) must divide evenly over {world} ranks"
    n = N // world
    assert n % multiple == 0, f"per-rank N ({n}) must be a multiple of {multiple}"
    return rank * n, n


def linear_rows(x_local: torch.Tensor, compute: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
    """Row-sharded linear: each rank applies the whole linear to its own rows.  No communication."""
    return compute(x_local)


def linear_columns(x: torch.Tensor, compute_slab: Callable[[torch.Tensor], torch.Tensor], N: int,
                   group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Column-sharded (tensor-parallel) linear.

    `compute_slab(x)` returns this rank's `[M, N / world]` slab of y (its weight rows); the slabs
    are all-gathered and laid side by side.  One collective per call: an all-gather of the
    `[M, N / world]` slabs (NCCL over NVLink on GPUs), then a strided copy into `[M, N]`."""
    world = dist.get_world_size(group)
    y_slab = compute_slab(x).contiguous()
    M, n = y_slab.shape
    assert n * world == N
    slabs = [torch.empty_like(y_slab) for _ in range(world)]
    dist.all_gather(slabs, y_slab, group=group)
    return torch.cat(slabs, dim=1)


class ColumnShardedLinear:
    """Tensor-parallel W4A4 linear whose all-gather is fused into the GEMM epilogue.

    Every rank holds rows `[col0, col0 + n)` of the weight-side tensors and a `[M, N]` result buffer in
    symmetric memory (torch.distributed._symmetric_memory).  `forward(act, ascales, lora_act)` launches
    the local GEMM in its column-sharded form (`svdq_gemm_w4a4_columns`): each finished 32 x 64 strip
    goes into the local buffer and, as one TMA store per peer over NVLink, into the same place of every peer's
    buffer.  A barrier over the ranks on the launch stream before the GEMM keeps a fast rank from
    overwriting a buffer a slow peer still reads; one after it makes every peer's strips visible.
    One process per GPU; at most 8 ranks.
    """

    def __init__(self, M: int, N: int, dtype: torch.dtype, *, wgt, wscales, lora_up=None, wcscales=None, bias=None,
                 group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        assert self.world <= 8
        self.M, self.N, self.dtype = M, N, dtype
        self.col0, self.n = column_slab(N, self.world, self.rank)
        assert wgt.shape[0] == self.n, "pass this rank's slab of the weight-side tensors"
        self.wgt, self.wscales, self.lora_up, self.wcscales, self.bias = wgt, wscales, lora_up, wcscales, bias
        self.y = symm_mem.empty((M, N), dtype=dtype, device=wgt.device)
        self.handle = symm_mem.rendezvous(self.y, self.group)
        self.peer_ptrs = [int(self.handle.buffer_ptrs[r]) for r in range(self.world) if r != self.rank]

    def forward(self, act: torch.Tensor, ascales: torch.Tensor, lora_act: Optional[torch.Tensor]) -> torch.Tensor:
        from . import ops
        self.handle.barrier(channel=0)           # every rank is done reading the previous result
        ops.gemm_w4a4(act, self.wgt, ascales, self.wscales, lora_act, self.lora_up, self.wcscales, self.bias,
                      self.dtype, _columns=(self.y, self.peer_ptrs, self.col0))
        self.handle.barrier(channel=1)           # every rank's strips have landed everywhere
        return self.y
