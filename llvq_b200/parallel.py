"""Row-sharded (tensor-parallel) projections over `torch.distributed`.

Every output row of a projection is an independent dot product over its own codes, row
scale and tail (no cross-row state, llvq-cuda/kernels/planes_seg.cu:65-83), so rank g of G
holds rows [g * d_out / G, (g + 1) * d_out / G) and the activation is replicated. The only
exchange is an all-gather of the output shards (NCCL over NVLink on GPUs; gloo in the CPU
tests of the host logic). The reference is single-GPU; this layer is new.
"""
from __future__ import annotations

from typing import Callable

import numpy as np


def shard_rows(d_out: int, world: int, rank: int, multiple: int = 8):
    """[lo, hi) of `rank`: shards are equal multiples of `multiple` rows whenever d_out allows,
    so that every shard keeps the 8-row alignment the kernels tile by."""
    if d_out % (world * multiple) == 0:
        per = d_out // world
        return rank * per, (rank + 1) * per
    units = (d_out + multiple - 1) // multiple
    lo_u = units * rank // world
    hi_u = units * (rank + 1) // world
    return min(lo_u * multiple, d_out), min(hi_u * multiple, d_out)


class ShardedProj:
    """One projection split by rows across the ranks of a process group.

    `local_forward(x) -> tensor[hi - lo]` computes this rank's rows (on a GPU: a FusedProj
    through FusedRuntime.forward); `forward` all-gathers the shards into the full output.
    """

    def __init__(self, d_out: int, local_forward: Callable, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.d_out = d_out
        self.bounds = [shard_rows(d_out, self.world, r) for r in range(self.world)]
        self.lo, self.hi = self.bounds[self.rank]
        self.local_forward = local_forward
        self.equal = len({hi - lo for lo, hi in self.bounds}) == 1

    def forward(self, x):
        import torch
        y_local = self.local_forward(x)
        if y_local.numel() != self.hi - self.lo:
            raise ValueError("local_forward returned the wrong number of rows")
        if self.world == 1:
            return y_local
        if self.equal:
            out = torch.empty(self.d_out, dtype=y_local.dtype, device=y_local.device)
            self.dist.all_gather_into_tensor(out, y_local.contiguous(), group=self.group)
            return out
        # ragged shards: pad every shard to the longest one, gather, then drop the padding
        longest = max(hi - lo for lo, hi in self.bounds)
        padded = torch.zeros(longest, dtype=y_local.dtype, device=y_local.device)
        padded[: self.hi - self.lo] = y_local
        buf = torch.empty(self.world * longest, dtype=y_local.dtype, device=y_local.device)
        self.dist.all_gather_into_tensor(buf, padded, group=self.group)
        return torch.cat([buf[r * longest: r * longest + (hi - lo)] for r, (lo, hi) in enumerate(self.bounds)])


def shard_matrix(m, world: int, rank: int):
    """The rows of a synthetic / archive matrix that `rank` uploads."""
    lo, hi = shard_rows(m.d_out, world, rank)
    return m.rows(lo, hi), lo, hi


def check_partition(d_out: int, world: int) -> None:
    """Shards tile [0, d_out) in order without gaps or overlap."""
    b = [shard_rows(d_out, world, r) for r in range(world)]
    assert b[0][0] == 0 and b[-1][1] == d_out
    for (l0, h0), (l1, _) in zip(b, b[1:]):
        assert h0 == l1 and l0 <= h0
    assert all(lo % 8 == 0 for lo, _ in b)
    _ = np  # numpy kept for callers that shard host arrays
