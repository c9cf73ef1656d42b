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


class _DeviceBytes:
    """A raw device range for torch.as_tensor (CUDA array interface, zero-copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerExchange:
    """All-gather of small shards through peer memory (llvq_tp_exchange): one region per rank holding a flag
    area and one gather buffer per site, mapped into every peer through CUDA IPC. One process per GPU; the
    IPC handles travel through the process group once, at construction. `site_bytes[i]` is the size of the
    gathered buffer of site i (world shards)."""

    FLAG_BYTES, HANDLE_BYTES = 512, 64

    def __init__(self, lib, device: int, site_bytes, group=None, spin_limit: int = 0):
        import ctypes as C
        import torch
        import torch.distributed as dist
        from ._lib import check
        self.lib, self.device, self.group = lib, device, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if len(site_bytes) > 16:
            raise ValueError("at most 16 sites")
        self.offsets, off = [], self.FLAG_BYTES
        for n in site_bytes:
            self.offsets.append(off)
            off += (n + 255) // 256 * 256
        self.site_bytes, self.total = list(site_bytes), off
        own, handle = C.c_void_p(), (C.c_uint8 * self.HANDLE_BYTES)()
        check(lib.llvq_tp_region_create(device, off - self.FLAG_BYTES, C.byref(own), handle))
        self._own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._regions = (C.c_void_p * self.world)()
        self._opened = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self._regions[r] = self._own
                continue
            peer = C.c_void_p()
            check(lib.llvq_tp_region_open(device, (C.c_uint8 * self.HANDLE_BYTES).from_buffer_copy(h), C.byref(peer)))
            self._regions[r] = peer.value
            self._opened.append(peer.value)
        ctx = C.c_void_p()
        check(lib.llvq_tp_ctx_create(device, self.rank, self.world, self._regions, spin_limit, C.byref(ctx)))
        self._ctx = ctx
        self.mem = torch.as_tensor(_DeviceBytes(self._own, self.total), device=torch.device("cuda", device))
        dist.barrier(group=group)  # every rank has mapped every region before the first store

    def buffer(self, site: int, dtype):
        """The gathered buffer of `site` in this rank's region, as a 1-D tensor of `dtype`."""
        lo = self.offsets[site]
        return self.mem[lo:lo + self.site_bytes[site]].view(dtype)

    def exchange(self, site: int, shard):
        """Enqueue the gather of `shard` (this rank's contiguous part) on the current stream; returns the buffer."""
        import ctypes as C
        import torch
        from ._lib import check
        nbytes = shard.numel() * shard.element_size()
        if nbytes * self.world != self.site_bytes[site] or not shard.is_contiguous():
            raise ValueError(f"site {site}: a contiguous shard of {self.site_bytes[site] // self.world} bytes, got {nbytes}")
        check(self.lib.llvq_tp_exchange(self._ctx, site, self.offsets[site], C.c_void_p(shard.data_ptr()), nbytes,
                                        C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return self.buffer(site, shard.dtype)

    def poll_error(self) -> int:
        """Read and clear the error word (bit 2: a peer's flag did not arrive within the spin limit)."""
        import ctypes as C
        from ._lib import check
        v = C.c_int32()
        check(self.lib.llvq_tp_poll_error(self._ctx, C.byref(v)))
        return v.value

    def close(self) -> None:
        if self._ctx:
            self.lib.llvq_tp_ctx_destroy(self._ctx)
            self._ctx = None
            for p in self._opened:
                self.lib.llvq_tp_region_close(self.device, p)
            self.lib.llvq_tp_region_free(self.device, self._own)


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
