"""Host logic of the row-sharded (tensor-parallel) path on CPU: world size 2, gloo.

The per-rank compute is stood in for by the CPU oracle (tests may use it as the checker);
what is under test is the partition, the shard extraction and the all-gather reassembly.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def test_row_partition_tiles_every_shape():
    from llvq_b200.parallel import check_partition, shard_rows
    for d_out in (8, 16, 24, 40, 1024, 2560, 4096, 5120, 9728, 17408, 151936, 1000, 7):
        for world in (1, 2, 4, 8):
            check_partition(d_out, world)
    assert shard_rows(5120, 8, 3) == (1920, 2560)       # 14B q/o: 640 rows per GPU
    assert shard_rows(1024, 8, 7) == (896, 1024)        # 14B k/v: one KV head per GPU
    assert shard_rows(17408, 8, 0) == (0, 2176)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from llvq_b200 import synth
        from llvq_b200.parallel import ShardedProj, shard_matrix
        from oracle import ref
        results = {}
        for d_out, d_in in ((64, 24 * 6 + 5), (40, 48)):  # equal shards, then ragged shards
            m = synth.make_matrix(d_out, d_in, 0xD157 + d_out)
            x = synth.make_activation(d_in, 9).astype(np.float64)
            shard, lo, hi = shard_matrix(m, world, rank)

            def local_forward(xv, shard=shard):
                y = ref.gemv_f64(shard.codes, shard.d_out, shard.d_in, shard.centroids, shard.row_scales,
                                 shard.tail, xv.numpy(), threads=1)
                return torch.from_numpy(np.atleast_1d(y))

            sp = ShardedProj(d_out, local_forward)
            assert (sp.lo, sp.hi) == (lo, hi)
            y = sp.forward(torch.from_numpy(x))
            full = ref.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, m.tail, x, threads=1)
            results[d_out] = bool(np.array_equal(y.numpy(), full))
        q.put((rank, results))
    finally:
        dist.destroy_process_group()


def test_sharded_projection_gathers_the_full_output():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, results in got:
        assert results == {64: True, 40: True}, (rank, results)
