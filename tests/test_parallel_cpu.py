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


# ---- tensor-parallel decode loop: head-sharded attention, row-sharded MLP, sharded greedy head ----

def _dense_qwen3(cfg, weights, norms, embed, capacity, tp):
    """The decode loop on dense CPU weights (a stand-in for the fused projections), whole or sharded."""
    from llvq_b200.model import FusedQwen3, tp_rows
    world, rank = (tp.world, tp.rank) if tp else (1, 0)
    rows = tp_rows(cfg, world, rank)
    cut = lambda w, name: w[rows[name][0]:rows[name][1]]
    blocks = []
    for w, n in zip(weights, norms):
        blk = dict(n)
        blk["qkv"] = torch.cat([cut(w["q"], "q"), cut(w["k"], "k"), cut(w["v"], "v")])
        blk["o"], blk["down"] = cut(w["o"], "o"), cut(w["down"], "down")
        blk["gate_up"] = torch.cat([cut(w["gate"], "gate"), cut(w["up"], "up")])
        blocks.append(blk)
    lin = torch.nn.functional.linear

    def head(rows_e, h, off):
        logits = rows_e.float() @ h.float()
        i = logits.argmax().reshape(1)
        return logits[i].float(), i + off

    return FusedQwen3(cfg, blocks, embed, norms[0]["final"], capacity, gemv=lambda w, x: lin(x.float(), w.float()).half(),
                      gemm=lambda w, x: lin(x.float(), w.float()).half(), head=head, kv_int8=True, tp=tp, prefill_chunk=8)


def _tp_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from llvq_b200.model import Qwen3Config, TpGroup
        torch.manual_seed(11)  # the same weights on every rank
        cfg = Qwen3Config(hidden=64, inter=96, n_heads=4, n_kv=2, head_dim=64, layers=2, vocab=128)
        hd = cfg.head_dim
        shp = {"q": (cfg.n_heads * hd, cfg.hidden), "k": (cfg.n_kv * hd, cfg.hidden), "v": (cfg.n_kv * hd, cfg.hidden),
               "o": (cfg.hidden, cfg.n_heads * hd), "gate": (cfg.inter, cfg.hidden), "up": (cfg.inter, cfg.hidden),
               "down": (cfg.hidden, cfg.inter)}
        weights = [{n: (0.08 * torch.randn(*s)).half() for n, s in shp.items()} for _ in range(cfg.layers)]
        nrm = lambda n: (1.0 + 0.02 * torch.randn(n)).half()
        norms = [{"ln1": nrm(cfg.hidden), "ln2": nrm(cfg.hidden), "q_norm": nrm(hd), "k_norm": nrm(hd), "final": nrm(cfg.hidden)}
                 for _ in range(cfg.layers)]
        embed = (0.5 * torch.randn(cfg.vocab, cfg.hidden)).half()
        prompt = [int(t) for t in torch.randint(0, cfg.vocab, (19,))]  # three prefill chunks of 8, 8 and 3 tokens
        whole = _dense_qwen3(cfg, weights, norms, embed, 48, None).generate(prompt, 12)
        sharded_model = _dense_qwen3(cfg, weights, norms, embed, 48, TpGroup())
        sharded = sharded_model.generate(prompt, 12)
        q.put((rank, whole, sharded, sharded_model.caches[0].q[0].shape[1]))
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_decode_loop_picks_the_single_rank_tokens():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31000 + os.getpid() % 2000
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=150) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, whole, sharded, kv_local in got:
        assert len(whole) == 12 and whole == sharded, (rank, whole, sharded)
        assert kv_local == 1  # each rank caches only its own kv head
    assert got[0][1] == got[1][1]


def test_row_window_generator_equals_the_slice_of_the_whole_matrix():
    from llvq_b200 import synth
    m = synth.make_matrix(48, 24 * 5 + 7, 123)
    for lo, hi in ((0, 48), (8, 24), (40, 48), (16, 16)):
        a, b = m.rows(lo, hi), synth.make_matrix_rows(48, 24 * 5 + 7, 123, lo, hi)
        assert np.array_equal(a.codes, b.codes) and np.array_equal(a.row_scales, b.row_scales)
        assert np.array_equal(a.tail, b.tail) and np.array_equal(a.centroids, b.centroids)


def test_tp_layout_rejects_a_world_that_does_not_divide_the_heads():
    from llvq_b200.model import Qwen3Config, tp_rows
    cfg = Qwen3Config.named("qwen3-14b")
    r = tp_rows(cfg, 8, 3)
    assert r["q"] == (3 * 640, 4 * 640) and r["k"] == (3 * 128, 4 * 128) and r["gate"] == (3 * 2176, 4 * 2176)
    assert r["o"] == (1920, 2560)
