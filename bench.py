#!/usr/bin/env python
"""Benchmark of the fused Leech-lattice dequant-GEMV on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

Workload (`config.workload` = "qwen3-4b-layer-gemv"): benchmark configuration 1 — the seven
projections of a Qwen3-4B layer (q 4096x2560, k/v 1024x2560, o 2560x4096, gate/up
9728x2560, down 2560x9728) at batch 1 with f16 activations, on seeded synthetic
codes. One step = one pass over the seven projections of L distinct layers
(default 36 = every projection of the model once, 252 GEMVs, 904 MB of codes), so
every step streams far more than the 126 MB L2 and no matrix is re-read warm.

Reported: `value` = algorithmic GB/s (codes + f32 tails + f64 row scales + x + y
bytes over the device time of the pass, inputs resident in HBM); `e2e` = the same
metric through the host-buffer C ABI call (x copied in from pinned host memory and
y copied back inside the timed region, per GEMV); `roofline` for the GEMV kernel;
`cpu_baseline` = the CPU oracle (the C++ restatement of the reference's Rust path)
timed on this box's host cores on a bounded sample. `--impl reference` times that
CPU path alone, as the reference arm.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM bytes (read + write) the GEMV kernel moved for the four grouped launches of one layer in the
# ncu capture summarised in profiles/gemv_sorted_kernel_qwen3_4b_layer.md (5.16 + 3.62 + 14.31 + 7.34 MB).
NCU_DRAM_BYTES_PER_LAYER = 30.43e6
MODEL = "qwen3-4b"
PROJS = ["q", "k", "v", "o", "gate", "up", "down"]
CONFIG_ID = 1


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured", float(d.get("sm_max_mhz", 1965.0))
    return 6650.0, "fallback", 1965.0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes(mats, x_bytes, y_bytes):
    """codes + f32 tail + f64 row scales + x + y, per GEMV, summed."""
    return sum(m.codes.size + m.tail.size * 4 + m.d_out * 8 + m.d_in * x_bytes + m.d_out * y_bytes for m in mats)


def cpu_pass(ref, mats, xs, threads):
    t0 = time.perf_counter()
    for m, x in zip(mats, xs):
        ref.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, m.tail, x, threads=threads)
    return time.perf_counter() - t0


def cpu_baseline(layers_sample=1, min_seconds=6.0, max_seconds=30.0):
    """The oracle's decode + scale + dot on all host threads, over the seven projections of
    `layers_sample` layers, repeated until min_seconds have passed."""
    from oracle import ref
    from llvq_b200 import synth
    threads = ref.hw_threads()
    mats = [m for l in range(layers_sample) for m in synth.make_layer(MODEL, CONFIG_ID, l).values()]
    xs = [synth.make_activation(m.d_in, 0x1000 + i, np.float16).astype(np.float64) for i, m in enumerate(mats)]
    nbytes = algorithmic_bytes(mats, 2, 2)
    cpu_pass(ref, mats[:1], xs[:1], threads)  # builds the tables
    times, t_start = [], time.perf_counter()
    while (time.perf_counter() - t_start < min_seconds or len(times) < 2) and time.perf_counter() - t_start < max_seconds:
        times.append(cpu_pass(ref, mats, xs, threads))
    t = statistics.median(times)
    blocks = sum(m.n_blocks for m in mats)
    return {"value": nbytes / t / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{layers_sample} layer(s) x 7 projections = {blocks} blocks, median of {len(times)} passes",
            "ns_per_block_per_core": t * threads / blocks * 1e9, "ms_per_pass": t * 1e3}, nbytes


def gemm_section(rt, torch, synth, layers=3, iters=4):
    """benchmark configuration 3: batched dequant-GEMM (tcgen05) on Qwen3-8B projection shapes, B = 16 and 64.
    `layers` distinct layers per pass (152 MB of codes) so no matrix is re-read warm."""
    shapes = synth.layer_shapes("qwen3-8b")
    projs = []
    for l in range(layers):
        for name, (do, di) in shapes.items():
            projs.append(rt.upload(synth.make_matrix(do, di, synth.matrix_seed(3, l, synth.PROJ_IDS[name])), tail_f16=True))
    blocks = sum(p.n_blocks for p in projs)
    out = {"workload": "qwen3-8b-layer-gemm", "layers_per_pass": layers, "blocks_per_pass": blocks}
    for batch in (16, 64):
        xs = {di: torch.from_numpy(synth.make_activation(di, 0x3000 + batch, np.float16, batch=batch)).cuda()
              for di in {p.d_in for p in projs}}
        ys = [torch.empty(batch, p.d_out, dtype=torch.float16, device="cuda") for p in projs]
        for _ in range(2):
            for p, y in zip(projs, ys):
                rt.forward_batch(p, xs[p.d_in], out=y)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            for p, y in zip(projs, ys):
                rt.forward_batch(p, xs[p.d_in], out=y)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        flops = sum(2.0 * batch * p.d_out * p.d_in for p in projs)
        out[f"batch{batch}"] = {"ms_per_layer": ms / layers, "gblocks_per_s": blocks / ms / 1e6,
                                "tflops": flops / ms / 1e9, "tokens_x_layers_per_s": batch * layers / (ms * 1e-3)}
    for p in projs:
        p.free()
    return out


def decode_section(rt, torch, prompt_len=128, new_tokens=256, rotations=False, embed_q8=False):
    """benchmark configuration 2: Qwen3-4B-architecture greedy decode at batch 1 (36 layers, random LLVQ codes, f16
    tied embedding, int8 KV cache), 128 random prompt tokens then 256 generated; the token step is replayed
    from a CUDA graph. tok/s counts the generated tokens over the decode phase (prefill reported apart).
    With `rotations` the same model is timed a second time with an incoherence rotation in front of every
    projection group (4 more launches per layer), as a real artifact needs; the configuration itself has none."""
    from llvq_b200.model import Qwen3Config, synthetic_model
    cfg = Qwen3Config.named(MODEL)
    t0 = time.perf_counter()
    model, _ = synthetic_model(rt, cfg, config_id=2, capacity=prompt_len + new_tokens, rotations=rotations)
    setup = time.perf_counter() - t0
    rng = np.random.default_rng(0x2C0DE)
    prompt = [int(t) for t in rng.integers(0, cfg.vocab, prompt_len)]

    def timed():
        model._graph = None
        model.generate(prompt, 4, use_graph=True)  # captures the graph
        times = []
        for _ in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            nxt = model.pick(model._rms(model.prefill(prompt), model.final_norm)[0])
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            model.start_decode(nxt, prompt_len)
            out = [int(nxt)]
            while len(out) < new_tokens:
                model._graph_step()
                out.append(int(model._tok))
            torch.cuda.synchronize()
            times.append((t1 - t0, time.perf_counter() - t1))
        prefill_s, decode_s = min(t[0] for t in times), min(t[1] for t in times)
        return {"tok_per_s": (new_tokens - 1) / decode_s, "ms_per_token": decode_s / (new_tokens - 1) * 1e3,
                "prefill_ms": prefill_s * 1e3, "prefill_tok_per_s": prompt_len / prefill_s, "distinct_tokens": len(set(out))}

    held = [{k: blk.pop(k) for k in list(blk) if k.startswith("rot_")} for blk in model.blocks]
    res = {"workload": "qwen3-4b-greedy-decode", "prompt_tokens": prompt_len, "new_tokens": new_tokens, "kv_cache": "int8 g64",
           "graph": True, "setup_s": setup}
    res.update(timed())
    if embed_q8:  # the same model with the tied embedding carried as int8 g64 (the reference's embedq payload)
        from llvq_b200.model import Q8Embedding
        f16_emb, f16_head = model.emb, model.emb_head
        model.emb = Q8Embedding.quantize(rt.lib, model.emb.dense())
        model.emb_head = model.emb
        res["with_int8_head"] = timed()
        model.emb, model.emb_head = f16_emb, f16_head
    if rotations:
        for blk, rots in zip(model.blocks, held):
            blk.update(rots)
        res["with_rotations"] = timed()
    return res


def run_reference(args):
    """Reference arm: the reference's CPU path (oracle port) on the host cores; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    times = []
    from oracle import ref
    from llvq_b200 import synth
    threads = ref.hw_threads()
    mats = list(synth.make_layer(MODEL, CONFIG_ID, 0).values())
    xs = [synth.make_activation(m.d_in, 0x1000 + i, np.float16).astype(np.float64) for i, m in enumerate(mats)]
    nbytes = algorithmic_bytes(mats, 2, 2)
    for _ in range(args.warmup):
        cpu_pass(ref, mats, xs, threads)
    for _ in range(args.steps):
        times.append(cpu_pass(ref, mats, xs, threads))
    t = sum(times) / len(times)
    val = nbytes / t / 1e9
    sample = "each step = the 7 projections of one layer (4 185 600 blocks) on all host threads"
    emit(({
        "impl": "reference", "metric": "dequant_gemv_algorithmic_GBps", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "qwen3-4b-layer-gemv", "sample": sample},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def run_tp_decode(args):
    """benchmark configuration 4: Qwen3-14B-architecture greedy decode, tensor-parallel over the ranks (q/k/v by heads, the
    other projections and the tied head by rows, NCCL all-gathers of the row shards), int8 split-KV attention over a
    long random prompt, then `new_tokens` greedy tokens at batch 1 replayed from a CUDA graph. `value` = generated
    tokens per second over the decode phase (device-timed, max over ranks); the prefill is reported apart."""
    import torch
    import torch.distributed as dist
    from llvq_b200 import FusedRuntime
    from llvq_b200.model import Qwen3Config, TpGroup, synthetic_model
    rank, local_rank = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        # a rank that dies must end its peers' next collective with an error, not leave them waiting
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=300))
    rt = FusedRuntime(local_rank)
    cfg = Qwen3Config.named("qwen3-14b")
    layers = args.layers if args.layers != 36 else cfg.layers
    prompt_len, new_tokens = args.prompt, args.new_tokens
    t0 = time.perf_counter()
    model, _ = synthetic_model(rt, cfg, config_id=4, capacity=prompt_len + new_tokens, layers=layers,
                               tp=TpGroup(peer_lib=rt.lib if args.gather == "peer" else None) if world > 1 else None,
                               keep_host=False, device_codes=True)
    torch.cuda.synchronize()
    setup = time.perf_counter() - t0
    rng = np.random.default_rng(0x4C0DE)
    prompt = [int(t) for t in rng.integers(0, cfg.vocab, prompt_len)]
    sampler = ClockSampler(local_rank) if rank == 0 else None
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e[0].record()
    nxt = model.pick(model._rms(model.prefill(prompt), model.final_norm)[0])
    e[1].record()
    torch.cuda.synchronize()
    model.start_decode(nxt, prompt_len)
    step = model._eager_step if args.no_graph else model._graph_step
    for _ in range(max(args.warmup, 3)):  # the first call captures the graph; the position moves on, as in a real run
        step()
    model.start_decode(nxt, prompt_len)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    if sampler:
        sampler.start()
    out = [int(nxt)]
    e[2].record()
    t1 = time.perf_counter()
    while len(out) < new_tokens:
        step()
        out.append(int(model._tok))  # the per-token read-back of the reference's loop
    e[3].record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t1
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([e[2].elapsed_time(e[3]), wall * 1e3, e[0].elapsed_time(e[1])], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        toks = torch.tensor(out, device="cuda")
        ref = toks.clone()
        dist.broadcast(ref, 0)
        same = torch.tensor([int(torch.equal(ref, toks))], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        ranks_agree = bool(same.item())
    else:
        ranks_agree = True
    decode_ms, wall_ms, prefill_ms = t[0].item(), t[1].item(), t[2].item()
    if rank == 0:
        gen = new_tokens - 1
        kv_bytes = 2 * layers * (prompt_len + new_tokens // 2) * cfg.n_kv * (cfg.head_dim + 2 * 2 * cfg.head_dim // 64)
        emit(({
            "metric": "decode_tok_per_s", "value": gen / (decode_ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": gen, "warmup": max(args.warmup, 3), "ms_per_step": decode_ms / gen, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "qwen3-14b-tp-greedy-decode", "layers": layers, "prompt_tokens": prompt_len,
                       "new_tokens": new_tokens, "parallelism": f"tp{world}", "kv_cache": "int8 g64, split-KV attention",
                       "attn_splits": model.attn_splits, "graph": not args.no_graph,
                       "collective": ("none" if world == 1 else "peer-memory exchange kernel (stores + flags) x4 per layer + 1 per token"
                                      if args.gather == "peer" else "nccl all_gather_into_tensor x4 per layer + 1 per token")},
            "wall_tok_per_s": gen / (wall_ms * 1e-3), "prefill_ms": prefill_ms,
            "prefill_tok_per_s": prompt_len / (prefill_ms * 1e-3), "setup_s": setup, "ranks_agree": ranks_agree,
            "peer_errors": model.tp.peer.poll_error() if model.tp and model.tp.peer else None,
            "distinct_tokens": len(set(out)), "token_checksum": int(sum((i + 1) * t for i, t in enumerate(out)) % (1 << 31)),
            "kv_bytes_read_per_token": kv_bytes, "clocks": clocks}))
    if world > 1:
        # Every collective of this rank has completed (the reductions above were read on the host). Tearing the
        # process group down while a captured graph still holds its collectives did not return on this stack,
        # so the ranks leave without it: nothing is in flight and nothing waits on a peer.
        sys.stdout.flush()
        torch.cuda.synchronize()
        os._exit(0)


def run_tp(args):
    """benchmark configuration 4 (GEMV part): Qwen3-14B projections row-sharded over the ranks, f16 activations,
    NCCL all-gather of every output the next projection needs whole (4 per layer). Strong scaling:
    the job is the same 40-layer pass at every N; `value` = whole-job algorithmic GB/s."""
    import torch
    import torch.distributed as dist
    from llvq_b200 import FusedRuntime, synth
    from llvq_b200.parallel import shard_rows
    rank, local_rank = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        # a rank that dies must end its peers' next collective with an error, not leave them waiting
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=300))
    rt = FusedRuntime(local_rank)
    shapes = synth.layer_shapes("qwen3-14b")
    layers = args.layers if args.layers != 36 else 40
    order = [["q", "k", "v"], ["o"], ["gate", "up"], ["down"]]
    per_layer, job_bytes, job_blocks = [], 0, 0
    for l in range(layers):
        row = []
        for names in order:
            ms = []
            for n in names:
                do, di = shapes[n]
                lo, hi = shard_rows(do, world, rank)
                ms.append(synth.make_matrix(hi - lo, di, synth.matrix_seed(4, l, synth.PROJ_IDS[n]) ^ (rank << 40), n))
                job_bytes += do * (di // 24) * 6 + do * (di % 24) * 4 + do * 8 + do * 2
                job_blocks += do * (di // 24)
            job_bytes += shapes[names[0]][1] * 2
            proj = rt.upload_group(ms, tail_f16=True) if len(ms) > 1 else rt.upload(ms[0], tail_f16=True)
            full = sum(shapes[n][0] for n in names)
            row.append((proj, torch.empty(proj.d_out, dtype=torch.float16, device="cuda"),
                        torch.empty(proj.d_out * world, dtype=torch.float16, device="cuda"), full))
        per_layer.append(row)
    x_h = torch.from_numpy(synth.make_activation(5120, 0x4000, np.float16)).cuda()
    x_i = torch.from_numpy(synth.make_activation(17408, 0x4001, np.float16)).cuda()
    # the gathers of one layer: q|k|v -> context, o, gate|up -> SwiGLU product, down (all needed whole by what follows);
    # through peer memory by default (one site per gather of a layer), NCCL with --gather nccl
    peer = None
    if world > 1 and args.gather == "peer":
        from llvq_b200.parallel import PeerExchange
        peer = PeerExchange(rt.lib, local_rank, [row[gi][2].numel() * 2 for gi in range(4) for row in per_layer[:1]])

    def pass_once():
        for row in per_layer:
            for gi, (proj, y_loc, y_all, _full) in enumerate(row):
                rt.forward(proj, x_i if gi == 3 else x_h, out=y_loc)
                if peer is not None:
                    peer.exchange(gi, y_loc)
                elif world > 1:
                    dist.all_gather_into_tensor(y_all, y_loc)

    # one captured graph per rank, as the decode loop runs it: launch cost is not what is being measured
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        pass_once()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pass_once()

    def step():
        graph.replay()

    for _ in range(max(args.warmup, 3)):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    if rank == 0:
        peak, peak_kind, _ = measured_peaks()
        gbs = job_bytes / (ms * 1e-3) / 1e9
        emit(({
            "metric": "dequant_gemv_algorithmic_GBps", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "qwen3-14b-tp-layer-gemv", "layers_per_step": layers, "parallelism": f"tp{world}",
                       "collective": ("none" if world == 1 else "peer-memory exchange kernel x4 per layer" if peer is not None
                                      else "nccl all_gather_into_tensor x4 per layer"),
                       "blocks_per_step": job_blocks, "algorithmic_bytes_per_step": job_bytes},
            "token_equiv_per_s": (layers / 40.0) / (ms * 1e-3), "gblocks_per_s": job_blocks / (ms * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s", "frac": gbs / world / peak,
                         "traffic": None, "peak_kind": f"of {peak_kind}"},
            "peer_errors": peer.poll_error() if peer is not None else None, "graph": True}))
    if world > 1:
        # as in run_tp_decode: every collective has completed and been read; the ranks leave without tearing
        # the process group down under a captured graph
        sys.stdout.flush()
        torch.cuda.synchronize()
        os._exit(0)


_RESULT_FD = None


def _own_stdout():
    """The contract is ONE JSON line on stdout. Libraries write there too (NCCL prints a version banner at its
    VERSION and WARN debug levels), so the process keeps a private duplicate of stdout for the result and points
    file descriptor 1 at stderr for everything else."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(obj) -> None:
    line = (json.dumps(obj) + "\n").encode()
    sys.stdout.flush()
    if _RESULT_FD is None:
        os.write(1, line)
    else:
        os.write(_RESULT_FD, line)


def main():
    _own_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", action="store_true",
                    help="tensor-parallel mode: Qwen3-14B projections row-sharded over the ranks with all-gathers")
    ap.add_argument("--tp-decode", action="store_true",
                    help="config 4: Qwen3-14B tensor-parallel greedy decode over the ranks (prompt --prompt, --new-tokens)")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="--tp / --tp-decode: all-gathers of the row shards through peer memory (llvq_tp_exchange) or NCCL")
    ap.add_argument("--no-graph", action="store_true", help="--tp-decode: launch every token step eagerly")
    ap.add_argument("--prompt", type=int, default=32768)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=36, help="distinct layers per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gemm", action="store_true", help="skip the batched-GEMM (config 3) side measurement")
    ap.add_argument("--no-decode", action="store_true", help="skip the greedy-decode (config 2) side measurement")
    ap.add_argument("--embed-q8", action="store_true",
                    help="time the config-2 decode a second time with the tied embedding / head carried as int8 g64")
    ap.add_argument("--rotations", action="store_true",
                    help="time the config-2 decode a second time with an activation rotation per projection group")
    ap.add_argument("--no-groups", action="store_true",
                    help="launch q, k, v and gate, up separately instead of row-concatenated")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.tp_decode:
        return run_tp_decode(args)
    if args.tp:
        return run_tp(args)

    import torch
    import torch.distributed as dist
    from llvq_b200 import FusedRuntime, _lib, synth

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the measured path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # a rank that dies must end its peers' next collective with an error, not leave them waiting
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=300))
    rt = FusedRuntime(local_rank)
    lib = _lib.load()

    # Weak scaling: every rank holds its own `layers` distinct layers (no data-path collective;
    # the projections of different layers are independent units).
    t_gen = time.perf_counter()
    projs, xs_host, mats_meta = [], [], []
    # q|k|v and gate|up read the same activation, so each group is one row-concatenated launch
    # (llvq_matrix_upload_group); the seven projections are all computed either way.
    groups = [[n] for n in PROJS] if args.no_groups else [["q", "k", "v"], ["o"], ["gate", "up"], ["down"]]
    for l in range(args.layers):
        layer = synth.make_layer(MODEL, CONFIG_ID, rank * 1000 + l)
        for names in groups:
            ms = [layer[n] for n in names]
            projs.append(rt.upload_group(ms, tail_f16=True) if len(ms) > 1 else rt.upload(ms[0], tail_f16=True))
            mats_meta.append((sum(m.codes.size for m in ms), sum(m.tail.size for m in ms), sum(m.d_out for m in ms),
                              ms[0].d_in))
            xs_host.append(torch.from_numpy(synth.make_activation(ms[0].d_in, 0x2000 + len(xs_host), np.float16)).pin_memory())
    gen_s = time.perf_counter() - t_gen
    xs_dev = [x.cuda() for x in xs_host]
    ys_dev = [torch.empty(p.d_out, dtype=torch.float16, device="cuda") for p in projs]
    ys_host = [torch.empty(p.d_out, dtype=torch.float16).pin_memory() for p in projs]
    step_bytes = sum(c + t * 4 + do * 8 + di * 2 + do * 2 for c, t, do, di in mats_meta)
    step_blocks = sum(p.n_blocks for p in projs)
    codes_bytes = sum(c for c, _, _, _ in mats_meta)

    def step_device():
        for p, x, y in zip(projs, xs_dev, ys_dev):
            rt.forward(p, x, out=y)

    xs_np, ys_np = [x.numpy() for x in xs_host], [y.numpy() for y in ys_host]

    def step_e2e():
        # the C ABI call a host-side plugin makes for one token: every projection's x copied in from
        # pinned host memory, its GEMV, its y copied back, one synchronisation at the end
        rt.forward_host_many(projs, xs_np, ys_np)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    for _ in range(max(args.warmup, 3)):
        step_device()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = lib.llvq_launch_count()
    ms_total = timed(step_device, args.steps)
    launches = lib.llvq_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    assert not rt.poll_range_error(), "a synthetic index fell outside the ball"

    for _ in range(2):
        step_e2e()
    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e = timed(step_e2e, e2e_steps)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_step = ms_total / args.steps
    value = world * step_bytes / (ms_step * 1e-3) / 1e9
    e2e_value = world * step_bytes / (ms_e2e / e2e_steps * 1e-3) / 1e9
    peak, peak_kind, sm_max = measured_peaks()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    per_gpu_gbs = step_bytes / (ms_step * 1e-3) / 1e9
    # Two-term roofline of the path: T_roof = max(T_bytes, T_alu) with the agreed algorithmic
    # decode work of 184 lane-operations per block on SMs x 128 lanes at the max SM clock.
    t_bytes = step_bytes / (peak * 1e9)
    t_alu = step_blocks * 184.0 / (sms * 128 * sm_max * 1e6)
    out = {
        "metric": "dequant_gemv_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "qwen3-4b-layer-gemv", "layers_per_step": args.layers, "projections_per_step": 7 * args.layers,
                   "launches_per_step": len(projs), "grouping": "none" if args.no_groups else "q|k|v, o, gate|up, down",
                   "blocks_per_step": step_blocks, "algorithmic_bytes_per_step": step_bytes, "activations": "f16",
                   "l2": "every step streams %.0f MB of distinct codes (> 126 MB L2)" % (codes_bytes / 1e6),
                   "parallelism": f"replicas x{world}" if world > 1 else "single"},
        "token_equiv_per_s": world * (args.layers / 36.0) / (ms_step * 1e-3),
        "gblocks_per_s": world * step_blocks / (ms_step * 1e-3) / 1e9,
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                     "traffic": (NCU_DRAM_BYTES_PER_LAYER * args.layers / len(projs)) if not args.no_groups else None,
                     "algorithmic_bytes_per_launch": step_bytes / len(projs), "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBps": per_gpu_gbs / 8000.0,
                     "kernel": "gemv", "launches": launches, "avg_launch_us": ms_total * 1e3 / max(launches, 1),
                     "two_term": {"t_bytes_ms": t_bytes * 1e3, "t_alu_ms": t_alu * 1e3,
                                  "frac": max(t_bytes, t_alu) * 1e3 / ms_step, "ops_per_block": 184}},
        "e2e": {"value": e2e_value, "unit": "GB/s",
                "h2d_bytes_per_step": sum(di * 2 for _, _, _, di in mats_meta),
                "d2h_bytes_per_step": sum(do * 2 for _, _, do, _ in mats_meta), "ms_per_step": ms_e2e / e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks, "setup_s": gen_s,
    }
    for p in projs:
        p.free()
    # side measurements of the single-GPU configurations (3: batched GEMM, 2: greedy decode) and the CPU baseline
    # belong to the N = 1 line; a multi-rank run reports the replicated GEMV pass only
    if not args.no_gemm and world == 1:
        out["gemm"] = gemm_section(rt, torch, synth)
    if not args.no_decode and world == 1:
        out["decode"] = decode_section(rt, torch, rotations=args.rotations, embed_q8=args.embed_q8)
    if not args.no_cpu_baseline and world == 1:
        cb, _ = cpu_baseline()
        out["cpu_baseline"] = cb
    emit(out)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
