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
metric through the host-buffer C ABI call (every x copied in from pinned host memory
and every y copied back inside the timed region); `roofline` for the GEMV kernel;
`cpu_baseline` = the CPU oracle (the C++ restatement of the reference's Rust path)
timed on this box's host cores on a bounded sample; `gemm` = configuration 3 (batched
GEMM), `decode` = configuration 2 (greedy decode, with the token step split by phase),
`tp` = configuration 4 on the ranks of the run (row-sharded GEMV pass and tensor-parallel
decode; tp1 figures at N = 1). `--impl reference` times the CPU path alone, as the
reference arm, and adds as a side measurement the reference's own serving kernel on its
transcoded layout where that kernel was built from the reference's sources.
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

def ncu_dram_bytes_per_launch():
    """DRAM bytes (read + write) per GEMV launch of one Qwen3-4B layer, from the tracked summary of the ncu
    capture of this kernel (profiles/*.json, written when the profile is refreshed); None when it is missing."""
    path = os.path.join(ROOT, "profiles", "gemv_dram_traffic.json")
    try:
        d = json.load(open(path))
        return float(d["dram_bytes_per_layer"]) / float(d["launches_per_layer"])
    except (OSError, KeyError, ValueError):
        return None


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
        # the token step by phase, each phase's launches replayed apart at the last position (ms per token)
        model._pos -= 1
        phases = {k: round(v, 4) for k, v in model.phase_split().items()}
        model._pos += 1
        return {"tok_per_s": (new_tokens - 1) / decode_s, "ms_per_token": decode_s / (new_tokens - 1) * 1e3,
                "prefill_ms": prefill_s * 1e3, "prefill_tok_per_s": prompt_len / prefill_s, "distinct_tokens": len(set(out)),
                "phases_ms": phases}

    held = [{k: blk.pop(k) for k in list(blk) if k.startswith("rot_")} for blk in model.blocks]
    res = {"workload": "qwen3-4b-greedy-decode", "prompt_tokens": prompt_len, "new_tokens": new_tokens, "kv_cache": "int8 g64",
           "graph": True, "setup_s": setup,
           "deviations": "norm weights are 1 + N(0, 0.02) (the configuration says N(0, 0.02)) so that activations keep their "
                         "scale; with random weights the greedy loop settles on very few distinct tokens (see distinct_tokens)"}
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


def verify_before_timing(rt, torch, synth, rank):
    """Every row of one projection group per shape is checked against the f64 CPU reference before the clock
    starts, as the reference's kernel bench does (llvq-cuda/src/bin/matvec.rs:582-602): the four grouped launches
    of layer `rank * 1000` (the first one timed), f16 activations, relative L2 against the 1e-3 of the f16 path."""
    from oracle import ref
    layer = synth.make_layer(MODEL, CONFIG_ID, rank * 1000)
    worst = 0.0
    for gi, names in enumerate((["q", "k", "v"], ["o"], ["gate", "up"], ["down"])):
        ms = [layer[n] for n in names]
        proj = rt.upload_group(ms, tail_f16=True) if len(ms) > 1 else rt.upload(ms[0], tail_f16=True)
        x = synth.make_activation(ms[0].d_in, 0x2000 + gi, np.float16)
        y = rt.forward(proj, torch.from_numpy(x).cuda()).float().cpu().numpy().astype(np.float64)
        want = np.concatenate([ref.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales,
                                            m.tail.astype(np.float16).astype(np.float32), x.astype(np.float64)) for m in ms])
        rel = float(np.linalg.norm(y - want) / max(np.linalg.norm(want), 1e-300))
        proj.free()
        if not rel <= 1e-3:
            raise SystemExit(f"bench: group {'|'.join(names)} differs from the CPU reference (relative L2 {rel:.3g}); not timing")
        worst = max(worst, rel)
    return {"groups": 4, "rows": int(sum(layer[n].d_out for n in PROJS)), "worst_rel_l2": worst, "tolerance": 1e-3}


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
    blocks = sum(m.n_blocks for m in mats)
    gpu_kernel = reference_gpu_kernel(args)
    emit(({
        "impl": "reference", "metric": "dequant_gemv_algorithmic_GBps", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        # the keys of the GPU arm's config, with this arm's bounded sample (one layer per step instead of 36)
        "config": {"workload": "qwen3-4b-layer-gemv", "layers_per_step": 1, "projections_per_step": 7,
                   "launches_per_step": 0, "grouping": "none", "blocks_per_step": blocks,
                   "algorithmic_bytes_per_step": nbytes, "activations": "f16",
                   "l2": "host caches; each step decodes 25 MB of codes", "parallelism": "single", "sample": sample},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        # the reference's own serving kernel on its transcoded layout, where it was built (oracle/_ref): a side
        # measurement of another format on this GPU, not the path of `value`
        "reference_gpu_kernel": gpu_kernel,
    }))


def reference_gpu_kernel(args, layers=4):
    """The reference's serving GEMV (`tv_planes_h`, llvq-llm/kernels/tv_planes_h.cu:38-72, compiled by nvcc from the
    reference's sources into oracle/_ref/libref_planes.so) on its Planes14 layout (14 bytes per block, written from the
    same archive codes by oracle/planes14.py, the reference's own transcoder being Rust): one launch per projection,
    `layers` distinct layers of the Qwen3-4B shapes (235 MB of records per pass, larger than L2), f32 activations in and
    f16 out as its forward_rotated; device-timed. Reported with its parity against the f64 CPU reference."""
    try:
        import torch
        from oracle import planes14, ref
        from llvq_b200 import synth
        if not planes14.available():
            return {"unavailable": "oracle/_ref/libref_planes.so is not built (no checkout of the reference where the tree was built)"}
        if not torch.cuda.is_available():
            return {"unavailable": "no CUDA device"}
        runner = planes14.Planes14Runner(0)
        hs, xs, worst = [], [], 0.0
        for l in range(layers):
            for i, (name, m) in enumerate(synth.make_layer(MODEL, CONFIG_ID, l).items()):
                h = runner.upload(m)
                x = torch.from_numpy(synth.make_activation(m.d_in, 0x1000 + i, np.float32)).cuda()
                if l == 0:  # every projection shape once against the CPU reference, before anything is timed
                    y = runner.forward(h, x).float().cpu().numpy().astype(np.float64)
                    want = ref.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales,
                                        m.tail.astype(np.float16).astype(np.float32), x.cpu().numpy().astype(np.float64))
                    worst = max(worst, float(np.linalg.norm(y - want) / np.linalg.norm(want)))
                hs.append(h)
                xs.append(x)
        if not worst <= 1e-3:
            return {"unavailable": f"the reference kernel's result differs from the CPU reference (relative L2 {worst:.3g})"}
        ys = [torch.empty(h["d_out"], dtype=torch.float16, device="cuda") for h in hs]

        def run():
            for h, x, y in zip(hs, xs, ys):
                runner.forward(h, x, out=y)
        for _ in range(max(args.warmup, 3)):
            run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(max(args.steps, 5)):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / max(args.steps, 5)
        blocks = sum(h["d_out"] * h["nb"] for h in hs)
        return {"kernel": "tv_planes_h (reference, Planes14 layout, 14 bytes per block)", "layers_per_pass": layers,
                "launches_per_pass": len(hs), "ms_per_pass": ms, "gblocks_per_s": blocks / ms / 1e6,
                "layout_bytes_GBps": blocks * 14 / ms / 1e6, "archive_code_equiv_GBps": blocks * 6.54 / ms / 1e6,
                "worst_rel_l2_vs_cpu_reference": worst}
    except Exception as e:  # a side measurement must not take the arm down
        return {"unavailable": f"{type(e).__name__}: {e}"}


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


def tp_block(args, rt, torch, dist, world, rank, local_rank):
    """benchmark configuration 4 inside the line the driver runs: the Qwen3-14B-architecture model with its output rows
    sharded over the `world` ranks of this run (q/k/v by heads, the other projections and the tied head by rows; the
    same matrices at every N), measured twice: `gemv` = one pass over the 4 x 40 projection groups with the gather
    that follows each of them in a token step (captured in one CUDA graph per rank), `decode` = a 32 768-token
    prompt into the int8 KV cache, then 128 greedy tokens replayed from a graph. Strong scaling: the job does not
    change with N, so the N = 1 run of this same function gives the tp1 figures. Before any timing, every rank
    checks 64 rows of each of its shards against the CPU reference, and rank 0 checks rows it received through the
    gather against its own unsharded computation of the same rows, bit for bit."""
    from oracle import ref
    from llvq_b200 import synth
    from llvq_b200.model import Qwen3Config, TpGroup, synthetic_model, tp_rows
    cfg = Qwen3Config.named("qwen3-14b")
    layers = cfg.layers
    prompt_len, new_tokens = args.prompt, args.new_tokens
    t0 = time.perf_counter()
    model, _ = synthetic_model(rt, cfg, config_id=4, capacity=prompt_len + new_tokens, layers=layers,
                               tp=TpGroup(peer_lib=rt.lib if args.gather == "peer" else None) if world > 1 else None,
                               keep_host=False, device_codes=True)
    torch.cuda.synchronize()
    setup = time.perf_counter() - t0
    tp = model.tp
    hd = cfg.head_dim
    x_h = torch.from_numpy(synth.make_activation(cfg.hidden, 0x4000, np.float16)).cuda()
    x_i = torch.from_numpy(synth.make_activation(cfg.inter, 0x4001, np.float16)).cuda()
    shapes = {"q": (cfg.n_heads * hd, cfg.hidden), "k": (cfg.n_kv * hd, cfg.hidden), "v": (cfg.n_kv * hd, cfg.hidden),
              "o": (cfg.hidden, cfg.n_heads * hd), "gate": (cfg.inter, cfg.hidden), "up": (cfg.inter, cfg.hidden),
              "down": (cfg.hidden, cfg.inter)}
    rows = tp_rows(cfg, world, rank)

    # ---- verification, layer 0 ----
    def tile_rows(name, lo, n):
        """rows [lo, lo + n) of layer 0's projection `name`, as the model drew them (tiles of d_out / 8 rows)."""
        do, di = shapes[name]
        per = do // 8
        t = lo // per
        m = synth.make_matrix_rows_cuda(do, di, synth.matrix_seed(4, 0, synth.PROJ_IDS[name]), t * per, (t + 1) * per,
                                        device=torch.device("cuda", local_rank))
        return m.rows(lo - t * per, lo - t * per + n)

    blk0 = model.blocks[0]
    groups = (("qkv", ["q", "k", "v"], x_h), ("o", ["o"], x_h), ("gate_up", ["gate", "up"], x_h), ("down", ["down"], x_i))
    worst = 0.0
    for gname, names, x in groups:
        y = rt.forward(blk0[gname], x).float().cpu().numpy().astype(np.float64)
        at = 0
        for n in names:
            lo, hi = rows[n]
            m = tile_rows(n, lo, 64)
            want = ref.gemv_f64(m.codes, 64, m.d_in, m.centroids, m.row_scales, m.tail.astype(np.float16).astype(np.float32),
                                x.cpu().numpy().astype(np.float64))
            rel = float(np.linalg.norm(y[at:at + 64] - want) / max(np.linalg.norm(want), 1e-300))
            if not rel <= 1e-3:
                raise SystemExit(f"bench: rank {rank} shard of {n} differs from the CPU reference (relative L2 {rel:.3g})")
            worst = max(worst, rel)
            at += hi - lo
    gathered_ok = None
    if tp is not None:
        # rows of the LAST rank's o shard, as they arrive in this rank's gathered buffer, against a local GEMV
        # of the same rows: rows do not interact, so the bits must agree
        o_loc = rt.forward(blk0["o"], x_h, out=model._o_loc)
        tp.gather_into(1, model._o, o_loc)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        lo_last = tp_rows(cfg, world, world - 1)["o"][0]
        m = tile_rows("o", lo_last, 64)
        p64 = rt.upload(m, tail_f16=True)
        mine = rt.forward(p64, x_h)
        gathered_ok = bool(torch.equal(mine, model._o[lo_last:lo_last + 64]))
        p64.free()
        if not gathered_ok:
            raise SystemExit(f"bench: rank {rank}: gathered rows of the o projection differ from the unsharded GEMV")

    # ---- the GEMV pass: 4 projection groups + 4 gathers per layer, as a token step issues them ----
    q_loc, i_loc = model.h_loc * hd, model.inter_loc

    def pass_once():
        for blk in model.blocks:
            rt.forward(blk["qkv"], x_h, out=model._qkv)
            if tp is not None:
                tp.gather_into(0, model._ctx, model._qkv[:q_loc])
            rt.forward(blk["o"], x_h, out=model._o_loc)
            if tp is not None:
                tp.gather_into(1, model._o, model._o_loc)
            rt.forward(blk["gate_up"], x_h, out=model._gu)
            if tp is not None:
                tp.gather_into(2, model._act, model._gu[:i_loc])
            rt.forward(blk["down"], x_i, out=model._down_loc)
            if tp is not None:
                tp.gather_into(3, model._down, model._down_loc)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        pass_once()
    torch.cuda.current_stream().wait_stream(side)
    sync_all()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pass_once()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    sync_all()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_pass = t.item()
    job_bytes = job_blocks = 0
    for names, d_in in ((["q", "k", "v"], cfg.hidden), (["o"], cfg.n_heads * hd), (["gate", "up"], cfg.hidden), (["down"], cfg.inter)):
        job_bytes += d_in * 2
        for n in names:
            do, di = shapes[n]
            job_bytes += do * (di // 24) * 6 + do * (di % 24) * 4 + do * 8 + do * 2
            job_blocks += do * (di // 24)
    job_bytes *= layers
    job_blocks *= layers
    collective = ("none" if world == 1 else "peer-memory exchange kernel (stores + flags), 4 per layer" if args.gather == "peer"
                  else "nccl all_gather_into_tensor, 4 per layer")
    gemv = {"workload": "qwen3-14b-tp-layer-gemv", "layers_per_pass": layers, "ms_per_pass": ms_pass,
            "value": job_bytes / (ms_pass * 1e-3) / 1e9, "unit": "GB/s (whole job, algorithmic)",
            "gblocks_per_s": job_blocks / (ms_pass * 1e-3) / 1e9, "blocks_per_pass": job_blocks,
            "algorithmic_bytes_per_pass": job_bytes, "collective": collective, "graph": True, "steps": args.steps}

    # ---- the greedy decode ----
    rng = np.random.default_rng(0x4C0DE)
    prompt = [int(tk) for tk in rng.integers(0, cfg.vocab, prompt_len)]
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    sync_all()
    ev[0].record()
    nxt = model.pick(model._rms(model.prefill(prompt), model.final_norm)[0])
    ev[1].record()
    torch.cuda.synchronize()
    model.start_decode(nxt, prompt_len)
    for _ in range(3):  # the first call captures the graph; the position moves on, as in a real run
        model._graph_step()
    model.start_decode(nxt, prompt_len)
    sync_all()
    out = [int(nxt)]
    ev[2].record()
    while len(out) < new_tokens:
        model._graph_step()
        out.append(int(model._tok))  # the per-token read-back of the reference's loop
    ev[3].record()
    torch.cuda.synchronize()
    t = torch.tensor([ev[2].elapsed_time(ev[3]), ev[0].elapsed_time(ev[1])], device="cuda")
    ranks_agree = True
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        toks = torch.tensor(out, device="cuda")
        first = toks.clone()
        dist.broadcast(first, 0)
        same = torch.tensor([int(torch.equal(first, toks))], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        ranks_agree = bool(same.item())
    decode_ms, prefill_ms = t[0].item(), t[1].item()
    gen = new_tokens - 1
    decode = {"workload": "qwen3-14b-tp-greedy-decode", "prompt_tokens": prompt_len, "new_tokens": new_tokens,
              "tok_per_s": gen / (decode_ms * 1e-3), "ms_per_token": decode_ms / gen, "prefill_ms": prefill_ms,
              "kv_cache": "int8 g64, split-KV attention", "attn_splits": model.attn_splits, "graph": True,
              "collective": collective + (", 1 per token" if world > 1 else ""), "ranks_agree": ranks_agree,
              "distinct_tokens": len(set(out)),
              "token_checksum": int(sum((i + 1) * tk for i, tk in enumerate(out)) % (1 << 31))}
    peer_errors = tp.peer.poll_error() if tp is not None and tp.peer is not None else None
    return {"parallelism": f"tp{world}", "scaling": "strong", "setup_s": setup, "gemv": gemv, "decode": decode,
            "peer_errors": peer_errors,
            "verified_before_timing": {"shard_rows_vs_cpu_reference": 64 * 7, "worst_rel_l2": worst, "tolerance": 1e-3,
                                       "gathered_rows_bit_exact": gathered_ok}}


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
    ap.add_argument("--pass-eager", action="store_true",
                    help="the GEMV pass as one library call per projection from Python instead of a replayed CUDA graph")
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
    ap.add_argument("--no-tp", action="store_true",
                    help="skip the tensor-parallel block (configuration 4: Qwen3-14B sharded over the ranks of this run)")
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
        # NVLS off for the peer-memory gathers (plain peer stores); the communicator-init lines of NCCL's INFO log
        # show how many ranks joined
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("NCCL_DEBUG", "INFO")
        os.environ.setdefault("NCCL_DEBUG_SUBSYS", "INIT")
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

    verified = verify_before_timing(rt, torch, synth, rank) if rank == 0 else None

    # clocks and throttle reasons are sampled (100 ms apart) from before the warm-up to the end of the timed passes:
    # the warm-up runs the same passes, at least W of them and for at least 0.6 s, so that the samples see the load
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # the pass is replayed from a captured CUDA graph, as the decode loop replays its token step (--pass-eager:
    # one library call per projection from Python instead); the launches of a replay are those of its capture
    step_timed, launches_per_step = step_device, None
    if not args.pass_eager:
        step_device()
        torch.cuda.synchronize()
        launches0 = lib.llvq_launch_count()
        pass_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(pass_graph):
            step_device()
        launches_per_step = lib.llvq_launch_count() - launches0
        step_timed = pass_graph.replay
    t_warm, n_warm = time.perf_counter(), 0
    while n_warm < max(args.warmup, 3) or time.perf_counter() - t_warm < 0.6:
        step_timed()
        n_warm += 1
        if n_warm % 8 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    launches0 = lib.llvq_launch_count()
    ms_total = timed(step_timed, args.steps)
    launches = lib.llvq_launch_count() - launches0 if launches_per_step is None else launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    assert not rt.poll_range_error(), "a synthetic index fell outside the ball"

    for _ in range(2):
        step_e2e()
    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e = timed(step_e2e, e2e_steps)

    for p in projs:
        p.free()
    projs_n = len(projs)
    del xs_dev, ys_dev
    torch.cuda.empty_cache()
    # configuration 4 (tensor parallel over the ranks of this run; tp1 figures at N = 1): every rank takes part
    tp_res = None if args.no_tp else tp_block(args, rt, torch, dist, world, rank, local_rank)

    if rank != 0:
        if world > 1:
            sys.stdout.flush()
            torch.cuda.synchronize()
            os._exit(0)
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
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 activations in and out; int8 x int8 dot products (dp4a), f32 scaling",
        "data": "synthetic",
        "config": {"workload": "qwen3-4b-layer-gemv", "layers_per_step": args.layers, "projections_per_step": 7 * args.layers,
                   "launches_per_step": projs_n, "grouping": "none" if args.no_groups else "q|k|v, o, gate|up, down",
                   "launched_as": "one library call per projection" if args.pass_eager else "a captured CUDA graph of the pass, replayed per step",
                   "blocks_per_step": step_blocks, "algorithmic_bytes_per_step": step_bytes, "activations": "f16",
                   "l2": "every step streams %.0f MB of distinct codes (> 126 MB L2)" % (codes_bytes / 1e6),
                   "parallelism": f"replicas x{world}" if world > 1 else "single"},
        "token_equiv_per_s": world * (args.layers / 36.0) / (ms_step * 1e-3),
        "gblocks_per_s": world * step_blocks / (ms_step * 1e-3) / 1e9,
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                     "traffic": ncu_dram_bytes_per_launch() if not args.no_groups else None,
                     "algorithmic_bytes_per_launch": step_bytes / projs_n, "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBps": per_gpu_gbs / 8000.0,
                     "kernel": "gemv", "launches": launches, "avg_launch_us": ms_total * 1e3 / max(launches, 1),
                     "two_term": {"t_bytes_ms": t_bytes * 1e3, "t_alu_ms": t_alu * 1e3,
                                  "frac": max(t_bytes, t_alu) * 1e3 / ms_step, "ops_per_block": 184}},
        "e2e": {"value": e2e_value, "unit": "GB/s",
                "h2d_bytes_per_step": sum(di * 2 for _, _, _, di in mats_meta),
                "d2h_bytes_per_step": sum(do * 2 for _, _, do, _ in mats_meta), "ms_per_step": ms_e2e / e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks, "setup_s": gen_s, "verified_before_timing": verified,
        "kernels": [{"name": n, "registers": r, "local_bytes": lb} for n, r, lb, _, _ in rt.kernel_info()],
    }
    # side measurements of the single-GPU configurations (3: batched GEMM, 2: greedy decode) and the CPU baseline
    # belong to the N = 1 line; a multi-rank run reports the replicated GEMV pass only
    if not args.no_gemm and world == 1:
        out["gemm"] = gemm_section(rt, torch, synth)
    if not args.no_decode and world == 1:
        out["decode"] = decode_section(rt, torch, rotations=args.rotations, embed_q8=args.embed_q8)
    if not args.no_cpu_baseline and world == 1:
        cb, _ = cpu_baseline()
        out["cpu_baseline"] = cb
    if not args.no_tp:
        out["tp"] = tp_res
    emit(out)
    if world > 1:
        # every collective has completed and been read on the host; the ranks leave without tearing the process
        # group down under captured graphs (see run_tp_decode)
        sys.stdout.flush()
        torch.cuda.synchronize()
        os._exit(0)


if __name__ == "__main__":
    main()
