"""End-to-end gate of the decode loop: the same greedy loop run on fused projections and on dense
weights decoded by the CPU oracle must produce the same tokens (the reference's own gate,
llvq-llm/src/bin/fusedrun.rs:263-278), on a small Qwen3-shaped model."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dense_model(rt, oracle, cfg, mats, fused, capacity, kv_int8):
    import torch
    from llvq_b200.model import FusedQwen3
    dev = fused.device

    def dense(ms):
        rows = []
        for m in ms:
            w = oracle.decode_matrix(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales,
                                     m.tail.astype(np.float16).astype(np.float32))
            rows.append(torch.from_numpy(w))
        return torch.cat(rows).to(dev).half()

    blocks = []
    for blk, m in zip(fused.blocks, mats):
        d = dict(blk)
        d["qkv"], d["o"] = dense([m["q"], m["k"], m["v"]]), dense([m["o"]])
        d["gate_up"], d["down"] = dense([m["gate"], m["up"]]), dense([m["down"]])
        blocks.append(d)
    lin = torch.nn.functional.linear
    return FusedQwen3(cfg, blocks, fused.embed, fused.final_norm, capacity,
                      gemv=lambda w, x: lin(x.float(), w.float()).half(),
                      gemm=lambda w, x: lin(x.float(), w.float()).half(), head=fused.head, kv_int8=kv_int8,
                      rotate=fused.rotate, gemv_rotated=lambda w, xr, out=None: lin(xr, w.float()).half())


@pytest.mark.parametrize("kv_int8,rotations,embed_q8", [(True, False, False), (False, False, False), (True, True, False),
                                                        (True, False, True)])
def test_greedy_tokens_match_the_dense_decoded_run(rt, oracle, kv_int8, rotations, embed_q8):
    import torch
    from llvq_b200.model import Qwen3Config, synthetic_model
    # widths 256 (power of two: no odd mix) and 496 = 16 * 31 (the largest odd factors the rotation serves)
    cfg = Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 16, n_heads=4, n_kv=2, head_dim=64, layers=2, vocab=512)
    capacity = 64
    # row scales 40 times the configurations': the blocks then dominate the residual stream and the generated tokens
    # vary (with the plain scales a random model repeats one token, which most bugs past the first step survive)
    fused, mats = synthetic_model(rt, cfg, config_id=2, capacity=capacity, kv_int8=kv_int8, rotations=rotations, embed_q8=embed_q8,
                                  row_scale_gain=40.0)
    dense = _dense_model(rt, oracle, cfg, mats, fused, capacity, kv_int8)
    g = np.random.default_rng(5)
    prompt = [int(t) for t in g.integers(0, cfg.vocab, 20)]  # 20 >= 16: the prefill takes the tensor-core GEMM
    want = dense.generate(prompt, 24)
    got = fused.generate(prompt, 24)
    assert len(got) == 24 and all(0 <= t < cfg.vocab for t in got)
    assert len(set(want)) > 4, f"the dense run emits only {len(set(want))} distinct tokens: {want}"
    first_diff = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), None)
    assert first_diff is None, f"first divergence at token {first_diff}: {got} vs {want}"
    # the logits behind EVERY generated token agree closely, not just their argmax: both models re-read the
    # sequence so far (prompt + the tokens generated up to that step)
    for step in range(len(got)):
        seq = torch.tensor(prompt + got[:step], device=fused.device)
        lf = fused.logits_last(fused.hidden(seq, fused.positions[:seq.numel()]))
        ld = dense.logits_last(dense.hidden(seq, dense.positions[:seq.numel()]))
        # (the dense run holds its weights rounded to f16 and the amplified row scales carry that rounding
        # through two blocks: 2e-2 here, against 5e-3 at the configurations' own scales)
        assert ((lf - ld).norm() / ld.norm()).item() < 2e-2, step
        assert int(ld.argmax()) == want[step]
    assert not rt.poll_range_error()


def test_fused_decode_kernels_agree_with_the_tensor_op_step(rt):
    """Same model, token step once as four fused kernels per block and once as torch ops."""
    import torch
    from llvq_b200.model import Qwen3Config, synthetic_model
    for hd, heads, kv in ((64, 4, 2), (128, 4, 1)):
        cfg = Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 8, n_heads=heads, n_kv=kv, head_dim=hd, layers=2, vocab=512)
        prompt = list(range(40, 60))
        a, _ = synthetic_model(rt, cfg, config_id=2, capacity=64, fused_ops=True)
        b, _ = synthetic_model(rt, cfg, config_id=2, capacity=64, fused_ops=False)
        assert a.ops is not None and b.ops is None
        assert a.generate(prompt, 20) == b.generate(prompt, 20)
        # the hidden state after the step, not only the argmax
        a.start_decode(torch.tensor(7, device=a.device), 30)
        b.start_decode(torch.tensor(7, device=b.device), 30)
        a._fused_step()
        xb = b.hidden(torch.tensor([7], device=b.device), torch.tensor([30], device=b.device))
        ha = a._h.float()
        hb = b._rms(xb[-1:], b.final_norm)[0].float()
        assert ((ha - hb).norm() / hb.norm()).item() < 5e-3


def test_graph_replay_gives_the_eager_tokens(rt):
    from llvq_b200.model import Qwen3Config, synthetic_model
    cfg = Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 8, n_heads=4, n_kv=2, head_dim=64, layers=2, vocab=512)
    prompt = list(range(3, 23))
    a, _ = synthetic_model(rt, cfg, config_id=2, capacity=64)
    eager = a.generate(prompt, 16)
    b, _ = synthetic_model(rt, cfg, config_id=2, capacity=64)
    graphed = b.generate(prompt, 16, use_graph=True)
    assert eager == graphed
    assert b.generate(prompt, 16, use_graph=True) == eager  # a second generation replays the same graph
    assert a.generate(prompt, 0) == []


def test_phase_split_times_every_phase_and_leaves_the_model_untouched(rt):
    """phase_split replays each phase's launches apart (graphs of their own): every phase of a single-GPU step is
    reported, the sum is positive, and token, position and the tokens generated afterwards are what they were."""
    import torch
    from llvq_b200.model import Qwen3Config, synthetic_model
    cfg = Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 16, n_heads=4, n_kv=2, head_dim=64, layers=2, vocab=512)
    model, _ = synthetic_model(rt, cfg, config_id=2, capacity=64, row_scale_gain=40.0)
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    want = model.generate(prompt, 12, use_graph=True)
    first = model.generate(prompt, 5, use_graph=True)
    tok, pos = int(model._tok), int(model._pos)
    ph = model.phase_split(reps=3)
    assert set(ph) == {"embed", "norm", "projections", "rope_kv_write", "attention", "swiglu", "head", "sum"}
    assert all(v > 0 for v in ph.values()) and abs(ph["sum"] - sum(v for k, v in ph.items() if k != "sum")) < 1e-6
    assert (int(model._tok), int(model._pos)) == (tok, pos)
    assert first == want[:5] and model.generate(prompt, 12, use_graph=True) == want


def test_dependent_launches_do_not_change_a_token(rt):
    """Every kernel of the token step is launched as a programmatic dependent of the kernel before it (its preamble
    may run early; it waits for that kernel before touching memory). The tokens and the final hidden state are
    those of ordinary launches, eagerly and from a captured graph, with and without rotations."""
    import torch
    from llvq_b200.model import Qwen3Config, synthetic_model
    cfg = Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 16, n_heads=4, n_kv=2, head_dim=64, layers=3, vocab=512)
    prompt = [int(t) for t in np.random.default_rng(77).integers(0, cfg.vocab, 18)]
    for rotations in (False, True):
        runs = {}
        for overlap in (False, True):
            for use_graph in (False, True):
                rt.set_overlap(overlap)
                try:
                    model, _ = synthetic_model(rt, cfg, config_id=2, capacity=64, rotations=rotations, row_scale_gain=40.0)
                    toks = model.generate(prompt, 30, use_graph=use_graph)
                    torch.cuda.synchronize()
                    runs[(overlap, use_graph)] = (toks, model._x.clone())
                finally:
                    rt.set_overlap(True)
        want_t, want_x = runs[(False, False)]
        assert len(set(want_t)) > 4
        for key, (toks, x) in runs.items():
            assert toks == want_t, (rotations, key)
            assert torch.equal(x, want_x), (rotations, key)
    assert not rt.poll_range_error()


def test_norm_and_swiglu_inside_the_projection_do_not_change_a_token(rt):
    """Without rotations the token step lets the q/k/v and gate/up projections compute their RMSNorm (and the
    residual add) and the down projection its SwiGLU product in the kernel's staging step. The tokens and the
    final hidden state are those of the step with separate norm and SwiGLU kernels, eagerly and from a graph; the
    width 2560 has 16 tail columns, the small model's inter of 496 is a multiple of 8."""
    import torch
    from llvq_b200.model import Qwen3Config, synthetic_model
    for cfg, layers in ((Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 16, n_heads=4, n_kv=2, head_dim=64, layers=3, vocab=512), 3),
                        (Qwen3Config.named("qwen3-4b"), 2)):
        prompt = [int(t) for t in np.random.default_rng(5).integers(0, cfg.vocab, 12)]
        runs = {}
        for fuse in (False, True):
            for use_graph in (False, True):
                big = cfg.hidden > 1000  # drawn on the GPU, with the benchmark's row scales
                model, _ = synthetic_model(rt, cfg, config_id=2, capacity=64, layers=layers, row_scale_gain=1.0 if big else 40.0,
                                           device_codes=big, keep_host=False)
                model.fuse_x = fuse
                toks = model.generate(prompt, 20, use_graph=use_graph)
                torch.cuda.synchronize()
                runs[(fuse, use_graph)] = (toks, model._x.clone())
        want_t, want_x = runs[(False, False)]
        for key, (toks, x) in runs.items():
            assert toks == want_t, key
            assert torch.equal(x, want_x), key
    assert not rt.poll_range_error()


def test_int8_kv_cache_matches_the_reference_scheme():
    """u8 affine, groups of 64, f16 scale and bias, constant groups exact (llvq-llm/src/kvq.rs:110-165)."""
    import torch
    from llvq_b200.model import kv_dequantize, kv_quantize
    torch.manual_seed(0)
    x = torch.randn(5, 2, 128, device="cuda").half()
    x[0, 0, :64] = 0.375  # a constant group has nothing to grade
    q, s, b = kv_quantize(x)
    y = kv_dequantize(q, s, b)
    assert q.dtype == torch.uint8 and s.shape == (5, 2, 2) and y.dtype == torch.float16
    assert torch.equal(y[0, 0, :64], x[0, 0, :64])
    step = s.float().unsqueeze(-1).expand(5, 2, 2, 64).reshape(5, 2, 128)
    assert ((y.float() - x.float()).abs() <= 0.51 * step + 2e-3).all()
    q2, s2, b2 = kv_quantize(y)  # a second round trip moves nothing by more than one step
    assert ((kv_dequantize(q2, s2, b2).float() - y.float()).abs() <= step + 2e-3).all()


def test_int8_kv_cache_rounds_halves_away_from_zero(rt):
    """candle's round() (llvq-llm/src/kvq.rs:149-152) rounds k + 0.5 to k + 1; round-to-even would give k for even k.
    A group with minimum 0 and maximum 255 / 64 has scale 1 / 64 exactly (f16), so x = (k + 0.5) / 64 is an exact tie."""
    import torch
    from llvq_b200.model import Int8KvCache, kv_quantize
    k = torch.arange(62, dtype=torch.float32)
    g = torch.cat([torch.tensor([0.0, 255.0 / 64.0]), (k + 0.5) / 64.0]).half()  # 64 values, all exact in f16
    assert torch.equal(g.float()[2:] * 64.0, k + 0.5)
    x = g.repeat(2).reshape(1, 1, 128).cuda()
    q, s, b = kv_quantize(x)
    want = torch.cat([torch.tensor([0.0, 255.0]), k + 1.0]).to(torch.uint8)
    assert s.flatten().tolist() == [1.0 / 64.0] * 2 and b.flatten().tolist() == [0.0, 0.0]
    assert torch.equal(q.flatten()[:64].cpu(), want) and torch.equal(q.flatten()[64:].cpu(), want)
    # the kernel that writes the cache in the token step agrees with the mirror on the ties
    import ctypes as C
    n_heads, n_kv, hd = 1, 1, 128
    qkv = torch.zeros((n_heads + 2 * n_kv) * hd, dtype=torch.float16, device="cuda")
    qkv[2 * hd:] = x.flatten()  # the value head is stored as it comes (no norm, no rotary embedding)
    ones = torch.ones(hd, dtype=torch.float16, device="cuda")
    cos = torch.ones(4, hd // 2, device="cuda")
    sin = torch.zeros(4, hd // 2, device="cuda")
    pos = torch.zeros(1, dtype=torch.int64, device="cuda")
    cache = Int8KvCache(4, n_kv, hd, qkv.device)
    q_out = torch.empty(n_heads * hd, dtype=torch.float16, device="cuda")
    from llvq_b200._lib import check
    check(rt.lib.llvq_op_qkv_rope_cache_h(qkv.data_ptr(), ones.data_ptr(), ones.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                          pos.data_ptr(), q_out.data_ptr(), cache.q[0].data_ptr(), cache.s[0].data_ptr(),
                                          cache.b[0].data_ptr(), cache.q[1].data_ptr(), cache.s[1].data_ptr(),
                                          cache.b[1].data_ptr(), n_heads, n_kv, hd, C.c_float(1e-6), None))
    torch.cuda.synchronize()
    assert torch.equal(cache.q[1][0, 0, :64].cpu(), want) and torch.equal(cache.q[1][0, 0, 64:].cpu(), want)


@pytest.mark.parametrize("hd,heads,kv", [(128, 8, 2), (64, 4, 4), (128, 10, 2), (64, 6, 3), (128, 8, 1)])
def test_split_kv_attention_matches_a_float_reference_at_long_contexts(rt, hd, heads, kv):
    """The sliced attention equals softmax(q k^T / sqrt(d)) v over the dequantised cache for any slice
    count, including slices that hold no position (attention semantics of llvq-llm/src/model.rs:500-560)."""
    import torch
    from llvq_b200._lib import check
    from llvq_b200.model import kv_dequantize, kv_quantize
    L = rt.lib
    torch.manual_seed(3)
    cap = 4100
    k = (torch.randn(cap, kv, hd, device="cuda") * 1.5).half()
    v = torch.randn(cap, kv, hd, device="cuda").half()
    kq, ks, kb = kv_quantize(k)
    vq, vs, vb = kv_quantize(v)
    kd, vd = kv_dequantize(kq, ks, kb).float(), kv_dequantize(vq, vs, vb).float()
    q = torch.randn(heads, hd, device="cuda").half()
    p = lambda t: t.data_ptr()
    st = torch.cuda.current_stream().cuda_stream
    for last in (0, 5, 1023, 4099):
        pos = torch.tensor(last, device="cuda", dtype=torch.int64)
        rep = heads // kv
        kk = kd[: last + 1].repeat_interleave(rep, dim=1)  # [t, heads, hd]
        vv = vd[: last + 1].repeat_interleave(rep, dim=1)
        w = torch.softmax(torch.einsum("hd,thd->ht", q.float(), kk) / hd ** 0.5, dim=1)
        want = torch.einsum("ht,thd->hd", w, vv)
        outs = []
        for splits in (1, 3, 16, 200):
            out = torch.zeros(heads, hd, device="cuda", dtype=torch.float16)
            ws = torch.full((heads * splits * (hd + 2),), float("nan"), device="cuda")
            check(L.llvq_op_attn_decode_int8_h(p(q), p(kq), p(ks), p(kb), p(vq), p(vs), p(vb), p(pos), p(out),
                                               heads, kv, hd, splits, p(ws), st))
            torch.cuda.synchronize()
            assert ((out.float() - want).abs().max() <= 2e-3 + 2e-3 * want.abs().max()).item(), (last, splits)
            outs.append(out)
        for o in outs[1:]:
            assert (o.float() - outs[0].float()).abs().max().item() <= 2e-3
    bad = L.llvq_op_attn_decode_int8_h(p(q), p(kq), p(ks), p(kb), p(vq), p(vs), p(vb), p(pos), p(out), heads, kv, hd, 4, None, st)
    assert bad != 0  # several slices need the scratch buffer


def test_chunked_prefill_and_library_attention_keep_the_tokens(rt):
    """A prompt cut into chunks (each attending to the cache so far), the dense-transient GEMM route and the
    fused-attention route for large score matrices all continue with the tokens of the one-chunk run."""
    import torch
    from llvq_b200.model import Qwen3Config, synthetic_model
    cfg = Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 8, n_heads=4, n_kv=2, head_dim=64, layers=2, vocab=512)
    g = np.random.default_rng(8)
    prompt = [int(t) for t in g.integers(0, cfg.vocab, 150)]
    base, _ = synthetic_model(rt, cfg, config_id=2, capacity=192)
    want = base.generate(prompt, 12)
    chunked, _ = synthetic_model(rt, cfg, config_id=2, capacity=192)
    chunked.prefill_chunk = 64
    assert chunked.generate(prompt, 12) == want
    dense, _ = synthetic_model(rt, cfg, config_id=2, capacity=192, dense_prefill_from=32)
    hd = dense.prefill(prompt)
    hb = base.prefill(prompt)
    assert ((hd.float() - hb.float()).norm() / hb.float().norm()).item() < 1e-2
    # the fused-attention route (taken when the score matrix would be large) against the explicit softmax
    q = torch.randn(70, 4, 64, device="cuda").half()
    k = torch.randn(150, 2, 64, device="cuda").half()
    v = torch.randn(150, 2, 64, device="cuda").half()
    pos = torch.arange(80, 150, device="cuda")
    small = base._attend(q, k, v, pos, 150)
    base.sdpa_from = 0
    big = base._attend(q, k, v, pos, 150)
    assert ((big.float() - small.float()).abs().max()).item() < 5e-3


def test_rotated_prefill_stays_close_to_the_token_by_token_run(rt):
    """With rotations on, a prompt of several rows goes through the batched GEMM, which takes f16 activations: the
    rotated activation is rounded to f16 once per projection group, where the one-row path (and the reference,
    which serves prompt rows as f32-activation matvecs: llvq-llm/src/model.rs:497-536) keeps f32. The test bounds
    what that rounding costs: last-token logits of the prompt in one chunk against the same prompt fed row by row
    (each row through the one-row path, attending to the cache written so far), and the same greedy token."""
    import torch
    from llvq_b200.model import Qwen3Config, synthetic_model
    cfg = Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 16, n_heads=4, n_kv=2, head_dim=64, layers=2, vocab=512)
    g = np.random.default_rng(31)
    prompt = [int(t) for t in g.integers(0, cfg.vocab, 24)]
    batched, _ = synthetic_model(rt, cfg, config_id=2, capacity=64, rotations=True, row_scale_gain=40.0)
    rowwise, _ = synthetic_model(rt, cfg, config_id=2, capacity=64, rotations=True, row_scale_gain=40.0)
    rowwise.prefill_chunk = 1
    hb, hr = batched.prefill(prompt), rowwise.prefill(prompt)
    lb, lr = batched.logits_last(hb), rowwise.logits_last(hr)
    assert ((lb - lr).norm() / lr.norm()).item() < 1e-2
    assert int(lb.argmax()) == int(lr.argmax())


def _tp_gpu_worker(rank, world, port, q):
    """Child of the two-GPU test. Every outcome, an exception included, goes back through the queue, and the
    process leaves through os._exit so that a failed rank never waits on its peer in a teardown."""
    import datetime
    import os
    import traceback
    import torch
    import torch.distributed as dist
    try:
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                                timeout=datetime.timedelta(seconds=60))
        from llvq_b200 import FusedRuntime
        from llvq_b200.model import Qwen3Config, TpGroup, synthetic_model
        cfg = Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 16, n_heads=4, n_kv=2, head_dim=64, layers=2, vocab=512)
        rt = FusedRuntime(rank)
        g = np.random.default_rng(21)
        prompt = [int(t) for t in g.integers(0, cfg.vocab, 40)]
        whole, _ = synthetic_model(rt, cfg, config_id=4, capacity=96)
        want = whole.generate(prompt, 20)
        sharded, _ = synthetic_model(rt, cfg, config_id=4, capacity=96, tp=TpGroup())
        got = sharded.generate(prompt, 20)
        q.put((rank, "eager", want, got))
        graphed = sharded.generate(prompt, 20, use_graph=True)
        q.put((rank, "graph", want, graphed))
        # the same model with the token-step gathers through peer memory (llvq_tp_exchange)
        peer_tp = TpGroup(peer_lib=rt.lib)
        peered, _ = synthetic_model(rt, cfg, config_id=4, capacity=96, tp=peer_tp)
        q.put((rank, "peer eager", want, peered.generate(prompt, 20)))
        q.put((rank, "peer graph", want, peered.generate(prompt, 20, use_graph=True)))
        torch.cuda.synchronize()
        q.put((rank, "peer errors", 0, peer_tp.peer.poll_error()))
        torch.cuda.synchronize()
    except BaseException:  # noqa: BLE001 - reported to the parent, which fails the test
        q.put((rank, "error", traceback.format_exc(), None))
    finally:
        q.close()
        q.join_thread()
        os._exit(0)


def test_tensor_parallel_model_on_two_gpus_picks_the_single_gpu_tokens():
    """Head-sharded attention, row-sharded projections and the sharded greedy head over NCCL: the tokens of
    the whole model on one GPU, eagerly and from a captured graph (needs two GPUs; NVLS off)."""
    import os
    import queue
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 33000 + os.getpid() % 2000
    procs = [ctx.Process(target=_tp_gpu_worker, args=(r, 2, port, q), daemon=True) for r in range(2)]
    for p in procs:
        p.start()
    got = []
    try:
        while len(got) < 10:
            item = q.get(timeout=240)
            got.append(item)
            assert item[1] != "error", f"rank {item[0]} failed:\n{item[2]}"
    except queue.Empty:
        pytest.fail(f"ranks went silent; reports so far: {got}")
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()  # the exact children started above
    for rank, phase, want, tokens in got:
        assert tokens == want, (rank, phase, want, tokens)


def test_int8_embedding_kernels_follow_the_reference_arithmetic(rt):
    """emb_q8_gather: f16(scale * q + bias) with an f32 multiply then an f32 add, bit for bit; the greedy head over
    the same payload picks the argmax of the f32 logits of the dequantised rows (llvq-llm/kernels/emb_q8.cu:42-106);
    the quantiser follows quantize_affine (embedquant.rs:22-80): constant groups ungraded, codes within one step."""
    import torch
    from llvq_b200.model import Q8Embedding
    g = torch.Generator(device="cuda").manual_seed(6)
    for V, H in ((1000, 256), (151936 // 8, 2560), (16, 64)):
        w = (0.02 * torch.randn(V, H, device="cuda", generator=g)).half()
        w[3 % V, :64] = 0.25  # a constant group
        emb = Q8Embedding.quantize(rt.lib, w)
        assert emb.scales[3 % V, 0] == 1.0 and int(emb.wq[3 % V, :64].max()) == 0 and emb.biases[3 % V, 0] == 0.25
        deq = (emb.scales.float().unsqueeze(-1) * emb.wq.float().reshape(V, H // 64, 64) + emb.biases.float().unsqueeze(-1)).reshape(V, H)
        step = emb.scales.float().unsqueeze(-1).expand(V, H // 64, 64).reshape(V, H)
        assert ((deq - w.float()).abs() <= 0.51 * step + 1e-3).all()
        toks = torch.tensor([0, V - 1, 3 % V, 7 % V], device="cuda")
        assert torch.equal(emb.lookup(toks), deq.half().index_select(0, toks))
        assert torch.equal(emb.dense(), deq.half())
        h = torch.randn(H, device="cuda", generator=g).half()
        logits = deq @ h.float()
        val, idx = emb.pick(h, 100)
        torch.cuda.synchronize()
        assert int(idx) - 100 == int(logits.argmax()) and abs(float(val) - float(logits.max())) <= 1e-4 * max(1.0, float(logits.abs().max()))
        lo = V // 2
        v2, i2 = emb.shard(lo, V).pick(h, lo)
        if int(logits.argmax()) >= lo:
            assert int(i2) == int(logits.argmax())
