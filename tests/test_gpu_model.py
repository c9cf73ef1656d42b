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
                      gemm=lambda w, x: lin(x.float(), w.float()).half(), kv_int8=kv_int8)


@pytest.mark.parametrize("kv_int8", [True, False])
def test_greedy_tokens_match_the_dense_decoded_run(rt, oracle, kv_int8):
    import torch
    from llvq_b200.model import Qwen3Config, synthetic_model
    cfg = Qwen3Config(hidden=24 * 10 + 16, inter=24 * 20 + 8, n_heads=4, n_kv=2, head_dim=64, layers=2, vocab=512)
    capacity = 64
    fused, mats = synthetic_model(rt, cfg, config_id=2, capacity=capacity, kv_int8=kv_int8)
    dense = _dense_model(rt, oracle, cfg, mats, fused, capacity, kv_int8)
    g = np.random.default_rng(5)
    prompt = [int(t) for t in g.integers(0, cfg.vocab, 20)]  # 20 >= 16: the prefill takes the tensor-core GEMM
    want = dense.generate(prompt, 24)
    got = fused.generate(prompt, 24)
    assert len(got) == 24 and all(0 <= t < cfg.vocab for t in got)
    first_diff = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), None)
    assert first_diff is None, f"first divergence at token {first_diff}: {got} vs {want}"
    # the logits behind the first generated token agree closely, not just their argmax
    toks = torch.tensor(prompt, device=fused.device)
    lf = fused.logits_last(fused.hidden(toks, fused.positions[:20]))
    ld = dense.logits_last(dense.hidden(toks, dense.positions[:20]))
    assert ((lf - ld).norm() / ld.norm()).item() < 5e-3
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
