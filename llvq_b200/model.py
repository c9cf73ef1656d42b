"""Greedy decode loop of a Qwen3-architecture model whose projections are fused LLVQ GEMVs.

Mirror of the reference's `Qwen3::generate` / `Block::forward_cached`
(llvq-llm/src/model.rs:766-835, 1041-1073): like the reference, only the seven projections
of a block go through the fused operator; RMSNorm, per-head q/k norm, RoPE (theta 1e6,
rotate-half), grouped-query attention, SwiGLU, the tied f16 head and the argmax are stock
tensor ops (candle there, torch here). Two things differ from the reference's loop:

* the prompt is prefilled through the batched dequant-GEMM (`forward_batch`, tensor cores)
  instead of one matvec launch per prompt row;
* the KV cache really stores int8: u8 codes with an f16 scale and bias per group of 64 along
  head_dim, exactly the scheme of llvq-llm/src/kvq.rs:110-165 (round to nearest, range/255
  scale through f16, constant groups reconstruct to their bias); the reference only simulates
  it by a quantize-dequantize round trip in the cache dtype. Reads dequantize to f16, so the
  values attention sees are the ones the reference's simulation produces.

The per-token step has static shapes (fixed-capacity cache, position held in a device tensor),
so it can be captured once in a CUDA graph and replayed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import numpy as np

KV_GROUP = 64  # llvq-llm/src/kvq.rs: groups of 64 along head_dim


@dataclass
class Qwen3Config:
    hidden: int
    inter: int
    n_heads: int
    n_kv: int
    head_dim: int
    layers: int
    vocab: int
    rope_theta: float = 1e6
    eps: float = 1e-6

    @staticmethod
    def named(name: str) -> "Qwen3Config":
        from .synth import MODEL_SHAPES
        h, inter, qh, kvh, hd, layers, vocab = MODEL_SHAPES[name]
        return Qwen3Config(h, inter, qh, kvh, hd, layers, vocab)


def kv_quantize(x):
    """[..., head_dim] f16 -> (u8 codes, f16 scale, f16 bias), groups of 64 (kvq.rs:110-165)."""
    import torch
    g = x.float().unflatten(-1, (-1, KV_GROUP))
    mn = g.amin(-1, keepdim=True)
    mx = g.amax(-1, keepdim=True)
    s = ((mx - mn) / 255.0).half()
    mn = mn.half()
    sf = s.float()
    safe = torch.where(sf > 0, sf, torch.ones_like(sf))
    q = ((g - mn.float()) / safe).round().clamp_(0, 255)
    q = torch.where(sf > 0, q, torch.zeros_like(q)).to(torch.uint8)
    return q.flatten(-2), s.squeeze(-1), mn.squeeze(-1)


def kv_dequantize(q, s, mn):
    g = q.unflatten(-1, (-1, KV_GROUP)).float()
    return (g * s.float().unsqueeze(-1) + mn.float().unsqueeze(-1)).half().flatten(-2)


class Int8KvCache:
    """Fixed-capacity int8 KV cache of one block: [capacity, n_kv, head_dim] codes + per-group f16 scale/bias."""

    def __init__(self, capacity: int, n_kv: int, head_dim: int, device):
        import torch
        ng = head_dim // KV_GROUP
        self.q = [torch.zeros(capacity, n_kv, head_dim, dtype=torch.uint8, device=device) for _ in range(2)]
        self.s = [torch.zeros(capacity, n_kv, ng, dtype=torch.float16, device=device) for _ in range(2)]
        self.b = [torch.zeros(capacity, n_kv, ng, dtype=torch.float16, device=device) for _ in range(2)]

    def write(self, which: int, pos, x):
        """pos: int64 device tensor [L]; x: [L, n_kv, head_dim] f16."""
        q, s, b = kv_quantize(x)
        self.q[which].index_copy_(0, pos, q)
        self.s[which].index_copy_(0, pos, s)
        self.b[which].index_copy_(0, pos, b)

    def read(self, which: int):
        return kv_dequantize(self.q[which], self.s[which], self.b[which])

    def bytes_per_position(self) -> int:
        return 2 * (self.q[0][0].numel() + 2 * 2 * self.s[0][0].numel())


class FusedQwen3:
    """`proj(name_group, x)` hooks let the same loop run on fused projections or on a dense stand-in."""

    def __init__(self, cfg: Qwen3Config, blocks: Sequence[dict], embed, final_norm, capacity: int,
                 gemv: Callable, gemm: Callable, kv_int8: bool = True, ops=None):
        """blocks[i]: {"qkv", "o", "gate_up", "down": projection handles, "ln1", "ln2", "q_norm", "k_norm": f16 tensors}.
        gemv(handle, x[d_in]) -> y[d_out]; gemm(handle, X[L, d_in]) -> Y[L, d_out] (both f16 on the GPU)."""
        import torch
        self.cfg, self.blocks, self.embed, self.final_norm = cfg, list(blocks), embed, final_norm
        self.gemv, self.gemm, self.capacity, self.kv_int8 = gemv, gemm, capacity, kv_int8
        dev = embed.device
        self.device = dev
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=dev, dtype=torch.float32) / cfg.head_dim))
        ang = torch.arange(capacity, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.positions = torch.arange(capacity, device=dev)
        if kv_int8:
            self.caches = [Int8KvCache(capacity, cfg.n_kv, cfg.head_dim, dev) for _ in blocks]
        else:
            self.caches = [[torch.zeros(capacity, cfg.n_kv, cfg.head_dim, dtype=torch.float16, device=dev) for _ in range(2)]
                           for _ in blocks]
        self._graph = None
        # `ops`: the C library (llvq_op_* kernels). With it and an int8 cache the token step runs the fused
        # decode kernels; without it every non-projection step is a torch op (the prefill always is).
        self.ops = ops if kv_int8 else None
        if self.ops is not None:
            f16 = dict(dtype=torch.float16, device=dev)
            self._x, self._h = torch.zeros(cfg.hidden, **f16), torch.zeros(cfg.hidden, **f16)
            self._qkv = torch.zeros((cfg.n_heads + 2 * cfg.n_kv) * cfg.head_dim, **f16)
            self._q, self._ctx = (torch.zeros(cfg.n_heads * cfg.head_dim, **f16) for _ in range(2))
            self._o, self._down = torch.zeros(cfg.hidden, **f16), torch.zeros(cfg.hidden, **f16)
            self._gu, self._act = torch.zeros(2 * cfg.inter, **f16), torch.zeros(cfg.inter, **f16)
        # the token and its position live in fixed device tensors: a captured graph keeps their addresses
        self._tok = torch.zeros(1, dtype=torch.long, device=dev)
        self._pos = torch.zeros(1, dtype=torch.long, device=dev)

    # ---- pieces ------------------------------------------------------------------
    def _rms(self, x, w):
        xf = x.float()
        return (xf * (xf.pow(2).mean(-1, keepdim=True) + self.cfg.eps).rsqrt() * w.float()).half()

    def _rope(self, x, pos):
        """x: [L, heads, head_dim]; rotate-half convention (candle_nn::rotary_emb::rope)."""
        import torch
        c, s = self.cos.index_select(0, pos)[:, None, :], self.sin.index_select(0, pos)[:, None, :]
        x1, x2 = x.float().chunk(2, dim=-1)
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).half()

    def _proj(self, handle, h):
        return self.gemv(handle, h[0])[None, :] if h.shape[0] == 1 else self.gemm(handle, h)

    def _block(self, i: int, x, pos):
        """x: [L, hidden] f16, pos: int64 [L] absolute positions (consecutive)."""
        import torch
        cfg, blk = self.cfg, self.blocks[i]
        L = x.shape[0]
        h = self._rms(x, blk["ln1"])
        qkv = self._proj(blk["qkv"], h)
        nq, nk = cfg.n_heads * cfg.head_dim, cfg.n_kv * cfg.head_dim
        q = qkv[:, :nq].reshape(L, cfg.n_heads, cfg.head_dim)
        k = qkv[:, nq:nq + nk].reshape(L, cfg.n_kv, cfg.head_dim)
        v = qkv[:, nq + nk:].reshape(L, cfg.n_kv, cfg.head_dim)
        q = self._rope(self._rms(q, blk["q_norm"]), pos)
        k = self._rope(self._rms(k, blk["k_norm"]), pos)
        cache = self.caches[i]
        if self.kv_int8:
            cache.write(0, pos, k)
            cache.write(1, pos, v.contiguous())
            k_all, v_all = cache.read(0), cache.read(1)
        else:
            cache[0].index_copy_(0, pos, k)
            cache[1].index_copy_(0, pos, v.contiguous())
            k_all, v_all = cache[0], cache[1]
        groups = cfg.n_heads // cfg.n_kv
        kf = k_all.float().repeat_interleave(groups, dim=1)   # [T, heads, hd]
        vf = v_all.float().repeat_interleave(groups, dim=1)
        scores = torch.einsum("lhd,thd->hlt", q.float(), kf) * (1.0 / cfg.head_dim ** 0.5)
        visible = self.positions[None, None, :] <= pos[None, :, None]  # causal, and nothing beyond the write head
        scores = scores.masked_fill(~visible, float("-inf"))
        ctx = torch.einsum("hlt,thd->lhd", torch.softmax(scores, dim=-1), vf).half().reshape(L, nq)
        x = x + self._proj(blk["o"], ctx)
        h = self._rms(x, blk["ln2"])
        gu = self._proj(blk["gate_up"], h)
        gated = (torch.nn.functional.silu(gu[:, :cfg.inter].float()) * gu[:, cfg.inter:].float()).half()
        return x + self._proj(blk["down"], gated)

    def hidden(self, tokens, pos):
        x = self.embed.index_select(0, tokens)
        for i in range(len(self.blocks)):
            x = self._block(i, x, pos)
        return x

    def logits_last(self, x):
        h = self._rms(x[-1:], self.final_norm)
        return (h @ self.embed.t()).float()[0]

    # ---- the loop ----------------------------------------------------------------
    def generate(self, prompt: Sequence[int], max_new: int, use_graph: bool = False) -> List[int]:
        """Greedy continuation, `Qwen3::generate` (model.rs:1041-1073): prefill, then one token at a time."""
        import torch
        if max_new == 0:
            return []
        n = len(prompt)
        if n + max_new > self.capacity:
            raise ValueError(f"{n} prompt + {max_new} new tokens exceed the cache capacity {self.capacity}")
        toks = torch.tensor(list(prompt), device=self.device, dtype=torch.long)
        x = self.hidden(toks, self.positions[:n])
        nxt = self.logits_last(x).argmax()
        out = [int(nxt)]
        self.start_decode(nxt, n)
        step = self._graph_step if use_graph else self._eager_step
        while len(out) < max_new:
            step()
            out.append(int(self._tok))  # one scalar read-back per token, as model.rs:1064
        return out

    def start_decode(self, first_token, position: int) -> None:
        """Point the token step at `first_token` (device scalar) sitting at `position` (in place: graph-safe)."""
        self._tok.copy_(first_token.reshape(1))
        self._pos.fill_(position)

    def _eager_step(self):
        if self.ops is not None:
            return self._fused_step()
        x = self.hidden(self._tok, self._pos)
        self._tok.copy_(self.logits_last(x).argmax().reshape(1))
        self._pos += 1

    def _fused_step(self):
        """One token: 4 fused GEMV launches and 4 small fused kernels per block, nothing else."""
        import ctypes as C
        import torch
        from ._lib import check
        L, cfg = self.ops, self.cfg
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        p = lambda t: C.c_void_p(t.data_ptr())
        self._x.copy_(self.embed.index_select(0, self._tok)[0])
        delta = None
        for blk, cache in zip(self.blocks, self.caches):
            check(L.llvq_op_add_rmsnorm_h(p(self._x), p(delta) if delta is not None else None, p(blk["ln1"]), p(self._h),
                                          cfg.hidden, cfg.eps, st))
            self.gemv(blk["qkv"], self._h, out=self._qkv)
            check(L.llvq_op_qkv_rope_cache_h(p(self._qkv), p(blk["q_norm"]), p(blk["k_norm"]), p(self.cos), p(self.sin),
                                             p(self._pos), p(self._q), p(cache.q[0]), p(cache.s[0]), p(cache.b[0]),
                                             p(cache.q[1]), p(cache.s[1]), p(cache.b[1]), cfg.n_heads, cfg.n_kv,
                                             cfg.head_dim, cfg.eps, st))
            check(L.llvq_op_attn_decode_int8_h(p(self._q), p(cache.q[0]), p(cache.s[0]), p(cache.b[0]), p(cache.q[1]),
                                               p(cache.s[1]), p(cache.b[1]), p(self._pos), p(self._ctx), cfg.n_heads,
                                               cfg.n_kv, cfg.head_dim, st))
            self.gemv(blk["o"], self._ctx, out=self._o)
            check(L.llvq_op_add_rmsnorm_h(p(self._x), p(self._o), p(blk["ln2"]), p(self._h), cfg.hidden, cfg.eps, st))
            self.gemv(blk["gate_up"], self._h, out=self._gu)
            check(L.llvq_op_silu_mul_h(p(self._gu), p(self._act), cfg.inter, st))
            self.gemv(blk["down"], self._act, out=self._down)
            delta = self._down
        check(L.llvq_op_add_rmsnorm_h(p(self._x), p(delta), p(self.final_norm), p(self._h), cfg.hidden, cfg.eps, st))
        self._tok.copy_((self._h[None, :] @ self.embed.t()).float()[0].argmax().reshape(1))
        self._pos += 1

    def _graph_step(self):
        import torch
        if self._graph is None:
            tok0, pos0 = self._tok.clone(), self._pos.clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):  # warm-up outside the capture (lazy initialisations)
                self._eager_step()
            torch.cuda.current_stream().wait_stream(side)
            self._tok.copy_(tok0)
            self._pos.copy_(pos0)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._eager_step()
            self._tok.copy_(tok0)
            self._pos.copy_(pos0)
        self._graph.replay()


def synthetic_model(rt, cfg: Qwen3Config, config_id: int, capacity: int, seed: int = 0x51, layers: Optional[int] = None,
                    kv_int8: bool = True, fused_ops: bool = True):
    """Random-weight model of BASELINE config 2/4: LLVQ codes for every projection, f16 N(0, 0.02)
    norms and tied embedding (norm weights are 1 + N(0, 0.02) so that activations keep their scale)."""
    import torch
    from . import synth
    n_layers = layers or cfg.layers
    dev = torch.device("cuda", rt.device)
    g = synth.SplitMix64(seed)
    mats, blocks = [], []

    def f16(n, base=0.0):
        return torch.from_numpy((base + 0.02 * g.gaussian(n)).astype(np.float16)).to(dev)

    for l in range(n_layers):
        shp = {"q": (cfg.n_heads * cfg.head_dim, cfg.hidden), "k": (cfg.n_kv * cfg.head_dim, cfg.hidden),
               "v": (cfg.n_kv * cfg.head_dim, cfg.hidden), "o": (cfg.hidden, cfg.n_heads * cfg.head_dim),
               "gate": (cfg.inter, cfg.hidden), "up": (cfg.inter, cfg.hidden), "down": (cfg.hidden, cfg.inter)}
        m = {n: synth.make_matrix(do, di, synth.matrix_seed(config_id, l, synth.PROJ_IDS[n]), f"l{l}.{n}")
             for n, (do, di) in shp.items()}
        mats.append(m)
        blocks.append({"qkv": rt.upload_group([m["q"], m["k"], m["v"]], tail_f16=True), "o": rt.upload(m["o"], tail_f16=True),
                       "gate_up": rt.upload_group([m["gate"], m["up"]], tail_f16=True),
                       "down": rt.upload(m["down"], tail_f16=True),
                       "ln1": f16(cfg.hidden, 1.0), "ln2": f16(cfg.hidden, 1.0),
                       "q_norm": f16(cfg.head_dim, 1.0), "k_norm": f16(cfg.head_dim, 1.0)})
    embed = f16(cfg.vocab * cfg.hidden).reshape(cfg.vocab, cfg.hidden)
    final_norm = f16(cfg.hidden, 1.0)
    model = FusedQwen3(cfg, blocks, embed, final_norm, capacity, gemv=rt.forward, gemm=rt.forward_batch, kv_int8=kv_int8,
                       ops=rt.lib if fused_ops else None)
    return model, mats
