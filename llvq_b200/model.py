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
    t = (g - mn.float()) / safe
    # candle's round() rounds halves away from zero (kvq.rs:149-152); torch.round would round them to even
    q = torch.where(t >= 0, torch.floor(t + 0.5), -torch.floor(0.5 - t)).clamp_(0, 255)
    q = torch.where(sf > 0, q, torch.zeros_like(q)).to(torch.uint8)
    return q.flatten(-2), s.squeeze(-1), mn.squeeze(-1)


def kv_dequantize(q, s, mn):
    g = q.unflatten(-1, (-1, KV_GROUP)).float()
    return (g * s.float().unsqueeze(-1) + mn.float().unsqueeze(-1)).half().flatten(-2)


def _silu(x):
    import torch
    return torch.nn.functional.silu(x)


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

    def read(self, which: int, end: Optional[int] = None):
        return kv_dequantize(self.q[which][:end], self.s[which][:end], self.b[which][:end])

    def bytes_per_position(self) -> int:
        return 2 * (self.q[0][0].numel() + 2 * 2 * self.s[0][0].numel())


class F16Embedding:
    """The tied f16 embedding: row gather for the input, `head(E, h, row_offset)` for the greedy pick."""

    def __init__(self, w, head: Callable):
        self.w, self.head, self.device, self.rows = w, head, w.device, w.shape[0]

    def lookup(self, tokens):
        return self.w.index_select(0, tokens)

    def shard(self, lo: int, hi: int) -> "F16Embedding":
        return F16Embedding(self.w[lo:hi], self.head)

    def pick(self, h, row_offset: int):
        return self.head(self.w, h, row_offset)

    def dense(self):
        return self.w


class Q8Embedding:
    """The tied embedding carried as int8 g64 (w = scale * q + bias per 64 values of a row, f16 scale and bias:
    the `embedq` payload of a sealed file, llvq-llm/src/embedquant.rs:22, kernels llvq-llm/kernels/emb_q8.cu)."""

    def __init__(self, lib, wq, scales, biases):
        import torch
        if wq.dtype != torch.uint8 or scales.dtype != torch.float16 or biases.dtype != torch.float16 or wq.shape[1] % 64:
            raise ValueError("Q8Embedding: u8 codes [V, H] with H % 64 == 0, f16 scales and biases [V, H / 64]")
        self.lib, self.wq, self.scales, self.biases = lib, wq.contiguous(), scales.contiguous(), biases.contiguous()
        self.device, self.rows, self.hidden = wq.device, wq.shape[0], wq.shape[1]
        self._scratch = torch.zeros(8192, dtype=torch.uint8, device=self.device)
        self._val = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._idx = torch.zeros(1, dtype=torch.long, device=self.device)

    @staticmethod
    def quantize(lib, w):
        """f16 [V, H] -> Q8Embedding by the reference's quantize_affine (embedquant.rs:22-80): per group the
        range over 255 through f16, constant groups ungraded (scale 1, q 0), round half away from zero."""
        import torch
        V, H = w.shape
        g = w.float().reshape(V, H // 64, 64)
        mn, mx = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
        s = ((mx - mn) / 255.0).half()
        graded = s.float() > 0
        s = torch.where(graded, s, torch.ones_like(s))
        b = mn.half()
        t = (g - b.float()) / s.float()
        q = torch.where(graded, (torch.sign(t) * torch.floor(t.abs() + 0.5)).clamp(0, 255), torch.zeros_like(t))
        return Q8Embedding(lib, q.to(torch.uint8).reshape(V, H), s.reshape(V, H // 64), b.reshape(V, H // 64))

    def lookup(self, tokens):
        import ctypes as C
        import torch
        from ._lib import check
        tokens = tokens.to(torch.long).contiguous()
        y = torch.empty(tokens.numel(), self.hidden, dtype=torch.float16, device=self.device)
        p = lambda t: C.c_void_p(t.data_ptr())
        check(self.lib.llvq_op_embed_gather_q8_h(p(self.wq), p(self.scales), p(self.biases), p(tokens), tokens.numel(), self.rows,
                                                 self.hidden, p(y), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return y

    def shard(self, lo: int, hi: int) -> "Q8Embedding":
        return Q8Embedding(self.lib, self.wq[lo:hi], self.scales[lo:hi], self.biases[lo:hi])

    def pick(self, h, row_offset: int):
        import ctypes as C
        import torch
        from ._lib import check
        p = lambda t: C.c_void_p(t.data_ptr())
        check(self.lib.llvq_op_lm_head_argmax_q8_h(p(self.wq), p(self.scales), p(self.biases), p(h), self.rows, self.hidden, row_offset,
                                                   p(self._scratch), p(self._val), p(self._idx),
                                                   C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return self._val, self._idx

    def dense(self):
        """Dequantised f16 copy (diagnostics and tests): f16(scale * q + bias), f32 multiply then add."""
        V, H = self.wq.shape
        w = self.wq.float().reshape(V, H // 64, 64) * self.scales.float().unsqueeze(-1) + self.biases.float().unsqueeze(-1)
        return w.reshape(V, H).half()


class TpGroup:
    """Rank layout of a tensor-parallel model: rank r of `world` holds q heads [r H/world, (r+1) H/world),
    the matching kv heads, rows [r I/world, ...) of gate/up, rows [r D/world, ...) of o/down and rows
    [r V/world, ...) of the tied head. Every exchange is an all-gather of row shards in rank order: NCCL
    by default; with `peer_lib` (the C library) the gathers of the token step go through peer memory
    (llvq_tp_exchange: peer stores + flags), the prompt's 2-D gathers stay on NCCL."""

    def __init__(self, group=None, peer_lib=None, spin_limit: int = 0):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.peer_lib, self.spin_limit, self.peer = peer_lib, spin_limit, None

    def check(self, cfg: Qwen3Config) -> None:
        for name, n in (("q heads", cfg.n_heads), ("kv heads", cfg.n_kv), ("intermediate rows", cfg.inter),
                        ("hidden rows", cfg.hidden), ("vocabulary rows", cfg.vocab)):
            if n % self.world:
                raise ValueError(f"{n} {name} do not split over {self.world} ranks")

    def alloc(self, device, specs):
        """Gathered buffers of the token step, one per site: specs = [(numel, dtype), ...] -> tensors."""
        import torch
        if self.peer_lib is None:
            return [torch.zeros(n, dtype=dt, device=device) for n, dt in specs]
        from .parallel import PeerExchange
        sizes = [n * torch.empty(0, dtype=dt).element_size() for n, dt in specs]
        self.peer = PeerExchange(self.peer_lib, device.index, sizes, group=self.group, spin_limit=self.spin_limit)
        return [self.peer.buffer(i, dt) for i, (_, dt) in enumerate(specs)]

    def gather_into(self, site: int, out, shard):
        """out[world * n] <- shards [n] in rank order (1-D, preallocated by `alloc`: safe inside a graph capture)."""
        if self.peer is not None:
            self.peer.exchange(site, shard)
        else:
            self.dist.all_gather_into_tensor(out, shard, group=self.group)
        return out

    def gather_cols(self, shard):
        """[L, n] shards -> [L, world * n]."""
        import torch
        L, n = shard.shape
        buf = torch.empty(self.world * L, n, dtype=shard.dtype, device=shard.device)
        self.dist.all_gather_into_tensor(buf, shard.contiguous(), group=self.group)
        return buf.view(self.world, L, n).permute(1, 0, 2).reshape(L, self.world * n)


class FusedQwen3:
    """`gemv` / `gemm` / `head` hooks let the same loop run on fused projections or on a dense stand-in.
    With a `TpGroup` the handles in `blocks` are this rank's row shards and `embed_head` its vocabulary rows."""

    def __init__(self, cfg: Qwen3Config, blocks: Sequence[dict], embed, final_norm, capacity: int,
                 gemv: Callable, gemm: Callable, head: Callable, kv_int8: bool = True, ops=None,
                 tp: Optional[TpGroup] = None, prefill_chunk: int = 2048, rotate: Optional[Callable] = None,
                 gemv_rotated: Optional[Callable] = None):
        """blocks[i]: {"qkv", "o", "gate_up", "down": projection handles, "ln1", "ln2", "q_norm", "k_norm": f16 tensors}.
        gemv(handle, x[d_in]) -> y[d_out]; gemm(handle, X[L, d_in]) -> Y[L, d_out] (both f16);
        head(E[rows, hidden], h[hidden], row_offset) -> (best logit f32 [1], its row int64 [1]).
        A block may carry "rot_qkv", "rot_o", "rot_gate_up", "rot_down": the rotation of the activation that
        group consumes (one per shared activation, llvq-llm/src/rotplan.rs); then rotate(rot, x f16 [.., n]) ->
        f32 and gemv_rotated(handle, xr f32 [d_in], out=) -> f16 are used, as FusedRuntime::rotate and
        forward_rotated are in the reference (llvq-llm/src/fused_cuda.rs:362-402)."""
        import torch
        self.cfg, self.blocks, self.embed, self.final_norm = cfg, list(blocks), embed, final_norm
        self.gemv, self.gemm, self.head, self.capacity, self.kv_int8 = gemv, gemm, head, capacity, kv_int8
        self.rotate, self.gemv_rotated = rotate, gemv_rotated
        self.tp = tp if tp is not None and tp.world > 1 else None
        self.world = self.tp.world if self.tp else 1
        self.rank = self.tp.rank if self.tp else 0
        if self.tp:
            self.tp.check(cfg)
        self.h_loc, self.kv_loc, self.inter_loc = cfg.n_heads // self.world, cfg.n_kv // self.world, cfg.inter // self.world
        self.prefill_chunk = prefill_chunk
        self.sdpa_from = 1 << 28  # bytes of f32 scores above which the prompt attention is the library's fused kernel
        # `embed`: the tied f16 embedding as a tensor, or an embedding object (F16Embedding, Q8Embedding)
        self.emb = embed if hasattr(embed, "lookup") else F16Embedding(embed, head)
        dev = self.emb.device
        self.device = dev
        v_loc = cfg.vocab // self.world
        self.emb_head = self.emb.shard(self.rank * v_loc, (self.rank + 1) * v_loc)
        self.head_offset = self.rank * v_loc
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=dev, dtype=torch.float32) / cfg.head_dim))
        ang = torch.arange(capacity, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.positions = torch.arange(capacity, device=dev)
        if kv_int8:
            self.caches = [Int8KvCache(capacity, self.kv_loc, cfg.head_dim, dev) for _ in blocks]
        else:
            self.caches = [[torch.zeros(capacity, self.kv_loc, cfg.head_dim, dtype=torch.float16, device=dev) for _ in range(2)]
                           for _ in blocks]
        self._graph = None
        # `ops`: the C library (llvq_op_* kernels). With it and an int8 cache the token step runs the fused
        # decode kernels; without it every non-projection step is a torch op (the prefill always is).
        self.ops = ops if kv_int8 else None
        if self.ops is not None:
            f16 = dict(dtype=torch.float16, device=dev)
            hd, w = cfg.head_dim, self.world
            self._x, self._h = torch.zeros(cfg.hidden, **f16), torch.zeros(cfg.hidden, **f16)
            # a projection that follows a norm or the SwiGLU product computes that step in its own staging
            # (llvq_gemv_norm_h / llvq_gemv_silu_h); the residual stream then alternates between _x and _x2
            self._x2 = torch.zeros(cfg.hidden, **f16)
            self.fuse_x = True
            self._qkv = torch.zeros((self.h_loc + 2 * self.kv_loc) * hd, **f16)
            self._q = torch.zeros(self.h_loc * hd, **f16)
            gathered = [(cfg.n_heads * hd, torch.float16), (cfg.hidden, torch.float16), (cfg.inter, torch.float16),
                        (cfg.hidden, torch.float16), (2 * self.world, torch.long)]
            bufs = self.tp.alloc(dev, gathered) if self.tp else [torch.zeros(n, dtype=dt, device=dev) for n, dt in gathered]
            self._ctx, self._o, self._act, self._down, self._best_all = bufs
            self._gu = torch.zeros(2 * self.inter_loc, **f16)
            # f32 staging of a rotated activation, one buffer per width
            self._xr = {n: torch.zeros(n, dtype=torch.float32, device=dev) for n in {cfg.hidden, cfg.n_heads * hd, cfg.inter}}
            # the shard a rank computes before the gather; the full buffer itself when there is one rank
            self._ctx_loc = torch.zeros(self.h_loc * hd, **f16) if w > 1 else self._ctx
            self._o_loc = torch.zeros(cfg.hidden // w, **f16) if w > 1 else self._o
            self._down_loc = torch.zeros(cfg.hidden // w, **f16) if w > 1 else self._down
            self._act_loc = torch.zeros(self.inter_loc, **f16) if w > 1 else self._act
            # split-KV attention: a CTA serves one KV head over one slice of the positions with 8 warps of 32
            # positions each, so slices go down to 256 positions until there are two CTAs per SM
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            self.attn_splits = max(1, min(-(-capacity // 256), (2 * sms) // self.kv_loc))
            self._attn_ws = torch.zeros(self.h_loc * self.attn_splits * (hd + 2), dtype=torch.float32, device=dev)
        # the token and its position live in fixed device tensors: a captured graph keeps their addresses
        self._tok = torch.zeros(1, dtype=torch.long, device=dev)
        self._pos = torch.zeros(1, dtype=torch.long, device=dev)
        self._best = torch.zeros(2, dtype=torch.long, device=dev)        # (logit bits, row) of this rank's shard
        if self.ops is None:
            self._best_all = torch.zeros(2 * self.world, dtype=torch.long, device=dev)

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

    def _proj(self, blk, name, h):
        handle, rot = blk[name], blk.get("rot_" + name)
        if rot is None:
            return self.gemv(handle, h[0])[None, :] if h.shape[0] == 1 else self.gemm(handle, h.contiguous())
        xr = self.rotate(rot, h.contiguous())  # f32, one rotation for every projection of the group
        return self.gemv_rotated(handle, xr[0])[None, :] if h.shape[0] == 1 else self.gemm(handle, xr.half())

    def _all(self, shard):
        return self.tp.gather_cols(shard) if self.tp else shard

    def _attend(self, q, k_all, v_all, pos, end):
        """q: [L, heads, hd]; k_all, v_all: [T, kv heads, hd] (cache contents); causal over absolute positions."""
        import torch
        cfg = self.cfg
        L, T = q.shape[0], k_all.shape[0]
        groups = q.shape[1] // k_all.shape[1]
        visible = self.positions[None, :T] <= pos[:, None]  # causal, and nothing beyond the write head
        if L * T * q.shape[1] * 4 > self.sdpa_from:
            # long prompts: the library's fused attention on f16 operands, scores never materialised
            kh = k_all.repeat_interleave(groups, dim=1).permute(1, 0, 2)[None]
            vh = v_all.repeat_interleave(groups, dim=1).permute(1, 0, 2)[None]
            out = torch.nn.functional.scaled_dot_product_attention(q.permute(1, 0, 2)[None], kh, vh, attn_mask=visible[None, None])
            return out[0].permute(1, 0, 2).reshape(L, -1)
        kf = k_all.float().repeat_interleave(groups, dim=1)   # [T, heads, hd]
        vf = v_all.float().repeat_interleave(groups, dim=1)
        scores = torch.einsum("lhd,thd->hlt", q.float(), kf) * (1.0 / cfg.head_dim ** 0.5)
        scores = scores.masked_fill(~visible[None], float("-inf"))
        return torch.einsum("hlt,thd->lhd", torch.softmax(scores, dim=-1), vf).half().reshape(L, -1)

    def _block(self, i: int, x, pos, end: Optional[int] = None):
        """x: [L, hidden] f16, pos: int64 [L] absolute positions (consecutive); attention reads cache
        positions [0, end) (the whole cache when the caller does not know the write head on the host)."""
        cfg, blk = self.cfg, self.blocks[i]
        L, hd = x.shape[0], cfg.head_dim
        end = self.capacity if end is None else end
        h = self._rms(x, blk["ln1"])
        qkv = self._proj(blk, "qkv", h)
        nq, nk = self.h_loc * hd, self.kv_loc * hd
        q = qkv[:, :nq].reshape(L, self.h_loc, hd)
        k = qkv[:, nq:nq + nk].reshape(L, self.kv_loc, hd)
        v = qkv[:, nq + nk:].reshape(L, self.kv_loc, hd)
        q = self._rope(self._rms(q, blk["q_norm"]), pos)
        k = self._rope(self._rms(k, blk["k_norm"]), pos)
        cache = self.caches[i]
        if self.kv_int8:
            cache.write(0, pos, k)
            cache.write(1, pos, v.contiguous())
            k_all, v_all = cache.read(0, end), cache.read(1, end)
        else:
            cache[0].index_copy_(0, pos, k)
            cache[1].index_copy_(0, pos, v.contiguous())
            k_all, v_all = cache[0][:end], cache[1][:end]
        ctx = self._all(self._attend(q, k_all, v_all, pos, end))
        x = x + self._all(self._proj(blk, "o", ctx))
        h = self._rms(x, blk["ln2"])
        gu = self._proj(blk, "gate_up", h)
        gated = (_silu(gu[:, :self.inter_loc].float()) * gu[:, self.inter_loc:].float()).half()
        return x + self._all(self._proj(blk, "down", self._all(gated)))

    def hidden(self, tokens, pos, end: Optional[int] = None):
        x = self.emb.lookup(tokens)
        for i in range(len(self.blocks)):
            x = self._block(i, x, pos, end)
        return x

    def prefill(self, prompt: Sequence[int]):
        """Run the prompt through the blocks in chunks of `prefill_chunk` tokens (each chunk attends to the
        cache written so far); returns the hidden state of the last prompt token, [1, hidden]."""
        import torch
        toks = torch.tensor(list(prompt), device=self.device, dtype=torch.long)
        x = None
        for lo in range(0, len(prompt), self.prefill_chunk):
            hi = min(len(prompt), lo + self.prefill_chunk)
            x = self.hidden(toks[lo:hi], self.positions[lo:hi], end=hi)
        return x[-1:]

    def pick(self, h):
        """Greedy token of the normalised hidden state h [hidden] -> int64 [1] (device)."""
        val, idx = self.emb_head.pick(h, self.head_offset)
        if not self.tp:
            return idx
        self._best[0:1].view(val.dtype)[0:1].copy_(val)
        self._best[1:2].copy_(idx)
        self.tp.gather_into(4, self._best_all, self._best)
        pairs = self._best_all.view(self.world, 2)
        vals = pairs[:, 0:1].contiguous().view(val.dtype)[:, 0]
        return pairs[:, 1].index_select(0, vals.argmax().reshape(1))  # first rank on ties = lowest row

    def logits_last(self, x):
        """Full logits of the last row (diagnostics; the loop itself uses `pick`)."""
        h = self._rms(x[-1:], self.final_norm)
        return (h @ self.emb.dense().t()).float()[0]

    # ---- the loop ----------------------------------------------------------------
    def generate(self, prompt: Sequence[int], max_new: int, use_graph: bool = False) -> List[int]:
        """Greedy continuation, `Qwen3::generate` (model.rs:1041-1073): prefill, then one token at a time."""
        if max_new == 0:
            return []
        n = len(prompt)
        if n + max_new > self.capacity:
            raise ValueError(f"{n} prompt + {max_new} new tokens exceed the cache capacity {self.capacity}")
        nxt = self.pick(self._rms(self.prefill(prompt), self.final_norm)[0])
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
        self._tok.copy_(self.pick(self._rms(x[-1:], self.final_norm)[0]))
        self._pos += 1

    def _gemv(self, blk, name, x, out):
        """Token-step projection into a fixed buffer, through the group's rotation when it has one."""
        rot = blk.get("rot_" + name)
        if rot is None:
            self.gemv(blk[name], x, out=out)
        else:
            xr = self._xr[x.numel()]
            self.rotate(rot, x, out=xr)
            self.gemv_rotated(blk[name], xr, out=out)

    def _fused_step(self):
        """One token: 4 fused GEMV launches and 4 small fused kernels per block (2 when the projections form
        their own norm and SwiGLU product, see fuse_x; + 4 all-gathers of row shards on a tensor-parallel
        model), then the greedy head. With self._only set to a phase name only that phase's launches are
        issued (phase_split times them apart)."""
        import ctypes as C
        import torch
        from ._lib import check
        L, cfg, tp = self.ops, self.cfg, self.tp
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        p = lambda t: C.c_void_p(t.data_ptr())
        only = getattr(self, "_only", None)
        on = lambda phase: only is None or only == phase
        if on("embed"):
            self._x.copy_(self.emb.lookup(self._tok)[0])
        delta = None
        stream = [self._x, self._x2]  # stream[0] holds the residual stream

        def fusable(proj):
            return self.fuse_x and getattr(proj, "_h", None) is not None and proj.d_in >= 24

        def norm_then(blk, name, ln, delta, out):
            """x += delta; RMSNorm; the group's projection: without a rotation the projection's kernel does all three
            (x + delta lands in the other stream buffer), with one normalisation and rotation are one kernel."""
            rot = blk.get("rot_" + name)
            dp = p(delta) if delta is not None else None
            if rot is None and fusable(blk[name]):
                if on("projections"):
                    check(L.llvq_gemv_norm_h(blk[name]._h, p(stream[0]), dp, p(blk[ln]), cfg.eps, p(stream[1]), p(out), st))
                stream.reverse()
            elif rot is None:
                if on("norm"):
                    check(L.llvq_op_add_rmsnorm_h(p(stream[0]), dp, p(blk[ln]), p(self._h), cfg.hidden, cfg.eps, st))
                if on("projections"):
                    self.gemv(blk[name], self._h, out=out)
            else:
                xr = self._xr[cfg.hidden]
                if on("norm"):
                    check(L.llvq_op_add_rmsnorm_rotate_h(p(stream[0]), dp, p(blk[ln]), rot._h, p(xr), cfg.hidden, cfg.eps, st))
                if on("projections"):
                    self.gemv_rotated(blk[name], xr, out=out)

        for blk, cache in zip(self.blocks, self.caches):
            norm_then(blk, "qkv", "ln1", delta, self._qkv)
            if on("rope_kv_write"):
                check(L.llvq_op_qkv_rope_cache_h(p(self._qkv), p(blk["q_norm"]), p(blk["k_norm"]), p(self.cos), p(self.sin),
                                                 p(self._pos), p(self._q), p(cache.q[0]), p(cache.s[0]), p(cache.b[0]),
                                                 p(cache.q[1]), p(cache.s[1]), p(cache.b[1]), self.h_loc, self.kv_loc,
                                                 cfg.head_dim, cfg.eps, st))
            if on("attention"):
                check(L.llvq_op_attn_decode_int8_h(p(self._q), p(cache.q[0]), p(cache.s[0]), p(cache.b[0]), p(cache.q[1]),
                                                   p(cache.s[1]), p(cache.b[1]), p(self._pos), p(self._ctx_loc), self.h_loc,
                                                   self.kv_loc, cfg.head_dim, self.attn_splits, p(self._attn_ws), st))
            if tp and on("gathers"):
                tp.gather_into(0, self._ctx, self._ctx_loc)
            if on("projections"):
                self._gemv(blk, "o", self._ctx, self._o_loc)
            if tp and on("gathers"):
                tp.gather_into(1, self._o, self._o_loc)
            norm_then(blk, "gate_up", "ln2", self._o, self._gu)
            rot_down = blk.get("rot_down")
            if rot_down is not None and not tp:  # one rank holds the whole SwiGLU product: gate, rotate, project
                xr = self._xr[cfg.inter]
                if on("swiglu"):
                    check(L.llvq_op_silu_mul_rotate_h(p(self._gu), rot_down._h, p(xr), cfg.inter, st))
                if on("projections"):
                    self.gemv_rotated(blk["down"], xr, out=self._down_loc)
            elif rot_down is None and not tp and fusable(blk["down"]) and cfg.inter % 8 == 0:
                if on("projections"):  # the SwiGLU product is formed in the projection's staging
                    check(L.llvq_gemv_silu_h(blk["down"]._h, p(self._gu), p(self._down_loc), st))
            else:
                if on("swiglu"):
                    check(L.llvq_op_silu_mul_h(p(self._gu), p(self._act_loc), self.inter_loc, st))
                if tp and on("gathers"):
                    tp.gather_into(2, self._act, self._act_loc)
                if on("projections"):
                    self._gemv(blk, "down", self._act, self._down_loc)
            if tp and on("gathers"):
                tp.gather_into(3, self._down, self._down_loc)
            delta = self._down
        if stream[0] is not self._x:  # an odd number of in-kernel norms: bring the stream home
            self._x.copy_(stream[0])
        if on("head"):
            check(L.llvq_op_add_rmsnorm_h(p(self._x), p(delta), p(self.final_norm), p(self._h), cfg.hidden, cfg.eps, st))
            self._tok.copy_(self.pick(self._h))
        if only is None:
            self._pos += 1

    PHASES = ("embed", "norm", "projections", "rope_kv_write", "attention", "swiglu", "gathers", "head")

    def phase_split(self, reps: int = 10) -> dict:
        """Device time of one token step by phase, in ms: every phase's launches (all layers) captured as a graph
        of their own and replayed `reps` times between two events, at the current position and token. The
        phases run apart here, so their sum leaves out what the whole step gains by overlapping a kernel's
        preamble with its predecessor and adds nothing for the gaps between kernels of different phases. The
        counterpart of the reference's per-phase token timing (llvq-llm/tests/phase_timing.rs). Not for a
        tensor-parallel model under NCCL gathers (a collective inside a partial graph needs every rank)."""
        import warnings
        import torch
        out = {}
        tok0 = self._tok.clone()
        for phase in self.PHASES:
            if phase == "gathers" and not self.tp:
                continue
            self._only = phase
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self._fused_step()
                torch.cuda.current_stream().wait_stream(side)
                g = torch.cuda.CUDAGraph()
                with warnings.catch_warnings():
                    # a phase whose work the projections' kernels have absorbed captures nothing
                    warnings.filterwarnings("ignore", message="The CUDA Graph is empty")
                    with torch.cuda.graph(g):
                        self._fused_step()
                g.replay()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                for _ in range(reps):
                    g.replay()
                e1.record()
                torch.cuda.synchronize()
                out[phase] = e0.elapsed_time(e1) / reps
            finally:
                self._only = None
                self._tok.copy_(tok0)
        out["sum"] = sum(out.values())
        return out

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


def kernel_head(lib):
    """The greedy-head hook backed by llvq_op_lm_head_argmax_h (scratch and outputs allocated once per device)."""
    import ctypes as C
    import torch
    from ._lib import check
    state = {}

    def head(embed_rows, h, row_offset):
        dev = embed_rows.device
        if dev not in state:
            state[dev] = (torch.zeros(8192, dtype=torch.uint8, device=dev), torch.zeros(1, dtype=torch.float32, device=dev),
                          torch.zeros(1, dtype=torch.long, device=dev))
        scratch, val, idx = state[dev]
        if not embed_rows.is_contiguous() or h.dtype != torch.float16 or embed_rows.dtype != torch.float16:
            raise ValueError("head: contiguous f16 embedding rows and an f16 hidden state")
        check(lib.llvq_op_lm_head_argmax_h(C.c_void_p(embed_rows.data_ptr()), C.c_void_p(h.data_ptr()), embed_rows.shape[0],
                                           embed_rows.shape[1], row_offset, C.c_void_p(scratch.data_ptr()),
                                           C.c_void_p(val.data_ptr()), C.c_void_p(idx.data_ptr()),
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return val, idx

    return head


def tp_rows(cfg: Qwen3Config, world: int, rank: int) -> dict:
    """[lo, hi) of the rows of each projection that `rank` holds (whole heads for q, k, v)."""
    hd = cfg.head_dim
    hq, hk, it, hid = cfg.n_heads // world * hd, cfg.n_kv // world * hd, cfg.inter // world, cfg.hidden // world
    return {"q": (rank * hq, (rank + 1) * hq), "k": (rank * hk, (rank + 1) * hk), "v": (rank * hk, (rank + 1) * hk),
            "o": (rank * hid, (rank + 1) * hid), "gate": (rank * it, (rank + 1) * it), "up": (rank * it, (rank + 1) * it),
            "down": (rank * hid, (rank + 1) * hid)}


def synthetic_model(rt, cfg: Qwen3Config, config_id: int, capacity: int, seed: int = 0x51, layers: Optional[int] = None,
                    kv_int8: bool = True, fused_ops: bool = True, tp: Optional[TpGroup] = None, dense_prefill_from: int = 1024,
                    keep_host: bool = True, device_codes: bool = False, rotations: bool = False, embed_q8: bool = False,
                    row_scale_gain: float = 1.0):
    """Random-weight model of benchmark configurations 2 and 4: LLVQ codes for every projection, f16 N(0, 0.02)
    norms and tied embedding (norm weights are 1 + N(0, 0.02) so that activations keep their scale).
    With `tp` every rank draws and uploads only its own rows of each matrix (the same matrices for any
    world size; `device_codes` draws the codes on the GPU, for models too large to draw on the host in
    reasonable time). `rotations` gives every group its incoherence rotation (one per shared activation, seeded
    per layer and group), as every real artifact has; the benchmark configurations are drawn without.
    `row_scale_gain` multiplies every row scale (host-drawn matrices only): with the configurations' |N(0, 0.02)| scales
    a random model's residual stream stays close to the embedding of its input token and greedy decoding repeats one
    token, which makes a weak test; a gain of some tens lets the blocks dominate and the tokens vary. Prompts of `dense_prefill_from` rows or more go through a transient dense copy of each
    projection and a library GEMM. Returns (model, host matrices per layer or [] when keep_host is off)."""
    import torch
    from . import synth
    n_layers = layers or cfg.layers
    dev = torch.device("cuda", rt.device)
    g = synth.SplitMix64(seed)
    world, rank = (tp.world, tp.rank) if tp else (1, 0)
    if tp:
        tp.check(cfg)
    rows = tp_rows(cfg, world, rank)
    mats, blocks = [], []

    def f16(n, base=0.0):
        return torch.from_numpy((base + 0.02 * g.gaussian(n)).astype(np.float16)).to(dev)

    shp = {"q": (cfg.n_heads * cfg.head_dim, cfg.hidden), "k": (cfg.n_kv * cfg.head_dim, cfg.hidden),
           "v": (cfg.n_kv * cfg.head_dim, cfg.hidden), "o": (cfg.hidden, cfg.n_heads * cfg.head_dim),
           "gate": (cfg.inter, cfg.hidden), "up": (cfg.inter, cfg.hidden), "down": (cfg.hidden, cfg.inter)}
    for l in range(n_layers):
        if device_codes:
            m = {n: synth.make_matrix_rows_cuda(do, di, synth.matrix_seed(config_id, l, synth.PROJ_IDS[n]), *rows[n], device=dev,
                                                name=f"l{l}.{n}") for n, (do, di) in shp.items()}
        else:
            m = {n: synth.make_matrix_rows(do, di, synth.matrix_seed(config_id, l, synth.PROJ_IDS[n]), *rows[n], name=f"l{l}.{n}")
                 for n, (do, di) in shp.items()}
        if row_scale_gain != 1.0:
            if device_codes:
                raise ValueError("row_scale_gain applies to host-drawn matrices only")
            for mat in m.values():
                mat.row_scales = mat.row_scales * row_scale_gain
        if keep_host:
            mats.append(m)
        blocks.append({"qkv": rt.upload_group([m["q"], m["k"], m["v"]], tail_f16=True), "o": rt.upload(m["o"], tail_f16=True),
                       "gate_up": rt.upload_group([m["gate"], m["up"]], tail_f16=True),
                       "down": rt.upload(m["down"], tail_f16=True),
                       "ln1": f16(cfg.hidden, 1.0), "ln2": f16(cfg.hidden, 1.0),
                       "q_norm": f16(cfg.head_dim, 1.0), "k_norm": f16(cfg.head_dim, 1.0)})
        if rotations:
            widths = {"qkv": cfg.hidden, "o": cfg.n_heads * cfg.head_dim, "gate_up": cfg.hidden, "down": cfg.inter}
            for gi, (name, width) in enumerate(widths.items()):
                blocks[-1]["rot_" + name] = rt.rotation(width, synth.matrix_seed(config_id, l, 16 + gi))
    if device_codes:
        gen = torch.Generator(device=dev).manual_seed(seed)
        embed = (0.02 * torch.randn(cfg.vocab, cfg.hidden, device=dev, generator=gen)).half()
    else:
        embed = f16(cfg.vocab * cfg.hidden).reshape(cfg.vocab, cfg.hidden)
    final_norm = f16(cfg.hidden, 1.0)
    if embed_q8:  # carry the tied embedding as int8 g64, as a file sealed with the reference's embedq does
        embed = Q8Embedding.quantize(rt.lib, embed)

    def gemm(proj, x):
        return rt.forward_batch_dense(proj, x) if x.shape[0] >= dense_prefill_from else rt.forward_batch(proj, x)

    model = FusedQwen3(cfg, blocks, embed, final_norm, capacity, gemv=rt.forward, gemm=gemm, head=kernel_head(rt.lib),
                       kv_int8=kv_int8, ops=rt.lib if fused_ops else None, tp=tp, rotate=rt.rotate,
                       gemv_rotated=rt.forward_rotated)
    return model, mats


def load_archive_model(rt, ar, capacity: int, kv_int8: bool = True, fused_ops: bool = True, dense_prefill_from: int = 1024):
    """A decode loop over a sealed container (`llvq_b200.archive.LvqArchive`): what the reference's fusedrun does
    with a `.llvq` file (llvq-llm/src/bin/fusedrun.rs, fused::load at llvq-llm/src/fused.rs:1147). The projections
    `model.layers.{i}.self_attn.{q,k,v,o}_proj.weight` / `mlp.{gate,up,down}_proj.weight` are uploaded straight
    from the file (q|k|v and gate|up as row groups), every group gets the rotation its records name (the records
    of a group must agree on it, as they consume one activation), the raw tensors give the tied f16 embedding and
    the norms, and `config.json` the shape. An embedding stored group-affine quantised (tag 1) is served when it
    is int8 with groups of 64 (the `embedq` payload); other quantised raw tensors are refused."""
    import ctypes as C
    import json
    import torch
    from ._lib import MatrixDesc, check
    from .runtime import FusedProj
    blobs = dict(ar.blob(i) for i in range(ar.n_blobs))
    if "config.json" not in blobs:
        raise ValueError("the container carries no config.json: not a sealed, self-contained file")
    c = json.loads(blobs["config.json"])
    hd = c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"]
    cfg = Qwen3Config(c["hidden_size"], c["intermediate_size"], c["num_attention_heads"], c["num_key_value_heads"], hd,
                      c["num_hidden_layers"], c["vocab_size"], float(c.get("rope_theta", 1e6)), float(c.get("rms_norm_eps", 1e-6)))
    dev = torch.device("cuda", rt.device)
    index = {ar.matrix(i)["name"]: i for i in range(ar.n_matrices)}
    raws = {}
    for i in range(ar.n_raw):
        t = ar.raw(i)
        if t["tag"] == 0:
            raws[t["name"]] = torch.from_numpy(t["data"].astype(np.float16)).to(dev)
        elif t["name"] == "model.embed_tokens.weight" and t["bits"] == 8 and t["group"] == 64 and len(t["dims"]) == 2:
            V, H = t["dims"]
            raws[t["name"]] = Q8Embedding(rt.lib, torch.from_numpy(t["packed"].copy()).reshape(V, H).to(dev),
                                          torch.from_numpy(t["scales"].astype(np.float16)).reshape(V, H // 64).to(dev),
                                          torch.from_numpy(t["biases"].astype(np.float16)).reshape(V, H // 64).to(dev))
        else:
            raise ValueError(f"{t['name']}: group-affine {t['bits']}-bit g{t['group']}; only an int8 g64 embedding is served")

    def group(layer: int, names):
        ids = [index[f"model.layers.{layer}.{n}.weight"] for n in names]
        descs = (MatrixDesc * len(ids))()
        for k, i in enumerate(ids):
            check(ar.lib.llvq_archive_matrix_desc(ar._h, i, 1, C.byref(descs[k])))
        h = C.c_void_p()
        check(rt.lib.llvq_matrix_upload_group(rt._h, descs, len(ids), C.byref(h)))
        seeds = {ar.matrix(i)["rotation_seed"] for i in ids}
        if len(seeds) != 1:
            raise ValueError(f"layer {layer} {names}: the records of one group name different rotations {seeds}")
        seed = seeds.pop()
        proj = FusedProj(rt, h.value, "|".join(names), [descs[k].d_out for k in range(len(ids))])
        return proj, (rt.rotation(descs[0].d_in, seed) if seed is not None else None)

    blocks = []
    for l in range(cfg.layers):
        blk = {"ln1": raws[f"model.layers.{l}.input_layernorm.weight"], "ln2": raws[f"model.layers.{l}.post_attention_layernorm.weight"],
               "q_norm": raws[f"model.layers.{l}.self_attn.q_norm.weight"], "k_norm": raws[f"model.layers.{l}.self_attn.k_norm.weight"]}
        for key, names in (("qkv", ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"]), ("o", ["self_attn.o_proj"]),
                           ("gate_up", ["mlp.gate_proj", "mlp.up_proj"]), ("down", ["mlp.down_proj"])):
            blk[key], rot = group(l, names)
            if rot is not None:
                blk["rot_" + key] = rot
        blocks.append(blk)

    def gemm(proj, x):
        return rt.forward_batch_dense(proj, x) if x.shape[0] >= dense_prefill_from else rt.forward_batch(proj, x)

    emb = raws["model.embed_tokens.weight"]
    return FusedQwen3(cfg, blocks, emb if isinstance(emb, Q8Embedding) else emb.contiguous(), raws["model.norm.weight"], capacity,
                      gemv=rt.forward, gemm=gemm, head=kernel_head(rt.lib), kv_int8=kv_int8, ops=rt.lib if fused_ops else None,
                      rotate=rt.rotate, gemv_rotated=rt.forward_rotated)
