"""Seeded synthetic LLVQ matrices with the shapes of the benchmark configurations.

The published Qwen3 artifact is not available offline, so every measurement and
parity case runs on synthetic matrices drawn the way the reference's own kernel
bench draws them (uniform indices over the ball, llvq-cuda/src/bin/matvec.rs:399-421)
from the reference's generator, SplitMix64 with Box-Muller normals
(llvq-core/src/rng.rs:21-41), restated here in vectorised numpy.

Draw order of one matrix (one generator per matrix):
  1. idx[b]  = next() mod (N(12) + 1), row-major over d_out x nblocks
  2. gain[b] = next() & 1, same order;  record = (idx << 1 | gain), 6 bytes big-endian
  3. two centroids 0.5 + U[0,1), sorted, rounded to f32
  4. row_scale[r] = |0.02 * N(0,1)|  (f64)
  5. tail[r,t]    = f32(0.02 * N(0,1))
Activations come from a separate generator (seed | 0xFF): x[c] = f32(N(0,1)).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

N12 = 111_043_117_458_000  # |Lambda24(12)|; the ball with the origin has N12 + 1 points
DIM = 24
_GAMMA = np.uint64(0x9E3779B97F4A7C15)
SEED_BASE = 0x4C4C5651_00000000

PROJ_IDS = {"q": 0, "k": 1, "v": 2, "o": 3, "gate": 4, "up": 5, "down": 6}


class SplitMix64:
    """Vectorised SplitMix64: `take(n)` returns the next n outputs of the scalar generator."""

    def __init__(self, seed: int):
        self.state = np.uint64(seed & 0xFFFFFFFFFFFFFFFF)

    def take(self, n: int) -> np.ndarray:
        with np.errstate(over="ignore"):
            k = np.arange(1, n + 1, dtype=np.uint64)
            z = self.state + k * _GAMMA
            self.state = np.uint64(self.state + np.uint64(n) * _GAMMA)
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            return z ^ (z >> np.uint64(31))

    def skip(self, n: int) -> None:
        """Jump over n outputs (the generator is a counter: state advances by n * gamma)."""
        with np.errstate(over="ignore"):
            self.state = np.uint64(self.state + np.uint64(n) * _GAMMA)

    def uniform(self, n: int) -> np.ndarray:
        return (self.take(n) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)

    def gaussian(self, n: int) -> np.ndarray:
        r = self.take(2 * n)
        u1 = ((r[0::2] >> np.uint64(11)).astype(np.float64) + 1.0) * (1.0 / 9007199254740993.0)
        u2 = (r[1::2] >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)
        return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def pack_codes(idx: np.ndarray, gain: np.ndarray) -> np.ndarray:
    """(idx << 1 | gain) as 6 big-endian bytes per block: the archive's 47+1-bit stream."""
    v = (idx.astype(np.uint64) << np.uint64(1)) | gain.astype(np.uint64)
    return np.ascontiguousarray(v.astype(">u8").view(np.uint8).reshape(-1, 8)[:, 2:]).reshape(-1)


def unpack_codes(codes: np.ndarray):
    b = np.asarray(codes, np.uint8).reshape(-1, 6)
    full = np.zeros((b.shape[0], 8), np.uint8)
    full[:, 2:] = b
    v = full.view(">u8").reshape(-1).astype(np.uint64)
    return v >> np.uint64(1), (v & np.uint64(1)).astype(np.uint8)


@dataclass
class SynthMatrix:
    name: str
    d_out: int
    d_in: int
    codes: np.ndarray       # uint8 [d_out * nb * 6]
    centroids: np.ndarray   # float64 [2]
    row_scales: np.ndarray  # float64 [d_out]
    tail: np.ndarray        # float32 [d_out, d_in % 24]
    shell_cap: int = 12

    @property
    def nb(self) -> int:
        return self.d_in // DIM

    @property
    def n_blocks(self) -> int:
        return self.d_out * self.nb

    def rows(self, lo: int, hi: int) -> "SynthMatrix":
        """Row shard [lo, hi): what one rank of a row-sharded projection holds."""
        nb6 = self.nb * 6
        return SynthMatrix(f"{self.name}[{lo}:{hi}]", hi - lo, self.d_in, self.codes[lo * nb6:hi * nb6],
                           self.centroids, self.row_scales[lo:hi], self.tail[lo:hi], self.shell_cap)


def matrix_seed(config: int, layer: int, proj: int) -> int:
    return SEED_BASE | (config << 24) | (layer << 8) | proj


def make_matrix_rows(d_out: int, d_in: int, seed: int, lo: int, hi: int, name: str = "w") -> SynthMatrix:
    """Rows [lo, hi) of make_matrix(d_out, d_in, seed), drawn without generating the other rows: what one
    rank of a row-sharded projection needs (equal to make_matrix(...).rows(lo, hi) bit for bit)."""
    g = SplitMix64(seed)
    nb, tw = d_in // DIM, d_in % DIM
    n_loc = hi - lo

    def window(per_row, draw):
        g.skip(lo * per_row)
        out = draw(n_loc * per_row)
        g.skip((d_out - hi) * per_row)
        return out

    idx = window(nb, lambda k: g.take(k)) % np.uint64(N12 + 1)
    gain = window(nb, lambda k: g.take(k)) & np.uint64(1)
    cen = np.sort(0.5 + g.uniform(2)).astype(np.float32).astype(np.float64)
    # a normal consumes two outputs: the windows below skip in units of two
    g.skip(2 * lo)
    rs = np.abs(0.02 * g.gaussian(n_loc))
    g.skip(2 * (d_out - hi))
    g.skip(2 * lo * tw)
    tail = (0.02 * g.gaussian(n_loc * tw)).astype(np.float32).reshape(n_loc, tw)
    return SynthMatrix(f"{name}[{lo}:{hi}]", n_loc, d_in, pack_codes(idx, gain), cen, rs, tail)


def make_matrix_rows_cuda(d_out: int, d_in: int, seed: int, lo: int, hi: int, device, tiles: int = 8,
                          name: str = "w") -> SynthMatrix:
    """Rows [lo, hi) of a large synthetic matrix whose codes are drawn on the GPU (torch's seeded generator:
    uniform indices over the ball and uniform gain bits, as make_matrix, but another stream). The matrix is
    cut into `tiles` equal row tiles, each with its own seed, so any rank layout whose shards are whole tiles
    sees the same matrix. Centroids, row scales and tails come from the host generator as in make_matrix."""
    import torch
    if d_out % tiles or lo % (d_out // tiles) or hi % (d_out // tiles):
        raise ValueError(f"rows [{lo}, {hi}) of {d_out} are not whole tiles of {d_out // tiles}")
    nb, tw, per = d_in // DIM, d_in % DIM, d_out // tiles
    parts = []
    for t in range(lo // per, hi // per):
        gen = torch.Generator(device=device).manual_seed((seed * 0x9E3779B1 + t) & 0x7FFFFFFFFFFFFFFF)
        idx = torch.randint(0, N12 + 1, (per * nb,), dtype=torch.int64, device=device, generator=gen)
        gain = torch.randint(0, 2, (per * nb,), dtype=torch.int64, device=device, generator=gen)
        v = (idx << 1) | gain
        shifts = torch.tensor([40, 32, 24, 16, 8, 0], dtype=torch.int64, device=device)
        parts.append(((v[:, None] >> shifts[None, :]) & 0xFF).to(torch.uint8).reshape(-1).cpu().numpy())
    g = SplitMix64(seed)
    cen = np.sort(0.5 + g.uniform(2)).astype(np.float32).astype(np.float64)
    g.skip(2 * lo)
    rs = np.abs(0.02 * g.gaussian(hi - lo))
    g.skip(2 * (d_out - hi))
    g.skip(2 * lo * tw)
    tail = (0.02 * g.gaussian((hi - lo) * tw)).astype(np.float32).reshape(hi - lo, tw)
    codes = np.concatenate(parts) if parts else np.zeros(0, np.uint8)
    return SynthMatrix(f"{name}[{lo}:{hi}]", hi - lo, d_in, codes, cen, rs, tail)


def make_matrix(d_out: int, d_in: int, seed: int, name: str = "w") -> SynthMatrix:
    g = SplitMix64(seed)
    nb, tw = d_in // DIM, d_in % DIM
    n = d_out * nb
    idx = g.take(n) % np.uint64(N12 + 1)
    gain = g.take(n) & np.uint64(1)
    cen = np.sort(0.5 + g.uniform(2)).astype(np.float32).astype(np.float64)
    rs = np.abs(0.02 * g.gaussian(d_out))
    tail = (0.02 * g.gaussian(d_out * tw)).astype(np.float32).reshape(d_out, tw)
    return SynthMatrix(name, d_out, d_in, pack_codes(idx, gain), cen, rs, tail)


def make_activation(d_in: int, seed: int, dtype=np.float32, batch: int | None = None) -> np.ndarray:
    g = SplitMix64(seed | 0xFF)
    n = d_in * (batch or 1)
    x = g.gaussian(n).astype(np.float32)
    if dtype == np.float16:
        x = x.astype(np.float16)
    return x.reshape(batch, d_in) if batch else x


# name -> (hidden, intermediate, q_heads, kv_heads, head_dim, layers, vocab)
MODEL_SHAPES = {
    "qwen3-4b": (2560, 9728, 32, 8, 128, 36, 151936),
    "qwen3-8b": (4096, 12288, 32, 8, 128, 36, 151936),
    "qwen3-14b": (5120, 17408, 40, 8, 128, 40, 151936),
}


def layer_shapes(model: str) -> dict:
    """(d_out, d_in) of the seven projections of one layer."""
    h, inter, qh, kvh, hd, _, _ = MODEL_SHAPES[model]
    return {"q": (qh * hd, h), "k": (kvh * hd, h), "v": (kvh * hd, h), "o": (h, qh * hd),
            "gate": (inter, h), "up": (inter, h), "down": (h, inter)}


def make_layer(model: str, config: int, layer: int) -> dict:
    return {p: make_matrix(do, di, matrix_seed(config, layer, PROJ_IDS[p]), f"{model}.l{layer}.{p}")
            for p, (do, di) in layer_shapes(model).items()}
