"""CPU restatement of the reference's incoherence rotation Q = (Q_odd (x) H_m) D. TEST INFRASTRUCTURE ONLY:
imported by tests/ (the checker of the CUDA rotation kernel and of the library's host-side table
builder), never by the product.

Follows llvq-quant/src/rotation.rs:
  * Rotation::new (rotation.rs:51-68): m = largest power of two dividing n, k = n / m; n signs, each
    -1 when next_gaussian() < 0; then Q_odd by Gram-Schmidt on Gaussian rows (orthonormal, rotation.rs:215-235);
  * SplitMix64 + Box-Muller cosine branch (llvq-core/src/rng.rs:21-41);
  * apply / apply_transpose (rotation.rs:101-124), mix (rotation.rs:128-150), wht (rotation.rs:193-212).
All arithmetic in f64, scalar order as in the reference (sums left to right).

Parity status: UNPINNED against reference outputs. The reference holds no golden vector for a rotation
(its own GPU test compares the kernel with this same Rust routine, llvq-cuda/tests/rotation_matches_rust.rs:
relative L2 < 1e-5, worst element < 1e-3 of the typical magnitude) and the Rust toolchain is absent here; what
pins this file are the structural properties the reference tests (orthogonality, Q^T Q = I, k = 1 for powers
of two, determinism in the seed).
"""
from __future__ import annotations

import math

import numpy as np

_MASK = (1 << 64) - 1


class SplitMix64:
    """Scalar generator, llvq-core/src/rng.rs:21-41."""

    def __init__(self, seed: int):
        self.state = seed & _MASK

    def next(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def next_f64(self) -> float:
        return (self.next() >> 11) * (1.0 / 9007199254740992.0)

    def next_gaussian(self) -> float:
        u1 = ((self.next() >> 11) + 1.0) * (1.0 / 9007199254740993.0)
        u2 = self.next_f64()
        return math.sqrt(-2.0 * math.log(u1)) * math.cos(math.tau * u2)


def _orthonormal(k: int, rng: SplitMix64) -> np.ndarray:
    q = np.zeros((k, k))
    for i in range(k):
        row = [rng.next_gaussian() for _ in range(k)]
        for p in range(i):
            prev = q[p]
            d = 0.0
            for a, b in zip(row, prev):
                d += a * b
            row = [r - d * b for r, b in zip(row, prev)]
        nrm = math.sqrt(sum(a * a for a in row))
        assert nrm > 1e-9
        q[i] = [r / nrm for r in row]
    return q


class Rotation:
    def __init__(self, n: int, seed: int):
        assert n > 0
        self.n = n
        self.m = n & -n  # 1 << trailing_zeros(n)
        self.k = n // self.m
        rng = SplitMix64(seed)
        self.signs = np.array([-1.0 if rng.next_gaussian() < 0.0 else 1.0 for _ in range(n)])
        self.small = _orthonormal(self.k, rng)

    def signbits(self) -> np.ndarray:
        """Bit i & 31 of word i >> 5 set = negative (llvq-llm/src/fused.rs:704-709)."""
        out = np.zeros((self.n + 31) // 32, np.uint32)
        for i in np.nonzero(self.signs < 0)[0]:
            out[i >> 5] |= np.uint32(1 << (int(i) & 31))
        return out

    @staticmethod
    def _wht(v: np.ndarray) -> None:
        n, length = v.size, 1
        while length < n:
            w = v.reshape(-1, 2, length)
            a, b = w[:, 0, :].copy(), w[:, 1, :].copy()
            w[:, 0, :], w[:, 1, :] = a + b, a - b
            length <<= 1
        v *= 1.0 / math.sqrt(n)

    def _mix(self, v: np.ndarray, transpose: bool) -> None:
        if self.k == 1:
            return
        q = self.small.T if transpose else self.small
        cols = v.reshape(self.k, self.m).copy()
        out = np.zeros_like(cols)
        for t in range(self.k):  # acc += q[g][t] * col[t], t ascending as in the reference
            out += q[:, t:t + 1] * cols[t:t + 1, :]
        v[:] = out.reshape(-1)

    def apply(self, x) -> np.ndarray:
        v = np.array(x, np.float64) * self.signs
        for g in range(self.k):
            self._wht(v[g * self.m:(g + 1) * self.m])
        self._mix(v, False)
        return v

    def apply_transpose(self, x) -> np.ndarray:
        v = np.array(x, np.float64)
        self._mix(v, True)
        for g in range(self.k):
            self._wht(v[g * self.m:(g + 1) * self.m])
        return v * self.signs
