"""The reference's own host drivers of its CUDA kernel text, as checkers (test infrastructure only).

The reference executes the scalar parts of three kernels on the CPU by compiling the kernel text as
plain C++ behind a small shim (llvq-cuda/tests/host_shim.h): the rotation (llvq-cuda/tests/host_rotate.cpp
over kernels/llvq_rot.cuh + rotate.cu), the q8 embedding dequantiser and gather (llvq-llm/tests/host_embq8.cpp
over kernels/emb_q8.cu) and the f16 tail epilogue (llvq-llm/tests/host_tail_h.cpp over tail_dot_h,
llvq-cuda/kernels/matvec.cu:329-341). `make -C oracle ref` builds the three from a checkout of the reference;
this module writes their stdin fixtures, runs them and parses their stdout, and holds the numpy
restatements of the same arithmetic that the tests compare with them.

Nothing here is on the product path: only tests and the build entry point import it.
"""
from __future__ import annotations

import os
import struct
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")
DRIVERS = ("host_rotate", "host_embq8", "host_tail_h")
ROT_KMAX = 32       # LLVQ_ROT_KMAX, llvq-cuda/kernels/llvq_rot.cuh:49
ROT_SMAX = 16384    # the driver's own vector bound, llvq-cuda/tests/host_rotate.cpp:43


def reference_checkout() -> str | None:
    """Directory of a checkout of the reference (LLVQ_REFERENCE_DIR, else `reference` beside this repository)."""
    cand = os.environ.get("LLVQ_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isfile(os.path.join(cand, "llvq-cuda", "tests", "host_rotate.cpp")) else None


def build(force: bool = False) -> bool:
    """Build the three drivers when a checkout of the reference is present; False when there is none."""
    ref = reference_checkout()
    if ref is None:
        return False
    cmd = ["make", "-C", _HERE, "REF=" + ref, "ref"] + (["-B"] if force else ["-s"])
    subprocess.check_call(cmd)
    return True


def driver(name: str) -> str | None:
    p = os.path.join(REF_DIR, name)
    return p if os.access(p, os.X_OK) else None


def available() -> bool:
    return all(driver(d) for d in DRIVERS)


def _run(name: str, fixture: bytes) -> bytes:
    exe = driver(name)
    if exe is None:
        raise FileNotFoundError(f"oracle/_ref/{name} is not built (make -C oracle ref)")
    return subprocess.run([exe], input=fixture, stdout=subprocess.PIPE, check=True, timeout=120).stdout


def fma32(a, b, c):
    """Single-rounded a * b + c on float32 arrays (the device's fma.rn.f32, std::fma on the host). The product of
    two float32 is exact in float64; the float64 sum is then rounded to odd (its rounding error is recovered with
    the two-sum identity, and an inexact even result moves one step towards the true value), after which the
    narrowing to float32 rounds once, correctly."""
    p = np.asarray(a, np.float32).astype(np.float64) * np.asarray(b, np.float32).astype(np.float64)
    c = np.broadcast_to(np.asarray(c, np.float32).astype(np.float64), p.shape)
    s = p + c
    bb = s - p
    err = (p - (s - bb)) + (c - bb)
    even = (s.view(np.uint64) & np.uint64(1)) == 0
    fix = even & (err != 0) & np.isfinite(s)
    toward = np.where(err > 0, np.inf, -np.inf)
    s = np.where(fix, np.nextafter(s, toward), s)
    return s.astype(np.float32)


# ---- rotation -----------------------------------------------------------------------------------------

def run_host_rotate(n: int, m: int, k: int, inv: np.float32, signbits: np.ndarray, small: np.ndarray, xin_bits: np.ndarray):
    """rot_apply of the reference on one f16 vector (bits in `xin_bits`): returns float32 [4, n], the kernel
    replayed with 1, 7, 32 and 256 threads (fixture layout: llvq-cuda/tests/host_rotate.cpp:22-30). `small`
    is the k x k odd mix; the driver wants it at row stride LLVQ_ROT_KMAX, zero padded."""
    assert n == m * k and n <= ROT_SMAX and k <= ROT_KMAX
    pad = np.zeros((ROT_KMAX, ROT_KMAX), np.float32)
    pad[:k, :k] = np.asarray(small, np.float32).reshape(k, k)
    fx = struct.pack("<IIIf", n, m, k, float(inv)) + np.asarray(signbits, "<u4").tobytes() + pad.tobytes() \
        + np.asarray(xin_bits, "<u2").tobytes()
    out = np.frombuffer(_run("host_rotate", fx), "<f4")
    assert out.size == 4 * n, out.size
    return out.reshape(4, n).copy()


def rotate_f32_replay(n: int, m: int, k: int, inv: np.float32, signbits: np.ndarray, small: np.ndarray, xin_bits: np.ndarray):
    """The same expression tree in numpy float32 (llvq_rot.cuh:114-235): sign, Walsh-Hadamard stages len = 1, 2,
    4 ... over each group of m, then s * inv (k == 1) or, per column j, out[g m + j] = sum_t Q[g][t] (s[t m + j] inv)
    as an ascending chain of single-rounded fused multiply-adds."""
    x = np.asarray(xin_bits, np.uint16).view(np.float16).astype(np.float32)
    i = np.arange(n)
    neg = (np.asarray(signbits, np.uint32)[i >> 5] >> (i & 31).astype(np.uint32)) & 1
    s = np.where(neg == 1, -x, x).astype(np.float32)
    ln = 1
    while ln < m:
        v = s.reshape(-1, 2, ln)
        a, b = v[:, 0, :].copy(), v[:, 1, :].copy()
        v[:, 0, :], v[:, 1, :] = a + b, a - b
        ln <<= 1
    inv = np.float32(inv)
    if k == 1:
        return (s * inv).astype(np.float32)
    col = (s.reshape(k, m) * inv).astype(np.float32)
    q = np.asarray(small, np.float32).reshape(k, k)
    out = np.zeros((k, m), np.float32)
    for g in range(k):
        acc = np.zeros(m, np.float32)
        for t in range(k):
            acc = fma32(q[g, t], col[t], acc)
        out[g] = acc
    return out.reshape(n)


# ---- q8 embedding --------------------------------------------------------------------------------------

def run_host_embq8(words: np.ndarray, scales_bits: np.ndarray, biases_bits: np.ndarray, ids: np.ndarray, x_bits: np.ndarray):
    """emb_q8_gather, q8_deq over every weight and the lane-ordered row dot of tv_q8_h
    (fixture layout: llvq-llm/tests/host_embq8.cpp:8-17). `words` uint32 [rows, d / 4] (four codes per word,
    low byte first), scales / biases f16 bits [rows, d / 64]. Returns (y f16 bits [ntok, d], deq float32 [rows, d],
    dot float32 [rows])."""
    rows, dw = words.shape
    d, gpr, ntok = dw * 4, scales_bits.shape[1], ids.size
    fx = struct.pack("<IIII", rows, d, gpr, ntok) + np.asarray(words, "<u4").tobytes() + np.asarray(scales_bits, "<u2").tobytes() \
        + np.asarray(biases_bits, "<u2").tobytes() + np.asarray(ids, "<u4").tobytes() + np.asarray(x_bits, "<u2").tobytes()
    raw = _run("host_embq8", fx)
    assert len(raw) == 2 * ntok * d + 4 * rows * d + 4 * rows
    y = np.frombuffer(raw, "<u2", ntok * d).reshape(ntok, d).copy()
    deq = np.frombuffer(raw, "<f4", rows * d, 2 * ntok * d).reshape(rows, d).copy()
    dot = np.frombuffer(raw, "<f4", rows, 2 * ntok * d + 4 * rows * d).copy()
    return y, deq, dot


def q8_dequant_f32(codes_u8: np.ndarray, scales_bits: np.ndarray, biases_bits: np.ndarray):
    """q8_deq (llvq-llm/kernels/emb_q8.cu:42-52): f32(scale) * f32(code) rounded, + f32(bias) rounded; groups of 64."""
    rows, d = codes_u8.shape
    s = np.asarray(scales_bits, np.uint16).view(np.float16).astype(np.float32).repeat(64, axis=1)
    b = np.asarray(biases_bits, np.uint16).view(np.float16).astype(np.float32).repeat(64, axis=1)
    prod = (s * codes_u8.astype(np.float32)).astype(np.float32)
    return (prod + b).astype(np.float32)


# ---- f16 tail epilogue ---------------------------------------------------------------------------------

def run_host_tail_h(tail_bits: np.ndarray, xt: np.ndarray):
    """tail_dot_h per row (fixture layout: llvq-llm/tests/host_tail_h.cpp:8-13): tail f16 bits [d_out, tail_w],
    xt float32 [tail_w] -> float32 [d_out]."""
    d_out, tail_w = tail_bits.shape
    fx = struct.pack("<II", d_out, tail_w) + np.asarray(tail_bits, "<u2").tobytes() + np.asarray(xt, "<f4").tobytes()
    out = np.frombuffer(_run("host_tail_h", fx), "<f4")
    assert out.size == d_out
    return out.copy()


def tail_dot_f32(tail_bits: np.ndarray, xt: np.ndarray, fused: bool):
    """tv = sum_i f32(tail[row][i]) * xt[i], i ascending from 0.0f in float32 (matvec.cu:329-341).
    fused=False rounds the product and the sum separately: what the host driver computes under
    -ffp-contract=off. fused=True is the chain of fused multiply-adds the same text becomes on a GPU, where
    the reference compiles it with NVRTC's default --fmad=true (llvq-cuda/src/gpu.rs:10-12)."""
    t = np.asarray(tail_bits, np.uint16).view(np.float16).astype(np.float32)
    xt = np.asarray(xt, np.float32)
    tv = np.zeros(t.shape[0], np.float32)
    for i in range(t.shape[1]):
        if fused:
            tv = fma32(t[:, i], xt[i], tv)
        else:
            tv = (tv + (t[:, i] * xt[i]).astype(np.float32)).astype(np.float32)
    return tv
