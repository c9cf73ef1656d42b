"""ctypes front end of the CPU oracle (test infrastructure only).

The arithmetic lives in ``llvq_oracle.cpp``; every function there cites the
reference file it restates. This module only builds/loads the shared object and
wraps the calls in numpy.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")
_SRC = os.path.join(_HERE, "llvq_oracle.cpp")

PUBLISHED_FINGERPRINT = 0x338F420F11866319  # llvq-artifact/tests/codebook_fingerprint.rs:58
N13 = 280_974_212_784_720                    # llvq-core/src/leech.rs:54
N12 = 111_043_117_458_000                    # README.md:832


def build(force: bool = False) -> str:
    """Compile liboracle.so with g++ if it is missing or older than its source."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s", "liboracle.so"])
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        u8p, i8p = C.POINTER(C.c_uint8), C.POINTER(C.c_int8)
        i32p, u32p = C.POINTER(C.c_int32), C.POINTER(C.c_uint32)
        u64p, f64p, f32p = C.POINTER(C.c_uint64), C.POINTER(C.c_double), C.POINTER(C.c_float)
        L.oracle_fingerprint.restype = C.c_uint64
        L.oracle_ball_size.restype = C.c_uint64
        L.oracle_ball_size.argtypes = [C.c_int]
        L.oracle_n_classes.restype = C.c_int
        L.oracle_n_classes.argtypes = [C.c_int]
        L.oracle_pack_bits.restype = C.c_int64
        L.oracle_pack_bits.argtypes = [u64p, C.c_int64, C.c_int, u8p, C.c_int64]
        L.oracle_unpack_bits.argtypes = [u8p, C.c_int64, C.c_int, u64p]
        L.oracle_class_range.argtypes = [C.c_int, C.c_int, u64p, u64p]
        L.oracle_class_desc.argtypes = [C.c_int, C.c_int, i32p]
        L.oracle_golay_table.argtypes = [u32p]
        for name in ("oracle_decode_index", "oracle_decode_index_fast"):
            f = getattr(L, name)
            f.restype = C.c_int
            f.argtypes = [C.c_int, C.c_uint64, i32p]
        L.oracle_encode_point.restype = C.c_int
        L.oracle_encode_point.argtypes = [C.c_int, i32p, u64p]
        L.oracle_leech_contains.restype = C.c_int
        L.oracle_leech_contains.argtypes = [i32p]
        L.oracle_decode_codes.restype = C.c_int64
        L.oracle_decode_codes.argtypes = [u8p, C.c_int64, i8p, u8p, u8p, C.c_int, C.c_int]
        L.oracle_decode_matrix.restype = C.c_int
        L.oracle_decode_matrix.argtypes = [u8p, C.c_int, C.c_int, f64p, f64p, f32p, f32p, C.c_int]
        L.oracle_gemv_f64.restype = C.c_int
        L.oracle_gemv_f64.argtypes = [u8p, C.c_int, C.c_int, f64p, f64p, f32p, f64p, C.c_int,
                                      f64p, f64p, C.c_int, C.c_int]
        L.oracle_hw_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def hw_threads() -> int:
    return int(lib().oracle_hw_threads())


def fingerprint() -> int:
    return int(lib().oracle_fingerprint())


def ball_size(cap: int = 12) -> int:
    return int(lib().oracle_ball_size(cap))


def n_classes(cap: int = 12) -> int:
    return int(lib().oracle_n_classes(cap))


def class_range(ci: int, cap: int = 12):
    lo, hi = C.c_uint64(), C.c_uint64()
    lib().oracle_class_range(cap, ci, C.byref(lo), C.byref(hi))
    return int(lo.value), int(hi.value)


def class_desc(ci: int, cap: int = 12) -> dict:
    raw = np.zeros(32, np.int32)
    lib().oracle_class_desc(cap, ci, _p(raw, C.c_int32))
    d = dict(shell=int(raw[0]), odd=bool(raw[1]), w=int(raw[2]), p_req=int(raw[3]))
    if d["odd"]:
        k = int(raw[4])
        d["vals"] = [(int(raw[8 + t]), int(raw[16 + t])) for t in range(k)]
    else:
        d["word"] = [(int(raw[8 + t]), int(raw[16 + t])) for t in range(int(raw[4]))]
        d["free"] = [(int(raw[12 + t]), int(raw[20 + t])) for t in range(int(raw[5]))]
        d["n0"] = int(raw[24])
    return d


def golay_table() -> np.ndarray:
    out = np.zeros(4096, np.uint32)
    lib().oracle_golay_table(_p(out, C.c_uint32))
    return out


def decode_index(idx: int, cap: int = 12, fast: bool = False):
    """Point of one index, or None when the index is outside the ball."""
    p = np.zeros(24, np.int32)
    f = lib().oracle_decode_index_fast if fast else lib().oracle_decode_index
    ok = f(cap, C.c_uint64(idx), _p(p, C.c_int32))
    return p if ok else None


def encode_point(p, cap: int = 12):
    p = np.ascontiguousarray(p, np.int32)
    out = C.c_uint64()
    ok = lib().oracle_encode_point(cap, _p(p, C.c_int32), C.byref(out))
    return int(out.value) if ok else None


def leech_contains(p) -> bool:
    p = np.ascontiguousarray(p, np.int32)
    return bool(lib().oracle_leech_contains(_p(p, C.c_int32)))


def pack_bits(vals, width: int) -> np.ndarray:
    vals = np.ascontiguousarray(vals, np.uint64)
    cap = (len(vals) * width + 7) // 8
    out = np.zeros(max(cap, 1), np.uint8)
    n = lib().oracle_pack_bits(_p(vals, C.c_uint64), len(vals), width, _p(out, C.c_uint8), cap)
    return out[:n]


def unpack_bits(buf, n: int, width: int) -> np.ndarray:
    buf = np.ascontiguousarray(buf, np.uint8)
    out = np.zeros(n, np.uint64)
    lib().oracle_unpack_bits(_p(buf, C.c_uint8), n, width, _p(out, C.c_uint64))
    return out


def decode_codes(codes, use_ref: bool = False, threads: int = 0):
    """(points int8 [n,24], shell u8 [n], gain u8 [n], n_bad) of packed 6-byte records."""
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    n = codes.size // 6
    pts = np.zeros((n, 24), np.int8)
    shell = np.zeros(n, np.uint8)
    gain = np.zeros(n, np.uint8)
    bad = lib().oracle_decode_codes(_p(codes, C.c_uint8), n, _p(pts, C.c_int8), _p(shell, C.c_uint8),
                                    _p(gain, C.c_uint8), int(use_ref), threads or hw_threads())
    return pts, shell, gain, int(bad)


def decode_matrix(codes, d_out, d_in, centroids, row_scales, tail, threads: int = 0) -> np.ndarray:
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    cen = np.ascontiguousarray(centroids, np.float64)
    rs = np.ascontiguousarray(row_scales, np.float64)
    tl = np.ascontiguousarray(tail, np.float32).reshape(-1)
    if tl.size == 0:
        tl = np.zeros(1, np.float32)
    out = np.zeros((d_out, d_in), np.float32)
    err = lib().oracle_decode_matrix(_p(codes, C.c_uint8), d_out, d_in, _p(cen, C.c_double),
                                     _p(rs, C.c_double), _p(tl, C.c_float), _p(out, C.c_float),
                                     threads or hw_threads())
    if err:
        raise ValueError("index outside the ball in the code stream")
    return out


def gemv_f64(codes, d_out, d_in, centroids, row_scales, tail, x, use_ref: bool = False,
             threads: int = 0, want_absdot: bool = False):
    """f64 reference y = decode(W) @ x for one vector [d_in] or a batch [nx, d_in]."""
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    cen = np.ascontiguousarray(centroids, np.float64)
    rs = np.ascontiguousarray(row_scales, np.float64)
    tl = np.ascontiguousarray(tail, np.float32).reshape(-1)
    if tl.size == 0:
        tl = np.zeros(1, np.float32)
    x = np.ascontiguousarray(x, np.float64)
    single = x.ndim == 1
    xb = x.reshape(1, -1) if single else x
    nx = xb.shape[0]
    y = np.zeros((nx, d_out), np.float64)
    ad = np.zeros((nx, d_out), np.float64)
    err = lib().oracle_gemv_f64(_p(codes, C.c_uint8), d_out, d_in, _p(cen, C.c_double), _p(rs, C.c_double),
                                _p(tl, C.c_float), _p(xb, C.c_double), nx, _p(y, C.c_double),
                                _p(ad, C.c_double), int(use_ref), threads or hw_threads())
    if err:
        raise ValueError("index outside the ball in the code stream")
    if single:
        y, ad = y[0], ad[0]
    return (y, ad) if want_absdot else y
