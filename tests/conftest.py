import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import ref
    ref.lib()
    return ref


@pytest.fixture(scope="session")
def shim():
    """The library's scalar decoders compiled as host C++ (tests/host_shim)."""
    d = os.path.join(ROOT, "tests", "host_shim")
    so, src = os.path.join(d, "libshim.so"), os.path.join(d, "shim.cpp")
    deps = [src] + [os.path.join(ROOT, "llvq_b200", "csrc", f) for f in os.listdir(os.path.join(ROOT, "llvq_b200", "csrc"))]
    if not os.path.exists(so) or any(os.path.getmtime(p) > os.path.getmtime(so) for p in deps):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-o", so, src])
    L = C.CDLL(so)
    L.shim_fingerprint.restype = C.c_uint64
    return L


@pytest.fixture(scope="session")
def rt():
    """One runtime on cuda:0 for the GPU tests."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from llvq_b200 import FusedRuntime
    r = FusedRuntime(0)
    yield r
    r.close()


def probe_indices(oracle, per_class_random=0, seed=1, cap=12):
    """Both ends of every class, their neighbours, the origin and the last index."""
    rng = np.random.default_rng(seed)
    out = [0, 1, 2]
    for ci in range(oracle.n_classes(cap)):
        lo, hi = oracle.class_range(ci, cap)
        out += [lo, min(lo + 1, hi), max(hi - 1, lo), hi, (lo + hi) // 2]
        if per_class_random:
            out += list(rng.integers(lo, hi + 1, per_class_random, dtype=np.uint64))
    return np.array(out, np.uint64)
