"""The allocation-free host-buffer GEMV (llvq_gemv_f32_host_static).

Some callers of this library are not allowed to trigger a device allocation on the
call path: a thread that runs while another thread of the process is capturing a
CUDA graph, or a plugin inside a server that budgets device memory once at
start-up. For them the library stages x and y in a fixed array inside its own
image instead of in cudaMalloc'd buffers. This test calls that entry point through
the C ABI twice in a row and compares each result with the ordinary host-buffer
entry point: same kernel, same inputs, so the bits must be identical.

The file name sorts last on purpose: if this test fails, a run that stops at the
first failure has already executed everything else.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_staging_matches_the_allocating_entry_point(rt):
    from llvq_b200 import _lib, synth
    L = _lib.load()
    m = synth.make_matrix(264, 24 * 50 + 11, 0x57A71C)
    proj = rt.upload(m)
    for call in range(2):  # the second call meets whatever the first one left in the array
        x = synth.make_activation(m.d_in, 0x100 + call)
        want = np.full(m.d_out, np.nan, np.float32)
        got = np.full(m.d_out, np.nan, np.float32)
        assert L.llvq_gemv_f32_host(proj._h, x.ctypes.data, want.ctypes.data, None) == 0
        assert L.llvq_gemv_f32_host_static(proj._h, x.ctypes.data, got.ctypes.data, None) == 0
        assert np.isfinite(want).all() and np.array_equal(got, want)
    # the property the entry point exists for: once the first call has resolved the array's address, a call
    # takes no device memory (cudaMemGetInfo before and after; the allocating entry would not show either, its
    # buffers being the matrix's own, but a regression that allocates on this path would)
    import torch
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    x = synth.make_activation(m.d_in, 0x1FF)
    assert L.llvq_gemv_f32_host_static(proj._h, x.ctypes.data, got.ctypes.data, None) == 0
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    # a second, smaller matrix right after: nothing stale from the larger one leaks into it
    m2 = synth.make_matrix(16, 48, 0x57A71D)
    p2 = rt.upload(m2)
    x = synth.make_activation(48, 7)
    want, got = np.empty(16, np.float32), np.empty(16, np.float32)
    assert L.llvq_gemv_f32_host(p2._h, x.ctypes.data, want.ctypes.data, None) == 0
    assert L.llvq_gemv_f32_host_static(p2._h, x.ctypes.data, got.ctypes.data, None) == 0
    assert np.array_equal(got, want)


def test_static_staging_at_the_documented_limit(rt):
    """d_in == LLVQ_STATIC_MAX_D_IN: the activation fills its part of the array up to the first float of y."""
    from llvq_b200 import _lib, synth
    L = _lib.load()
    m = synth.make_matrix(16, 65536, 0x57A71E)
    proj = rt.upload(m)
    x = synth.make_activation(m.d_in, 0x300)
    want, got = np.full(16, np.nan, np.float32), np.full(16, np.nan, np.float32)
    assert L.llvq_gemv_f32_host(proj._h, x.ctypes.data, want.ctypes.data, None) == 0
    assert L.llvq_gemv_f32_host_static(proj._h, x.ctypes.data, got.ctypes.data, None) == 0
    assert np.isfinite(want).all() and np.array_equal(got, want)


def test_static_staging_refuses_what_does_not_fit(rt):
    from llvq_b200 import _lib, synth
    L = _lib.load()
    wide = synth.make_matrix(8, 65536 + 24, 3)  # one block more than LLVQ_STATIC_MAX_D_IN
    proj = rt.upload(wide)
    x = np.zeros(wide.d_in, np.float32)
    y = np.zeros(8, np.float32)
    assert L.llvq_gemv_f32_host_static(proj._h, x.ctypes.data, y.ctypes.data, None) == _lib.ERR_INVALID
    assert b"exceeds" in L.llvq_last_error()
    assert L.llvq_gemv_f32_host_static(None, x.ctypes.data, y.ctypes.data, None) == _lib.ERR_INVALID
