"""The library's host-built tables and its scalar device decoder (compiled for the host by
tests/host_shim) against the CPU oracle; and the C ABI's exported symbols. No GPU needed."""
import ctypes as C
import os
import re

import numpy as np

from conftest import ROOT, probe_indices


class DevClass(C.Structure):
    _fields_ = [("offset", C.c_uint64), ("arr_a", C.c_uint64), ("arr_b", C.c_uint64), ("cnts_a", C.c_uint64),
                ("cnts_b", C.c_uint32), ("vals_a", C.c_uint32), ("vals_b", C.c_uint32), ("inv_norm", C.c_float),
                ("golay_base", C.c_uint16), ("odd", C.c_uint8), ("w", C.c_uint8), ("p_req", C.c_uint8),
                ("free_n", C.c_uint8), ("n_a", C.c_uint8), ("n_b", C.c_uint8), ("shell", C.c_uint8), ("pad", C.c_uint8 * 7)]


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "llvq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(llvq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from llvq_b200 import _lib
    L = _lib.load()
    names = _declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/llvq_b200.h but not exported"
    for n in _lib._SIGNATURES:
        assert n in names, f"{n} is bound in Python but not declared in the header"
    assert L.llvq_version().decode().count(".") == 2
    assert L.llvq_last_error() is not None


def test_null_arguments_are_refused_without_a_gpu():
    from llvq_b200 import _lib
    L = _lib.load()
    assert L.llvq_codebook_class_record(-1, None) == _lib.ERR_INVALID
    assert L.llvq_codebook_class_record(383, C.create_string_buffer(64)) == _lib.ERR_INVALID
    assert b"class" in L.llvq_last_error()
    assert L.llvq_gemv_f32(None, None, None, None) == _lib.ERR_INVALID
    assert L.llvq_matrix_upload(None, None, None) == _lib.ERR_INVALID
    assert L.llvq_decode_blocks(None, None, 0, None, None, None, None) == _lib.ERR_INVALID
    assert L.llvq_runtime_create(0, None) == _lib.ERR_INVALID
    L.llvq_matrix_free(None)
    L.llvq_runtime_destroy(None)


def test_class_records_match_the_oracle(oracle):
    from llvq_b200 import _lib
    L = _lib.load()
    assert C.sizeof(DevClass) == 64
    for ci in range(383):
        rec = DevClass()
        assert L.llvq_codebook_class_record(ci, C.byref(rec)) == 0
        lo, hi = oracle.class_range(ci, 13)
        d = oracle.class_desc(ci, 13)
        assert rec.offset == lo - 1
        assert bool(rec.odd) == d["odd"] and rec.shell == d["shell"]
        assert abs(rec.inv_norm - 1.0 / np.sqrt(16.0 * d["shell"])) < 1e-7
        kinds_a = [((rec.vals_a >> (4 * j)) & 15, (rec.cnts_a >> (8 * j)) & 255) for j in range(rec.n_a)]
        if d["odd"]:
            assert kinds_a == d["vals"]
            assert hi - lo + 1 == 4096 * rec.arr_a
        else:
            assert kinds_a == d["word"] and rec.w == d["w"] and rec.p_req == d["p_req"]
            kinds_b = [((rec.vals_b >> (4 * j)) & 15, (rec.cnts_b >> (8 * j)) & 255) for j in range(rec.n_b)]
            assert kinds_b == d["free"] + [(0, d["n0"])]
            assert rec.free_n == sum(n for _, n in d["free"])
            gam = {0: 1, 8: 759, 12: 2576, 16: 759, 24: 1}[rec.w]
            sw = 1 if rec.w == 0 else 1 << (rec.w - 1)
            assert hi - lo + 1 == gam * rec.arr_a * rec.arr_b * sw * (1 << rec.free_n)
            assert rec.golay_base == {0: 0, 8: 1, 12: 760, 16: 3336, 24: 4095}[rec.w]
    g = np.zeros(4096, np.uint32)
    assert L.llvq_codebook_golay(g.ctypes.data) == 0
    assert np.array_equal(g, oracle.golay_table())


def test_host_compiled_device_decoder_reproduces_the_fingerprint(shim, oracle):
    assert shim.shim_fingerprint() == oracle.PUBLISHED_FINGERPRINT


def _shim_decode(shim, idx, cap):
    idx = np.ascontiguousarray(idx, np.uint64)
    pts = np.zeros((idx.size, 24), np.int8)
    shell = np.zeros(idx.size, np.uint8)
    shim.shim_decode_indices(idx.ctypes.data_as(C.c_void_p), C.c_int64(idx.size), pts.ctypes.data_as(C.c_void_p),
                             shell.ctypes.data_as(C.c_void_p), cap)
    return pts, shell


def test_host_compiled_device_decoder_matches_oracle(shim, oracle):
    from llvq_b200 import synth
    for cap in (12, 13):
        idx = probe_indices(oracle, per_class_random=20, cap=cap)
        pts, shell = _shim_decode(shim, idx, cap)
        for k, i in enumerate(idx):
            assert np.array_equal(pts[k], oracle.decode_index(int(i), cap)), int(i)
    g = synth.SplitMix64(7)
    idx = g.take(100_000) % np.uint64(oracle.N12 + 1)
    pts, shell = _shim_decode(shim, idx, 12)
    ref_pts, ref_shell, _, bad = oracle.decode_codes(synth.pack_codes(idx, np.zeros_like(idx)))
    assert bad == 0 and np.array_equal(pts, ref_pts) and np.array_equal(shell, ref_shell)
    # refused indices: shell 255, zero point
    pts, shell = _shim_decode(shim, np.array([oracle.N12 + 1, oracle.N13, 1 << 47], np.uint64), 12)
    assert np.all(shell == 255) and not pts.any()
    pts, shell = _shim_decode(shim, np.array([oracle.N13, oracle.N13 + 1], np.uint64), 13)
    assert shell[0] == 13 and shell[1] == 255


def test_synthetic_generator_is_the_scalar_splitmix64():
    from llvq_b200 import synth

    def scalar(seed, n):
        out, s = [], seed
        for _ in range(n):
            s = (s + 0x9E3779B97F4A7C15) & (2 ** 64 - 1)
            z = s
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & (2 ** 64 - 1)
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & (2 ** 64 - 1)
            out.append(z ^ (z >> 31))
        return out

    g = synth.SplitMix64(0xDEADBEEF)
    assert [int(v) for v in g.take(5)] + [int(v) for v in g.take(4)] == scalar(0xDEADBEEF, 9)
    m = synth.make_matrix(8, 24 * 3 + 5, 42)
    idx, gain = synth.unpack_codes(m.codes)
    assert idx.max() <= synth.N12 and set(gain.tolist()) <= {0, 1}
    assert np.array_equal(synth.pack_codes(idx, gain), m.codes)
    assert m.centroids[0] <= m.centroids[1] and m.tail.shape == (8, 5) and (m.row_scales >= 0).all()
    sh = m.rows(2, 6)
    assert sh.d_out == 4 and sh.codes.size == 4 * 3 * 6 and np.array_equal(sh.tail, m.tail[2:6])


def _shim_decode_tab(shim, idx):
    idx = np.ascontiguousarray(idx, np.uint64)
    pts = np.zeros((idx.size, 24), np.int8)
    fam = np.zeros(idx.size, np.int8)
    scale = np.zeros(idx.size, np.float32)
    shim.shim_decode_tab(idx.ctypes.data_as(C.c_void_p), C.c_int64(idx.size), pts.ctypes.data_as(C.c_void_p),
                         fam.ctypes.data_as(C.c_void_p), scale.ctypes.data_as(C.c_void_p))
    return pts, fam, scale


def test_state_table_decoders_match_oracle_on_every_class(shim, oracle):
    """The decoders the fused kernels run (decode_tab.cuh): both ends of all 301 classes, their
    neighbours and 300 draws inside each; every family, the rare classes included."""
    idx = probe_indices(oracle, per_class_random=300, cap=12)
    pts, fam, scale = _shim_decode_tab(shim, idx)
    ref_pts, ref_shell = _shim_decode(shim, idx, 12)  # generic decoder, itself pinned to the oracle above
    assert np.array_equal(pts, ref_pts)
    for k in range(0, idx.size, 41):
        assert np.array_equal(pts[k], oracle.decode_index(int(idx[k])))
    assert set(fam.tolist()) >= {-1, 0, 1, 2, 3}
    ok = ref_shell > 0
    assert np.allclose(scale[ok], 1.0 / np.sqrt(16.0 * ref_shell[ok]), rtol=1e-6)
    pts, fam, _ = _shim_decode_tab(shim, np.array([0, oracle.N12 + 1, (1 << 47) - 1, 1 << 47, (1 << 63) + 5], np.uint64))
    assert fam.tolist() == [-1, -2, -2, -2, -2] and not pts.any()


def test_state_table_decoders_match_oracle_on_uniform_draws(shim, oracle):
    from llvq_b200 import synth
    g = synth.SplitMix64(0x7AB1E)
    idx = g.take(600_000) % np.uint64(oracle.N12 + 1)
    pts, fam, _ = _shim_decode_tab(shim, idx)
    ref_pts, _, _, bad = oracle.decode_codes(synth.pack_codes(idx, np.zeros_like(idx)))
    assert bad == 0 and np.array_equal(pts, ref_pts)
    frac = {f: float((fam == f).mean()) for f in (0, 1, 2, 3)}
    assert frac[0] < 2e-3 and frac[3] > 0.45 and frac[1] > 0.2 and frac[2] > 0.2


def test_state_tables_cover_the_ball_and_fit_shared_memory(shim):
    out = (C.c_int64 * 9)()
    shim.shim_tab_table_sizes(out)
    assert out[0] < 120_000            # bytes of the blob the kernels keep in shared memory
    assert out[1] < out[0] // 2         # what classification needs lands first
    assert out[2] < 400_000             # entries of the off-support arrangement table (global memory)
    assert out[7] == 0                  # no class is left without a decoder
    assert abs(sum(out[3:7]) / 1e12 - 1.0) < 1e-9
