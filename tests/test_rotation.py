"""The incoherence rotation Q = (Q_odd (x) H_m) D: the oracle's structural properties (the reference holds
no golden vector for it: its own tests check the same properties, llvq-quant/src/rotation.rs tests and
llvq-cuda/tests/rotation_matches_rust.rs), the library's host-side table builder against the oracle, and
the CUDA kernel against the oracle within the reference's own bound (relative L2 < 1e-5, worst element
< 1e-3 of the typical magnitude)."""
import ctypes as C

import numpy as np
import pytest

WIDTHS = [(24, 8, 3), (2560, 512, 5), (4096, 4096, 1), (9728, 512, 19), (5120, 1024, 5), (17408, 1024, 17), (96, 32, 3),
          (7, 1, 7), (1, 1, 1), (48, 16, 3)]


def test_oracle_rotation_is_orthogonal_and_deterministic():
    from oracle.rotation import Rotation
    for n, m, k in WIDTHS[:3] + WIDTHS[6:]:
        r = Rotation(n, 0xABC0 + n)
        assert (r.m, r.k) == (m, k)
        g = np.random.default_rng(n)
        x = g.standard_normal(n)
        y = r.apply(x)
        assert abs(np.linalg.norm(y) - np.linalg.norm(x)) <= 1e-12 * max(1.0, np.linalg.norm(x))
        assert np.abs(r.apply_transpose(y) - x).max() <= 1e-12
        assert np.abs(r.small @ r.small.T - np.eye(k)).max() <= 1e-12
        r2 = Rotation(n, 0xABC0 + n)
        assert np.array_equal(r2.signs, r.signs) and np.array_equal(r2.small, r.small)
        if n > 8:
            assert not np.array_equal(Rotation(n, 0xABC1 + n).signs, r.signs)
    # a power of two has no odd factor: the rotation is the scaled Hadamard transform of the signed vector
    r = Rotation(8, 5)
    e = np.zeros(8)
    e[0] = 1.0
    assert np.allclose(np.abs(r.apply(e)), 1 / np.sqrt(8)) and r.small.shape == (1, 1) and abs(r.small[0, 0]) == 1.0


def test_library_host_tables_match_the_oracle():
    """llvq_rotation_build_tables (C++ on the host, no GPU): sign bitmap identical, Q_odd = f32(oracle's),
    1/sqrt(m) narrowed once (RotationTables::build, llvq-llm/src/fused.rs:678-725)."""
    from llvq_b200._lib import check, load
    from oracle.rotation import Rotation
    L = load()
    for n, m, k in WIDTHS:
        seed = 0x5EED0000 + 17 * n
        want = Rotation(n, seed)
        sb = np.zeros((n + 31) // 32, np.uint32)
        small = np.zeros((k, k), np.float32)
        inv = C.c_float()
        check(L.llvq_rotation_build_tables(n, seed, sb.ctypes.data, small.ctypes.data, C.byref(inv)))
        assert np.array_equal(sb, want.signbits()), n
        assert np.abs(small.astype(np.float64) - want.small).max() <= 1e-7, n
        assert inv.value == np.float32(1.0 / np.sqrt(float(m)))
    assert L.llvq_rotation_build_tables(0, 1, None, None, None) != 0


@pytest.mark.gpu
@pytest.mark.parametrize("n,m,k", WIDTHS)
def test_rotation_kernel_matches_the_oracle(rt, n, m, k):
    import torch
    from oracle.rotation import Rotation
    seed = 0x77000 + n
    rot = rt.rotation(n, seed)
    assert (rot.m, rot.k) == (m, k)
    want = Rotation(n, seed)
    sb, small = rot.tables()
    assert np.array_equal(sb, want.signbits())
    g = np.random.default_rng(n + 1)
    for scale in (1.0, 30.0):
        x = (scale * g.standard_normal(n)).astype(np.float16)
        y = rt.rotate(rot, torch.from_numpy(x).cuda()).cpu().numpy().astype(np.float64)
        ref = want.apply(x.astype(np.float64))
        rel = np.linalg.norm(y - ref) / max(np.linalg.norm(ref), 1e-300)
        typical = np.sqrt(np.mean(ref * ref)) if n > 1 else max(abs(ref[0]), 1e-300)
        assert rel < 1e-5 and np.abs(y - ref).max() / max(typical, 1e-300) < 1e-3, (n, rel)
        assert abs(np.linalg.norm(y) - np.linalg.norm(x.astype(np.float64))) <= 1e-5 * np.linalg.norm(x.astype(np.float64)) + 1e-6
    xb = (g.standard_normal((5, n))).astype(np.float16)  # a batch: one CTA per row, same bits as row by row
    yb = rt.rotate(rot, torch.from_numpy(xb).cuda())
    for i in (0, 4):
        assert torch.equal(yb[i], rt.rotate(rot, torch.from_numpy(xb[i]).cuda()))
    rot.free()


@pytest.mark.gpu
def test_rotate_then_fused_gemv_equals_the_unrotated_product(rt, oracle):
    """y = W' (Q x) with the f32 rotated activation going into the f32-in / f16-out GEMV (rotate +
    forward_rotated, llvq-llm/src/fused_cuda.rs:362-402) against the f64 oracle of both steps."""
    import torch
    from llvq_b200 import synth
    from oracle.rotation import Rotation
    d_out, d_in = 96, 2560
    m = synth.make_matrix(d_out, d_in, 0xA0A0)
    proj = rt.upload(m, tail_f16=True)
    rot = rt.rotation(d_in, 0xBEEF)
    x = synth.make_activation(d_in, 21, np.float16)
    xr = rt.rotate(rot, torch.from_numpy(x).cuda())
    y = rt.forward_rotated(proj, xr).cpu().numpy()
    tail16 = m.tail.astype(np.float16).astype(np.float32)
    xr_ref = Rotation(d_in, 0xBEEF).apply(x.astype(np.float64))
    ref = oracle.gemv_f64(m.codes, d_out, d_in, m.centroids, m.row_scales, tail16, xr_ref)
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) <= 1e-3


@pytest.mark.gpu
def test_rotation_refuses_what_it_cannot_serve(rt):
    from llvq_b200._lib import LlvqError
    with pytest.raises(LlvqError):
        rt.rotation(37 * 8, 1)          # odd factor 37 > 32
    with pytest.raises(LlvqError):
        rt.rotation(1 << 17, 1)         # 512 KB of shared memory
    with pytest.raises(ValueError):
        import torch
        rot = rt.rotation(64, 1)
        rt.rotate(rot, torch.zeros(63, dtype=torch.float16, device="cuda"))


@pytest.mark.gpu
@pytest.mark.parametrize("n", [2560, 4096, 9728, 496])
def test_fused_norm_and_gate_kernels_equal_the_two_kernel_sequence(rt, n):
    """add+RMSNorm+rotate and SiLU*up+rotate keep the f16 rounding of the intermediate activation, so they
    give exactly the bits of the separate kernel followed by the rotation."""
    import ctypes as C
    import torch
    from llvq_b200._lib import check
    L = rt.lib
    rot = rt.rotation(n, 0x9000 + n)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    g = torch.Generator(device="cuda").manual_seed(n)
    for with_delta in (True, False):
        x0 = torch.randn(n, device="cuda", generator=g).half()
        delta = (0.3 * torch.randn(n, device="cuda", generator=g)).half()
        w = (1.0 + 0.02 * torch.randn(n, device="cuda", generator=g)).half()
        xa, xb = x0.clone(), x0.clone()
        h = torch.empty(n, device="cuda", dtype=torch.float16)
        check(L.llvq_op_add_rmsnorm_h(p(xa), p(delta) if with_delta else None, p(w), p(h), n, 1e-6, st))
        want = rt.rotate(rot, h)
        got = torch.empty(n, device="cuda", dtype=torch.float32)
        check(L.llvq_op_add_rmsnorm_rotate_h(p(xb), p(delta) if with_delta else None, p(w), rot._h, p(got), n, 1e-6, st))
        torch.cuda.synchronize()
        assert torch.equal(got, want) and torch.equal(xa, xb)
    gu = torch.randn(2 * n, device="cuda", generator=g).half()
    act = torch.empty(n, device="cuda", dtype=torch.float16)
    check(L.llvq_op_silu_mul_h(p(gu), p(act), n, st))
    want = rt.rotate(rot, act)
    got = torch.empty(n, device="cuda", dtype=torch.float32)
    check(L.llvq_op_silu_mul_rotate_h(p(gu), rot._h, p(got), n, st))
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    other = rt.rotation(64, 1)
    assert L.llvq_op_silu_mul_rotate_h(p(gu), other._h, p(got), n, st) != 0  # width mismatch is a status
