"""The reference's own host drivers of its CUDA kernel text as the pin of three restatements.

tests/golden/ref_driver_vectors.npz holds seeded inputs and what the reference's drivers computed from them
(llvq-cuda/tests/host_rotate.cpp, llvq-llm/tests/host_embq8.cpp, llvq-llm/tests/host_tail_h.cpp compiled as the
reference's tests compile them; tests/golden/make_ref_driver_vectors.py wrote the file). CPU tests hold the
oracle's restatements to those outputs and, where the built drivers are present, re-run them; GPU tests hold
the CUDA kernels to the same outputs. The rotation TABLES are this library's (the reference builds them in
Rust, which does not run here): what is pinned is the kernel arithmetic on given tables."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_driver_vectors.npz")
ROT_WIDTHS = [24, 96, 7, 64, 2560, 4096, 9728]
TAIL_WIDTHS = [16, 8, 23, 1]


@pytest.fixture(scope="module")
def vec():
    return dict(np.load(GOLDEN))


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def q8_words(codes):
    w = codes.reshape(codes.shape[0], -1, 4).astype(np.uint32)
    return w[..., 0] | w[..., 1] << 8 | w[..., 2] << 16 | w[..., 3] << 24


# ---- CPU: restatements against the drivers' outputs -------------------------------------------------------

@pytest.mark.parametrize("n", ROT_WIDTHS)
def test_rotation_restatements_match_the_reference_kernel_text(vec, n):
    """The float32 replay of the kernel's expression tree gives the driver's bits; the float64 oracle
    (oracle/rotation.py, built from the seed alone) stays within the reference's own bound of it
    (relative L2 < 1e-5, llvq-cuda/tests/rotation_matches_rust.rs)."""
    from oracle import ref_drivers as D
    from oracle.rotation import Rotation
    p = f"rot{n}_"
    m, k = (int(v) for v in vec[p + "mk"])
    want = vec[p + "out"]
    got = D.rotate_f32_replay(n, m, k, vec[p + "inv"], vec[p + "signbits"], vec[p + "small"], vec[p + "xin"])
    assert np.array_equal(bits(got), bits(want))
    r = Rotation(n, int(vec[p + "seed"]))
    assert (r.m, r.k) == (m, k) and np.array_equal(r.signbits(), vec[p + "signbits"])
    ref = r.apply(vec[p + "xin"].view(np.float16).astype(np.float64))
    assert np.linalg.norm(want - ref) <= 1e-5 * max(np.linalg.norm(ref), 1e-300)


def test_q8_dequantiser_restatement_matches_the_reference_kernel_text(vec):
    """q8_deq: one f32 multiply, one f32 add, never fused (llvq-llm/kernels/emb_q8.cu:42-52); the gather narrows
    it to f16 once; the row dot of tv_q8_h agrees with a float64 dot of the dequantised row."""
    from oracle import ref_drivers as D
    deq = D.q8_dequant_f32(vec["q8_codes"], vec["q8_scales"], vec["q8_biases"])
    assert np.array_equal(bits(deq), bits(vec["q8_deq"]))
    assert np.array_equal(deq[vec["q8_ids"]].astype(np.float16).view(np.uint16), vec["q8_gather"])
    x = vec["q8_x"].view(np.float16).astype(np.float64)
    dot64 = deq.astype(np.float64) @ x
    assert np.abs(vec["q8_dot"] - dot64).max() <= 1e-5 * np.abs(deq.astype(np.float64) * x).sum(axis=1).max()


@pytest.mark.parametrize("tw", TAIL_WIDTHS)
def test_tail_epilogue_restatement_matches_the_reference_kernel_text(vec, tw):
    """tail_dot_h on the host is multiply-then-add in f32 (matvec.cu:329-341 under -ffp-contract=off): the
    unfused replay gives its bits. The fused replay, which is what the text becomes on a GPU under NVRTC's
    default --fmad=true and what this library's kernels compute, stays within one rounding per term of it."""
    from oracle import ref_drivers as D
    tail, xt, want = vec[f"tail{tw}_tail"], vec[f"tail{tw}_xt"], vec[f"tail{tw}_tv"]
    assert np.array_equal(bits(D.tail_dot_f32(tail, xt, fused=False)), bits(want))
    fused = D.tail_dot_f32(tail, xt, fused=True)
    mag = (np.abs(tail.view(np.float16).astype(np.float64)) * np.abs(xt.astype(np.float64))).sum(axis=1)
    assert (np.abs(fused.astype(np.float64) - want) <= tw * 2.0 ** -24 * mag + 1e-45).all()


def test_built_drivers_reproduce_the_committed_vectors(vec):
    """Where oracle/_ref holds the drivers built from a checkout of the reference, they give the committed
    outputs again, at every thread count the rotation driver replays."""
    from oracle import ref_drivers as D
    if not D.available():
        pytest.skip("oracle/_ref is not built (no checkout of the reference on this machine)")
    for n in ROT_WIDTHS:
        p = f"rot{n}_"
        m, k = (int(v) for v in vec[p + "mk"])
        res = D.run_host_rotate(n, m, k, vec[p + "inv"], vec[p + "signbits"], vec[p + "small"], vec[p + "xin"])
        for i in range(4):
            assert np.array_equal(bits(res[i]), bits(vec[p + "out"])), (n, i)
    y, deq, dot = D.run_host_embq8(q8_words(vec["q8_codes"]), vec["q8_scales"], vec["q8_biases"], vec["q8_ids"], vec["q8_x"])
    assert np.array_equal(y, vec["q8_gather"]) and np.array_equal(bits(deq), bits(vec["q8_deq"]))
    assert np.array_equal(bits(dot), bits(vec["q8_dot"]))
    for tw in TAIL_WIDTHS:
        assert np.array_equal(bits(D.run_host_tail_h(vec[f"tail{tw}_tail"], vec[f"tail{tw}_xt"])), bits(vec[f"tail{tw}_tv"]))


def test_fused_multiply_add_emulation_rounds_once():
    """fma32 against exact rational arithmetic on operands chosen to defeat a double rounding."""
    from fractions import Fraction
    from oracle.ref_drivers import fma32
    g = np.random.default_rng(5)
    a = g.standard_normal(4000).astype(np.float32)
    b = g.standard_normal(4000).astype(np.float32)
    c = (-(a.astype(np.float64) * b.astype(np.float64)) * (1 + g.choice([0.0, 2.0 ** -24, 2.0 ** -30, 1e-3], 4000))).astype(np.float32)
    got = fma32(a, b, c)
    for i in range(0, 4000, 7):
        exact = Fraction(float(a[i])) * Fraction(float(b[i])) + Fraction(float(c[i]))
        lo, hi = np.nextafter(got[i], np.float32(-np.inf)), np.nextafter(got[i], np.float32(np.inf))
        e = abs(Fraction(float(got[i])) - exact)
        assert e <= abs(Fraction(float(lo)) - exact) and e <= abs(Fraction(float(hi)) - exact), i


# ---- GPU: the CUDA kernels against the drivers' outputs ---------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("n", ROT_WIDTHS)
def test_rotation_kernel_gives_the_bits_of_the_reference_kernel_text(rt, vec, n):
    """rot_apply_kernel takes the Walsh-Hadamard stages three at a time in registers, but every output is the
    same expression tree as the reference kernel's: identical float32 bits on the same tables and input."""
    import torch
    p = f"rot{n}_"
    rot = rt.rotation(n, int(vec[p + "seed"]))
    sb, small = rot.tables()
    assert np.array_equal(sb, vec[p + "signbits"]) and np.array_equal(bits(small), bits(vec[p + "small"]))
    assert np.float32(rot.inv) == vec[p + "inv"]
    x = torch.from_numpy(vec[p + "xin"].view(np.float16).copy()).cuda()
    y = rt.rotate(rot, x).cpu().numpy()
    assert np.array_equal(bits(y), bits(vec[p + "out"]))
    rot.free()


@pytest.mark.gpu
def test_q8_embedding_kernels_give_the_bits_of_the_reference_kernel_text(rt, vec):
    """Gather and dense dequantisation: f16(scale * q + bias) bit for bit; the greedy head's best logit is the
    driver's lane-ordered dot up to the order of the f32 sum."""
    import torch
    from llvq_b200.model import Q8Embedding
    dev = "cuda"
    emb = Q8Embedding(rt.lib, torch.from_numpy(vec["q8_codes"].copy()).to(dev),
                      torch.from_numpy(vec["q8_scales"].view(np.float16).copy()).to(dev),
                      torch.from_numpy(vec["q8_biases"].view(np.float16).copy()).to(dev))
    ids = torch.from_numpy(vec["q8_ids"].astype(np.int64)).to(dev)
    got = emb.lookup(ids).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, vec["q8_gather"])
    assert np.array_equal(emb.dense().cpu().numpy().view(np.uint16), vec["q8_deq"].astype(np.float16).view(np.uint16))
    h = torch.from_numpy(vec["q8_x"].view(np.float16).copy()).to(dev)
    val, idx = emb.pick(h, 0)
    torch.cuda.synchronize()
    dot = vec["q8_dot"]
    assert int(idx) == int(dot.argmax()) and abs(float(val) - float(dot.max())) <= 1e-5 * np.abs(dot).max() + 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("tw", TAIL_WIDTHS)
def test_gemv_tail_epilogue_against_the_reference_kernel_text(rt, vec, tw):
    """With every row scale zero the f32 GEMV returns the tail term alone: bit for bit the fused replay of
    tail_dot_h (the form the reference's text takes on a GPU), and within one rounding per term of the
    host driver's unfused sum."""
    import dataclasses
    import torch
    from llvq_b200 import synth
    from oracle import ref_drivers as D
    tail, xt, want = vec[f"tail{tw}_tail"], vec[f"tail{tw}_xt"], vec[f"tail{tw}_tv"]
    d_out, nb = tail.shape[0], 5
    m = synth.make_matrix(d_out, nb * 24 + tw, 0x7A11 + tw)
    m = dataclasses.replace(m, row_scales=np.zeros(d_out), tail=tail.view(np.float16).astype(np.float32))
    proj = rt.upload(m, tail_f16=True)
    x = np.concatenate([synth.make_activation(nb * 24, 3, np.float32), xt]).astype(np.float32)
    y = rt.forward(proj, torch.from_numpy(x).cuda()).cpu().numpy()
    proj.free()
    assert np.array_equal(bits(y), bits(D.tail_dot_f32(tail, xt, fused=True)))
    mag = (np.abs(tail.view(np.float16).astype(np.float64)) * np.abs(xt.astype(np.float64))).sum(axis=1)
    assert (np.abs(y.astype(np.float64) - want) <= tw * 2.0 ** -24 * mag + 1e-45).all()


# ---- the reference's served layout and its own serving kernel ---------------------------------------------

def test_planes14_transcoder_round_trips_every_class(oracle):
    """oracle/planes14.py writes the reference's 14-byte records (llvq-cuda/kernels/llvq_planes.cuh:1-40) from archive
    codes; read back with the kernel's own field arithmetic they give the oracle's weights, on both ends of every class."""
    from conftest import probe_indices
    from llvq_b200 import synth
    from oracle import planes14
    idx = probe_indices(oracle, per_class_random=20, cap=12)
    idx = idx[idx <= oracle.N12]
    gain = (np.arange(idx.size) & 1).astype(np.uint64)
    codes = synth.pack_codes(idx, gain)
    words = planes14.transcode(codes)
    assert words.dtype == np.uint32 and words.size * 4 == idx.size * 14 + 16
    w, g = planes14.decode_stream(words, idx.size)
    pts, shell, gain_ref, bad = oracle.decode_codes(codes)
    assert bad == 0 and np.array_equal(g, gain_ref)
    want = np.where(shell[:, None] > 0, pts / np.sqrt(16.0 * np.maximum(shell[:, None], 1)), 0.0).astype(np.float32)
    assert np.array_equal(w, want)
    tab, _, _ = planes14.class_tables()
    assert tab.shape == (512, 6) and tab[:302, :5].max() <= 1.0 and (tab[302:, :5] == 0).all()


@pytest.mark.gpu
def test_reference_serving_kernel_agrees_with_the_fused_gemv(rt, oracle):
    """The reference's own tv_planes_h (llvq-llm/kernels/tv_planes_h.cu:38-72), compiled from its sources and run on
    its Planes14 layout of the same weights, against the f64 oracle and against this library's GEMV on the archive
    codes: both within the f16 tolerance of the path, and of each other."""
    import torch
    from llvq_b200 import synth
    from oracle import planes14
    if not planes14.available():
        pytest.skip("oracle/_ref/libref_planes.so is not built (no checkout of the reference where the tree was built)")
    runner = planes14.Planes14Runner(0)
    for d_out, d_in in ((256, 2560), (64, 24 * 140 + 8), (8, 24 * 3)):
        m = synth.make_matrix(d_out, d_in, 0x914 + d_out)
        x32 = synth.make_activation(d_in, 5, np.float32)
        tail16 = m.tail.astype(np.float16).astype(np.float32)
        ref = oracle.gemv_f64(m.codes, d_out, d_in, m.centroids, m.row_scales, tail16, x32.astype(np.float64))
        h = runner.upload(m)
        y_ref = runner.forward(h, torch.from_numpy(x32).cuda())
        proj = rt.upload(m, tail_f16=True)
        y_own = rt.forward_rotated(proj, torch.from_numpy(x32).cuda())  # f32 in, f16 out: the same signature
        torch.cuda.synchronize()
        a, b = y_ref.float().cpu().numpy().astype(np.float64), y_own.float().cpu().numpy().astype(np.float64)
        assert np.linalg.norm(a - ref) <= 1e-3 * np.linalg.norm(ref)
        assert np.linalg.norm(b - ref) <= 1e-3 * np.linalg.norm(ref)
        assert np.linalg.norm(a - b) <= 1e-3 * np.linalg.norm(ref)
        proj.free()
