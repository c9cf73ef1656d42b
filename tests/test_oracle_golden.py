"""The CPU oracle against the reference's own known answers (tests/golden/reference_constants.json)
and against itself (two independent restatements of the decode)."""
import json
import os

import numpy as np

from conftest import probe_indices

HERE = os.path.dirname(os.path.abspath(__file__))
CONST = json.load(open(os.path.join(HERE, "golden", "reference_constants.json")))
VEC = json.load(open(os.path.join(HERE, "golden", "decode_vectors.json")))


def test_published_fingerprint(oracle):
    assert oracle.fingerprint() == int(CONST["published_fingerprint"]["value"], 16)


def test_ball_sizes_and_class_counts(oracle):
    assert oracle.ball_size(13) == CONST["n13"]["value"]
    assert oracle.ball_size(12) == CONST["n12"]["value"]
    assert oracle.n_classes(12) == CONST["classes_cap12"]["value"]
    assert oracle.n_classes(13) == CONST["classes_cap13"]["value"]
    assert (oracle.ball_size(12) + 1).bit_length() == CONST["index_bits"]["cap12"]
    assert (oracle.ball_size(13) + 1).bit_length() == CONST["index_bits"]["cap13"]


def test_theta_series_from_class_ranges(oracle):
    per_shell = {}
    for ci in range(oracle.n_classes(13)):
        lo, hi = oracle.class_range(ci, 13)
        s = oracle.class_desc(ci, 13)["shell"]
        per_shell[s] = per_shell.get(s, 0) + hi - lo + 1
    for m, n in CONST["theta"]["value"]:
        assert per_shell[m] == n


def test_golay_table(oracle):
    g = oracle.golay_table()
    w = np.array([bin(int(v)).count("1") for v in g])
    for k, n in CONST["golay_weight_buckets"]["value"].items():
        assert int((w == int(k)).sum()) == n
    assert len(set(g.tolist())) == 4096
    assert np.all(np.diff(w) >= 0)  # weight-major
    for k in (8, 12, 16):
        assert np.all(np.diff(g[w == k].astype(np.int64)) > 0)  # ascending inside a weight
    # closed under xor (linearity), minimum distance 8
    s = set(g.tolist())
    for i in range(0, 4096, 97):
        for j in range(0, 4096, 89):
            assert int(g[i]) ^ int(g[j]) in s
    assert min(w[w > 0]) == 8


def test_msb_first_packing(oracle):
    c = CONST["pack_three_3bit"]
    assert oracle.pack_bits(c["values"], c["width"]).tobytes().hex() == c["bytes_hex"]
    d = CONST["pack_density"]
    rng = np.random.default_rng(0)
    vals = rng.integers(0, 1 << 48, d["blocks"], dtype=np.uint64)
    buf = oracle.pack_bits(vals, d["bits"])
    assert buf.size == d["bytes"]
    assert np.array_equal(oracle.unpack_bits(buf, d["blocks"], d["bits"]), vals)
    # the 47+1 split of a record is the same stream as one 48-bit field
    from llvq_b200 import synth
    idx = vals >> np.uint64(1)
    gain = vals & np.uint64(1)
    interleaved = np.stack([idx, gain], 1).reshape(-1)
    two = np.zeros(d["blocks"] * 6, np.uint8)
    # push(idx, 47); push(gain, 1) per block
    bits = np.zeros(d["blocks"] * 48, np.uint8)
    for b in range(64):  # a prefix is enough for the bit-level check
        v = (int(idx[b]) << 1) | int(gain[b])
        for k in range(48):
            bits[b * 48 + k] = (v >> (47 - k)) & 1
    two = np.packbits(bits[:64 * 48])
    assert np.array_equal(two, synth.pack_codes(idx[:64], gain[:64]))
    assert np.array_equal(two, buf[:64 * 6])
    assert interleaved.size == 2 * d["blocks"]


def test_origin_and_bounds(oracle):
    assert not oracle.decode_index(0).any()
    assert oracle.decode_index(oracle.N13, 13) is not None
    assert oracle.decode_index(oracle.N13 + 1, 13) is None
    assert oracle.decode_index(oracle.N12, 12) is not None
    assert oracle.decode_index(oracle.N12 + 1, 12) is None
    # cap 12 is a prefix of cap 13
    for i in (1, 196560, 196561, oracle.N12 // 3, oracle.N12):
        assert np.array_equal(oracle.decode_index(i, 12), oracle.decode_index(i, 13))
    bad = np.zeros(24, np.int32)
    bad[:2] = 2
    assert oracle.encode_point(bad) is None
    far = np.zeros(24, np.int32)
    far[0] = 16
    assert oracle.encode_point(far, 13) is None


def test_shell2_is_exactly_the_first_196560_indices(oracle):
    lo, hi = CONST["shell2_index_range"]["lo"], CONST["shell2_index_range"]["hi"]
    from llvq_b200 import synth
    idx = np.arange(lo, hi + 1, dtype=np.uint64)
    pts, shell, _, bad = oracle.decode_codes(synth.pack_codes(idx, np.zeros_like(idx)), use_ref=True)
    assert bad == 0
    assert np.all(shell == 2)
    assert np.all((pts.astype(np.int32) ** 2).sum(1) == 32)
    assert len({p.tobytes() for p in pts}) == hi - lo + 1  # no collision: a bijection onto Shell(2)
    for p in pts[::997]:
        assert oracle.leech_contains(p.astype(np.int32))
    assert oracle.decode_index(hi + 1, 12) is not None and (oracle.decode_index(hi + 1, 12).astype(int) ** 2).sum() == 48


def test_reference_and_fast_decoders_agree_on_every_class_boundary(oracle):
    for cap in (12, 13):
        for i in probe_indices(oracle, per_class_random=3, cap=cap):
            a, b = oracle.decode_index(int(i), cap), oracle.decode_index(int(i), cap, fast=True)
            assert np.array_equal(a, b), int(i)


def test_decoders_agree_and_roundtrip_on_uniform_draws(oracle):
    from llvq_b200 import synth
    g = synth.SplitMix64(0x630001)
    idx = g.take(200_000) % np.uint64(oracle.N12 + 1)
    codes = synth.pack_codes(idx, np.zeros_like(idx))
    pa, sa, _, bad_a = oracle.decode_codes(codes, use_ref=True)
    pb, sb, _, bad_b = oracle.decode_codes(codes, use_ref=False)
    assert bad_a == bad_b == 0
    assert np.array_equal(pa, pb) and np.array_equal(sa, sb)
    assert np.array_equal((pa.astype(np.int32) ** 2).sum(1), 16 * sa.astype(np.int32))
    for k in range(0, idx.size, 40):  # encode(decode(i)) == i and membership
        p = pa[k].astype(np.int32)
        assert oracle.encode_point(p) == int(idx[k])
        assert int(idx[k]) == 0 or oracle.leech_contains(p)


def test_class_boundaries_roundtrip(oracle):
    for i in probe_indices(oracle, cap=13):
        p = oracle.decode_index(int(i), 13)
        assert oracle.encode_point(p, 13) == int(i)


def test_committed_decode_vectors(oracle):
    assert VEC["fingerprint"] == CONST["published_fingerprint"]["value"]
    for v in VEC["decode"]:
        assert oracle.decode_index(v["idx"]).tolist() == v["point"]
        assert oracle.decode_index(v["idx"], fast=True).tolist() == v["point"]


def test_committed_gemv_vector(oracle):
    from llvq_b200 import synth
    gv = VEC["gemv"]
    m = synth.make_matrix(gv["d_out"], gv["d_in"], gv["seed"], "golden")
    assert m.codes.tobytes().hex() == gv["codes_hex"]
    x = synth.make_activation(m.d_in, gv["seed"]).astype(np.float64)
    y = oracle.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, m.tail, x)
    assert np.allclose(y, gv["y"], rtol=1e-13, atol=0)
    # the f64 product equals dense decode times x (decode_matrix narrows to f32 at the end)
    w = oracle.decode_matrix(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, m.tail)
    assert np.allclose(w.astype(np.float64) @ x, y, rtol=1e-5, atol=1e-9)


def test_reconstruct_scale(oracle):
    """w_j = p_j * centroid[gain] * row_scale / sqrt(16 m); the origin decodes to zeros."""
    from llvq_b200 import synth
    idx = np.array([0, 1, 196561, oracle.N12], np.uint64)
    gain = np.array([1, 0, 1, 1], np.uint64)
    cen = np.array([0.75, 1.25])
    rs = np.array([0.5])
    w = oracle.decode_matrix(synth.pack_codes(idx, gain), 1, 96, cen, rs, np.zeros((1, 0), np.float32))[0]
    assert not w[:24].any()
    p1 = oracle.decode_index(1).astype(np.float64)
    assert np.array_equal(w[24:48], (p1 * (0.75 * 0.5 / np.sqrt(32.0))).astype(np.float32))
    p3 = oracle.decode_index(oracle.N12).astype(np.float64)
    assert np.array_equal(w[72:96], (p3 * (1.25 * 0.5 / np.sqrt(192.0))).astype(np.float32))
