"""The container reader (llvq_archive_*) against a writer that restates the reference's format
(tests/lvq_writer.py). No file of the reference is available offline, so this pins the reader to the format
as written in llvq-artifact/src/format.rs and src/sealed.rs, and to the packing vectors of g6_pack.rs
(already pinned in the oracle tests): a 47 + 1 bit stream is byte for byte the 6-byte records of the kernels."""
import os
import struct

import numpy as np
import pytest

import lvq_writer as W


def _matrix(seed, d_out=16, d_in=24 * 5 + 7, rotation=True):
    from llvq_b200 import synth
    m = synth.make_matrix(d_out, d_in, seed)
    idx, gain = synth.unpack_codes(m.codes)
    rec = W.matrix_record(f"model.layers.{seed}.self_attn.q_proj.weight", d_out, d_in, idx, gain, m.centroids, m.row_scales,
                          m.tail, rotation_seed=0xABCD00 + seed if rotation else None)
    return m, rec


def test_stream_of_47_plus_1_bits_is_the_six_byte_record_layout():
    from llvq_b200 import synth
    m = synth.make_matrix(8, 24 * 9, 5)
    idx, gain = synth.unpack_codes(m.codes)
    assert W.pack_stream(idx, gain, 47, 1) == m.codes.tobytes()
    assert W.pack_stream([0b101, 0b011, 0b110], [0, 0, 0], 3, 0) == bytes([0xAF, 0x00])  # g6_pack.rs:17-27


@pytest.mark.parametrize("version", [1, 2, 3, 4])
def test_reader_round_trips_every_section(tmp_path, version):
    from llvq_b200.archive import LvqArchive
    mats = [_matrix(1), _matrix(2, d_out=8, d_in=48, rotation=False)]
    emb = (np.arange(24, dtype=np.float32).reshape(4, 6) / 7).astype(np.float16)
    raws = [W.raw_f16("model.embed_tokens.weight", emb, version), W.raw_f16("model.norm.weight", np.ones(6, np.float16), version)]
    if version >= 3:
        raws.append(W.raw_quant("q8", [2, 64], 8, 64, bytes(range(128)), [0.5, 0.25], [-1.0, 2.0]))
    blobs = [W.blob("config.json", b'{"hidden_size": 6}'), W.blob("tokenizer.json", b"")]
    data = W.container(version, [r for _, r in mats], raws, blobs)
    path = os.path.join(tmp_path, "model.llvq")
    with open(path, "wb") as f:
        f.write(data)
    for ar in (LvqArchive(path=path), LvqArchive(data=data)):
        with ar:
            assert (ar.version, ar.n_matrices, ar.n_raw, ar.n_blobs) == (version, 2, len(raws), 2)
            assert ar.fingerprint == (0x338F420F11866319 if version >= 4 else None)
            for i, (m, _) in enumerate(mats):
                got = ar.matrix(i)
                assert got["d_out"] == m.d_out and got["d_in"] == m.d_in and got["shell_cap"] == 12
                assert (got["index_bits"], got["gain_bits"]) == (47, 1)
                assert np.array_equal(got["codes"], m.codes) and np.array_equal(got["centroids"], m.centroids)
                assert np.array_equal(got["row_scales"], m.row_scales) and np.array_equal(got["tail"], m.tail)
            assert ar.matrix(0)["rotation_seed"] == 0xABCD01 and ar.matrix(1)["rotation_seed"] is None
            assert ar.names()[0] == "model.layers.1.self_attn.q_proj.weight"
            r0 = ar.raw(0)
            assert r0["name"] == "model.embed_tokens.weight" and r0["dims"] == [4, 6] and np.array_equal(r0["data"], emb)
            if version >= 3:
                q = ar.raw(2)
                assert (q["bits"], q["group"], q["dims"]) == (8, 64, [2, 64]) and bytes(q["packed"]) == bytes(range(128))
                assert q["scales"].tolist() == [0.5, 0.25] and q["biases"].tolist() == [-1.0, 2.0]
            assert ar.blob(0) == ("config.json", b'{"hidden_size": 6}') and ar.blob(1) == ("tokenizer.json", b"")


def test_reader_refuses_what_the_reference_refuses():
    from llvq_b200._lib import LlvqError
    from llvq_b200.archive import LvqArchive
    _, rec = _matrix(3)
    good = W.container(4, [rec])
    with LvqArchive(data=good) as ar:
        assert ar.n_matrices == 1
    cases = {
        "not an artifact": b"GGUF" + good[4:],
        "codebook mismatch": W.header(4, 1, fingerprint=0x1234) + rec + struct.pack("<II", 0, 0),
        "truncated while reading code stream": good[:len(good) - 30],
        "truncated while reading matrix count": good[:6],
        "truncated while reading raw tensor count": W.header(4, 1) + rec,
        "shell cap 14": W.container(4, [rec.replace(struct.pack("<IIII", 16, 127, 12, 2), struct.pack("<IIII", 16, 127, 14, 2), 1)]),
        "bad raw encoding": W.header(4, 0) + struct.pack("<I", 1) + struct.pack("<I", 7) + b"\0" * 40,
    }
    for what, data in cases.items():
        with pytest.raises(LlvqError) as e:
            LvqArchive(data=data)
        assert what in str(e.value), (what, str(e.value))
    # a stream shorter than the dimensions promise: d_out doubled in the header of the record
    lied = rec.replace(struct.pack("<II", 16, 127), struct.pack("<II", 16, 24 * 50), 1)
    with pytest.raises(LlvqError):
        LvqArchive(data=W.container(4, [lied]))
    with pytest.raises(LlvqError):
        LvqArchive(path="/nonexistent/model.llvq")


def test_records_the_kernels_do_not_serve_are_refused_at_the_descriptor():
    import ctypes as C
    from llvq_b200._lib import LlvqError, MatrixDesc, check
    from llvq_b200.archive import LvqArchive
    rng = np.random.default_rng(0)
    rec13 = W.matrix_record("m13", 8, 24, rng.integers(0, 1 << 47, 8), [0] * 8, [0.9, 1.1], np.ones(8), [], shell_cap=13)
    rec4 = W.matrix_record("m4", 8, 24, rng.integers(0, 1 << 40, 8), [3] * 8, [0.7, 0.9, 1.1, 1.3], np.ones(8), [])
    with LvqArchive(data=W.container(4, [rec13, rec4])) as ar:
        assert ar.matrix(0)["index_bits"] == 48 and ar.matrix(1)["gain_bits"] == 2
        for i in (0, 1):
            with pytest.raises(LlvqError):
                check(ar.lib.llvq_archive_matrix_desc(ar._h, i, 1, C.byref(MatrixDesc())))


@pytest.mark.gpu
def test_projection_uploaded_from_the_file_equals_the_direct_upload(rt, oracle, tmp_path):
    import torch
    from llvq_b200 import synth
    from llvq_b200.archive import LvqArchive
    m, rec = _matrix(9, d_out=64, d_in=24 * 40 + 16)
    path = os.path.join(tmp_path, "one.llvq")
    with open(path, "wb") as f:
        f.write(W.container(4, [rec]))
    x = torch.from_numpy(synth.make_activation(m.d_in, 4, np.float16)).cuda()
    with LvqArchive(path=path) as ar:
        proj = ar.upload(rt, 0)
        y = rt.forward(proj, x)
        torch.cuda.synchronize()
    direct = rt.forward(rt.upload(m, tail_f16=True), x)
    assert torch.equal(y, direct)
    tail16 = m.tail.astype(np.float16).astype(np.float32)
    ref = oracle.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, tail16, x.cpu().numpy().astype(np.float64))
    assert np.linalg.norm(y.cpu().numpy() - ref) / np.linalg.norm(ref) <= 1e-3
