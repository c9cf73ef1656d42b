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


@pytest.mark.gpu
def test_decode_loop_from_a_sealed_file_matches_the_loop_built_from_the_same_arrays(rt, tmp_path):
    """file -> tokens: write a small self-contained model with the format-restating writer (rotation seed per
    group, f16 embedding and norms, config.json), load it with load_archive_model, and compare the greedy tokens
    with the loop assembled directly from the same matrices."""
    import json
    import torch
    from llvq_b200 import synth
    from llvq_b200.archive import LvqArchive
    from llvq_b200.model import FusedQwen3, Qwen3Config, kernel_head, load_archive_model
    cfg = Qwen3Config(hidden=256, inter=496, n_heads=4, n_kv=2, head_dim=64, layers=2, vocab=384)
    g = np.random.default_rng(3)
    f16 = lambda *s, base=0.0: (base + 0.02 * g.standard_normal(s)).astype(np.float16)
    shp = {"self_attn.q_proj": (256, 256), "self_attn.k_proj": (128, 256), "self_attn.v_proj": (128, 256),
           "self_attn.o_proj": (256, 256), "mlp.gate_proj": (496, 256), "mlp.up_proj": (496, 256), "mlp.down_proj": (256, 496)}
    groups = {"qkv": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], "o": ["self_attn.o_proj"],
              "gate_up": ["mlp.gate_proj", "mlp.up_proj"], "down": ["mlp.down_proj"]}
    recs, raws, host = [], [], []
    emb, final = f16(cfg.vocab, cfg.hidden), f16(cfg.hidden, base=1.0)
    raws += [W.raw_f16("model.embed_tokens.weight", emb), W.raw_f16("model.norm.weight", final)]
    for l in range(cfg.layers):
        layer = {"mats": {}, "seeds": {}}
        for gi, (key, names) in enumerate(groups.items()):
            seed = 0x5000 + 16 * l + gi
            layer["seeds"][key] = seed
            for n in names:
                m = synth.make_matrix(*shp[n], 900 + 10 * l + len(layer["mats"]))
                layer["mats"][n] = m
                idx, gain = synth.unpack_codes(m.codes)
                recs.append(W.matrix_record(f"model.layers.{l}.{n}.weight", m.d_out, m.d_in, idx, gain, m.centroids, m.row_scales,
                                            m.tail, rotation_seed=seed))
        for nm, arr in (("input_layernorm", f16(cfg.hidden, base=1.0)), ("post_attention_layernorm", f16(cfg.hidden, base=1.0)),
                        ("self_attn.q_norm", f16(64, base=1.0)), ("self_attn.k_norm", f16(64, base=1.0))):
            layer[nm] = arr
            raws.append(W.raw_f16(f"model.layers.{l}.{nm}.weight", arr))
        host.append(layer)
    config = {"hidden_size": 256, "intermediate_size": 496, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
              "num_hidden_layers": 2, "vocab_size": 384, "rope_theta": 1e6, "rms_norm_eps": 1e-6}
    path = os.path.join(tmp_path, "tiny.llvq")
    with open(path, "wb") as f:
        f.write(W.container(4, recs, raws, [W.blob("config.json", json.dumps(config).encode()), W.blob("tokenizer.json", b"{}")]))
    prompt = [int(t) for t in g.integers(0, cfg.vocab, 24)]
    with LvqArchive(path=path) as ar:
        model = load_archive_model(rt, ar, capacity=64)
        assert model.cfg == cfg and "rot_down" in model.blocks[0]
        got = model.generate(prompt, 16)
        graphed = model.generate(prompt, 16, use_graph=True)
    dev = torch.device("cuda")
    t = lambda a: torch.from_numpy(a).to(dev)
    blocks = []
    for layer in host:
        blk = {"ln1": t(layer["input_layernorm"]), "ln2": t(layer["post_attention_layernorm"]),
               "q_norm": t(layer["self_attn.q_norm"]), "k_norm": t(layer["self_attn.k_norm"])}
        for key, names in groups.items():
            ms = [layer["mats"][n] for n in names]
            blk[key] = rt.upload_group(ms, tail_f16=True) if len(ms) > 1 else rt.upload(ms[0], tail_f16=True)
            blk["rot_" + key] = rt.rotation(ms[0].d_in, layer["seeds"][key])
        blocks.append(blk)
    direct = FusedQwen3(cfg, blocks, t(emb), t(final), 64, gemv=rt.forward, gemm=rt.forward_batch, head=kernel_head(rt.lib),
                        ops=rt.lib, rotate=rt.rotate, gemv_rotated=rt.forward_rotated)
    want = direct.generate(prompt, 16)
    assert got == want and graphed == want and len(set(want)) >= 1
    # the same file with the embedding carried as int8 g64 (tag 1): loaded, and equal to the loop built on the
    # same quantised payload
    from llvq_b200.model import Q8Embedding
    q = Q8Embedding.quantize(rt.lib, t(emb))
    raws_q = [W.raw_quant("model.embed_tokens.weight", [cfg.vocab, cfg.hidden], 8, 64, q.wq.cpu().numpy().tobytes(),
                          q.scales.cpu().numpy().reshape(-1), q.biases.cpu().numpy().reshape(-1))] + raws[1:]
    path_q = os.path.join(tmp_path, "tiny_q8.llvq")
    with open(path_q, "wb") as f:
        f.write(W.container(4, recs, raws_q, [W.blob("config.json", json.dumps(config).encode())]))
    with LvqArchive(path=path_q) as ar:
        got_q = load_archive_model(rt, ar, capacity=64).generate(prompt, 16)
    direct_q = FusedQwen3(cfg, blocks, q, t(final), 64, gemv=rt.forward, gemm=rt.forward_batch, head=kernel_head(rt.lib),
                          ops=rt.lib, rotate=rt.rotate, gemv_rotated=rt.forward_rotated)
    assert got_q == direct_q.generate(prompt, 16)
