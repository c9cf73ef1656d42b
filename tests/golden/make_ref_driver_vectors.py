"""Writes tests/golden/ref_driver_vectors.npz: seeded inputs and the outputs of the reference's own host
drivers of its kernel text (oracle/_ref/host_rotate, host_embq8, host_tail_h; `make -C oracle ref` builds
them from a checkout of the reference). Run from the repository root where those binaries exist:

    python tests/golden/make_ref_driver_vectors.py

The rotation tables of a case come from this library's host-side builder (llvq_rotation_build_tables): the
reference builds them in Rust, which does not run here, so the drivers pin the KERNEL arithmetic on given
tables, not the tables. Every array of a case is stored, so the tests need neither the drivers nor the
reference."""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

ROTATION_CASES = [(24, 8, 3), (96, 32, 3), (7, 1, 7), (64, 64, 1), (2560, 512, 5), (4096, 4096, 1), (9728, 512, 19)]


def main() -> None:
    from llvq_b200._lib import check, load
    from oracle import ref_drivers as D
    assert D.available(), "build the drivers first: make -C oracle ref"
    L = load()
    out = {}
    g = np.random.default_rng(0x11F0)
    for n, m, k in ROTATION_CASES:
        seed = 0xC0DE00 + n
        sb = np.zeros((n + 31) // 32, np.uint32)
        small = np.zeros((k, k), np.float32)
        inv = C.c_float()
        check(L.llvq_rotation_build_tables(n, seed, sb.ctypes.data, small.ctypes.data, C.byref(inv)))
        x = (g.standard_normal(n) * g.choice([0.02, 1.0, 30.0])).astype(np.float16)
        x[g.integers(0, n)] = np.float16(6.0e-8)  # a subnormal half
        res = D.run_host_rotate(n, m, k, np.float32(inv.value), sb, small, x.view(np.uint16))
        assert all(np.array_equal(res[0].view(np.uint32), res[i].view(np.uint32)) for i in range(1, 4)), n
        p = f"rot{n}_"
        out[p + "seed"], out[p + "mk"], out[p + "inv"] = np.uint64(seed), np.array([m, k], np.int32), np.float32(inv.value)
        out[p + "signbits"], out[p + "small"], out[p + "xin"], out[p + "out"] = sb, small, x.view(np.uint16), res[0]
    # q8 embedding: 12 rows of 256 columns (4 groups), codes over the whole byte range, signed f16 scales and
    # biases with a subnormal and a zero among them
    rows, d = 12, 256
    codes = g.integers(0, 256, (rows, d), dtype=np.uint8)
    codes[0, :4] = (0, 255, 1, 128)
    scales = (g.uniform(1e-4, 3e-3, (rows, d // 64)) * g.choice([-1.0, 1.0], (rows, d // 64))).astype(np.float16)
    biases = g.uniform(-0.2, 0.2, (rows, d // 64)).astype(np.float16)
    scales[1, 0], biases[1, 1], scales[2, 2] = np.float16(5.0e-8), np.float16(0.0), np.float16(1.0)
    ids = np.array([3, 0, 11, 3, 7], np.uint32)
    x = g.standard_normal(d).astype(np.float16)
    words = codes.reshape(rows, d // 4, 4).astype(np.uint32)
    words = words[..., 0] | words[..., 1] << 8 | words[..., 2] << 16 | words[..., 3] << 24
    y, deq, dot = D.run_host_embq8(words, scales.view(np.uint16), biases.view(np.uint16), ids, x.view(np.uint16))
    out.update(q8_codes=codes, q8_scales=scales.view(np.uint16), q8_biases=biases.view(np.uint16), q8_ids=ids,
               q8_x=x.view(np.uint16), q8_gather=y, q8_deq=deq, q8_dot=dot)
    # f16 tail epilogue: the tail widths of the model's projections (2560 % 24 = 16, 9728 % 24 = 8) and the widest
    for tw in (16, 8, 23, 1):
        d_out = 40
        tail = (0.05 * g.standard_normal((d_out, tw))).astype(np.float16)
        tail[0, 0] = np.float16(3.0e-7)
        xt = (3.0 * g.standard_normal(tw)).astype(np.float32)
        out[f"tail{tw}_tail"], out[f"tail{tw}_xt"] = tail.view(np.uint16), xt
        out[f"tail{tw}_tv"] = D.run_host_tail_h(tail.view(np.uint16), xt)
    path = os.path.join(ROOT, "tests", "golden", "ref_driver_vectors.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
