"""Writes tests/golden/decode_vectors.json from the CPU oracle.

The reference is Rust and cannot run in the build environment, so these vectors
are regression anchors produced by the oracle *after* it reproduced the
reference's published fingerprint (0x338f420f11866319,
llvq-artifact/tests/codebook_fingerprint.rs:58). The primary pins are the
constants in reference_constants.json, which come from the reference's own test
files. Run from the repository root:  python tests/golden/make_vectors.py
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref  # noqa: E402
from llvq_b200 import synth  # noqa: E402


def main():
    assert ref.fingerprint() == ref.PUBLISHED_FINGERPRINT
    vec = []
    # both ends and the middle of every cap-12 class, the origin, and seeded uniform draws
    idxs = [0]
    for ci in range(ref.n_classes(12)):
        lo, hi = ref.class_range(ci, 12)
        idxs += [lo, (lo + hi) // 2, hi]
    g = synth.SplitMix64(0x600D)
    idxs += [int(v) for v in g.take(200) % np.uint64(ref.N12 + 1)]
    for i in idxs:
        p = ref.decode_index(int(i), 12)
        vec.append({"idx": int(i), "point": [int(v) for v in p]})
    # one small matrix with its f64 product, for the GEMV path
    m = synth.make_matrix(16, 24 * 5 + 7, 0xABCDEF, "golden")
    x = synth.make_activation(m.d_in, 0xABCDEF)
    y = ref.gemv_f64(m.codes, m.d_out, m.d_in, m.centroids, m.row_scales, m.tail, x.astype(np.float64), use_ref=True)
    out = {
        "fingerprint": hex(ref.fingerprint()),
        "decode": vec,
        "gemv": {"d_out": m.d_out, "d_in": m.d_in, "seed": 0xABCDEF,
                 "codes_hex": m.codes.tobytes().hex(), "y": [float(v) for v in y]},
    }
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "decode_vectors.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))


if __name__ == "__main__":
    main()
