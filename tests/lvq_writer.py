"""Writer of the reference's container format, for the reader's tests only (TEST INFRASTRUCTURE: the product
never writes this format). Restates write_header (llvq-artifact/src/format.rs:560-575), write_matrix_raw
(format.rs:239-297: name, d_out, d_in, shell cap, centroid count, rotation seed + flag, centroids f64, row
scales f64, tail f32, byte length + MSB-first stream of index_bits + gain_bits per block, llvq-search/src/pack.rs),
write_raw (src/sealed.rs:224-286) and write_blob (sealed.rs:331-336). Little-endian throughout."""
import struct

import numpy as np

MAGIC = {1: b"LVQ1", 2: b"LVQ2", 3: b"LVQ3", 4: b"LVQ4"}
INDEX_BITS = {12: 47, 13: 48}


def pack_stream(indices, gains, index_bits, gain_bits) -> bytes:
    """MSB-first dense bit stream: push(idx, index_bits); push(gain, gain_bits) per block, zero padded."""
    width = index_bits + gain_bits
    acc, nbits, out = 0, 0, bytearray()
    for i, g in zip(indices, gains):
        acc = (acc << width) | (int(i) << gain_bits) | int(g)
        nbits += width
        while nbits >= 8:
            nbits -= 8
            out.append((acc >> nbits) & 0xFF)
        acc &= (1 << nbits) - 1
    if nbits:
        out.append((acc << (8 - nbits)) & 0xFF)
    return bytes(out)


def header(version: int, n_matrices: int, fingerprint: int = 0x338F420F11866319) -> bytes:
    b = MAGIC[version] + struct.pack("<I", n_matrices)
    if version >= 4:
        b += struct.pack("<Q", fingerprint)
    return b


def matrix_record(name, d_out, d_in, indices, gains, centroids, row_scales, tail, shell_cap=12, rotation_seed=None) -> bytes:
    nm = name.encode()
    gb = max(0, (len(centroids) - 1).bit_length())
    b = struct.pack("<I", len(nm)) + nm + struct.pack("<IIII", d_out, d_in, shell_cap, len(centroids))
    b += struct.pack("<QI", rotation_seed or 0, 1 if rotation_seed is not None else 0)
    b += np.asarray(centroids, "<f8").tobytes() + np.asarray(row_scales, "<f8").tobytes()
    b += np.asarray(tail, "<f4").tobytes()
    stream = pack_stream(indices, gains, INDEX_BITS[shell_cap], gb)
    return b + struct.pack("<Q", len(stream)) + stream


def raw_f16(name, array, version=4) -> bytes:
    a = np.asarray(array, "<f2")
    nm = name.encode()
    b = struct.pack("<I", 0) if version >= 3 else b""
    b += struct.pack("<I", len(nm)) + nm + struct.pack("<I", a.ndim) + b"".join(struct.pack("<Q", d) for d in a.shape)
    return b + struct.pack("<Q", a.size) + a.tobytes()


def raw_quant(name, dims, bits, group, packed, scales, biases) -> bytes:
    nm = name.encode()
    b = struct.pack("<I", 1) + struct.pack("<I", len(nm)) + nm + struct.pack("<I", len(dims))
    b += b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<II", bits, group)
    b += struct.pack("<Q", len(packed)) + bytes(packed) + struct.pack("<Q", len(scales))
    return b + np.asarray(scales, "<f2").tobytes() + np.asarray(biases, "<f2").tobytes()


def blob(name, data: bytes) -> bytes:
    nm = name.encode()
    return struct.pack("<I", len(nm)) + nm + struct.pack("<Q", len(data)) + data


def container(version, matrices, raws=(), blobs=()) -> bytes:
    b = header(version, len(matrices)) + b"".join(matrices)
    return b + struct.pack("<I", len(raws)) + b"".join(raws) + struct.pack("<I", len(blobs)) + b"".join(blobs)
