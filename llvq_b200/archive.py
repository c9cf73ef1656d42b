"""The reference's model container (`LVQ1`..`LVQ4`, llvq-artifact/src/format.rs, src/sealed.rs) opened through
the library's reader: matrices as undecoded records whose code streams are uploaded where they lie, raw tensors
(embedding, norms) and blobs (config.json, tokenizer.json). Needs no GPU until `upload`."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import numpy as np

from ._lib import ArchiveMatrixInfo, ArchiveRawInfo, MatrixDesc, check, load

TAIL_F32, TAIL_F16 = 0, 1


class LvqArchive:
    def __init__(self, path: Optional[str] = None, data: Optional[bytes] = None):
        self.lib = load()
        self._h = C.c_void_p()
        self._keep = None
        if (path is None) == (data is None):
            raise ValueError("LvqArchive: give a path or the bytes")
        if path is not None:
            check(self.lib.llvq_archive_open(path.encode(), C.byref(self._h)))
        else:
            self._keep = (C.c_uint8 * len(data)).from_buffer_copy(data)  # kept alive until close
            check(self.lib.llvq_archive_open_memory(self._keep, len(data), C.byref(self._h)))
        v, nm, nr, nb, hf = (C.c_int32() for _ in range(5))
        fp = C.c_uint64()
        check(self.lib.llvq_archive_counts(self._h, C.byref(v), C.byref(nm), C.byref(nr), C.byref(nb), C.byref(hf), C.byref(fp)))
        self.version, self.n_matrices, self.n_raw, self.n_blobs = v.value, nm.value, nr.value, nb.value
        self.fingerprint = fp.value if hf.value else None

    # -- matrices ---------------------------------------------------------------
    def matrix(self, i: int) -> dict:
        """Header fields and side arrays of record i (copies); the code stream as a read-only byte view."""
        info = ArchiveMatrixInfo()
        check(self.lib.llvq_archive_matrix(self._h, i, C.byref(info)))
        tail_w = info.d_in % 24
        as_np = lambda p, n, dt: np.ctypeslib.as_array(p, shape=(n,)).astype(dt, copy=True) if n else np.zeros(0, dt)
        return {"name": info.name.decode(), "d_out": info.d_out, "d_in": info.d_in, "shell_cap": info.shell_cap,
                "index_bits": info.index_bits, "gain_bits": info.gain_bits,
                "rotation_seed": info.rotation_seed if info.has_rotation else None,
                "centroids": as_np(info.centroids, info.n_centroids, np.float64),
                "row_scales": as_np(info.row_scales, info.d_out, np.float64),
                "tail": as_np(info.tail, info.d_out * tail_w, np.float32).reshape(info.d_out, tail_w),
                "codes": np.ctypeslib.as_array(info.stream, shape=(int(info.stream_bytes),)) if info.stream_bytes else np.zeros(0, np.uint8)}

    def names(self) -> List[str]:
        return [self.matrix(i)["name"] for i in range(self.n_matrices)]

    def upload(self, rt, i: int, tail_f16: bool = True):
        """Upload record i to the runtime's GPU straight from the mapped file (no decode, no re-packing)."""
        from .runtime import FusedProj
        d = MatrixDesc()
        check(self.lib.llvq_archive_matrix_desc(self._h, i, TAIL_F16 if tail_f16 else TAIL_F32, C.byref(d)))
        h = C.c_void_p()
        check(self.lib.llvq_matrix_upload(rt._h, C.byref(d), C.byref(h)))
        return FusedProj(rt, h.value, self.matrix(i)["name"], [d.d_out])

    # -- raw tensors and blobs -----------------------------------------------------
    def raw(self, i: int) -> dict:
        """Raw tensor i: f16 values as a numpy float16 array of its dims, or the group-affine fields
        (bits, group, packed u8, scales f16, biases f16) when it is stored quantised."""
        info = ArchiveRawInfo()
        check(self.lib.llvq_archive_raw(self._h, i, C.byref(info)))
        dims = [int(info.dims[k]) for k in range(info.rank)]
        take = lambda p, n: bytes(np.ctypeslib.as_array(p, shape=(int(n),))) if n else b""
        out = {"name": info.name.decode(), "dims": dims, "tag": info.tag}
        if info.tag == 0:
            out["data"] = np.frombuffer(take(info.data, info.data_bytes), dtype="<f2").reshape(dims)
        else:
            out.update(bits=info.bits, group=info.group, packed=np.frombuffer(take(info.data, info.data_bytes), np.uint8),
                       scales=np.frombuffer(take(info.scales, 2 * info.groups), "<f2"),
                       biases=np.frombuffer(take(info.biases, 2 * info.groups), "<f2"))
        return out

    def blob(self, i: int):
        name, data, n = C.c_char_p(), C.POINTER(C.c_uint8)(), C.c_uint64()
        check(self.lib.llvq_archive_blob(self._h, i, C.byref(name), C.byref(data), C.byref(n)))
        return name.value.decode(), bytes(np.ctypeslib.as_array(data, shape=(int(n.value),))) if n.value else b""

    def close(self) -> None:
        if self._h:
            self.lib.llvq_archive_close(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
