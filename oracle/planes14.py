"""The reference's served layout (Planes14) written from archive codes, and the launch of the reference's own
serving kernel on it (test and benchmark infrastructure only; the library never imports this).

The reference does not serve the 48-bit archive code: at load it decodes every block on the CPU and rewrites it
as a fixed 14-byte record (llvq-cuda/kernels/llvq_planes.cuh:1-40, host packer llvq-cuda/src/planes14_host.rs:47-95,
load-time transcode llvq-llm/src/fused.rs:1055):

    [ class : 9 ][ gain : 1 ][ smask : 24 ][ plane0 : 24 ][ plane1 : 24 ][ plane2 : 24 ][ 0 : 6 ]   (LSB first)

The level of slot j is plane0[j] | plane1[j] << 1 | plane2[j] << 2, an index into the class's table of absolute
values already divided by sqrt(16 * shell) (ClassRec, llvq-cuda/kernels/llvq_slot.cuh:38-41); smask[j] is the sign.
The class numbering is the transcoder's own business (the kernel only indexes the uploaded table with it): here
record id = class of the index map + 1, id 0 = the origin, levels = the class's distinct magnitudes in descending
order. The reference's transcoder is Rust and does not run here; this one decodes with the CPU oracle and packs with
numpy. `make -C oracle ref` builds the kernel (`tv_planes_h`, llvq-llm/kernels/tv_planes_h.cu:38-72) from the
reference's sources into oracle/_ref/libref_planes.so; `Planes14Runner` launches it through ctypes.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import ref

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_HERE, "_ref", "libref_planes.so")
STRIDE = 14  # bytes per record


def available() -> bool:
    return os.path.exists(LIB)


_tables = None


def class_tables():
    """(tab float32 [512, 6] as ClassRec {vals[5], len}, level_of uint8 [302, 16], starts uint64 [302]):
    record id -> level values / count; (record id, |value|) -> level; first index of every class."""
    global _tables
    if _tables is None:
        tab = np.zeros((512, 6), np.float32)
        tab[:, 5] = np.array([1], np.uint32).view(np.float32)[0]  # len = 1: a lone zero level (origin, unused ids)
        level_of = np.zeros((302, 16), np.uint8)
        starts = np.zeros(302, np.uint64)
        starts[0] = 0
        for ci in range(ref.n_classes(12)):
            d = ref.class_desc(ci, 12)
            lo, _ = ref.class_range(ci, 12)
            starts[ci + 1] = lo
            kinds = d["vals"] if d["odd"] else d["word"] + d["free"] + ([(0, d["n0"])] if d["n0"] else [])
            mags = sorted({abs(int(v)) for v, n in kinds if n > 0}, reverse=True)
            assert 1 <= len(mags) <= 5, (ci, mags)
            for lev, v in enumerate(mags):
                tab[ci + 1, lev] = np.float32(v / np.sqrt(16.0 * d["shell"]))
                level_of[ci + 1, v] = lev
            tab[ci + 1, 5] = np.array([len(mags)], np.uint32).view(np.float32)[0]
        _tables = (tab, level_of, starts)
    return _tables


def transcode(codes: np.ndarray) -> np.ndarray:
    """Archive code stream (uint8 [6 n], MSB-first 48-bit records) -> Planes14 stream as uint32 words, padded for
    the kernel's four-word window. One decode per block through the CPU oracle, as the reference's load does."""
    tab, level_of, starts = class_tables()
    pts, _, gain, bad = ref.decode_codes(codes)
    assert bad == 0
    n = pts.shape[0]
    c = np.ascontiguousarray(codes, np.uint8).reshape(n, 6).astype(np.uint64)
    v = (c[:, 0] << 40) | (c[:, 1] << 32) | (c[:, 2] << 24) | (c[:, 3] << 16) | (c[:, 4] << 8) | c[:, 5]
    idx = v >> np.uint64(1)
    rid = np.searchsorted(starts[1:], idx, side="right").astype(np.int64)  # 0 for the origin (index 0)
    lev = level_of[rid[:, None], np.abs(pts).astype(np.int64)].astype(np.uint64)  # [n, 24]
    bit = np.uint64(1) << np.arange(24, dtype=np.uint64)
    p0 = ((lev & np.uint64(1)) * bit).sum(axis=1, dtype=np.uint64)
    p1 = (((lev >> np.uint64(1)) & np.uint64(1)) * bit).sum(axis=1, dtype=np.uint64)
    p2 = (((lev >> np.uint64(2)) & np.uint64(1)) * bit).sum(axis=1, dtype=np.uint64)
    sm = ((pts < 0).astype(np.uint64) * bit).sum(axis=1, dtype=np.uint64)
    lo = rid.astype(np.uint64) | (gain.astype(np.uint64) << np.uint64(9)) | (sm << np.uint64(10)) | (p0 << np.uint64(34)) \
        | ((p1 & np.uint64(0x3F)) << np.uint64(58))
    hi = (p1 >> np.uint64(6)) | (p2 << np.uint64(18))
    out = np.zeros(n * STRIDE + 16, np.uint8)
    rec = out[:n * STRIDE].reshape(n, STRIDE)
    rec[:, :8] = lo.view(np.uint8).reshape(n, 8)
    rec[:, 8:] = hi.view(np.uint8).reshape(n, 8)[:, :6]
    return out.view(np.uint32)


def transcode_cuda(codes: np.ndarray, device, chunk: int = 1 << 20):
    """transcode() with the packing on a GPU (torch): the lattice decode stays the CPU oracle's, the bit packing of
    large matrices is what takes the time in numpy. Returns an int32 tensor on `device`, same bytes as transcode()."""
    import torch
    tab, level_of, starts = class_tables()
    pts, _, gain, bad = ref.decode_codes(codes)
    assert bad == 0
    n = pts.shape[0]
    lev_t = torch.from_numpy(level_of.astype(np.int64)).to(device)
    starts_t = torch.from_numpy(starts[1:].astype(np.int64)).to(device)
    shifts = torch.tensor([40, 32, 24, 16, 8, 0], dtype=torch.int64, device=device)
    bit = (torch.ones(24, dtype=torch.int64, device=device) << torch.arange(24, dtype=torch.int64, device=device))
    out = torch.zeros(n * STRIDE + 16, dtype=torch.uint8, device=device)
    c_all = np.ascontiguousarray(codes, np.uint8).reshape(n, 6)
    for lo_i in range(0, n, chunk):
        hi_i = min(n, lo_i + chunk)
        c = torch.from_numpy(c_all[lo_i:hi_i]).to(device).to(torch.int64)
        idx = ((c << shifts[None, :]).sum(dim=1)) >> 1
        rid = torch.searchsorted(starts_t, idx, right=True)
        p = torch.from_numpy(pts[lo_i:hi_i]).to(device).to(torch.int64)
        lev = lev_t[rid[:, None], p.abs()]
        p0 = ((lev & 1) * bit).sum(dim=1)
        p1 = (((lev >> 1) & 1) * bit).sum(dim=1)
        p2 = (((lev >> 2) & 1) * bit).sum(dim=1)
        sm = ((p < 0).to(torch.int64) * bit).sum(dim=1)
        g = torch.from_numpy(gain[lo_i:hi_i].astype(np.int64)).to(device)
        lo = rid | (g << 9) | (sm << 10) | (p0 << 34) | ((p1 & 0x3F) << 58)   # bit 63 may be set: two's complement keeps the bytes
        hi = (p1 >> 6) | (p2 << 18)
        rec = out[lo_i * STRIDE:hi_i * STRIDE].view(hi_i - lo_i, STRIDE)
        rec[:, :8] = lo.view(torch.uint8).view(-1, 8)
        rec[:, 8:] = hi.view(torch.uint8).view(-1, 8)[:, :6]
    return out.view(torch.int32)


def decode_stream(words: np.ndarray, n: int):
    """Planes14 stream -> (points int32 [n, 24] in units of the class values' numerators is not kept: returns the
    float32 weights per block before gain and row scale, [n, 24]) by the kernel's own field arithmetic; for tests."""
    tab, _, _ = class_tables()
    raw = words.view(np.uint8)[:n * STRIDE].reshape(n, STRIDE)
    lo = np.zeros((n, 8), np.uint8)
    lo[:] = raw[:, :8]
    hi = np.zeros((n, 8), np.uint8)
    hi[:, :6] = raw[:, 8:]
    lo, hi = lo.view(np.uint64)[:, 0], hi.view(np.uint64)[:, 0]
    rid = (lo & np.uint64(0x1FF)).astype(np.int64)
    gain = ((lo >> np.uint64(9)) & np.uint64(1)).astype(np.uint8)
    sm = (lo >> np.uint64(10)) & np.uint64(0xFFFFFF)
    p0 = (lo >> np.uint64(34)) & np.uint64(0xFFFFFF)
    p1 = ((lo >> np.uint64(58)) | (hi << np.uint64(6))) & np.uint64(0xFFFFFF)
    p2 = (hi >> np.uint64(18)) & np.uint64(0xFFFFFF)
    j = np.arange(24, dtype=np.uint64)
    lev = (((p0[:, None] >> j) & np.uint64(1)) | (((p1[:, None] >> j) & np.uint64(1)) << np.uint64(1))
           | (((p2[:, None] >> j) & np.uint64(1)) << np.uint64(2))).astype(np.int64)
    w = tab[rid[:, None], lev]
    w = np.where(((sm[:, None] >> j) & np.uint64(1)) == 1, -w, w)
    return w.astype(np.float32), gain


class Planes14Runner:
    """The reference kernel on one GPU: uploads the class table once, matrices as Planes14 streams, and launches
    tv_planes_h per matrix (f32 activation in, binary16 result out, as the reference's forward_rotated)."""

    def __init__(self, device: int = 0):
        import torch
        if not available():
            raise FileNotFoundError("oracle/_ref/libref_planes.so is not built (make -C oracle ref)")
        self.torch = torch
        self.dev = torch.device("cuda", device)
        self.lib = C.CDLL(LIB)
        self.lib.ref_tv_planes_h.restype = C.c_int
        self.lib.ref_tv_planes_h.argtypes = [C.c_void_p] * 7 + [C.c_uint, C.c_uint, C.c_uint, C.c_void_p]
        assert self.lib.ref_class_rec_bytes() == 24
        self.tab = torch.from_numpy(class_tables()[0].copy()).to(self.dev)

    def upload(self, m):
        """m: a synthetic matrix (codes, centroids, row_scales, tail; d_out a multiple of 8)."""
        torch = self.torch
        assert m.d_out % 8 == 0
        words = transcode_cuda(m.codes, self.dev)
        return {
            "words": words, "nb": m.d_in // 24, "tail_w": m.d_in % 24, "d_out": m.d_out, "d_in": m.d_in,
            "gscale": torch.tensor(np.asarray(m.centroids, np.float32), device=self.dev),
            "rscale": torch.tensor(np.asarray(m.row_scales, np.float32), device=self.dev),
            "tail": torch.from_numpy(np.ascontiguousarray(m.tail, np.float16).reshape(-1).view(np.int16).copy()).to(self.dev)
            if m.d_in % 24 else torch.zeros(8, dtype=torch.int16, device=self.dev),
        }

    def forward(self, h, x, out=None):
        """x: f32 [d_in] on the device -> f16 [d_out]."""
        torch = self.torch
        y = out if out is not None else torch.empty(h["d_out"], dtype=torch.float16, device=self.dev)
        st = torch.cuda.current_stream().cuda_stream
        rc = self.lib.ref_tv_planes_h(h["words"].data_ptr(), self.tab.data_ptr(), h["gscale"].data_ptr(), h["rscale"].data_ptr(),
                                      h["tail"].data_ptr(), x.data_ptr(), y.data_ptr(), h["nb"], h["tail_w"], h["d_out"], st)
        if rc:
            raise RuntimeError(f"tv_planes_h launch failed: CUDA error {rc}")
        return y
