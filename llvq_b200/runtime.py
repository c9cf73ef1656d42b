"""Host-side mirror of the reference's operator surface for the fused path.

`FusedRuntime` / `FusedProj` follow llvq-llm/src/fused_cuda.rs:119-160,182-402: a
runtime owns the per-GPU tables, a projection owns its resident device buffers
and `forward_rotated(proj, x)` is the one call the model makes per projection.
Everything is a thin layer over the C ABI of include/llvq_b200.h; PyTorch only
provides device memory and streams. There is no CPU path: without the CUDA
library or a GPU these classes raise.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _lib
from ._lib import MatrixDesc, TAIL_F16, TAIL_F32, check


def _desc(m, tail_mode: int, keep: list) -> MatrixDesc:
    codes = np.ascontiguousarray(m.codes, np.uint8)
    cen = np.ascontiguousarray(m.centroids, np.float64)
    rs = np.ascontiguousarray(m.row_scales, np.float64)
    tail = np.ascontiguousarray(m.tail, np.float32).reshape(-1)
    if cen.size != 2:
        # the fused path serves exactly one gain bit (llvq-llm/src/fused.rs:1171-1177)
        raise ValueError(f"{m.name}: {cen.size} centroids; the fused path needs exactly 2")
    keep += [codes, cen, rs, tail]
    return MatrixDesc(m.d_out, m.d_in, int(getattr(m, "shell_cap", 12)), tail_mode,
                      codes.ctypes.data if codes.size else None, cen.ctypes.data, rs.ctypes.data,
                      tail.ctypes.data if tail.size else None)


class FusedProj:
    """One resident projection (or a row-concatenated group of projections)."""

    def __init__(self, rt: "FusedRuntime", handle: int, name: str, splits: Sequence[int]):
        self.rt, self._h, self.name = rt, C.c_void_p(handle), name
        self.splits = list(splits)  # d_out of every segment, in order
        d_out, d_in = C.c_int32(), C.c_int32()
        check(rt.lib.llvq_matrix_dims(self._h, C.byref(d_out), C.byref(d_in)))
        self.d_out, self.d_in = d_out.value, d_in.value

    def algorithmic_bytes(self, x_bytes: int, y_bytes: int) -> int:
        out = C.c_uint64()
        check(self.rt.lib.llvq_matrix_algorithmic_bytes(self._h, x_bytes, y_bytes, C.byref(out)))
        return out.value

    @property
    def n_blocks(self) -> int:
        return self.d_out * (self.d_in // 24)

    def free(self) -> None:
        if self._h:
            self.rt.lib.llvq_matrix_free(self._h)
            self._h = C.c_void_p(None)

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class DeviceRotation:
    """Handle of one uploaded rotation (sign bitmap, odd mix, 1/sqrt(m))."""

    def __init__(self, rt: "FusedRuntime", handle: int, n: int):
        self.rt, self._h, self.n = rt, C.c_void_p(handle), n
        m, k, inv = C.c_int32(), C.c_int32(), C.c_float()
        check(rt.lib.llvq_rotation_info(self._h, None, C.byref(m), C.byref(k), C.byref(inv)))
        self.m, self.k, self.inv = m.value, k.value, inv.value

    def tables(self):
        """(signbits uint32 [ceil(n/32)], small float32 [k, k]) as uploaded."""
        sb = np.zeros((self.n + 31) // 32, np.uint32)
        small = np.zeros((self.k, self.k), np.float32)
        check(self.rt.lib.llvq_rotation_tables(self._h, sb.ctypes.data, small.ctypes.data))
        return sb, small

    def free(self) -> None:
        if self._h:
            self.rt.lib.llvq_rotation_free(self._h)
            self._h = C.c_void_p(None)


class FusedRuntime:
    """Per-GPU decoder tables, verified against the published codebook fingerprint on creation."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        self.device = device
        h = C.c_void_p()
        check(self.lib.llvq_runtime_create(device, C.byref(h)))
        self._h = h

    # -- codebook ---------------------------------------------------------------
    def fingerprint(self) -> int:
        out = C.c_uint64()
        check(self.lib.llvq_codebook_fingerprint(self._h, C.byref(out)))
        return out.value

    def codebook_info(self, shell_cap: int = 12):
        n, size = C.c_int32(), C.c_uint64()
        check(self.lib.llvq_codebook_info(self._h, shell_cap, C.byref(n), C.byref(size)))
        return n.value, size.value

    def kernel_info(self):
        """[(name, registers, local bytes, static shared bytes, binary version)] of the hot kernels, as read back
        from the loaded module when the runtime was created (local bytes are always 0: a spill is refused)."""
        out, i = [], 0
        while True:
            name, regs, loc, smem, ver = C.c_char_p(), C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
            if self.lib.llvq_runtime_kernel_info(self._h, i, C.byref(name), C.byref(regs), C.byref(loc), C.byref(smem),
                                                 C.byref(ver)) != 0:
                return out
            out.append((name.value.decode(), regs.value, loc.value, smem.value, ver.value))
            i += 1

    def set_overlap(self, on: bool) -> None:
        """Consecutive fused GEMV launches overlap the next launch's table and code prologue with the previous
        launch's tail (programmatic dependent launch); on by default, off gives ordinary launches."""
        check(self.lib.llvq_runtime_set_overlap(self._h, 1 if on else 0))

    def poll_range_error(self) -> bool:
        flag = C.c_int32()
        check(self.lib.llvq_runtime_poll_error(self._h, C.byref(flag)))
        return bool(flag.value)

    # -- upload -----------------------------------------------------------------
    def upload(self, m, tail_f16: bool = False) -> FusedProj:
        keep: list = []
        d = _desc(m, TAIL_F16 if tail_f16 else TAIL_F32, keep)
        h = C.c_void_p()
        check(self.lib.llvq_matrix_upload(self._h, C.byref(d), C.byref(h)))
        return FusedProj(self, h.value, m.name, [m.d_out])

    def upload_group(self, ms: Sequence, tail_f16: bool = False) -> FusedProj:
        keep: list = []
        arr = (MatrixDesc * len(ms))(*[_desc(m, TAIL_F16 if tail_f16 else TAIL_F32, keep) for m in ms])
        h = C.c_void_p()
        check(self.lib.llvq_matrix_upload_group(self._h, arr, len(ms), C.byref(h)))
        return FusedProj(self, h.value, "|".join(m.name for m in ms), [m.d_out for m in ms])

    # -- rotation ---------------------------------------------------------------
    def rotation(self, n: int, seed: int) -> "DeviceRotation":
        """The incoherence rotation of width n built from a matrix's rotation seed (RotationTables::build)."""
        h = C.c_void_p()
        check(self.lib.llvq_rotation_create(self._h, n, seed & 0xFFFFFFFFFFFFFFFF, C.byref(h)))
        return DeviceRotation(self, h.value, n)

    def rotate(self, rot: "DeviceRotation", x, out=None):
        """f16 activation [n] or [B, n] -> the same in the rotated basis, f32; FusedRuntime::rotate.
        Its output is what forward_rotated consumes; one rotation serves every projection of a group."""
        import torch
        if not x.is_cuda or x.dtype != torch.float16 or not x.is_contiguous() or x.shape[-1] != rot.n or x.dim() > 2:
            raise ValueError(f"rotate: a contiguous CUDA f16 activation of {rot.n} elements (or a batch of them)")
        xr = out if out is not None else torch.empty(x.shape, dtype=torch.float32, device=x.device)
        check(self.lib.llvq_rotate_h(rot._h, x.data_ptr(), xr.data_ptr(), x.numel() // rot.n, self._stream()))
        return xr

    # -- forward ----------------------------------------------------------------
    @staticmethod
    def _stream():
        import torch
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def forward_rotated(self, proj: FusedProj, xr, out=None):
        """f32 activation [d_in] -> f16 result [d_out]; FusedRuntime::forward_rotated."""
        import torch
        self._check_x(proj, xr, torch.float32)
        y = out if out is not None else torch.empty(proj.d_out, dtype=torch.float16, device=xr.device)
        check(self.lib.llvq_gemv_f32x_h(proj._h, xr.data_ptr(), y.data_ptr(), self._stream()))
        return y

    def forward(self, proj: FusedProj, x, out=None):
        """Same dtype in and out: f32 -> f32 (kernel bench path) or f16 -> f16 (model path)."""
        import torch
        if x.dtype == torch.float32:
            fn = self.lib.llvq_gemv_f32
        elif x.dtype == torch.float16:
            fn = self.lib.llvq_gemv_h
        else:
            raise TypeError(f"activation dtype {x.dtype}: the fused path takes f32 or f16")
        self._check_x(proj, x, x.dtype)
        y = out if out is not None else torch.empty(proj.d_out, dtype=x.dtype, device=x.device)
        check(fn(proj._h, x.data_ptr(), y.data_ptr(), self._stream()))
        return y

    def forward_norm(self, proj: FusedProj, resid, delta, norm_w, eps: float, resid_out, out=None):
        """y = W (RMSNorm(resid + delta) * norm_w) with the norm computed in the projection's kernel; resid + delta goes
        to resid_out (not resid itself). f16 throughout; the bits of add_rmsnorm followed by forward. `delta` may be None."""
        import torch
        self._check_x(proj, resid, torch.float16)
        for t in (delta, norm_w, resid_out):
            if t is not None:
                self._check_x(proj, t, torch.float16)
        y = out if out is not None else torch.empty(proj.d_out, dtype=torch.float16, device=resid.device)
        check(self.lib.llvq_gemv_norm_h(proj._h, resid.data_ptr(), delta.data_ptr() if delta is not None else None,
                                        norm_w.data_ptr(), eps, resid_out.data_ptr(), y.data_ptr(), self._stream()))
        return y

    def forward_silu(self, proj: FusedProj, gate_up, out=None):
        """y = W (silu(gate) * up) for gate_up = [gate | up] (f16, 2 d_in values), the product formed in the projection's
        kernel; the bits of silu_mul followed by forward."""
        import torch
        if gate_up.dtype != torch.float16 or gate_up.numel() != 2 * proj.d_in or not gate_up.is_contiguous() or not gate_up.is_cuda:
            raise ValueError("forward_silu: gate_up must be a contiguous f16 CUDA tensor of 2 d_in values")
        y = out if out is not None else torch.empty(proj.d_out, dtype=torch.float16, device=gate_up.device)
        check(self.lib.llvq_gemv_silu_h(proj._h, gate_up.data_ptr(), y.data_ptr(), self._stream()))
        return y

    def forward_batch(self, proj: FusedProj, x, out=None):
        """f16 [B, d_in] -> f16 [B, d_out]; every code is decoded once per batch."""
        import torch
        if x.dim() != 2 or x.shape[1] != proj.d_in or x.dtype != torch.float16 or not x.is_contiguous():
            raise ValueError("forward_batch: x must be a contiguous f16 [B, d_in] tensor")
        y = out if out is not None else torch.empty(x.shape[0], proj.d_out, dtype=torch.float16, device=x.device)
        check(self.lib.llvq_gemm_h(proj._h, x.data_ptr(), y.data_ptr(), x.shape[0], self._stream()))
        return y

    def dequant(self, proj: FusedProj, out=None):
        """The projection as dense f16 [d_out, d_in] (a transient operand: nothing keeps it)."""
        import torch
        w = out if out is not None else torch.empty(proj.d_out, proj.d_in, dtype=torch.float16,
                                                    device=torch.device("cuda", self.device))
        if w.dtype != torch.float16 or w.numel() != proj.d_out * proj.d_in or not w.is_contiguous():
            raise ValueError("dequant: out must be a contiguous f16 tensor of d_out * d_in elements")
        check(self.lib.llvq_matrix_dequant_h(proj._h, w.data_ptr(), self._stream()))
        return w.view(proj.d_out, proj.d_in)

    def forward_batch_dense(self, proj: FusedProj, x):
        """f16 [B, d_in] -> f16 [B, d_out] for long prompts: the codes are decoded once into a transient
        dense matrix (one reused buffer per runtime) and the contraction is a library GEMM."""
        import torch
        if x.dim() != 2 or x.shape[1] != proj.d_in or x.dtype != torch.float16:
            raise ValueError("forward_batch_dense: x must be an f16 [B, d_in] tensor")
        need = proj.d_out * proj.d_in
        if getattr(self, "_dense_buf", None) is None or self._dense_buf.numel() < need:
            self._dense_buf = torch.empty(need, dtype=torch.float16, device=x.device)
        w = self.dequant(proj, out=self._dense_buf[:need])
        return x @ w.t()

    def forward_host(self, proj: FusedProj, x_host: np.ndarray, y_host: np.ndarray):
        """Host buffers in and out (copies inside the call); returns after the result has landed."""
        if x_host.dtype == np.float32:
            fn = self.lib.llvq_gemv_f32_host
        elif x_host.dtype == np.float16:
            fn = self.lib.llvq_gemv_h_host
        else:
            raise TypeError("forward_host: f32 or f16 activations")
        if x_host.size != proj.d_in or y_host.size != proj.d_out or y_host.dtype != x_host.dtype:
            raise ValueError("forward_host: shape or dtype mismatch")
        check(fn(proj._h, x_host.ctypes.data, y_host.ctypes.data, self._stream()))
        return y_host

    def forward_host_many(self, projs, xs_host, ys_host) -> None:
        """f16 host buffers for a list of projections: everything is enqueued, one synchronisation at the end."""
        from ._lib import HostCall
        n = len(projs)
        arr = (HostCall * n)()
        for i, (p, x, y) in enumerate(zip(projs, xs_host, ys_host)):
            if x.dtype != np.float16 or y.dtype != np.float16 or x.size != p.d_in or y.size != p.d_out:
                raise ValueError("forward_host_many: f16 buffers of d_in / d_out elements")
            arr[i].m, arr[i].x_host, arr[i].y_host = p._h, x.ctypes.data, y.ctypes.data
        check(self.lib.llvq_gemv_h_host_many(arr, n, self._stream()))

    @staticmethod
    def _check_x(proj: FusedProj, x, dtype) -> None:
        # the reference's own preconditions: contiguous, len == d_in (fused_cuda.rs:768-787)
        if not x.is_cuda or x.dtype != dtype or not x.is_contiguous() or x.numel() != proj.d_in:
            raise ValueError(f"{proj.name}: activation must be a contiguous CUDA {dtype} tensor of {proj.d_in} elements")

    # -- probes -----------------------------------------------------------------
    def decode_blocks(self, codes_dev):
        """uint8 CUDA tensor of 6-byte records -> (points int8 [n,24], shell u8 [n], gain u8 [n])."""
        import torch
        n = codes_dev.numel() // 6
        pts = torch.empty((n, 24), dtype=torch.int8, device=codes_dev.device)
        shell = torch.empty(n, dtype=torch.uint8, device=codes_dev.device)
        gain = torch.empty(n, dtype=torch.uint8, device=codes_dev.device)
        check(self.lib.llvq_decode_blocks(self._h, codes_dev.data_ptr(), n, pts.data_ptr(), shell.data_ptr(),
                                          gain.data_ptr(), self._stream()))
        return pts, shell, gain

    def forward_probe(self, proj: FusedProj, x, mode: int, out=None):
        """The f16 GEMV kernel with parts left out (mode 1: no decoders, 2: no class search, 3: neither)."""
        import torch
        self._check_x(proj, x, torch.float16)
        y = out if out is not None else torch.empty(proj.d_out, dtype=torch.float16, device=x.device)
        check(self.lib.llvq_gemv_probe_h(proj._h, x.data_ptr(), y.data_ptr(), mode, self._stream()))
        return y

    def forward_trace(self, proj: FusedProj, x, mode: int = 0, max_ctas: int = 256):
        """One traced launch of the f16 GEMV kernel: (y, stamps[n_ctas, 64] in ns; 0 = event absent)."""
        import torch
        self._check_x(proj, x, torch.float16)
        y = torch.empty(proj.d_out, dtype=torch.float16, device=x.device)
        stamps = np.zeros((max_ctas, 64), np.uint64)
        n = C.c_int32(0)
        check(self.lib.llvq_gemv_trace_h(proj._h, x.data_ptr(), y.data_ptr(), mode, stamps.ctypes.data, max_ctas,
                                         C.byref(n), self._stream()))
        return y, stamps[:n.value]

    def decode_blocks_fast(self, codes_dev):
        """decode_blocks through the decoders the fused kernels run (cap-12 ball)."""
        import torch
        n = codes_dev.numel() // 6
        pts = torch.empty((n, 24), dtype=torch.int8, device=codes_dev.device)
        shell = torch.empty(n, dtype=torch.uint8, device=codes_dev.device)
        gain = torch.empty(n, dtype=torch.uint8, device=codes_dev.device)
        check(self.lib.llvq_decode_blocks_fast(self._h, codes_dev.data_ptr(), n, pts.data_ptr(), shell.data_ptr(),
                                               gain.data_ptr(), self._stream()))
        return pts, shell, gain

    def decode_indices(self, idx_dev):
        """int64/uint64 CUDA tensor of indices (cap-13 ball) -> (points int8 [n,24], shell u8 [n])."""
        import torch
        n = idx_dev.numel()
        pts = torch.empty((n, 24), dtype=torch.int8, device=idx_dev.device)
        shell = torch.empty(n, dtype=torch.uint8, device=idx_dev.device)
        check(self.lib.llvq_decode_indices(self._h, idx_dev.data_ptr(), n, pts.data_ptr(), shell.data_ptr(), self._stream()))
        return pts, shell

    def close(self) -> None:
        if self._h:
            self.lib.llvq_runtime_destroy(self._h)
            self._h = C.c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
