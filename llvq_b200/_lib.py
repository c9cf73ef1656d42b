"""ctypes binding of libllvq_b200.so — the same declarations as include/llvq_b200.h."""
from __future__ import annotations

import ctypes as C
import os

from . import _build

OK = 0
ERR_INVALID, ERR_CUDA, ERR_CODEBOOK, ERR_RANGE, ERR_UNSUPPORTED = -1, -2, -3, -4, -5
TAIL_F32, TAIL_F16 = 0, 1
PUBLISHED_FINGERPRINT = 0x338F420F11866319


class MatrixDesc(C.Structure):
    """llvq_matrix_desc of include/llvq_b200.h."""
    _fields_ = [
        ("d_out", C.c_int32), ("d_in", C.c_int32), ("shell_cap", C.c_int32), ("tail_mode", C.c_int32),
        ("codes", C.c_void_p), ("centroids", C.c_void_p), ("row_scales", C.c_void_p), ("tail", C.c_void_p),
    ]


class HostCall(C.Structure):
    """llvq_host_call of include/llvq_b200.h."""
    _fields_ = [("m", C.c_void_p), ("x_host", C.c_void_p), ("y_host", C.c_void_p)]


class ArchiveMatrixInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("d_out", C.c_int32), ("d_in", C.c_int32), ("shell_cap", C.c_int32),
                ("n_centroids", C.c_int32), ("index_bits", C.c_int32), ("gain_bits", C.c_int32), ("has_rotation", C.c_int32),
                ("rotation_seed", C.c_uint64), ("centroids", C.POINTER(C.c_double)), ("row_scales", C.POINTER(C.c_double)),
                ("tail", C.POINTER(C.c_float)), ("stream", C.POINTER(C.c_uint8)), ("stream_bytes", C.c_uint64)]


class ArchiveRawInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("tag", C.c_int32), ("rank", C.c_int32), ("bits", C.c_int32), ("group", C.c_int32),
                ("dims", C.POINTER(C.c_uint64)), ("data", C.POINTER(C.c_uint8)), ("data_bytes", C.c_uint64),
                ("scales", C.POINTER(C.c_uint8)), ("biases", C.POINTER(C.c_uint8)), ("groups", C.c_uint64)]


class LlvqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"llvq status {status}: {message}")
        self.status = status
        self.message = message


_SIGNATURES = {
    "llvq_last_error": (C.c_char_p, []),
    "llvq_version": (C.c_char_p, []),
    "llvq_launch_count": (C.c_uint64, []),
    "llvq_runtime_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "llvq_runtime_destroy": (None, [C.c_void_p]),
    "llvq_runtime_poll_error": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32)]),
    "llvq_codebook_fingerprint": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "llvq_codebook_info": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int32), C.POINTER(C.c_uint64)]),
    "llvq_codebook_class_record": (C.c_int, [C.c_int32, C.c_void_p]),
    "llvq_codebook_golay": (C.c_int, [C.c_void_p]),
    "llvq_matrix_upload": (C.c_int, [C.c_void_p, C.POINTER(MatrixDesc), C.POINTER(C.c_void_p)]),
    "llvq_matrix_upload_group": (C.c_int, [C.c_void_p, C.POINTER(MatrixDesc), C.c_int32, C.POINTER(C.c_void_p)]),
    "llvq_matrix_free": (None, [C.c_void_p]),
    "llvq_matrix_dims": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "llvq_matrix_algorithmic_bytes": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_uint64)]),
    "llvq_gemv_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_gemv_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_gemv_f32x_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_gemv_norm_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_gemv_silu_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_gemm_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "llvq_gemv_f32_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_gemv_h_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_op_add_rmsnorm_h": (C.c_int, [C.c_void_p] * 4 + [C.c_int32, C.c_float, C.c_void_p]),
    "llvq_op_qkv_rope_cache_h": (C.c_int, [C.c_void_p] * 13 + [C.c_int32] * 3 + [C.c_float, C.c_void_p]),
    "llvq_archive_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "llvq_archive_open_memory": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "llvq_archive_close": (None, [C.c_void_p]),
    "llvq_archive_counts": (C.c_int, [C.c_void_p] + [C.POINTER(C.c_int32)] * 5 + [C.POINTER(C.c_uint64)]),
    "llvq_archive_matrix": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(ArchiveMatrixInfo)]),
    "llvq_archive_matrix_desc": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(MatrixDesc)]),
    "llvq_archive_raw": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(ArchiveRawInfo)]),
    "llvq_archive_blob": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_char_p), C.POINTER(C.POINTER(C.c_uint8)),
                                   C.POINTER(C.c_uint64)]),
    "llvq_rotation_create": (C.c_int, [C.c_void_p, C.c_int32, C.c_uint64, C.POINTER(C.c_void_p)]),
    "llvq_rotation_create_from_tables": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "llvq_rotation_build_tables": (C.c_int, [C.c_int32, C.c_uint64, C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]),
    "llvq_rotation_free": (None, [C.c_void_p]),
    "llvq_rotation_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                    C.POINTER(C.c_float)]),
    "llvq_rotation_tables": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_rotate_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "llvq_op_add_rmsnorm_rotate_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_float,
                                              C.c_void_p]),
    "llvq_op_silu_mul_rotate_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "llvq_tp_region_create": (C.c_int, [C.c_int32, C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]),
    "llvq_tp_region_open": (C.c_int, [C.c_int32, C.c_void_p, C.POINTER(C.c_void_p)]),
    "llvq_tp_region_close": (C.c_int, [C.c_int32, C.c_void_p]),
    "llvq_tp_region_free": (C.c_int, [C.c_int32, C.c_void_p]),
    "llvq_tp_ctx_create": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_void_p), C.c_uint32, C.POINTER(C.c_void_p)]),
    "llvq_tp_ctx_destroy": (None, [C.c_void_p]),
    "llvq_tp_exchange": (C.c_int, [C.c_void_p, C.c_int32, C.c_size_t, C.c_void_p, C.c_uint32, C.c_void_p]),
    "llvq_tp_exchange_emulated": (C.c_int, [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_size_t, C.POINTER(C.c_void_p),
                                            C.c_uint32, C.c_void_p]),
    "llvq_tp_poll_error": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32)]),
    "llvq_op_lm_head_argmax_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p]),
    "llvq_op_lm_head_argmax_q8_h": (C.c_int, [C.c_void_p] * 4 + [C.c_int32, C.c_int32, C.c_int64] + [C.c_void_p] * 4),
    "llvq_op_embed_gather_q8_h": (C.c_int, [C.c_void_p] * 4 + [C.c_int32] * 3 + [C.c_void_p, C.c_void_p]),
    "llvq_matrix_dequant_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_op_attn_decode_int8_h": (C.c_int, [C.c_void_p] * 9 + [C.c_int32] * 4 + [C.c_void_p, C.c_void_p]),
    "llvq_op_silu_mul_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "llvq_gemv_h_host_many": (C.c_int, [C.POINTER(HostCall), C.c_int32, C.c_void_p]),
    "llvq_gemv_f32_host_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_decode_blocks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_runtime_set_overlap": (C.c_int, [C.c_void_p, C.c_int32]),
    "llvq_runtime_kernel_info": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_gemv_probe_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "llvq_gemv_trace_h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "llvq_decode_blocks_fast": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "llvq_decode_indices": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def load(build: bool = True) -> C.CDLL:
    """Load the library (building it first when asked and stale). Fails loudly when it is missing."""
    global _lib
    if _lib is None:
        path = _build.build() if build else _build.LIB
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: the CUDA library was not built; there is no fallback")
        L = C.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            f = getattr(L, name)
            f.restype = res
            f.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise LlvqError(status, load().llvq_last_error().decode())
