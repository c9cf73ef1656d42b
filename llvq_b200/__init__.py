"""llvq_b200: fused Leech-lattice dequant-GEMV for NVIDIA B200 (sm_100a)."""
from ._lib import LlvqError, PUBLISHED_FINGERPRINT  # noqa: F401
from .runtime import FusedProj, FusedRuntime  # noqa: F401

__all__ = ["FusedRuntime", "FusedProj", "LlvqError", "PUBLISHED_FINGERPRINT"]
