"""Fused compute + collective operators built on hand-written tcgen05 kernels."""

from . import gemm

__all__ = ["gemm"]
