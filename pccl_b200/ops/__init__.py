"""Fused compute + collective operators built on hand-written tcgen05 kernels."""

from . import gemm
from .tensor_parallel import AllGatherGemm, AllReduceResidualRMSNorm, GemmReduceScatter

__all__ = ["gemm", "GemmReduceScatter", "AllGatherGemm", "AllReduceResidualRMSNorm"]
