"""Fused compute + collective operators built on hand-written tcgen05 kernels."""

from . import gemm, moe
from .moe import FusedMoE
from .tensor_parallel import AllGatherGemm, AllReduceResidualRMSNorm, GemmReduceScatter

__all__ = ["gemm", "moe", "FusedMoE", "GemmReduceScatter", "AllGatherGemm", "AllReduceResidualRMSNorm"]
