"""bf16 GEMM on the tcgen05 tensor cores (hand-written kernel, no cuBLAS).

``matmul_nt(a, b)`` computes ``a @ b.T`` for ``a[M, K]`` and ``b[N, K]`` — the
``nn.Linear`` weight layout — with fp32 accumulation in tensor memory.  It is the
core of the fused operators in this package and is exposed on its own for tests
and roofline measurements.
"""

from __future__ import annotations

from typing import Optional

import torch


def _native():
    from ..engine import load_native
    return load_native().fused


def available() -> bool:
    try:
        return torch.cuda.is_available() and hasattr(_native(), "matmul_nt")
    except ImportError:
        return False


def matmul_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, ctas: int = 0,
              sms_per_tile: int = 0) -> torch.Tensor:
    """``sms_per_tile``: 2 = pairs of SMs share 256 x 256 tiles (``tcgen05.mma.cta_group::2``), 1 = one SM per
    128 x 256 tile, 0 = the default (``PCCL_GEMM_SMS_PER_TILE``, 2)."""
    return _native().matmul_nt(a, b, out, ctas, sms_per_tile)


def check() -> None:
    """Raise if any kernel of the GEMM family recorded a device-side timeout."""
    code = _native().read_error()
    if code:
        _native().clear_error()
        role = {0: "TMA producer", 1: "MMA issuer", 2: "epilogue", 3: "reducer (peer flag)", 4: "copier (peer shard ready)",
                5: "copier (peers done reading)"}.get(code & 0xFF, str(code & 0xFF))
        raise RuntimeError(f"tcgen05 GEMM kernel gave up waiting (code {code >> 8}, role {role})")
