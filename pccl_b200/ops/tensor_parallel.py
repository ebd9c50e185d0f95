"""Tensor-parallel linear layers whose collective is fused into the GEMM kernel.

``GemmReduceScatter``  row-parallel linear + sequence-parallel output:
    ``y[M/W, N] = reduce_scatter_rows(x[M, K/W] @ w[N, K/W].T)``.
``AllGatherGemm``      sequence-parallel input + column-parallel linear:
    ``y[M, N/W] = all_gather_rows(x[M/W, K]) @ w[N/W, K].T``.

Both own their symmetric buffers (allocated once from the engine's arena, identical
offsets on every rank because every rank constructs the same operators in the same
order) and count calls: flags are never reset, a call number travels to the kernel.
Construction is collective (it ends with a barrier so that no peer can signal a rank
whose flags are not zeroed yet).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import engine as _engine

_BLOCK = 128


def _native():
    return _engine.load_native().fused


def _fence(group) -> None:
    torch.cuda.synchronize()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.barrier(group=group)


class GemmReduceScatter:
    def __init__(self, m: int, n: int, k_local: int, group=None):
        self.engine = _engine.get_engine()
        self.world, self.rank = self.engine.world, self.engine.rank
        if m % (self.world * _BLOCK):
            raise ValueError(f"M={m} must be a multiple of world*{_BLOCK}")
        self.m, self.n, self.k = m, n, k_local
        rows = m // self.world
        self.recv = self.engine.empty_symmetric((2, self.world, rows, n), torch.bfloat16)
        self.flags = self.engine.empty_symmetric((self.world * (rows // _BLOCK),), torch.int32)
        self.flags.zero_()
        self.block_counter = torch.zeros(m // _BLOCK, dtype=torch.int32, device="cuda")
        self.epoch = 0
        self.group = group
        _fence(group)

    def __call__(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor = None, ctas: int = 0) -> torch.Tensor:
        if out is None:
            out = torch.empty(self.m // self.world, self.n, dtype=torch.bfloat16, device=x.device)
        self.epoch += 1
        _native().gemm_reduce_scatter(x, w, out, self.recv.heap_offset, self.flags.heap_offset,
                                      self.block_counter, self.epoch, ctas)
        return out


class AllGatherGemm:
    """``swiglu=True``: ``w`` stacks the gate and up projections interleaved in groups of 16 rows
    (``pccl_b200.ops.moe.interleave_gate_up``) and the result is ``[M, n_local / 2] = silu(gate) * up``,
    computed in the GEMM's epilogue."""

    def __init__(self, m: int, n_local: int, k: int, group=None, copy_ctas: int = 0, swiglu: bool = False):
        self.engine = _engine.get_engine()
        self.world, self.rank = self.engine.world, self.engine.rank
        if m % (self.world * _BLOCK):
            raise ValueError(f"M={m} must be a multiple of world*{_BLOCK}")
        self.m, self.n, self.k = m, n_local, k
        self.rows = m // self.world
        self.gathered = self.engine.empty_symmetric((m, k), torch.bfloat16)
        self.flags = self.engine.empty_symmetric((2 * self.world,), torch.int32)
        self.flags.zero_()
        self.ready = torch.zeros(m // _BLOCK, dtype=torch.int32, device="cuda")
        self.copy_ctas = copy_ctas
        self.swiglu = bool(swiglu)
        if self.swiglu and n_local % 32:
            raise ValueError("with swiglu the stacked gate/up weight has a multiple of 32 rows")
        self.epoch = 0
        self.group = group
        _fence(group)

    @property
    def local_shard(self) -> torch.Tensor:
        """View of this rank's rows inside the gathered matrix: write activations here to skip the copy."""
        return self.gathered[self.rank * self.rows:(self.rank + 1) * self.rows]

    def __call__(self, x_shard: torch.Tensor, w: torch.Tensor, out: torch.Tensor = None, ctas: int = 0) -> torch.Tensor:
        if x_shard.data_ptr() != self.local_shard.data_ptr():
            self.local_shard.copy_(x_shard)
        if out is None:
            out = torch.empty(self.m, self.n // 2 if self.swiglu else self.n, dtype=torch.bfloat16, device=w.device)
        self.epoch += 1
        _native().all_gather_gemm(self.gathered.heap_offset, self.m, self.k, w, out, self.flags.heap_offset,
                                  self.ready, self.epoch, self.copy_ctas, ctas, self.swiglu)
        return out


class AllReduceResidualRMSNorm:
    """``h = residual + all_reduce(x); y = rmsnorm(h) * gamma`` in one kernel.

    ``self.x`` (this rank's partial, written by the caller), ``self.residual`` (read and
    updated in place) and ``self.y`` (result) are ``[tokens, hidden]`` bf16 tensors in
    symmetric memory owned by the operator.  ``use_nvls``: True = in-switch reduction when the
    engine has multicast and there are more than two ranks, "force" = whenever it has multicast,
    False = peer loads / stores only.
    """

    def __init__(self, tokens: int, hidden: int, eps: float = 1e-5, group=None, use_nvls: bool = True):
        self.engine = _engine.get_engine()
        self.world, self.rank = self.engine.world, self.engine.rank
        # With two ranks the in-switch reduction moves 1.5x the bytes of the peer path: keep it for W > 2.
        self.tokens, self.hidden, self.eps = tokens, hidden, eps
        self.use_nvls = bool(use_nvls) and (self.world > 2 or use_nvls == "force")
        self.x = self.engine.empty_symmetric((tokens, hidden), torch.bfloat16)
        self.y = self.engine.empty_symmetric((tokens, hidden), torch.bfloat16)
        self.residual = self.engine.empty_symmetric((tokens, hidden), torch.bfloat16)
        self.flags = self.engine.empty_symmetric((2 * self.world,), torch.int32)
        self.flags.zero_()
        self.cta_counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.epoch = 0
        _fence(group)

    def __call__(self, gamma: torch.Tensor, x: torch.Tensor = None, residual: torch.Tensor = None, ctas: int = 0):
        if x is not None and x.data_ptr() != self.x.data_ptr():
            self.x.copy_(x)
        if residual is not None and residual.data_ptr() != self.residual.data_ptr():
            self.residual.copy_(residual)
        self.epoch += 1
        _native().ar_residual_rmsnorm(self.x.heap_offset, self.y.heap_offset, self.residual.heap_offset,
                                      self.flags.heap_offset, gamma, self.cta_counter, self.tokens, self.hidden,
                                      self.eps, self.epoch, self.use_nvls, ctas)
        return self.y, self.residual
