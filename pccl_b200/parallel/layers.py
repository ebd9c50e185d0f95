"""Tensor-, sequence-, expert- and data-parallel building blocks on top of the fused operators.

Inference-side modules (no autograd through the fused kernels):

``ColumnParallelLinear``   sequence-parallel input ``[T/W, K]`` -> all-gather fused into the GEMM ->
                           ``[T, N/W]`` (weight ``[N/W, K]``).
``RowParallelLinear``      ``[T, K/W]`` -> GEMM with the reduce-scatter fused into its epilogue ->
                           ``[T/W, N]`` (weight ``[N, K/W]``).
``ExpertParallelMoE``      top-2 routed SwiGLU experts spread over the ranks (`pccl_b200.ops.moe`).
``GradientBuckets``        data-parallel gradient averaging: gradients are packed into buckets that
                           live in the symmetric working buffer and reduced in place, one plan per
                           bucket size, all on the caller's stream.

The reference ships collectives only and no strategy code; these are the strategies its
collectives exist for.
"""

from __future__ import annotations

from typing import Iterable, List, Sequence

import torch

from ..ops import AllGatherGemm, FusedMoE, GemmReduceScatter
from . import collectives as _c


class ColumnParallelLinear:
    def __init__(self, tokens: int, in_features: int, out_features_local: int, weight: torch.Tensor = None):
        self.op = AllGatherGemm(tokens, out_features_local, in_features)
        self.weight = weight if weight is not None else torch.empty(
            out_features_local, in_features, dtype=torch.bfloat16, device="cuda")

    @property
    def input_shard(self) -> torch.Tensor:
        """Write this rank's rows here to skip the staging copy."""
        return self.op.local_shard

    def __call__(self, x_shard: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        return self.op(x_shard, self.weight, out)


class RowParallelLinear:
    def __init__(self, tokens: int, in_features_local: int, out_features: int, weight: torch.Tensor = None):
        self.op = GemmReduceScatter(tokens, out_features, in_features_local)
        self.weight = weight if weight is not None else torch.empty(
            out_features, in_features_local, dtype=torch.bfloat16, device="cuda")

    def __call__(self, x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        return self.op(x, self.weight, out)


class ExpertParallelMoE:
    def __init__(self, tokens: int, hidden: int, ffn: int, experts: int, local: bool = False):
        self.op = FusedMoE(tokens, hidden, ffn, experts, local=local)

    def load(self, wg, w1, w3, w2) -> None:
        self.op.set_weights(wg, w1, w3, w2)

    def __call__(self, x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        return self.op(x, out)


def partition_buckets(sizes: Sequence[int], bucket_elems: int) -> List[List[int]]:
    """Greedy in-order packing: indices of consecutive tensors whose element counts sum to at most
    ``bucket_elems`` (a tensor larger than that gets a bucket of its own)."""
    buckets: List[List[int]] = []
    current: List[int] = []
    used = 0
    for i, n in enumerate(sizes):
        if current and used + n > bucket_elems:
            buckets.append(current)
            current, used = [], 0
        current.append(i)
        used += n
    if current:
        buckets.append(current)
    return buckets


class GradientBuckets:
    """Average gradients over the data-parallel ranks through the plan engine.

    Parameters are packed, in order, into buckets of at most ``bucket_bytes``; each bucket is a slice
    of the symmetric working buffer, so the all-reduce runs in place with no staging copy.  Buckets
    are sized for launch latency and overlap (NVSwitch gives every pair full bandwidth, so there is
    no per-link reason to split further).
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], bucket_bytes: int = 64 << 20,
                 dtype: torch.dtype = torch.bfloat16):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        self.dtype = dtype
        esize = torch.empty((), dtype=dtype).element_size()
        world = int(_c._state["world"])          # the engine is already connected (pccl_b200.parallel.init)
        self.buckets: List[Sequence[int]] = partition_buckets([p.numel() for p in self.params], bucket_bytes // esize)
        # every bucket's element count is rounded up so that it divides over ranks and 16-byte vectors
        self.sizes = []
        for idxs in self.buckets:
            n = sum(self.params[i].numel() for i in idxs)
            unit = world * 8
            self.sizes.append((n + unit - 1) // unit * unit)
        self.capacity = max(self.sizes)
        self.buffer = _c.working_tensor(self.capacity, dtype)

    def reduce(self) -> None:
        """Average every parameter's ``.grad`` in place (call after backward)."""
        for idxs, size in zip(self.buckets, self.sizes):
            flat = self.buffer[:size]
            offset = 0
            for i in idxs:
                g = self.params[i].grad
                n = g.numel()
                flat[offset:offset + n].copy_(g.reshape(-1))
                offset += n
            if offset < size:
                flat[offset:].zero_()
            _c.all_reduce(flat, op="avg")
            offset = 0
            for i in idxs:
                g = self.params[i].grad
                n = g.numel()
                g.copy_(flat[offset:offset + n].view_as(g))
                offset += n
