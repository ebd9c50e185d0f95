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

import os

from typing import Iterable, List, Sequence

import torch

from ..ops import AllGatherGemm, FusedMoE, GemmReduceScatter
from . import collectives as _c


class ColumnParallelLinear:
    """``swiglu=True`` makes it the gated first half of a SwiGLU feed-forward: ``weight`` holds
    the gate and up projections interleaved in groups of 16 rows and the output is
    ``[T, out_features_local / 2] = silu(gate) * up`` straight from the GEMM's epilogue."""

    def __init__(self, tokens: int, in_features: int, out_features_local: int, weight: torch.Tensor = None,
                 swiglu: bool = False):
        self.op = AllGatherGemm(tokens, out_features_local, in_features, swiglu=swiglu)
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

    Parameters are packed, in order, into buckets of at most ``bucket_bytes``.  A bucket is gathered
    into the head of the symmetric working buffer, where its all-reduce runs in place with no staging
    copy (buckets take turns there: they are reduced one after the other on one side stream);
    packing and unpacking are one kernel launch per bucket (the table of gradient addresses travels
    in the kernel's parameters).  Buckets are sized for launch latency and overlap (NVSwitch gives
    every pair full bandwidth, so there is no per-link reason to split further).

    Two ways to use it:

    * ``reduce()`` after backward: every bucket is packed, reduced and unpacked on a side stream and
      the current stream waits for the result.
    * ``attach()`` once, then ``finish()`` after every backward: a hook on each parameter marks its
      gradient ready; when the last gradient of a bucket arrives (buckets are filled in reverse
      parameter order, the order backward produces them) the bucket is reduced on the side stream
      while backward goes on computing.  ``finish()`` reduces what is left and makes the current
      stream wait.  Every rank must produce its gradients for the same buckets, in any order.

    Hooked reductions use a lean instance of the push kernel (12 CTAs on a high-priority stream): a
    collective that takes most of the SMs does not overlap with a GEMM, it displaces it.  Measured
    (bench/dp_overlap_bench.py, 8 x 32 MB of gradients on 2 and 4 GPUs): 17-36 % of the reduction time
    hides under backward, the step is 0.93-0.97x of torch DDP over NCCL.  The collective's grid is
    launched as a whole (its CTAs wait on one another), so it starts in the gaps between GEMMs rather
    than inside them; launching it piecemeal is far worse (CTAs that got an SM spin for those that
    did not: 12.5 ms per step against 5.5).
    The collectives' kernels run next to whatever backward has on the GPU; they are launched so that
    all their CTAs are resident at once (see ``csrc/common/launch.h``), so a GEMM holding most of the
    SMs delays them but cannot starve them.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], bucket_bytes: int = 32 << 20,
                 dtype: torch.dtype = torch.bfloat16):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        self.dtype = dtype
        esize = torch.empty((), dtype=dtype).element_size()
        self.esize = esize
        world = int(_c._state["world"])          # the engine is already connected (pccl_b200.parallel.init)
        self.world = world
        self.buckets: List[Sequence[int]] = partition_buckets([p.numel() for p in self.params], bucket_bytes // esize)
        # every bucket's element count is rounded up so that it divides over ranks and 16-byte vectors
        self.sizes = []
        unit = world * 8
        for idxs in self.buckets:
            n = sum(self.params[i].numel() for i in idxs)
            self.sizes.append((n + unit - 1) // unit * unit)
        self.capacity = max(self.sizes)
        self.buffer = _c.working_tensor(self.capacity, dtype)
        self.offsets: List[List[int]] = []           # byte offset of every parameter inside its bucket
        for idxs in self.buckets:
            at, row = 0, []
            for i in idxs:
                row.append(at * esize)
                at += self.params[i].numel()
            self.offsets.append(row)
        self.bucket_of = {i: b for b, idxs in enumerate(self.buckets) for i in idxs}
        # High priority: when SMs free up under a running backward GEMM, the collective's CTAs are placed
        # before the GEMM's remaining ones, so a bucket's reduction starts inside the kernel that follows
        # its last gradient instead of after it.
        self.stream = torch.cuda.Stream(priority=-1)
        # Hooked reductions run beside backward's GEMMs: a lean grid for them (collective allocation).
        self._lean = _c.ensure_lean_push()
        # PCCL_DP_TRANSPORT=ce: no grid at all for the transfer: the copy engines gather every rank's
        # bucket and a plain element-wise kernel sums the copies (W - 1 buckets cross the link per rank
        # instead of 2 (W - 1) / W).  Correct, but measured slower than the lean push grid (6.6 ms against
        # 5.5 ms per step for 8 x 32 MB on two GPUs: the host-driven plan forks into per-channel streams
        # and its signal segments queue behind the GEMMs like any other kernel), so it is not the default.
        self._gather = None
        if os.environ.get("PCCL_DP_TRANSPORT", "push") == "ce" and world > 1 and torch.cuda.is_available() \
                and os.environ.get("PCCL_EXECUTOR") != "cpu":
            try:
                self._gather = _c.working_tensor(world * self.capacity, dtype)
            except Exception:                      # the working buffer is too small for W buckets
                self._gather = None
        self._native = None
        self._hooks: list = []
        self._pending = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)

    # -- one bucket ------------------------------------------------------------------------------
    def _fused(self):
        if self._native is None:
            from .. import engine as _engine
            self._native = _engine.load_native().fused
        return self._native

    def _grads(self, b: int) -> List[torch.Tensor]:
        grads = []
        for i in self.buckets[b]:
            g = self.params[i].grad
            if g is None:
                raise RuntimeError(f"parameter {i} has no gradient")
            if g.dtype != self.dtype or not g.is_contiguous():
                raise RuntimeError("GradientBuckets reduces contiguous gradients of its own dtype "
                                   f"({self.dtype}); parameter {i} has {g.dtype}")
            grads.append(g)
        return grads

    def _reduce_bucket(self, b: int, overlap: bool = False) -> None:
        """Pack, all-reduce (average) and unpack bucket ``b`` on the side stream, after everything
        the current stream has queued so far."""
        flat = self.buffer[:self.sizes[b]]
        grads = self._grads(b)
        used = sum(g.numel() for g in grads)
        self.stream.wait_stream(torch.cuda.current_stream())
        if overlap and self._gather is not None:
            n, world, rank = self.sizes[b], self.world, int(_c._state["rank"])
            region = self._gather[:world * n]
            mine = region[rank * n:(rank + 1) * n]
            with torch.cuda.stream(self.stream):
                if used < n:
                    mine[used:].zero_()
                self._fused().bucket_pack(grads, self.offsets[b], mine, False)
                _c.all_gather(region, mine, executor="ce", async_op=True)
                total = torch.sum(region.view(world, n), dim=0, dtype=torch.float32)      # rank order on every rank
                flat = total.mul_(1.0 / world).to(self.dtype)
                self._fused().bucket_pack(grads, self.offsets[b], flat, True)
            for g in grads:
                g.record_stream(self.stream)
            self._launched[b] = True
            return
        if len(grads) == 1 and used == self.sizes[b]:
            # A bucket that is one gradient needs no packing: it is reduced where it lies.
            with torch.cuda.stream(self.stream):
                _c.all_reduce(grads[0].view(-1), op="avg", async_op=True, overlap=overlap and self._lean)
            grads[0].record_stream(self.stream)
            self._launched[b] = True
            return
        with torch.cuda.stream(self.stream):
            if used < self.sizes[b]:
                flat[used:].zero_()
            self._fused().bucket_pack(grads, self.offsets[b], flat, False)
            _c.all_reduce(flat, op="avg", async_op=True, overlap=overlap and self._lean)
            self._fused().bucket_pack(grads, self.offsets[b], flat, True)
        for g in grads:
            g.record_stream(self.stream)
        self._launched[b] = True

    # -- after backward --------------------------------------------------------------------------
    def reduce(self) -> None:
        """Average every parameter's ``.grad`` in place (call after backward)."""
        for b in range(len(self.buckets)):
            self._reduce_bucket(b)
        self._join()

    def _join(self) -> None:
        torch.cuda.current_stream().wait_stream(self.stream)
        self._launched = [False] * len(self.buckets)
        self._pending = [len(idxs) for idxs in self.buckets]

    # -- during backward -------------------------------------------------------------------------
    def attach(self) -> "GradientBuckets":
        """Install the hooks that start a bucket's reduction as soon as its last gradient exists."""
        if self._hooks:
            return self
        self._pending = [len(idxs) for idxs in self.buckets]

        def make(i: int):
            def ready(_param):
                b = self.bucket_of[i]
                self._pending[b] -= 1
                if self._pending[b] == 0 and not self._launched[b]:
                    self._reduce_bucket(b, overlap=True)
            return ready

        for i, p in enumerate(self.params):
            self._hooks.append(p.register_post_accumulate_grad_hook(make(i)))
        return self

    def detach(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def finish(self) -> None:
        """Reduce the buckets backward did not complete (unused parameters keep their old gradient
        out of it only if every rank skips them alike) and make the current stream wait."""
        for b in range(len(self.buckets)):
            if not self._launched[b] and all(self.params[i].grad is not None for i in self.buckets[b]):
                self._reduce_bucket(b)
        self._join()
