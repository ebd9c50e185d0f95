"""Switch-native templates: one-shot, two-shot, direct RS / AG / all-to-all, NVLS.

On an NVSwitch fabric every peer is one hop away at full per-GPU bandwidth, so
a rank can talk to all peers *in the same step* without the N-1 serial hops of
a ring.  These templates have a constant number of synchronisation points:

* **one-shot allreduce** — barrier, every rank reduces the whole vector from
  all ranks into scratch, barrier, local copy back.  N× the traffic of a
  bandwidth-optimal algorithm but a single round trip: the small-message choice.
* **two-shot allreduce** — barrier, reduce *my 1/N slice* from all ranks in
  place, barrier, pull every peer's finished slice, barrier.  Bandwidth-optimal
  (2(N-1)/N of the vector crosses each link) with three synchronisations.
* **direct reduce-scatter / allgather / all-to-all** — the two halves of
  two-shot on their own, and pairwise pulls for all-to-all, each bracketed by
  barriers so that back-to-back collectives cannot race on the shared buffer.
* **NVLS allreduce / reduce-scatter / allgather** — the same shape, with the
  switch doing the arithmetic: ``multimem.reduce`` (ld_reduce over every rank's
  copy) and ``multimem.store`` (one store delivered to every rank).

The reference has no counterpart; its ring templates are in
pccl/dsl/algorithms/ring.py.  Barriers use ``all_pairs_barrier`` with disjoint
signal-id blocks (+200, +300, +400 above the channel's base) so a fast rank's
posts for a later barrier can never satisfy an earlier one.
"""

from __future__ import annotations

from typing import Callable, List

from ..decorators import CommunicationOp, Stream
from ..graph import PrimitiveIRGraph
from ..nodes import DeviceType
from .base import CollectiveAlgorithm, all_pairs_barrier, channel_slices, finish

_BARRIER_A, _BARRIER_B, _BARRIER_C = 200, 300, 400


def _rotated(rank: int, world_size: int, include_self: bool) -> List[int]:
    """Peers starting after ``rank`` so that simultaneous requests of all ranks
    spread over all destinations instead of converging on rank 0."""
    start = 0 if include_self else 1
    return [(rank + i) % world_size for i in range(start, world_size)]


def _shard_piece(tensor_size: int, world_size: int, c: int, nc: int):
    """(elements per piece, offset of piece c inside a shard).  For collectives whose
    result or input is a *contiguous shard per rank* (reduce-scatter, allgather,
    all-to-all) channels cut every rank's shard into ``nc`` pieces, so that the
    union over channels is still the contiguous shard the engine reads or writes."""
    shard = tensor_size // world_size
    piece = shard // nc
    return shard, piece, c * piece


def _per_channel(name: str, kind: str, algorithm: str, rank: int, world_size: int,
                 tensor_size: int, dtype: str, num_channels: int,
                 body: Callable[..., None]) -> PrimitiveIRGraph:
    with CommunicationOp(name=f"{name}_c{num_channels}_rank{rank}", device=DeviceType.CUDA) as op:
        op.tensor(dtype=dtype, shape=(tensor_size,))
        for c, base, span, sig in channel_slices(tensor_size, num_channels):
            with Stream(f"ch{c}"):
                op.set_channel(c)
                body(op, base, span, sig, c, num_channels)
        return finish(op, kind, algorithm)


class OneShotAllreduce(CollectiveAlgorithm):
    name: str = "oneshot"

    @property
    def step_count(self) -> str:
        return "O(1)"

    def build_allreduce(self, rank, world_size, tensor_size, dtype="bfloat16", executor="sm",
                        num_channels=1) -> PrimitiveIRGraph:
        def body(op, base, span, sig, c=0, nc=1):
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
            # Result goes to scratch behind the tensor: peers are still reading [0, n).
            op.sm_reduce_multi(source_ranks=_rotated(rank, world_size, True),
                               remote_offset=base, dst_offset=tensor_size + base, count=span)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_B)
            op.sm_copy(source_rank=rank, src_offset=tensor_size + base, dst_offset=base, size=span)
        return _per_channel("oneshot_ar", "allreduce", "oneshot", rank, world_size, tensor_size,
                            dtype, num_channels, body)


class TwoShotAllreduce(CollectiveAlgorithm):
    name: str = "twoshot"

    @property
    def step_count(self) -> str:
        return "O(1)"

    @property
    def bandwidth_optimal(self) -> bool:
        return True

    def build_allreduce(self, rank, world_size, tensor_size, dtype="bfloat16", executor="sm",
                        num_channels=1) -> PrimitiveIRGraph:
        def body(op, base, span, sig, c=0, nc=1):
            piece = span // world_size
            mine = base + rank * piece
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
            op.sm_reduce_multi(source_ranks=_rotated(rank, world_size, True),
                               remote_offset=mine, dst_offset=mine, count=piece)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_B)
            for peer in _rotated(rank, world_size, False):
                off = base + peer * piece
                op.sm_copy(source_rank=peer, src_offset=off, dst_offset=off, size=piece)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_C)
        return _per_channel("twoshot_ar", "allreduce", "twoshot", rank, world_size, tensor_size,
                            dtype, num_channels, body)

    def build_reduce_scatter(self, rank, world_size, tensor_size, dtype="bfloat16",
                             executor="sm", num_channels=1) -> PrimitiveIRGraph:
        def body(op, base, span, sig, c=0, nc=1):
            shard, piece, within = _shard_piece(tensor_size, world_size, c, nc)
            mine = rank * shard + within
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
            op.sm_reduce_multi(source_ranks=_rotated(rank, world_size, True),
                               remote_offset=mine, dst_offset=mine, count=piece)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_B)
        return _per_channel("direct_rs", "reduce_scatter", "direct", rank, world_size,
                            tensor_size, dtype, num_channels, body)

    def build_allgather(self, rank, world_size, tensor_size, dtype="bfloat16", executor="sm",
                        num_channels=1) -> PrimitiveIRGraph:
        copy = "ce_copy" if executor == "ce" else "sm_copy"

        def body(op, base, span, sig, c=0, nc=1):
            shard, piece, within = _shard_piece(tensor_size, world_size, c, nc)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
            for peer in _rotated(rank, world_size, False):
                off = peer * shard + within
                getattr(op, copy)(source_rank=peer, src_offset=off, dst_offset=off, size=piece)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_B)
        return _per_channel("direct_ag", "allgather", "direct", rank, world_size, tensor_size,
                            dtype, num_channels, body)

    def build_alltoall(self, rank, world_size, tensor_size, dtype="bfloat16", executor="sm",
                       num_channels=1) -> PrimitiveIRGraph:
        copy = "ce_copy" if executor == "ce" else "sm_copy"

        def body(op, base, span, sig, c=0, nc=1):
            shard, piece, within = _shard_piece(tensor_size, world_size, c, nc)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
            for peer in _rotated(rank, world_size, False):
                getattr(op, copy)(source_rank=peer, src_offset=rank * shard + within,
                                  dst_offset=tensor_size + peer * shard + within, size=piece)
            # Trailing barrier: the next collective must not overwrite [0, n)
            # while a slower peer is still pulling from it.
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_B)
        return _per_channel("direct_a2a", "alltoall", "direct", rank, world_size, tensor_size,
                            dtype, num_channels, body)


class NvlsAllreduce(CollectiveAlgorithm):
    """In-switch reduction.  ``multimem.reduce`` reads a slice through the
    multicast address (the switch returns the sum over all ranks' copies) and
    stores it locally; ``multimem.store`` writes a local slice through the
    multicast address (the switch delivers it to every rank)."""

    name: str = "nvls"

    @property
    def step_count(self) -> str:
        return "O(1)"

    @property
    def bandwidth_optimal(self) -> bool:
        return True

    def build_allreduce(self, rank, world_size, tensor_size, dtype="bfloat16",
                        executor="multimem", num_channels=1) -> PrimitiveIRGraph:
        def body(op, base, span, sig, c=0, nc=1):
            piece = span // world_size
            mine = base + rank * piece
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
            op.multimem_reduce(source_rank=rank, src_offset=mine, dst_offset=mine,
                               remote_offset=mine, count=piece)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_B)
            op.multimem_store(source_rank=rank, src_offset=mine, dst_offset=mine, size=piece)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_C)
        return _per_channel("nvls_ar", "allreduce", "nvls", rank, world_size, tensor_size,
                            dtype, num_channels, body)

    def build_reduce_scatter(self, rank, world_size, tensor_size, dtype="bfloat16",
                             executor="multimem", num_channels=1) -> PrimitiveIRGraph:
        def body(op, base, span, sig, c=0, nc=1):
            shard, piece, within = _shard_piece(tensor_size, world_size, c, nc)
            mine = rank * shard + within
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
            op.multimem_reduce(source_rank=rank, src_offset=mine, dst_offset=mine,
                               remote_offset=mine, count=piece)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_B)
        return _per_channel("nvls_rs", "reduce_scatter", "nvls", rank, world_size, tensor_size,
                            dtype, num_channels, body)

    def build_allgather(self, rank, world_size, tensor_size, dtype="bfloat16",
                        executor="multimem", num_channels=1) -> PrimitiveIRGraph:
        def body(op, base, span, sig, c=0, nc=1):
            shard, piece, within = _shard_piece(tensor_size, world_size, c, nc)
            mine = rank * shard + within
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
            op.multimem_store(source_rank=rank, src_offset=mine, dst_offset=mine, size=piece)
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_B)
        return _per_channel("nvls_ag", "allgather", "nvls", rank, world_size, tensor_size,
                            dtype, num_channels, body)


#: direct RS / AG / A2A live on the two-shot class; this alias names them for what they are
DirectCollectives = TwoShotAllreduce
