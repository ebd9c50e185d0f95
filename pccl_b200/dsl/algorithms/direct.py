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
from .base import SIGNAL_STRIDE, CollectiveAlgorithm, all_pairs_barrier, channel_slices, finish

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
    """In-switch reduction.

    All-reduce is one pass per rank over its 1/N slice: ``multimem.allreduce`` fetches each vector
    with ``multimem.ld_reduce`` (the switch returns the sum over all ranks' copies) and writes it
    straight back with ``multimem.st`` (the switch delivers it to every rank).  Per GPU and
    direction (1 + 1/N) of the message crosses NVLink, and the outbound reduce traffic overlaps
    the inbound broadcast traffic.  ``one_pass=False`` keeps the two halves apart
    (``multimem.reduce`` into local memory, barrier, ``multimem.store``), which serialises an
    outbound-bound phase and an inbound-bound phase and measured about twice as slow; it remains
    as ``nvls_twopass`` for comparison.  Reduce-scatter and all-gather are those halves on their own.
    """

    name: str = "nvls"
    one_pass: bool = True

    @property
    def step_count(self) -> str:
        return "O(1)"

    @property
    def bandwidth_optimal(self) -> bool:
        return True

    def build_allreduce(self, rank, world_size, tensor_size, dtype="bfloat16",
                        executor="multimem", num_channels=1) -> PrimitiveIRGraph:
        one_pass = self.one_pass

        def body(op, base, span, sig, c=0, nc=1):
            piece = span // world_size
            mine = base + rank * piece
            all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
            if one_pass:
                op.multimem_allreduce(offset=mine, count=piece)
            else:
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


class NvlsTwoPassAllreduce(NvlsAllreduce):
    """The in-switch all-reduce as two separate passes (reduce, barrier, broadcast)."""

    name: str = "nvls_twopass"
    one_pass: bool = False


def hybrid_split(tensor_size: int, world_size: int, fraction: float, nvls_channels: int,
                 peer_channels: int, align: int = 16):
    """Element ranges of the hybrid all-reduce: ``[(channel, base, span, kind), ...]``.

    The first ``fraction`` of the tensor (rounded so that every channel's span splits into
    ``world_size`` pieces of a multiple of ``align`` elements) goes to the in-switch channels,
    the rest to the peer (two-shot) channels; what rounding leaves over joins the last peer
    channel's range as a tail that is reduced by the two-shot steps of that channel."""
    unit = world_size * align
    out = []
    nvls_elems = int(tensor_size * max(0.0, min(1.0, fraction)))
    per_nvls = (nvls_elems // max(1, nvls_channels)) // unit * unit if nvls_channels else 0
    base = 0
    for c in range(nvls_channels):
        if per_nvls:
            out.append((len(out), base, per_nvls, "nvls"))
            base += per_nvls
    rest = tensor_size - base
    per_peer = (rest // max(1, peer_channels)) // unit * unit if peer_channels else 0
    for c in range(peer_channels):
        if per_peer:
            out.append((len(out), base, per_peer, "peer"))
            base += per_peer
    return out, base


class HybridAllreduce(CollectiveAlgorithm):
    """In-switch and peer-memory all-reduce side by side in one launch.

    Channels ``[0, k)`` run the one-pass ``multimem.allreduce`` on the first ``nvls_fraction`` of
    the message; channels ``[k, C)`` run the two-shot schedule (``sm.reduce_multi`` of this rank's
    piece from every peer, then pulls of the finished pieces) on the rest.  The two paths load
    different parts of the fabric (the switch's reduction engines and multicast replication
    against plain unicast reads), so where the in-switch path alone does not fill the links the
    peer path uses what is left.  ``nvls_fraction`` (``PCCL_NVLS_FRACTION``) is the *byte* split;
    the CTA split follows it because the engine hands CTAs to chains in proportion to their bytes.
    Elements that the rounding of the split leaves over (fewer than ``C * world * 16``) are
    reduced by a small two-shot tail on the last channel.
    """

    name: str = "hybrid"

    def __init__(self, nvls_fraction: float = None):
        import os
        if nvls_fraction is None:
            nvls_fraction = float(os.environ.get("PCCL_NVLS_FRACTION", "0.7"))
        self.nvls_fraction = nvls_fraction

    @property
    def step_count(self) -> str:
        return "O(1)"

    @property
    def bandwidth_optimal(self) -> bool:
        return True

    def build_allreduce(self, rank, world_size, tensor_size, dtype="bfloat16", executor="multimem",
                        num_channels=2) -> PrimitiveIRGraph:
        num_channels = max(2, num_channels)
        k = min(num_channels - 1, max(1, round(num_channels * self.nvls_fraction)))
        ranges, covered = hybrid_split(tensor_size, world_size, self.nvls_fraction, k, num_channels - k)
        with CommunicationOp(name=f"hybrid_ar_c{num_channels}_rank{rank}", device=DeviceType.CUDA) as op:
            op.tensor(dtype=dtype, shape=(tensor_size,))

            def two_shot(base, span, sig):
                piece = span // world_size
                mine = base + rank * piece
                op.sm_reduce_multi(source_ranks=_rotated(rank, world_size, True),
                                   remote_offset=mine, dst_offset=mine, count=piece)
                all_pairs_barrier(op, rank, world_size, sig + _BARRIER_B)
                for peer in _rotated(rank, world_size, False):
                    off = base + peer * piece
                    op.sm_copy(source_rank=peer, src_offset=off, dst_offset=off, size=piece)

            for c, base, span, kind in ranges:
                sig = c * SIGNAL_STRIDE
                with Stream(f"ch{c}"):
                    op.set_channel(c)
                    all_pairs_barrier(op, rank, world_size, sig + _BARRIER_A)
                    if kind == "nvls":
                        piece = span // world_size
                        op.multimem_allreduce(offset=base + rank * piece, count=piece)
                    else:
                        two_shot(base, span, sig)
                    if c == len(ranges) - 1 and covered < tensor_size:
                        # Tail left by rounding: rank 0 reduces it, everyone pulls it.
                        tail = tensor_size - covered
                        if rank == 0:
                            op.sm_reduce_multi(source_ranks=list(range(world_size)), remote_offset=covered,
                                               dst_offset=covered, count=tail)
                        all_pairs_barrier(op, rank, world_size, sig + 500)
                        if rank != 0:
                            op.sm_copy(source_rank=0, src_offset=covered, dst_offset=covered, size=tail)
                    all_pairs_barrier(op, rank, world_size, sig + _BARRIER_C)
            return finish(op, "allreduce", "hybrid")


#: direct RS / AG / A2A live on the two-shot class; this alias names them for what they are
DirectCollectives = TwoShotAllreduce
