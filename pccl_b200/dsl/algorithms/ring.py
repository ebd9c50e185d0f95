"""Ring templates: allreduce, reduce-scatter, allgather, all-to-all.

All data movement is *pull*: in every step a rank reads one chunk from its left
neighbour's buffer.  Two counting semaphores per channel order the steps:
``S+100`` is a one-off "my input is in place" handshake, ``S`` is posted to the
right neighbour after every step ("the chunk you will read next is final").
The emitted primitive sequences are identical to the reference's, so plans are
interchangeable between the two libraries (reference:
pccl/dsl/algorithms/ring.py:27-89 allreduce, :91-141 reduce-scatter,
:143-193 allgather, :195-246 all-to-all).
"""

from __future__ import annotations

from ..decorators import CommunicationOp, Stream
from ..graph import PrimitiveIRGraph
from ..nodes import DeviceType
from .base import CollectiveAlgorithm, channel_slices, finish


class _RingChannel:
    """Emits the steps of one channel of a ring collective."""

    def __init__(self, op: CommunicationOp, rank: int, world: int, executor: str,
                 base: int, chunk: int, sig: int):
        self.op, self.rank, self.world = op, rank, world
        self.left, self.right = (rank - 1) % world, (rank + 1) % world
        self.base, self.chunk, self.sig = base, chunk, sig
        self.tma = executor == "tma"

    def handshake(self) -> None:
        self.op.notify(signal_id=self.sig + 100, target_rank=self.right)
        self.op.wait_notify(signal_id=self.sig + 100, source_rank=self.left)

    def step(self, chunk_index: int, reduce: bool, wait_first: bool) -> None:
        op, off = self.op, self.base + (chunk_index % self.world) * self.chunk
        if wait_first:
            op.wait_notify(signal_id=self.sig, source_rank=self.left)
        if reduce:
            emit = op.tma_reduce if self.tma else op.sm_reduce
            emit(reduce_op="sum", source_rank=self.left, src_offset=off, dst_offset=off,
                 remote_offset=off, count=self.chunk)
        else:
            emit = op.tma_copy if self.tma else op.sm_copy
            emit(source_rank=self.left, src_offset=off, dst_offset=off, size=self.chunk)
        op.notify(signal_id=self.sig, target_rank=self.right)

    def drain(self) -> None:
        self.op.wait_notify(signal_id=self.sig, source_rank=self.left)


class RingAllreduce(CollectiveAlgorithm):
    name: str = "ring"

    @property
    def step_count(self) -> str:
        return "O(2(N-1))"

    @property
    def bandwidth_optimal(self) -> bool:
        return True

    def _build(self, kind: str, tag: str, rank: int, world: int, n: int, dtype: str,
               executor: str, channels: int, body) -> PrimitiveIRGraph:
        with CommunicationOp(name=f"ring_{tag}_{executor}_c{channels}_rank{rank}",
                             device=DeviceType.CUDA) as op:
            op.tensor(dtype=dtype, shape=(n,))
            for c, base, span, sig in channel_slices(n, channels):
                with Stream(f"ch{c}"):
                    op.set_channel(c)
                    body(_RingChannel(op, rank, world, executor, base, span // world, sig))
            return finish(op, kind, "ring")

    def build_allreduce(self, rank, world_size, tensor_size, dtype="bfloat16", executor="tma",
                        num_channels=1) -> PrimitiveIRGraph:
        def body(ch: _RingChannel) -> None:
            ch.handshake()
            for s in range(world_size - 1):          # reduce-scatter half
                ch.step(rank - s - 1, reduce=True, wait_first=s > 0)
            for s in range(world_size - 1):          # allgather half
                ch.step(rank - s, reduce=False, wait_first=True)
            ch.drain()
        return self._build("allreduce", "ar", rank, world_size, tensor_size, dtype, executor,
                           num_channels, body)

    def build_reduce_scatter(self, rank, world_size, tensor_size, dtype="bfloat16",
                             executor="tma", num_channels=1) -> PrimitiveIRGraph:
        def body(ch: _RingChannel) -> None:
            ch.handshake()
            # One chunk further back than in allreduce, so that the chunk that
            # ends up fully reduced on this rank is chunk ``rank``.
            for s in range(world_size - 1):
                ch.step(rank - s - 2, reduce=True, wait_first=s > 0)
            ch.drain()
        return self._build("reduce_scatter", "rs", rank, world_size, tensor_size, dtype,
                           executor, num_channels, body)

    def build_allgather(self, rank, world_size, tensor_size, dtype="bfloat16", executor="tma",
                        num_channels=1) -> PrimitiveIRGraph:
        def body(ch: _RingChannel) -> None:
            ch.handshake()
            for s in range(world_size - 1):          # step 0 fetches the left neighbour's own shard
                ch.step(rank - s - 1, reduce=False, wait_first=s > 0)
            ch.drain()
        return self._build("allgather", "ag", rank, world_size, tensor_size, dtype, executor,
                           num_channels, body)

    def build_alltoall(self, rank, world_size, tensor_size, dtype="bfloat16", executor="tma",
                       num_channels=1) -> PrimitiveIRGraph:
        """Pairwise exchange.  Chunk ``rank`` of every peer is pulled into a
        scratch area behind the tensor (``n + peer*chunk``), so reads (of
        ``[0, n)``) and writes never overlap.  Always SM copies: the scratch
        area lies outside the tensor the TMA path is described over."""
        def body(ch: _RingChannel) -> None:
            op = ch.op
            for i in range(world_size - 1):          # N-1 ring rounds == full barrier
                op.notify(signal_id=ch.sig + 100 + i, target_rank=ch.right)
                op.wait_notify(signal_id=ch.sig + 100 + i, source_rank=ch.left)
            for s in range(world_size - 1):
                peer = (rank + s + 1) % world_size
                op.sm_copy(source_rank=peer, src_offset=ch.base + rank * ch.chunk,
                           dst_offset=ch.base + tensor_size + peer * ch.chunk, size=ch.chunk)

        with CommunicationOp(name=f"ring_a2a_sm_c{num_channels}_rank{rank}",
                             device=DeviceType.CUDA) as op:
            op.tensor(dtype=dtype, shape=(tensor_size,))
            for c, base, span, sig in channel_slices(tensor_size, num_channels):
                with Stream(f"ch{c}"):
                    op.set_channel(c)
                    body(_RingChannel(op, rank, world_size, "sm", base, span // world_size, sig))
            return finish(op, "alltoall", "ring")
