"""Recursive halving / doubling (Rabenseifner) templates, power-of-two ranks.

Allreduce: log2(N) halving steps (each rank reduces the half of its active
region selected by one bit of its rank, reading it from the partner across
that bit), then log2(N) doubling steps in reverse that copy the partner's
finished half back.  Signals carry the *sender's* rank as id
(reference: pccl/dsl/algorithms/recursive_hd.py:21-145; the allreduce emitted
here is primitive-for-primitive the same plan).

Reduce-scatter and allgather (additions): the same recursion, but pairing
across the *highest* bit first so that the slice a rank ends up owning is
slice ``rank`` — the layout the engine's I/O convention expects.
"""

from __future__ import annotations

from ..decorators import CommunicationOp, Stream
from ..graph import PrimitiveIRGraph
from ..nodes import DeviceType
from .base import CollectiveAlgorithm, finish, is_power_of_two


def _log2(n: int) -> int:
    return n.bit_length() - 1


class RecursiveHalvingDoubling(CollectiveAlgorithm):
    name: str = "rhd"

    @property
    def step_count(self) -> str:
        return "O(2 log N)"

    @property
    def bandwidth_optimal(self) -> bool:
        return True

    @staticmethod
    def _check(world_size: int) -> int:
        if not is_power_of_two(world_size):
            raise ValueError(
                f"RecursiveHalvingDoubling requires power-of-2 world_size, got {world_size}")
        return _log2(world_size)

    @staticmethod
    def _exchange(op: CommunicationOp, rank: int, partner: int) -> None:
        op.notify(signal_id=rank, target_rank=partner)
        op.wait_notify(signal_id=partner, source_rank=partner)

    def build_allreduce(self, rank, world_size, tensor_size, dtype="bfloat16", executor="tma",
                        num_channels=1) -> PrimitiveIRGraph:
        levels = self._check(world_size)
        tma = executor == "tma"

        def region_start(k: int) -> int:
            """Start of the region this rank is still responsible for before step k."""
            return sum(tensor_size >> (j + 1) for j in range(k) if rank >> j & 1)

        with CommunicationOp(name=f"rhd_ar_{executor}_rank{rank}", device=DeviceType.CUDA) as op:
            op.tensor(dtype=dtype, shape=(tensor_size,))
            with Stream("main"):
                op.set_channel(0)
                for k in range(levels):                       # halving: reduce my half
                    partner, half = rank ^ (1 << k), tensor_size >> (k + 1)
                    mine = region_start(k) + (half if rank >> k & 1 else 0)
                    self._exchange(op, rank, partner)
                    (op.tma_reduce if tma else op.sm_reduce)(
                        reduce_op="sum", source_rank=partner, src_offset=mine, dst_offset=mine,
                        remote_offset=mine, count=half)
                for k in reversed(range(levels)):             # doubling: fetch the other half
                    partner, half = rank ^ (1 << k), tensor_size >> (k + 1)
                    theirs = region_start(k) + (0 if rank >> k & 1 else half)
                    self._exchange(op, rank, partner)
                    (op.tma_copy if tma else op.sm_copy)(
                        source_rank=partner, src_offset=theirs, dst_offset=theirs, size=half)
                    if k == 0:
                        # Only the last step acknowledges, which keeps every
                        # semaphore balanced so the plan can be re-run.
                        op.notify(signal_id=rank, target_rank=partner)
                op.wait_notify(signal_id=rank ^ 1, source_rank=rank ^ 1)
            return finish(op, "allreduce", "rhd")

    # -- additions: natural-order reduce-scatter / allgather --------------------
    def build_reduce_scatter(self, rank, world_size, tensor_size, dtype="bfloat16",
                             executor="tma", num_channels=1) -> PrimitiveIRGraph:
        levels = self._check(world_size)
        tma = executor == "tma"
        with CommunicationOp(name=f"rhd_rs_{executor}_rank{rank}", device=DeviceType.CUDA) as op:
            op.tensor(dtype=dtype, shape=(tensor_size,))
            with Stream("main"):
                op.set_channel(0)
                start = 0
                for k in range(levels):
                    bit = levels - 1 - k
                    partner, half = rank ^ (1 << bit), tensor_size >> (k + 1)
                    mine = start + (half if rank >> bit & 1 else 0)
                    self._exchange(op, rank, partner)
                    (op.tma_reduce if tma else op.sm_reduce)(
                        reduce_op="sum", source_rank=partner, src_offset=mine, dst_offset=mine,
                        remote_offset=mine, count=half)
                    start = mine
                # Closing handshake with every partner: nobody may start the next
                # collective (and overwrite its input) while a partner still reads it.
                for k in range(levels):
                    self._exchange(op, rank, rank ^ (1 << k))
            return finish(op, "reduce_scatter", "rhd")

    def build_allgather(self, rank, world_size, tensor_size, dtype="bfloat16", executor="tma",
                        num_channels=1) -> PrimitiveIRGraph:
        levels = self._check(world_size)
        tma = executor == "tma"
        shard = tensor_size // world_size
        with CommunicationOp(name=f"rhd_ag_{executor}_rank{rank}", device=DeviceType.CUDA) as op:
            op.tensor(dtype=dtype, shape=(tensor_size,))
            with Stream("main"):
                op.set_channel(0)
                for bit in range(levels):                     # doubling, lowest bit first
                    partner, span = rank ^ (1 << bit), shard << bit
                    # Partner holds the aligned block of ``span`` elements that contains its rank.
                    theirs = (partner >> bit << bit) * shard
                    self._exchange(op, rank, partner)
                    (op.tma_copy if tma else op.sm_copy)(
                        source_rank=partner, src_offset=theirs, dst_offset=theirs, size=span)
                for bit in range(levels):
                    self._exchange(op, rank, rank ^ (1 << bit))
            return finish(op, "allgather", "rhd")
