"""Common interface of the collective algorithm templates.

A template turns ``(rank, world_size, tensor_size, dtype, executor,
num_channels)`` into the per-rank ``PrimitiveIRGraph`` of one collective
(reference: pccl/dsl/algorithms/base.py:7-64).  ``tensor_size`` counts elements
of the *full* tensor (all shards).  Buffer conventions, shared with the engine:

=============== ============================== =================================
collective      input in the working buffer    output in the working buffer
=============== ============================== =================================
allreduce       ``[0, n)``                     ``[0, n)``
reduce_scatter  ``[0, n)``                     ``[rank*n/W, (rank+1)*n/W)``
allgather       shard at ``[rank*n/W, ...)``   ``[0, n)``
alltoall        ``[0, n)``                     chunk p at ``[n + p*n/W, ...)`` for
                                               p != rank, own chunk stays in place
=============== ============================== =================================
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Iterator, Tuple

from ..decorators import CommunicationOp
from ..graph import PrimitiveIRGraph

#: signal ids of channel c live in [c * SIGNAL_STRIDE, (c + 1) * SIGNAL_STRIDE)
SIGNAL_STRIDE = 1000


def channel_slices(tensor_size: int, num_channels: int) -> Iterator[Tuple[int, int, int, int]]:
    """Yields ``(channel, base_offset, elements, signal_base)`` per channel."""
    per_channel = tensor_size // num_channels
    for c in range(num_channels):
        yield c, c * per_channel, per_channel, c * SIGNAL_STRIDE


def all_pairs_barrier(op: CommunicationOp, rank: int, world_size: int, signal_base: int) -> None:
    """Every rank posts one signal to every peer, then consumes one from each.

    The signal id encodes the *sender* (``signal_base + sender``) because the
    runtime indexes a rank's semaphores by id only.  Peers are visited in
    rotated order so the N*(N-1) posts do not all target rank 0 first.
    """
    peers = [(rank + i) % world_size for i in range(1, world_size)]
    for peer in peers:
        op.notify(signal_id=signal_base + rank, target_rank=peer)
    for peer in peers:
        op.wait_notify(signal_id=signal_base + peer, source_rank=peer)


def is_power_of_two(n: int) -> bool:
    return n > 0 and n & (n - 1) == 0


class CollectiveAlgorithm(ABC):
    name: str = ""

    @abstractmethod
    def build_allreduce(self, rank: int, world_size: int, tensor_size: int,
                        dtype: str = "bfloat16", executor: str = "tma",
                        num_channels: int = 1) -> PrimitiveIRGraph:
        raise NotImplementedError

    def _unsupported(self, what: str):
        raise NotImplementedError(f"{type(self).__name__} does not implement {what}")

    def build_reduce_scatter(self, rank: int, world_size: int, tensor_size: int,
                             dtype: str = "bfloat16", executor: str = "tma",
                             num_channels: int = 1) -> PrimitiveIRGraph:
        self._unsupported("reduce_scatter")

    def build_allgather(self, rank: int, world_size: int, tensor_size: int,
                        dtype: str = "bfloat16", executor: str = "tma",
                        num_channels: int = 1) -> PrimitiveIRGraph:
        self._unsupported("allgather")

    def build_alltoall(self, rank: int, world_size: int, tensor_size: int,
                       dtype: str = "bfloat16", executor: str = "tma",
                       num_channels: int = 1) -> PrimitiveIRGraph:
        self._unsupported("alltoall")

    @property
    def step_count(self) -> str:
        return "unknown"

    @property
    def bandwidth_optimal(self) -> bool:
        return False


def finish(op: CommunicationOp, collective_type: str, algorithm: str) -> PrimitiveIRGraph:
    graph = op.get_graph()
    graph.collective_type = collective_type
    graph.algorithm = algorithm
    return graph
