"""Automatic channelization.

Finds maximal runs of same-type data primitives on channel 0 whose source
ranges are back-to-back (signal primitives in between are skipped over), and —
only when the channel-aware cost model says it pays — deals the run out to
``num_channels`` channels in contiguous blocks (reference:
pccl/dsl/passes/channelize.py:42-203).
"""

from __future__ import annotations

from collections import deque
from typing import List, Optional, Set

from ..graph import PrimitiveIRGraph
from ..nodes import IRNodeVariant, PrimitiveOpType as Op
from ..superopt.cost_model import GpuProfile, H100_PROFILE, critical_path_cost
from ..superopt.rule import PatternEdge, PatternNode

_DATA_OPS = frozenset({Op.SM_COPY, Op.TMA_COPY, Op.CE_COPY, Op.SM_REDUCE, Op.TMA_REDUCE,
                       Op.RDMA_WRITE, Op.RDMA_READ})
_SYNC_OPS = frozenset({Op.NOTIFY, Op.WAIT_NOTIFY, Op.NOOP})


def _extent(node: IRNodeVariant) -> int:
    params = node.to_params()
    return params.get("size", params.get("count", 0))


class ChannelizePass:
    def __init__(self, num_channels: int = 2, min_data_size: int = 4096,
                 profile: GpuProfile = H100_PROFILE):
        self.num_channels = num_channels
        self.min_data_size = min_data_size
        self.profile = profile

    def run(self, graph: PrimitiveIRGraph) -> PrimitiveIRGraph:
        for chain in self._find_channelizable_chains(graph):
            self._try_channelize_chain(graph, chain)
        return graph

    # -- discovery ---------------------------------------------------------
    def _find_channelizable_chains(self, graph: PrimitiveIRGraph) -> List[List[IRNodeVariant]]:
        claimed: Set[str] = set()
        chains: List[List[IRNodeVariant]] = []
        for head in graph.topological_sort():
            if head.op_id in claimed or head.op_type not in _DATA_OPS or head.channel != 0:
                continue
            chain = [head]
            claimed.add(head.op_id)
            while True:
                nxt = self._next_data_op(graph, chain[-1])
                if (nxt is None or nxt.op_id in claimed or nxt.op_type != head.op_type
                        or nxt.channel != 0 or not self._is_contiguous(chain[-1], nxt)):
                    break
                chain.append(nxt)
                claimed.add(nxt.op_id)
            if len(chain) > self.num_channels:
                chains.append(chain)
        return chains

    @staticmethod
    def _next_data_op(graph: PrimitiveIRGraph, node: IRNodeVariant) -> Optional[IRNodeVariant]:
        """Nearest data primitive downstream of ``node``, looking through signals."""
        frontier, seen = deque(node.next_ops), set()
        while frontier:
            nid = frontier.popleft()
            if nid in seen or nid not in graph.nodes:
                continue
            seen.add(nid)
            candidate = graph.nodes[nid]
            if candidate.op_type in _DATA_OPS:
                return candidate
            if candidate.op_type in _SYNC_OPS:
                frontier.extend(candidate.next_ops)
        return None

    @staticmethod
    def _is_contiguous(a: IRNodeVariant, b: IRNodeVariant) -> bool:
        pa, pb = a.to_params(), b.to_params()
        for key in ("size", "count"):
            if key in pa and key in pb:
                return pb.get("src_offset", 0) == pa.get("src_offset", 0) + pa[key]
        return False

    # -- decision ------------------------------------------------------------
    def _chain_data_size(self, chain: List[IRNodeVariant]) -> int:
        return sum(_extent(node) for node in chain)

    def _data_size_of(self, node: IRNodeVariant) -> int:
        return _extent(node)

    def _try_channelize_chain(self, graph: PrimitiveIRGraph, chain: List[IRNodeVariant]) -> bool:
        length, lanes = len(chain), self.num_channels
        if length <= lanes:
            return False
        total = self._chain_data_size(chain)
        if total < self.min_data_size:
            return False
        per_op = total // length
        block = -(-length // lanes)

        def pattern(lane_of):
            nodes = [PatternNode(op_type=n.op_type, rank=0, chunk_id=0, channel=lane_of(i))
                     for i, n in enumerate(chain)]
            edges = [PatternEdge(i, i + 1) for i in range(length - 1)
                     if lane_of(i) == lane_of(i + 1)]
            return nodes, edges

        serial = critical_path_cost(*pattern(lambda i: 0), self.profile, per_op)
        spread = critical_path_cost(*pattern(lambda i: min(i // block, lanes - 1)),
                                    self.profile, per_op)
        if spread >= serial:
            return False
        self._apply_channelization(graph, chain, lanes)
        return True

    @staticmethod
    def _apply_channelization(graph: PrimitiveIRGraph, chain: List[IRNodeVariant], nc: int) -> None:
        block = -(-len(chain) // nc)
        for i, node in enumerate(chain):
            node.channel = min(i // block, nc - 1)
