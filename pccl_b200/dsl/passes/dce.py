"""Dead-code elimination.

Roots are the exit nodes plus every node with an externally visible effect
(remote writes, signal posts, host barriers); everything not backwards-reachable
from a root is dropped (reference: pccl/dsl/passes/dce.py:8-46).
"""

from __future__ import annotations

from typing import List, Set

from ..graph import PrimitiveIRGraph
from ..nodes import NotifyNode, OcsBarrierNode, RdmaWriteNode, SmPutNode

_SIDE_EFFECTS = (RdmaWriteNode, NotifyNode, OcsBarrierNode, SmPutNode)


class DeadCodeEliminationPass:
    def __init__(self, keep_side_effects: bool = True):
        self.keep_side_effects = keep_side_effects
        self._removed_nodes: List[str] = []

    def run(self, graph: PrimitiveIRGraph) -> PrimitiveIRGraph:
        self._removed_nodes = []
        if graph.is_empty():
            return graph
        live = self._live_set(graph)
        for nid in [n for n in graph.nodes if n not in live]:
            graph.remove_node(nid)
            self._removed_nodes.append(nid)
        if self._removed_nodes:
            graph._update_boundary_points()
        return graph

    def _live_set(self, graph: PrimitiveIRGraph) -> Set[str]:
        work = [nid for nid, node in graph.nodes.items()
                if not node.next_ops
                or (self.keep_side_effects and isinstance(node, _SIDE_EFFECTS))]
        live: Set[str] = set()
        while work:
            nid = work.pop()
            if nid in live or nid not in graph.nodes:
                continue
            live.add(nid)
            work.extend(graph.nodes[nid].dependencies)
        return live
