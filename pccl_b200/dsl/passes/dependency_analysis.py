"""Dependency analysis: check references, rebuild forward edges, index the order.

``dependencies`` is the source of truth; ``next_ops`` is regenerated from it so
later passes may edit dependencies only (reference:
pccl/dsl/passes/dependency_analysis.py:8-69).
"""

from __future__ import annotations

from typing import Dict

from ..graph import PrimitiveIRGraph


class DependencyAnalysisPass:
    def __init__(self, strict: bool = True):
        self.strict = strict
        self._topological_order: Dict[str, int] = {}

    def _complain(self, message: str) -> None:
        if self.strict:
            raise ValueError(message)

    def run(self, graph: PrimitiveIRGraph) -> PrimitiveIRGraph:
        if graph.is_empty():
            self._complain("Cannot analyze empty graph")
            return graph

        known = graph.nodes
        for nid, node in known.items():
            for dep in node.dependencies:
                if dep not in known:
                    self._complain(f"Node '{nid}' has dependency on non-existent node '{dep}'")
            for nxt in node.next_ops:
                if nxt not in known:
                    self._complain(
                        f"Node '{nid}' has next_op reference to non-existent node '{nxt}'")

        # Regenerate successors from predecessors, in node insertion order.
        for node in known.values():
            node.next_ops.clear()
        for nid, node in known.items():
            for dep in node.dependencies:
                if dep in known:
                    known[dep].add_next_op(nid)

        if graph._has_cycle():
            self._complain("Graph contains a cycle")
            return graph
        self._topological_order = {
            node.op_id: position for position, node in enumerate(graph.topological_sort())}
        return graph
