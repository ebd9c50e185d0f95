"""The per-rank primitive DAG.

A ``PrimitiveIRGraph`` owns the nodes of one rank's plan, keyed by op id, and
keeps the ``dependencies`` / ``next_ops`` adjacency that the code generator
serialises.  It offers the same surface as the reference container
(reference: pccl/dsl/graph.py:24-227): add/remove nodes, cycle-checked edge
insertion, validation, a stable Kahn ordering, and the splitting of a graph at
OCS barriers into host-separated phases.

Cycle detection here is iterative (three-colour DFS on an explicit stack), so
32-channel plans with tens of thousands of chained nodes do not hit Python's
recursion limit.
"""

from __future__ import annotations

import uuid
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional

from .nodes import IRNodeVariant, OcsBarrierNode, PrimitiveOpType


@dataclass
class OcsPhase:
    """Nodes that run between two host barriers, plus the barrier that ends them."""

    index: int
    nodes: List[IRNodeVariant]
    barrier: Optional[OcsBarrierNode] = None


@dataclass(init=False)
class PrimitiveIRGraph:
    nodes: Dict[str, IRNodeVariant]
    graph_name: str
    graph_id: str
    entry_points: List[str]
    exit_points: List[str]
    collective_type: str

    def __init__(self, nodes: Optional[Dict[str, IRNodeVariant]] = None,
                 graph_name: str = "unnamed_graph", graph_id: str = "",
                 entry_points: Optional[List[str]] = None,
                 exit_points: Optional[List[str]] = None,
                 collective_type: str = "",
                 # README-style keywords, accepted and recorded but not required.
                 device_type=None, num_ranks: Optional[int] = None):
        self.nodes = {} if nodes is None else nodes
        self.graph_name = graph_name
        self.graph_id = graph_id or f"{graph_name}_{uuid.uuid4().hex[:8]}"
        self.entry_points = [] if entry_points is None else entry_points
        self.exit_points = [] if exit_points is None else exit_points
        self.collective_type = collective_type
        #: name of the algorithm template that built the graph ("" if hand-built)
        self.algorithm = ""
        self.device_type = device_type
        self.num_ranks = num_ranks

    # -- container ---------------------------------------------------------
    def add_node(self, node: IRNodeVariant) -> IRNodeVariant:
        if node.op_id in self.nodes:
            raise ValueError(f"Node with id '{node.op_id}' already exists in graph")
        self.nodes[node.op_id] = node
        return node

    def get_node(self, node_id: str) -> IRNodeVariant:
        try:
            return self.nodes[node_id]
        except KeyError:
            raise KeyError(f"Node with id '{node_id}' not found in graph") from None

    def remove_node(self, node_id: str) -> None:
        self.get_node(node_id)
        del self.nodes[node_id]
        for other in self.nodes.values():
            if node_id in other.dependencies:
                other.dependencies.remove(node_id)
            if node_id in other.next_ops:
                other.next_ops.remove(node_id)

    def add_edge(self, src_id: str, dst_id: str) -> None:
        if src_id not in self.nodes:
            raise KeyError(f"Source node '{src_id}' not found in graph")
        if dst_id not in self.nodes:
            raise KeyError(f"Destination node '{dst_id}' not found in graph")
        if src_id == dst_id:
            raise ValueError(f"Cannot add self-loop on node '{src_id}'")
        src, dst = self.nodes[src_id], self.nodes[dst_id]
        if dst_id in src.next_ops:
            return
        # A new edge src->dst closes a cycle exactly when src is reachable from dst.
        if self._reaches(dst_id, src_id):
            raise ValueError(f"Adding edge {src_id} -> {dst_id} would create a cycle")
        dst.add_dependency(src_id)
        src.add_next_op(dst_id)

    def get_nodes_by_type(self, op_type: PrimitiveOpType) -> List[IRNodeVariant]:
        return [n for n in self.nodes.values() if n.op_type == op_type]

    def size(self) -> int:
        return len(self.nodes)

    def is_empty(self) -> bool:
        return not self.nodes

    def __repr__(self) -> str:
        return f"PrimitiveIRGraph(name={self.graph_name}, nodes={len(self.nodes)})"

    # -- structure ---------------------------------------------------------
    def _reaches(self, start: str, goal: str) -> bool:
        stack, seen = [start], {start}
        while stack:
            cur = stack.pop()
            if cur == goal:
                return True
            for nxt in self.nodes[cur].next_ops:
                if nxt in self.nodes and nxt not in seen:
                    seen.add(nxt)
                    stack.append(nxt)
        return False

    def _has_cycle(self) -> bool:
        WHITE, GREY, BLACK = 0, 1, 2
        colour = dict.fromkeys(self.nodes, WHITE)
        for root in self.nodes:
            if colour[root] != WHITE:
                continue
            colour[root] = GREY
            stack = [(root, iter(self.nodes[root].next_ops))]
            while stack:
                nid, successors = stack[-1]
                advanced = False
                for nxt in successors:
                    state = colour.get(nxt)
                    if state == GREY:
                        return True
                    if state == WHITE:
                        colour[nxt] = GREY
                        stack.append((nxt, iter(self.nodes[nxt].next_ops)))
                        advanced = True
                        break
                if not advanced:
                    colour[nid] = BLACK
                    stack.pop()
        return False

    def topological_sort(self) -> List[IRNodeVariant]:
        """Kahn's algorithm; ties resolve in insertion order, so the emitted
        plan order is deterministic for a given build sequence."""
        pending = {nid: len(n.dependencies) for nid, n in self.nodes.items()}
        ready = deque(nid for nid, deg in pending.items() if deg == 0)
        ordered: List[IRNodeVariant] = []
        while ready:
            nid = ready.popleft()
            node = self.nodes[nid]
            ordered.append(node)
            for nxt in node.next_ops:
                pending[nxt] -= 1
                if pending[nxt] == 0:
                    ready.append(nxt)
        if len(ordered) != len(self.nodes):
            raise ValueError("Cannot perform topological sort on graph with cycles")
        return ordered

    def _update_boundary_points(self) -> None:
        self.entry_points = [nid for nid, n in self.nodes.items() if not n.dependencies]
        self.exit_points = [nid for nid, n in self.nodes.items() if not n.next_ops]

    # -- validation --------------------------------------------------------
    def validate(self) -> bool:
        if not self.nodes:
            raise ValueError("Graph is empty (no nodes)")
        for nid, node in self.nodes.items():
            for dep in node.dependencies:
                if dep not in self.nodes:
                    raise ValueError(
                        f"Node '{nid}' has dependency on non-existent node '{dep}'")
            for nxt in node.next_ops:
                if nxt not in self.nodes:
                    raise ValueError(
                        f"Node '{nid}' has next_op reference to non-existent node '{nxt}'")
        if self._has_cycle():
            raise ValueError("Graph contains a cycle")
        for node in self.nodes.values():
            node.validate()
        self._update_boundary_points()
        self._validate_ocs_barrier_boundaries()
        return True

    # -- OCS phases --------------------------------------------------------
    def has_ocs_barriers(self) -> bool:
        return any(isinstance(n, OcsBarrierNode) for n in self.nodes.values())

    def split_ocs_phases(self) -> List[OcsPhase]:
        """Cut the graph at every OCS barrier (in topological order)."""
        order = self.topological_sort()
        if not self.has_ocs_barriers():
            return [OcsPhase(index=0, nodes=order)]
        self._validate_ocs_barrier_boundaries()
        phases: List[OcsPhase] = []
        bucket: List[IRNodeVariant] = []
        for node in order:
            if isinstance(node, OcsBarrierNode):
                phases.append(OcsPhase(index=len(phases), nodes=bucket, barrier=node))
                bucket = []
            else:
                bucket.append(node)
        phases.append(OcsPhase(index=len(phases), nodes=bucket))
        return phases

    def _validate_ocs_barrier_boundaries(self) -> None:
        """A barrier must be a clean cut of the whole graph.

        Because the host has to regain control between phases, (1) a barrier
        depends on every node of the phase it closes, (2) every entry node of
        the next phase depends on that barrier, and (3) no data edge jumps
        over a barrier.
        """
        if not self.has_ocs_barriers():
            return
        phase_of: Dict[str, int] = {}
        members: List[str] = []
        phase = 0
        last_barrier: Optional[str] = None
        for node in self.topological_sort():
            if isinstance(node, OcsBarrierNode):
                missing = sorted(set(members) - set(node.dependencies))
                if missing:
                    raise ValueError(
                        f"OCS barrier '{node.op_id}' must depend on every node in phase "
                        f"{phase}; missing {missing}")
                last_barrier, members, phase = node.op_id, [], phase + 1
                continue
            dep_phases = [phase_of.get(d) for d in node.dependencies]
            if phase > 0 and phase not in dep_phases and last_barrier not in node.dependencies:
                raise ValueError(
                    f"phase-{phase} entry node '{node.op_id}' must depend on OCS barrier "
                    f"'{last_barrier}'")
            for dep, dep_phase in zip(node.dependencies, dep_phases):
                if dep_phase is not None and dep_phase < phase:
                    raise ValueError(
                        f"data dependency '{dep}' -> '{node.op_id}' crosses an OCS barrier; "
                        "depend on the barrier node instead")
            phase_of[node.op_id] = phase
            members.append(node.op_id)

    # -- convenience -------------------------------------------------------
    def add_nodes(self, nodes: Iterable[IRNodeVariant]) -> None:
        for node in nodes:
            self.add_node(node)
