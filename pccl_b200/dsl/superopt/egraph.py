"""A small e-graph for equality saturation over plan primitives.

An e-graph stores many equivalent programs compactly: *e-nodes* (operator +
child e-class ids) are grouped into *e-classes* of nodes known to compute the
same thing.  Rewrites add e-nodes and merge e-classes; ``rebuild`` restores
congruence (equal operator + equal children => same class); ``extract`` picks
the cheapest representative per class under a cost function (reference:
pccl/dsl/superopt/egraph.py:18-275 defines the same public surface).
"""

from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field
from itertools import product
from typing import Any, Callable, Dict, Iterable, List, Optional, Set, Tuple

#: primitive name -> semantic family (members of a family differ only in executor)
OP_CATEGORY_MAP: Dict[str, str] = {
    "sm.copy": "copy", "tma.copy": "copy", "ce.copy": "copy",
    "sm.reduce": "reduce", "tma.reduce": "reduce", "multimem.reduce": "reduce",
    "multimem.store": "store",
    "rdma.write": "rdma_write", "rdma.read": "rdma_read",
    "notify": "notify", "wait_notify": "wait_notify", "noop": "noop",
}


class UnionFind:
    """Disjoint sets over integer ids with path halving and union by rank."""

    def __init__(self):
        self.parent: Dict[int, int] = {}
        self.rank: Dict[int, int] = {}

    def make_set(self, x: int) -> None:
        if x not in self.parent:
            self.parent[x] = x
            self.rank[x] = 0

    def find(self, x: int) -> int:
        parent = self.parent
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    def union(self, x: int, y: int) -> int:
        a, b = self.find(x), self.find(y)
        if a == b:
            return a
        if self.rank[a] < self.rank[b]:
            a, b = b, a
        self.parent[b] = a
        if self.rank[a] == self.rank[b]:
            self.rank[a] += 1
        return a


@dataclass(frozen=True)
class ENode:
    op_type: str
    rank: int
    children: Tuple[int, ...] = ()
    params: Tuple[Tuple[str, Any], ...] = ()

    def canonicalize(self, uf: UnionFind) -> "ENode":
        return ENode(self.op_type, self.rank, tuple(uf.find(c) for c in self.children),
                     self.params)

    @property
    def category(self) -> str:
        return OP_CATEGORY_MAP.get(self.op_type, self.op_type)


class Substitution(dict):
    """Pattern variable -> e-class id."""


@dataclass
class PatternExpr:
    """Either a variable (``var`` set) or an operator pattern with children.
    ``op_type``, ``op_category`` and ``rank`` constrain only when not None."""

    op_type: Optional[str] = None
    rank: Optional[int] = None
    children: List["PatternExpr"] = field(default_factory=list)
    var: Optional[str] = None
    op_category: Optional[str] = None

    def is_var(self) -> bool:
        return self.var is not None

    def admits(self, enode: ENode) -> bool:
        return ((self.op_type is None or enode.op_type == self.op_type)
                and (self.op_category is None or enode.category == self.op_category)
                and (self.rank is None or enode.rank == self.rank)
                and len(self.children) == len(enode.children))


def _unify(parts: Iterable[Substitution]) -> Optional[Substitution]:
    merged = Substitution()
    for part in parts:
        for var, eid in part.items():
            if merged.setdefault(var, eid) != eid:
                return None
    return merged


Rule = Tuple[PatternExpr, Callable[[Substitution], Optional[int]]]
CostFn = Callable[[ENode, Dict[int, float]], float]


class EGraph:
    def __init__(self):
        self.uf = UnionFind()
        self.eclass_nodes: Dict[int, Set[ENode]] = defaultdict(set)
        self.hashcons: Dict[ENode, int] = {}
        self.next_id = 0
        self.dirty = False

    # -- construction --------------------------------------------------------
    def find(self, eid: int) -> int:
        return self.uf.find(eid)

    def add(self, enode: ENode) -> int:
        enode = enode.canonicalize(self.uf)
        known = self.hashcons.get(enode)
        if known is not None:
            return self.uf.find(known)
        eid = self.next_id
        self.next_id += 1
        self.uf.make_set(eid)
        self.hashcons[enode] = eid
        self.eclass_nodes[eid].add(enode)
        return eid

    def merge(self, id1: int, id2: int) -> int:
        a, b = self.uf.find(id1), self.uf.find(id2)
        if a == b:
            return a
        keep = self.uf.union(a, b)
        drop = b if keep == a else a
        self.eclass_nodes[keep] |= self.eclass_nodes.pop(drop, set())
        self.dirty = True
        return keep

    def rebuild(self) -> None:
        """Re-canonicalise until congruence closure holds."""
        while self.dirty:
            self.dirty = False
            table: Dict[ENode, int] = {}
            for enode, eid in self.hashcons.items():
                canon, owner = enode.canonicalize(self.uf), self.uf.find(eid)
                other = table.get(canon)
                if other is None:
                    table[canon] = owner
                elif self.uf.find(other) != owner:
                    table[canon] = self.merge(other, owner)   # sets dirty again
            self.hashcons = table
            classes: Dict[int, Set[ENode]] = defaultdict(set)
            for enode, eid in table.items():
                classes[self.uf.find(eid)].add(enode.canonicalize(self.uf))
            self.eclass_nodes = classes

    # -- matching ------------------------------------------------------------
    def ematch(self, pattern: PatternExpr) -> List[Substitution]:
        found: List[Substitution] = []
        for eid in list(self.eclass_nodes):
            found.extend(self._match_eclass(pattern, eid))
        return found

    def _match_eclass(self, pattern: PatternExpr, eid: int) -> List[Substitution]:
        eid = self.uf.find(eid)
        if pattern.is_var():
            return [Substitution({pattern.var: eid})]
        out: List[Substitution] = []
        for enode in self.eclass_nodes.get(eid, ()):
            if not pattern.admits(enode):
                continue
            per_child = [self._match_eclass(p, c) for p, c in zip(pattern.children, enode.children)]
            for combo in product(*per_child):
                unified = _unify(combo)
                if unified is not None:
                    out.append(unified)
        return out

    def saturate(self, rules: List[Rule], limit: int = 30) -> int:
        """Apply rules until nothing changes or ``limit`` rounds ran; returns rounds."""
        rounds = 0
        while rounds < limit:
            fired = 0
            for pattern, applier in rules:
                for sub in self.ematch(pattern):
                    if applier(sub) is not None:
                        fired += 1
            self.rebuild()
            rounds += 1
            if not fired:
                break
        return rounds

    # -- extraction ----------------------------------------------------------
    def best_per_class(self, cost_fn: CostFn) -> Tuple[Dict[int, float], Dict[int, ENode]]:
        """Bellman-Ford style fix-point: cheapest e-node of every e-class."""
        cost: Dict[int, float] = {}
        choice: Dict[int, ENode] = {}
        for _ in range(len(self.eclass_nodes) + 1):
            improved = False
            for eid, enodes in self.eclass_nodes.items():
                eid = self.uf.find(eid)
                for enode in enodes:
                    kids = [self.uf.find(c) for c in enode.children]
                    if any(k not in cost for k in kids):
                        continue
                    value = cost_fn(enode, {k: cost[k] for k in kids})
                    if eid not in cost or value < cost[eid]:
                        cost[eid], choice[eid] = value, enode
                        improved = True
            if not improved:
                break
        return cost, choice

    def extract(self, root: int, cost_fn: CostFn) -> Tuple[float, Optional[ENode]]:
        cost, choice = self.best_per_class(cost_fn)
        root = self.uf.find(root)
        return cost.get(root, float("inf")), choice.get(root)

    def eclass_count(self) -> int:
        return len(self.eclass_nodes)

    def enode_count(self) -> int:
        return len(self.hashcons)
