"""Enumeration of small communication-DAG skeletons for rule discovery.

A skeleton of size k is a choice of k data primitives, an assignment of each to
a symbolic chunk (set partitions of k, so chunk labels are canonical), an
assignment to hardware channels, and orderings: primitives on the same chunk
and primitives on the same channel are chained; up to two extra ordering edges
between otherwise unordered pairs are also tried.  Signal primitives are not
enumerated (reference: pccl/dsl/superopt/enumerator.py:25-209).
"""

from __future__ import annotations

from collections import defaultdict
from enum import Enum
from itertools import combinations, product
from typing import Dict, Iterator, List, Sequence, Set, Tuple

from ..nodes import PrimitiveOpType
from .rule import PatternEdge, PatternNode


class LinkType(Enum):
    INTRA = "intra"
    INTER = "inter"


CANONICAL_OPS = {
    LinkType.INTRA: [
        PrimitiveOpType.SM_COPY,
        PrimitiveOpType.CE_COPY,
        PrimitiveOpType.SM_REDUCE,
        PrimitiveOpType.MULTIMEM_REDUCE,
        PrimitiveOpType.MULTIMEM_STORE,
    ],
    LinkType.INTER: [
        PrimitiveOpType.RDMA_WRITE,
        PrimitiveOpType.RDMA_READ,
    ],
}

#: executor upgrades that need no proof: identical semantics, never slower
EXECUTOR_UPGRADES = {
    PrimitiveOpType.SM_COPY: PrimitiveOpType.TMA_COPY,
    PrimitiveOpType.SM_REDUCE: PrimitiveOpType.TMA_REDUCE,
}

Skeleton = Tuple[List[PatternNode], List[PatternEdge]]
Pair = Tuple[int, int]


def _bell_partitions(n: int) -> List[List[int]]:
    """All set partitions of n items as restricted-growth strings, in
    lexicographic order (B(n) of them)."""
    if n == 0:
        return [[]]
    out: List[List[int]] = []
    labels = [0] * n

    def grow(pos: int, used: int) -> None:
        if pos == n:
            out.append(labels.copy())
            return
        for label in range(used + 1):
            labels[pos] = label
            grow(pos + 1, max(used, label + 1))

    grow(0, 0)
    return out


def _channel_assignments(k: int, max_channels: int) -> List[List[int]]:
    if max_channels <= 1:
        return [[0] * k]
    return [p for p in _bell_partitions(k) if max(p) < max_channels]


def _canonical_hash(nodes: Sequence[PatternNode], edges: Sequence[PatternEdge]) -> int:
    return hash((tuple((n.op_type.value, n.chunk_id, n.channel) for n in nodes),
                 tuple(sorted((e.src_idx, e.dst_idx) for e in edges))))


def _chain_same_label(labels: Sequence[int]) -> List[Pair]:
    """Consecutive members of every label class, as (earlier, later) pairs."""
    groups: Dict[int, List[int]] = defaultdict(list)
    for i, label in enumerate(labels):
        groups[label].append(i)
    return [pair for members in groups.values() for pair in zip(members, members[1:])]


def _derive_topology(chunk_ids: List[int]) -> List[Pair]:
    return _chain_same_label(chunk_ids)


def _channel_topology(channel_ids: List[int], base_edges: List[Pair]) -> List[Pair]:
    taken = {frozenset(e) for e in base_edges}
    extra = []
    for pair in _chain_same_label(channel_ids):
        if frozenset(pair) not in taken:
            taken.add(frozenset(pair))
            extra.append(pair)
    return extra


def _extra_orderings(k: int, base_edges: List[Pair]) -> Iterator[List[Pair]]:
    taken = {frozenset(e) for e in base_edges}
    free = [(i, j) for i in range(k) for j in range(i + 1, k) if frozenset((i, j)) not in taken]
    yield []
    most = min(1 if k <= 3 else 2, len(free))
    for r in range(1, most + 1):
        for combo in combinations(free, r):
            yield list(combo)


def enumerate_skeletons(k: int, link_type: LinkType = LinkType.INTRA,
                        max_channels: int = 1) -> Iterator[Skeleton]:
    if k <= 0:
        return
    seen: Set[int] = set()
    chunkings = _bell_partitions(k)
    channelings = _channel_assignments(k, max_channels)
    for ops in product(CANONICAL_OPS[link_type], repeat=k):
        for chunks in chunkings:
            chunk_edges = _derive_topology(chunks)
            for chans in channelings:
                base = chunk_edges + _channel_topology(chans, chunk_edges)
                nodes = [PatternNode(op_type=ops[i], rank=0, chunk_id=chunks[i],
                                     link_type=link_type.value, channel=chans[i])
                         for i in range(k)]
                for extra in _extra_orderings(k, base):
                    edges = [PatternEdge(s, d) for s, d in base + extra]
                    key = _canonical_hash(nodes, edges)
                    if key not in seen:
                        seen.add(key)
                        yield list(nodes), edges


def trivial_executor_rules():
    """One rule per entry of ``EXECUTOR_UPGRADES`` (intra-node only); they hold
    by construction and are never sent to the solver."""
    from .rule import RewriteRule

    def single(op: PrimitiveOpType) -> List[PatternNode]:
        return [PatternNode(op_type=op, rank=0, chunk_id=0, link_type=LinkType.INTRA.value)]

    return [
        RewriteRule(
            source_nodes=single(src), source_edges=[],
            replacement_nodes=single(dst), replacement_edges=[],
            param_constraints=["repl_n0_src_offset == src_n0_src_offset",
                               "repl_n0_dst_offset == src_n0_dst_offset"],
            link_type=LinkType.INTRA.value,
            rule_id=f"executor_upgrade_{src.value}_to_{dst.value}",
        )
        for src, dst in EXECUTOR_UPGRADES.items()
    ]
