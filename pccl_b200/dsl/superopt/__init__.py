"""Superoptimizer: offline rule discovery + e-graph rewriting of plans.

``discover_rules(k)`` enumerates all skeletons up to ``k`` primitives, filters
candidate (source, replacement) pairs with four cheap tests and proves the
survivors equivalent with z3; the rules are cached on disk and consumed by
``SuperoptPass`` (reference: pccl/dsl/superopt/__init__.py:42-277).

Candidate filters, in order of cost:
  1. *signature* — same number of reductions / chunks / remote writes;
  2. *fingerprint* — identical result of one concrete simulation;
  3. *cost* — replacement not more than 5 % slower than the source at any probe size;
  4. *minimality* — replacement must not contain an already-proven smaller one.
Replacements are searched only at sizes ``<=`` the source size.
"""

from __future__ import annotations

import logging
import time
from typing import Dict, Iterable, List, Optional, Sequence, Set, Tuple

from .cost_model import (
    B200_PROFILE, H100_PROFILE, NVLINK5_TOPOLOGY, NVLINK_TOPOLOGY, PCIE_TOPOLOGY, RDMA_TOPOLOGY,
    GpuProfile, TopologyProfile, critical_path_cost, egraph_node_cost,
)
from .domain_rules import (
    EXECUTOR_EQUIVALENCES, add_executor_equivalences, smt_rules_to_egraph, structural_rules,
)
from .egraph import EGraph, ENode, OP_CATEGORY_MAP, PatternExpr
from .egraph_bridge import egraph_to_ir, ir_to_egraph
from .enumerator import LinkType, enumerate_skeletons, trivial_executor_rules
from .rule import PatternEdge, PatternNode, RewriteRule
from .rule_db import load_rules as _load_rules
from .rule_db import save_rules
from .verifier import check_equivalence, concrete_fingerprint, signatures_compatible

logger = logging.getLogger(__name__)

Skeleton = Tuple[List[PatternNode], List[PatternEdge]]


def _skeleton_hash(nodes: Sequence[PatternNode], edges: Sequence[PatternEdge]) -> int:
    return hash((tuple((n.op_type.value, n.chunk_id, n.channel) for n in nodes),
                 tuple(sorted((e.src_idx, e.dst_idx) for e in edges))))


def _is_subsumed(repl_nodes: Sequence[PatternNode], repl_edges: Sequence[PatternEdge],
                 known_hashes: Set[int]) -> bool:
    """True if deleting any single node yields an already-proven replacement."""
    size = len(repl_nodes)
    if size <= 1:
        return False
    for gone in range(size):
        renumber = {old: new for new, old in enumerate(i for i in range(size) if i != gone)}
        nodes = [n for i, n in enumerate(repl_nodes) if i != gone]
        edges = [PatternEdge(renumber[e.src_idx], renumber[e.dst_idx]) for e in repl_edges
                 if gone not in (e.src_idx, e.dst_idx)]
        if _skeleton_hash(nodes, edges) in known_hashes:
            return True
    return False


class _Candidates:
    """Skeletons of one size with their fingerprints and cost bounds, computed once."""

    def __init__(self, skeletons: Iterable[Skeleton], profile: GpuProfile, sizes: Sequence[int]):
        self.items: List[Skeleton] = list(skeletons)
        self.fingerprint = [concrete_fingerprint(n, e) for n, e in self.items]
        costs = [[critical_path_cost(n, e, profile, s) for s in sizes] for n, e in self.items]
        self.cost_max = [max(c) for c in costs]
        self.cost_min = [min(c) for c in costs]

    def __len__(self) -> int:
        return len(self.items)


def _search(sources: _Candidates, repls: _Candidates, timeout: float, link_type: LinkType,
            stats: Dict[str, int], proven: Optional[Set[int]], rule_prefix: str = ""
            ) -> List[RewriteRule]:
    found: List[RewriteRule] = []
    for si, (s_nodes, s_edges) in enumerate(sources.items):
        for ri, (r_nodes, r_edges) in enumerate(repls.items):
            if not signatures_compatible(s_nodes, r_nodes):
                stats["skipped_sig"] += 1
                continue
            fa, fb = sources.fingerprint[si], repls.fingerprint[ri]
            if fa is not None and fb is not None and fa != fb:
                stats["skipped_fp"] += 1
                continue
            if repls.cost_min[ri] > sources.cost_max[si] * 1.05:
                stats["skipped_cost"] += 1
                continue
            if proven is not None and _is_subsumed(r_nodes, r_edges, proven):
                stats["skipped_minimal"] += 1
                continue
            stats["checked"] += 1
            rule = check_equivalence(s_nodes, s_edges, r_nodes, r_edges, timeout=timeout)
            if rule is None:
                continue
            rule.link_type = link_type.value
            if rule_prefix:
                rule.rule_id = rule_prefix + rule.rule_id
            found.append(rule)
            if proven is not None:
                proven.add(_skeleton_hash(r_nodes, r_edges))
    return found


def discover_rules(k: int, timeout_per_pair: float = 2.0, link_type: LinkType = LinkType.INTRA,
                   progress: bool = True,
                   data_sizes_for_cost: tuple = (1024, 1024 * 1024, 64 * 1024 * 1024),
                   max_channels: int = 1,
                   profile: GpuProfile = H100_PROFILE) -> List[RewriteRule]:
    """Discover and cache rules whose source has 1..k primitives.

    With ``max_channels > 1`` a second phase looks for *channelization* rules:
    single-channel sources with multi-channel replacements of the same size.
    ``profile`` selects the device the cost filter prices against.
    """
    started = time.time()
    rules: List[RewriteRule] = trivial_executor_rules() if link_type == LinkType.INTRA else []
    if progress:
        logger.info("generated %d trivial executor-upgrade rules", len(rules))

    single = {size: _Candidates(enumerate_skeletons(size, link_type, max_channels=1),
                                profile, data_sizes_for_cost) for size in range(1, k + 1)}
    if progress:
        for size, cands in single.items():
            logger.info("  skeletons k=%d: %d", size, len(cands))

    stats = dict.fromkeys(("checked", "skipped_sig", "skipped_fp", "skipped_cost",
                           "skipped_minimal"), 0)
    proven: Set[int] = set()
    for src_size in range(k, 0, -1):
        for repl_size in range(src_size, 0, -1):
            rules += _search(single[src_size], single[repl_size], timeout_per_pair,
                             link_type, stats, proven)
        if progress:
            logger.info("  after sk=%d: %d rules, %s, %.1fs", src_size, len(rules), stats,
                        time.time() - started)

    if max_channels > 1:
        ch_stats = dict.fromkeys(stats, 0)
        before = len(rules)
        for size in range(k, 1, -1):
            known = {_skeleton_hash(n, e) for n, e in single[size].items}
            multi = _Candidates(
                ((n, e) for n, e in enumerate_skeletons(size, link_type, max_channels=max_channels)
                 if len({node.channel for node in n}) > 1 and _skeleton_hash(n, e) not in known),
                profile, data_sizes_for_cost)
            if progress:
                logger.info("  multi-ch skeletons k=%d: %d", size, len(multi))
            if len(multi):
                rules += _search(single[size], multi, timeout_per_pair, link_type, ch_stats,
                                 None, rule_prefix="channelize_")
        if progress:
            logger.info("  channelization rules: %d found, %s", len(rules) - before, ch_stats)

    if progress:
        logger.info("discover_rules done: %d rules in %.1fs", len(rules), time.time() - started)
    save_rules(k, rules)
    return rules


def load_rules(k: int) -> List[RewriteRule]:
    return _load_rules(k)
