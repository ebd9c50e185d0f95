"""Hand-written rewrite knowledge for the e-graph.

A. *Executor equivalences*: primitives that differ only in which engine moves
   the bytes are interchangeable; for every such e-node the alternatives are
   added to its e-class up front.  The families are the reference's
   (reference: pccl/dsl/superopt/domain_rules.py:19-57): the multimem primitives stand alone here,
   because turning pulls into an in-switch broadcast or a run of reduces into an in-switch
   reduction changes several nodes at once; those rewrites live in ``fabric_rules.py``.
B. *Structural rules*: ``op(op(x, P), P) -> op(x, P)`` for idempotent
   re-application of the same primitive with identical parameters.
C. *Adapter for cached SMT-verified rules*: single-node rules become executor
   alternatives of matching e-nodes.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

from .egraph import EGraph, ENode, PatternExpr, Substitution
from .rule import RewriteRule
from .rule_db import load_all_rules

EXECUTOR_EQUIVALENCES: Dict[str, List[str]] = {
    "copy": ["sm.copy", "tma.copy", "ce.copy"],
    "reduce": ["sm.reduce", "tma.reduce"],
    "multimem_reduce": ["multimem.reduce"],
    "multimem_store": ["multimem.store"],
    "rdma_write": ["rdma.write"],
    "rdma_read": ["rdma.read"],
}

_FAMILY_OF: Dict[str, str] = {
    op: family for family, ops in EXECUTOR_EQUIVALENCES.items() for op in ops}

Rule = Tuple[PatternExpr, Callable[[Substitution], Optional[int]]]


def add_executor_equivalences(eg: EGraph) -> int:
    """Add every same-family alternative of every e-node; returns merges done."""
    merges = 0
    for eid, enodes in list(eg.eclass_nodes.items()):
        for enode in list(enodes):
            family = _FAMILY_OF.get(enode.op_type)
            if family is None:
                continue
            for alternative in EXECUTOR_EQUIVALENCES[family]:
                if alternative == enode.op_type:
                    continue
                twin = eg.add(ENode(alternative, enode.rank, enode.children, enode.params))
                if eg.find(twin) != eg.find(eid):
                    eg.merge(eid, twin)
                    merges += 1
    if merges:
        eg.rebuild()
    return merges


def structural_rules(eg: EGraph) -> List[Rule]:
    """Rules bound to ``eg``.  The duplicate-elimination rule needs parameter
    equality between parent and child, which a ``PatternExpr`` cannot state, so
    it is a whole-graph scan hung on a match-anything trigger."""

    fired_round = {"stamp": -1}

    def dedup(_sub: Substitution) -> Optional[int]:
        # The trigger matches once per e-class; scan only once per graph state.
        stamp = (eg.next_id, len(eg.eclass_nodes))
        if fired_round["stamp"] == stamp:
            return None
        fired_round["stamp"] = stamp
        merges = 0
        for eid, enodes in list(eg.eclass_nodes.items()):
            for parent in list(enodes):
                family = _FAMILY_OF.get(parent.op_type)
                if family is None:
                    continue
                for child_id in parent.children:
                    child_id = eg.find(child_id)
                    for child in list(eg.eclass_nodes.get(child_id, ())):
                        if (_FAMILY_OF.get(child.op_type) == family
                                and child.params == parent.params
                                and eg.find(eid) != eg.find(child_id)):
                            eg.merge(eid, child_id)
                            merges += 1
        return merges or None

    return [(PatternExpr(var="__dedup_any"), dedup)]


def smt_rules_to_egraph(eg: EGraph, rules: Optional[List[RewriteRule]] = None,
                        max_k: int = 6) -> List[Rule]:
    """Turn cached single-node rules ``A -> B`` into saturation rules that add
    ``B`` (same children, same params) next to every ``A`` e-node."""
    if rules is None:
        rules = load_all_rules(max_k=max_k)
    out: List[Rule] = []
    for rule in rules:
        if len(rule.source_nodes) != 1 or len(rule.replacement_nodes) != 1:
            continue
        src, repl = rule.source_nodes[0], rule.replacement_nodes[0]
        if src.op_type == repl.op_type:
            continue

        def make(src_name: str, repl_name: str):
            def applier(sub: Substitution) -> Optional[int]:
                added = 0
                for eid, enodes in list(eg.eclass_nodes.items()):
                    for enode in list(enodes):
                        if enode.op_type != src_name:
                            continue
                        twin = eg.add(ENode(repl_name, enode.rank, enode.children, enode.params))
                        if eg.find(twin) != eg.find(eid):
                            eg.merge(eid, twin)
                            added += 1
                return added or None
            return applier

        out.append((PatternExpr(op_type=src.op_type.value, rank=src.rank),
                    make(src.op_type.value, repl.op_type.value)))
    return out
