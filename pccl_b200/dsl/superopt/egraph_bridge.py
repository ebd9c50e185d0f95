"""Conversion between a ``PrimitiveIRGraph`` and an ``EGraph``.

``ir_to_egraph`` inserts one e-node per IR node, with the node's dependencies
as children and its plan parameters as the e-node payload.  ``egraph_to_ir``
runs cost-based extraction and materialises the chosen e-nodes as fresh IR
nodes, wiring edges from the e-node child relation and inheriting channel,
device and tensor info from the original node of the same e-class (reference:
pccl/dsl/superopt/egraph_bridge.py:46-252).
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

from ..graph import PrimitiveIRGraph
from ..nodes import (IRNodeVariant, NODE_CLASS_BY_OP, OcsBarrierNode, PrimitiveOpType,
                     node_from_params)
from .egraph import EGraph, ENode

CostFn = Callable[[ENode, Dict[int, float]], float]


def _params_to_frozen(params: dict) -> Tuple[Tuple[str, object], ...]:
    return tuple(sorted((k, tuple(v) if isinstance(v, list) else v) for k, v in params.items()))


def _enode_of(node: IRNodeVariant, class_of: Dict[str, int]) -> ENode:
    kids = tuple(class_of[d] for d in node.dependencies if d in class_of)
    name = node.op_type.value if node.op_type else "noop"
    return ENode(name, 0, kids, _params_to_frozen(node.to_params()))


def ir_to_egraph(graph: PrimitiveIRGraph) -> Tuple[EGraph, Dict[str, int], List[int]]:
    """Returns (e-graph, op_id -> e-class id, e-class ids of the exit nodes)."""
    eg = EGraph()
    class_of: Dict[str, int] = {}
    order = graph.topological_sort()
    for node in order:
        class_of[node.op_id] = eg.add(_enode_of(node, class_of))
    roots = [class_of[nid] for nid in graph.exit_points if nid in class_of]
    if not roots:
        roots = [class_of[n.op_id] for n in order if not n.next_ops]
    return eg, class_of, roots


def _extract_dag(eg: EGraph, roots: List[int], cost_fn: CostFn) -> Dict[int, ENode]:
    """Cheapest e-node of every e-class reachable from ``roots``."""
    _, choice = eg.best_per_class(cost_fn)
    picked: Dict[int, ENode] = {}
    work = [eg.find(r) for r in roots]
    while work:
        eid = work.pop()
        if eid in picked or eid not in choice:
            continue
        picked[eid] = choice[eid]
        work.extend(eg.find(c) for c in choice[eid].children)
    return picked


def _create_ir_node(enode: ENode, ref_node: Optional[IRNodeVariant] = None) -> Optional[IRNodeVariant]:
    try:
        op_type = PrimitiveOpType(enode.op_type)
    except ValueError:
        return None
    if op_type not in NODE_CLASS_BY_OP or NODE_CLASS_BY_OP[op_type] is OcsBarrierNode:
        return None
    params = dict(ref_node.to_params()) if ref_node is not None else {}
    params.update(dict(enode.params))
    # A node built without any rank information defaults to rank 0, not -1.
    for key in ("source_rank", "target_rank"):
        if key in getattr(NODE_CLASS_BY_OP[op_type], "PARAM_NAMES", ()):
            params.setdefault(key, 0)
    return node_from_params(op_type, params)


def egraph_to_ir(eg: EGraph, roots: List[int], cost_fn: CostFn,
                 original_graph: Optional[PrimitiveIRGraph] = None) -> PrimitiveIRGraph:
    picked = _extract_dag(eg, roots, cost_fn)

    # Locate, for each e-class, the original IR node that lives in it.
    origin: Dict[int, IRNodeVariant] = {}
    if original_graph is not None:
        class_of: Dict[str, int] = {}
        for node in original_graph.topological_sort():
            probe = _enode_of(node, class_of).canonicalize(eg.uf)
            eid = eg.hashcons.get(probe)
            if eid is None:
                continue
            eid = eg.find(eid)
            class_of[node.op_id] = eid
            origin.setdefault(eid, node)

    out = PrimitiveIRGraph(
        graph_name=original_graph.graph_name if original_graph else "extracted")
    if original_graph is not None:
        out.collective_type = original_graph.collective_type

    # Emit nodes in the original plan order where known, so ties in the later
    # topological sort resolve the same way as in the input graph.
    position = {id(n): i for i, n in enumerate(original_graph.nodes.values())} \
        if original_graph is not None else {}
    emit_order = sorted(picked, key=lambda e: position.get(id(origin.get(e)), len(position)))

    ir_id: Dict[int, str] = {}
    for eid in emit_order:
        ref = origin.get(eid)
        node = _create_ir_node(picked[eid], ref)
        if node is None:
            continue
        if ref is not None:
            node.channel, node.device, node.tensor_info = ref.channel, ref.device, ref.tensor_info
        out.add_node(node)
        ir_id[eid] = node.op_id

    for eid in emit_order:
        dst = ir_id.get(eid)
        if dst is None:
            continue
        for child in picked[eid].children:
            src = ir_id.get(eg.find(child))
            if src is not None and src != dst:
                try:
                    out.add_edge(src, dst)
                except (KeyError, ValueError):
                    pass
    out._update_boundary_points()
    return out
