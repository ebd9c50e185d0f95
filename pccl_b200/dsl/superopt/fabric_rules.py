"""Rewrites that retarget a plan to a switched fabric (NVLink 5 + NVSwitch, NVLS).

The e-graph of this package reasons about one node at a time (which engine moves the bytes of
*this* copy); what an NVSwitch changes is the shape of whole runs of nodes.  These rules work on
such runs in one rank's graph and are each applied only if the whole plan gets cheaper under
``plan_cost`` for the given device, fabric and message size, so the same pass keeps a small
message on peer loads and moves a large one into the switch:

F1  ``reduce_chain_to_multi``   a dependency chain of ``sm.reduce`` / ``tma.reduce`` nodes that fold
    different ranks' copies of ONE slice into it in place becomes a single ``sm.reduce_multi``:
    on a switch all sources are one hop away, so they can be read in the same step.
F2  ``reduce_multi_to_multimem``  an ``sm.reduce_multi`` over every rank becomes
    ``multimem.reduce`` (the switch folds the copies; this GPU receives one slice instead of W-1).
F3  ``gather_to_multimem_store``  the all-gather half of a direct all-reduce, seen from one rank as
    pulls of the other W-1 slices next to the slice this rank reduced itself, becomes one
    ``multimem.store`` of the own slice: the plan is the same program on every rank, so "everyone
    pulls everyone's slice" is "everyone broadcasts its slice".
F4  ``fuse_multimem_allreduce``   ``multimem.reduce`` of a slice into itself, a barrier, and the
    ``multimem.store`` of that slice become one ``multimem.allreduce`` (the barrier between the
    halves only protected slices that no other rank touches).

The reference's pass stops at the per-node executor upgrade ``sm -> tma``
(pccl/dsl/superopt/pass_.py:76-87, domain_rules.py:19-57); it has no structural rule.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..graph import PrimitiveIRGraph
from ..nodes import (DTYPE_BYTES, IRNodeVariant, MultimemAllreduceNode, MultimemReduceNode,
                     MultimemStoreNode, PrimitiveOpType as Op, SmReduceMultiNode, _dtype_name)
from .cost_model import GpuProfile, TopologyProfile, plan_cost

_REDUCES = (Op.SM_REDUCE, Op.TMA_REDUCE)
_PULLS = (Op.SM_COPY, Op.TMA_COPY, Op.CE_COPY)
_SIGNALS = (Op.NOTIFY, Op.WAIT_NOTIFY)
_MULTIMEM_DTYPES = ("float32", "float16", "bfloat16")


def world_size_of(graph: PrimitiveIRGraph) -> int:
    """Ranks a plan talks about: one more than the largest rank named in it."""
    top = 0
    for node in graph.nodes.values():
        params = node.to_params()
        for key in ("source_rank", "target_rank"):
            if isinstance(params.get(key), int):
                top = max(top, params[key])
        for rank in params.get("source_ranks", ()):
            top = max(top, rank)
    return top + 1


def _dtype(graph: PrimitiveIRGraph) -> str:
    for node in graph.nodes.values():
        if node.tensor_info is not None:
            return _dtype_name(node.tensor_info.dtype)
    return "float32"


def _replace(graph: PrimitiveIRGraph, old_ids: Sequence[str], new: Optional[IRNodeVariant]) -> None:
    """Splice ``new`` in for the run ``old_ids`` (a dependency chain, first to last): it inherits
    the first node's dependencies and the last node's successors.  ``new=None`` removes the run
    and connects its surroundings directly."""
    first, last = graph.nodes[old_ids[0]], graph.nodes[old_ids[-1]]
    inside = set(old_ids)
    deps = [d for d in first.dependencies if d not in inside]
    succs = [s for s in last.next_ops if s not in inside]
    rebuilt: Dict[str, IRNodeVariant] = {}
    for nid, node in graph.nodes.items():          # keep plan order: the new node takes the first one's place
        if nid == old_ids[0] and new is not None:
            rebuilt[new.op_id] = new
        if nid not in inside:
            rebuilt[nid] = node
    graph.nodes.clear()
    graph.nodes.update(rebuilt)
    if new is not None:
        new.channel, new.device, new.tensor_info = first.channel, first.device, first.tensor_info
        new.dependencies, new.next_ops = list(deps), list(succs)
    for nid in deps:
        node = graph.nodes[nid]
        node.next_ops = [n for n in node.next_ops if n not in inside]
        for target in ([new.op_id] if new is not None else succs):
            if target not in node.next_ops:
                node.next_ops.append(target)
    for nid in succs:
        node = graph.nodes[nid]
        node.dependencies = [d for d in node.dependencies if d not in inside]
        for source in ([new.op_id] if new is not None else deps):
            if source not in node.dependencies:
                node.dependencies.append(source)
    graph._update_boundary_points()


def _single_successor(graph: PrimitiveIRGraph, node: IRNodeVariant) -> Optional[IRNodeVariant]:
    if len(node.next_ops) != 1:
        return None
    nxt = graph.nodes.get(node.next_ops[0])
    return nxt if nxt is not None and len(nxt.dependencies) == 1 else None


# ---- F1 ------------------------------------------------------------------------------------------

def reduce_chain_to_multi(graph: PrimitiveIRGraph, rank: int) -> int:
    """Chains ``self[X] = peer_a[X] (op) self[X]; self[X] = peer_b[X] (op) self[X]; ...``."""
    done = 0
    for start in list(graph.nodes.values()):
        if start.op_id not in graph.nodes or start.op_type not in _REDUCES:
            continue
        if not (start.src_offset == start.dst_offset == start.remote_offset):
            continue
        prev = [graph.nodes[d] for d in start.dependencies if d in graph.nodes]
        if len(prev) == 1 and prev[0].op_type in _REDUCES and len(prev[0].next_ops) == 1 \
                and (prev[0].src_offset, prev[0].count, prev[0].reduce_op) == (start.src_offset, start.count,
                                                                              start.reduce_op) \
                and prev[0].src_offset == prev[0].dst_offset == prev[0].remote_offset:
            continue                                   # not the head of its chain
        chain, sources = [start], [start.source_rank]
        while True:
            nxt = _single_successor(graph, chain[-1])
            if nxt is None or nxt.op_type not in _REDUCES or nxt.channel != start.channel:
                break
            if (nxt.src_offset, nxt.dst_offset, nxt.remote_offset, nxt.count, nxt.reduce_op) != \
                    (start.src_offset, start.dst_offset, start.remote_offset, start.count, start.reduce_op):
                break
            if nxt.source_rank in sources or nxt.source_rank == rank:
                break
            chain.append(nxt)
            sources.append(nxt.source_rank)
        if len(chain) < 2 or rank in sources:
            continue
        fused = SmReduceMultiNode(reduce_op=start.reduce_op, source_ranks=tuple([rank] + sources),
                                  dst_offset=start.dst_offset, remote_offset=start.remote_offset,
                                  count=start.count)
        _replace(graph, [n.op_id for n in chain], fused)
        done += 1
    return done


# ---- F2 ------------------------------------------------------------------------------------------

def reduce_multi_to_multimem(graph: PrimitiveIRGraph, rank: int, world: int, dtype: str) -> int:
    if dtype not in _MULTIMEM_DTYPES:
        return 0
    done = 0
    for node in list(graph.nodes.values()):
        if node.op_type != Op.SM_REDUCE_MULTI or set(node.source_ranks) != set(range(world)):
            continue
        if node.reduce_op == "avg" or (dtype == "float32" and node.reduce_op != "sum"):
            continue                                   # fp32 has an in-switch sum only
        fused = MultimemReduceNode(reduce_op=node.reduce_op, source_rank=rank, src_offset=node.remote_offset,
                                   dst_offset=node.dst_offset, remote_offset=node.remote_offset, count=node.count)
        _replace(graph, [node.op_id], fused)
        done += 1
    return done


# ---- F3 ------------------------------------------------------------------------------------------

def _skip_signals(graph: PrimitiveIRGraph, node: IRNodeVariant) -> Tuple[List[IRNodeVariant], Optional[IRNodeVariant]]:
    """The run of notify / wait nodes that follows ``node`` on its chain, and the node after it."""
    run: List[IRNodeVariant] = []
    cur = _single_successor(graph, node)
    while cur is not None and cur.op_type in _SIGNALS:
        run.append(cur)
        cur = _single_successor(graph, cur)
    return run, cur


def gather_to_multimem_store(graph: PrimitiveIRGraph, rank: int, world: int) -> int:
    """``reduce(mine); barrier; pull slice p from p for every other p`` -> ``...; store(mine)``."""
    done = 0
    for head in list(graph.nodes.values()):
        if head.op_id not in graph.nodes or head.op_type not in (Op.MULTIMEM_REDUCE, Op.SM_REDUCE_MULTI):
            continue
        if head.dst_offset != head.remote_offset:
            continue
        _, first_pull = _skip_signals(graph, head)
        pulls: List[IRNodeVariant] = []
        cur = first_pull
        while cur is not None and cur.op_type in _PULLS and cur.channel == head.channel \
                and cur.src_offset == cur.dst_offset and cur.size == head.count and cur.source_rank != rank:
            pulls.append(cur)
            cur = _single_successor(graph, cur)
        if len(pulls) != world - 1 or {p.source_rank for p in pulls} != set(range(world)) - {rank}:
            continue
        # The slices must be the W pieces of one contiguous span, piece r belonging to rank r.
        base = head.dst_offset - rank * head.count
        if any(p.src_offset != base + p.source_rank * head.count for p in pulls):
            continue
        store = MultimemStoreNode(source_rank=rank, src_offset=head.dst_offset, dst_offset=head.dst_offset,
                                  size=head.count)
        _replace(graph, [p.op_id for p in pulls], store)
        done += 1
    return done


def _is_all_pairs_barrier(run: Sequence[IRNodeVariant], rank: int, world: int) -> bool:
    """W-1 notifies of one id to every peer, then W-1 waits whose ids name their senders the same
    way: the shape every rank of a symmetric plan holds, so every rank may drop it together."""
    notifies = [n for n in run if n.op_type == Op.NOTIFY]
    waits = [n for n in run if n.op_type == Op.WAIT_NOTIFY]
    peers = set(range(world)) - {rank}
    if len(run) != 2 * (world - 1) or {n.target_rank for n in notifies} != peers \
            or {n.source_rank for n in waits} != peers:
        return False
    ids = {n.signal_id for n in notifies}
    if len(ids) != 1:
        return False
    base = ids.pop() - rank
    return all(w.signal_id == base + w.source_rank for w in waits)


# ---- F4 ------------------------------------------------------------------------------------------

def fuse_multimem_allreduce(graph: PrimitiveIRGraph, rank: int, world: int) -> int:
    done = 0
    for head in list(graph.nodes.values()):
        if head.op_id not in graph.nodes or head.op_type != Op.MULTIMEM_REDUCE:
            continue
        if not (head.dst_offset == head.remote_offset):
            continue
        signals, store = _skip_signals(graph, head)
        if store is None or store.op_type != Op.MULTIMEM_STORE:
            continue
        if signals and not _is_all_pairs_barrier(signals, rank, world):
            continue                                   # signals some other part of the plan may rely on
        if (store.src_offset, store.dst_offset, store.size) != (head.dst_offset, head.dst_offset, head.count):
            continue
        fused = MultimemAllreduceNode(reduce_op=head.reduce_op, offset=head.dst_offset, count=head.count)
        _replace(graph, [head.op_id] + [s.op_id for s in signals] + [store.op_id], fused)
        done += 1
    return done


# ---- driver ----------------------------------------------------------------------------------------

def _snapshot(graph: PrimitiveIRGraph):
    import copy
    return copy.deepcopy(graph.nodes), list(graph.entry_points), list(graph.exit_points)


def _restore(graph: PrimitiveIRGraph, saved) -> None:
    graph.nodes.clear()
    graph.nodes.update(saved[0])
    graph.entry_points, graph.exit_points = saved[1], saved[2]


def apply_fabric_rules(graph: PrimitiveIRGraph, profile: GpuProfile, topology: TopologyProfile,
                       rank: Optional[int] = None, world_size: Optional[int] = None) -> Dict[str, int]:
    """Apply F1-F4 in order, keeping each only if ``plan_cost`` goes down.  Returns how often each
    rule fired and stayed.  ``rank`` defaults to the rank this plan does not name as a peer."""
    if not getattr(topology, "uniform_all_to_all", False):
        return {}
    world = world_size or world_size_of(graph)
    if rank is None:
        named = set()
        for node in graph.nodes.values():
            params = node.to_params()
            if node.op_type in _SIGNALS:
                named.add(params.get("target_rank", params.get("source_rank")))
        candidates = sorted(set(range(world)) - named)
        rank = candidates[0] if candidates else 0
    dtype = _dtype(graph)
    elem = DTYPE_BYTES.get(dtype, 4)

    def cost() -> float:
        return plan_cost(graph, profile, topology, elem, world)

    steps: List[Tuple[str, Callable[[], int]]] = [("reduce_chain_to_multi", lambda: reduce_chain_to_multi(graph, rank))]
    if getattr(topology, "in_switch_reduction", False):
        steps += [("reduce_multi_to_multimem", lambda: reduce_multi_to_multimem(graph, rank, world, dtype)),
                  ("gather_to_multimem_store", lambda: gather_to_multimem_store(graph, rank, world)),
                  ("fuse_multimem_allreduce", lambda: fuse_multimem_allreduce(graph, rank, world))]
    fired: Dict[str, int] = {}
    # The multimem rules only pay as a group (the reduce alone moves W slices outbound for the one it
    # saves inbound), so they are priced together: keep all of them or none.
    before, saved = cost(), _snapshot(graph)
    n = steps[0][1]()
    if n and cost() <= before:
        fired[steps[0][0]] = n
    elif n:
        _restore(graph, saved)
    if len(steps) > 1:
        before, saved = cost(), _snapshot(graph)
        counts = {name: fn() for name, fn in steps[1:]}
        if any(counts.values()) and cost() < before:
            fired.update({k: v for k, v in counts.items() if v})
        elif any(counts.values()):
            _restore(graph, saved)
    return fired
