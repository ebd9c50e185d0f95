"""Equivalence checking of two skeletons (2-rank model, rank 0 executes).

Pipeline per candidate pair: cheap signature filter -> concrete simulation on
integer-tagged slots for several chunk geometries -> bit-vector proof over named
slots with z3 (no arrays, no quantifiers).  A pair that survives all three
becomes a ``RewriteRule`` (reference: pccl/dsl/superopt/verifier.py:52-331).
"""

from __future__ import annotations

import hashlib
import uuid
from collections import defaultdict
from typing import Dict, List, Optional, Sequence, Tuple

from ..nodes import PrimitiveOpType as Op
from .rule import PatternEdge, PatternNode, RewriteRule

_COPY_LIKE = frozenset({Op.SM_COPY, Op.TMA_COPY, Op.CE_COPY, Op.MULTIMEM_STORE, Op.RDMA_READ})
_REDUCE_LIKE = frozenset({Op.SM_REDUCE, Op.TMA_REDUCE, Op.MULTIMEM_REDUCE})
_WRITE_REMOTE = frozenset({Op.RDMA_WRITE, Op.SM_PUT})
_SYNC_OPS = frozenset({Op.NOTIFY, Op.WAIT_NOTIFY, Op.NOOP})

_PULL_PARAMS = ["source_rank", "src_offset", "dst_offset", "size"]
_REDUCE_PARAMS = ["source_rank", "src_offset", "dst_offset", "remote_offset", "reduce_op", "count"]
_OP_PARAM_TEMPLATES: Dict[Op, List[str]] = {
    **{op: _PULL_PARAMS for op in _COPY_LIKE},
    **{op: _REDUCE_PARAMS for op in _REDUCE_LIKE},
    Op.RDMA_WRITE: ["target_rank", "src_offset", "dst_offset", "size"],
    Op.SM_PUT: ["target_rank", "src_offset", "dst_offset", "size"],
    Op.NOTIFY: ["target_rank", "signal_id"],
    Op.WAIT_NOTIFY: ["source_rank", "signal_id"],
    Op.NOOP: [],
}

NUM_SLOTS = 32
#: (chunk_size, base_offset) geometries the concrete filter runs
_TEST_PARAM_SETS = [
    {"chunk_size": 4096, "base_off": 0},
    {"chunk_size": 8192, "base_off": 0},
    {"chunk_size": 4096, "base_off": 4096},
    {"chunk_size": 1024, "base_off": 0},
    {"chunk_size": 16384, "base_off": 8192},
]


def _topo_sort(num_nodes: int, edges: Sequence[PatternEdge]) -> Optional[List[int]]:
    """FIFO Kahn order, or None if the edges contain a cycle."""
    outs = defaultdict(list)
    indeg = [0] * num_nodes
    for e in edges:
        outs[e.src_idx].append(e.dst_idx)
        indeg[e.dst_idx] += 1
    queue = [i for i in range(num_nodes) if indeg[i] == 0]
    head = 0
    while head < len(queue):
        for nxt in outs[queue[head]]:
            indeg[nxt] -= 1
            if indeg[nxt] == 0:
                queue.append(nxt)
        head += 1
    return queue if len(queue) == num_nodes else None


def _make_concrete_params(node: PatternNode, chunk_size: int, base_off: int) -> dict:
    off = base_off + node.chunk_id * chunk_size
    op = node.op_type
    if op in _COPY_LIKE:
        return {"source_rank": 1, "src_offset": off, "dst_offset": off, "size": chunk_size}
    if op in _REDUCE_LIKE:
        return {"source_rank": 1, "src_offset": off, "dst_offset": off, "remote_offset": off,
                "reduce_op": "sum", "count": chunk_size}
    if op in _WRITE_REMOTE:
        return {"target_rank": 1, "src_offset": off, "dst_offset": off, "size": chunk_size}
    if op == Op.NOTIFY:
        return {"target_rank": 1, "signal_id": node.chunk_id}
    if op == Op.WAIT_NOTIFY:
        return {"source_rank": 1, "signal_id": node.chunk_id}
    return {}


def _simulate(nodes: Sequence[PatternNode], edges: Sequence[PatternEdge],
              chunk_size: int, base_off: int) -> Optional[Tuple[list, list]]:
    """Run the skeleton on two 32-slot buffers of distinct integer tags."""
    order = _topo_sort(len(nodes), edges)
    if order is None:
        return None
    buf = {0: list(range(NUM_SLOTS)), 1: list(range(NUM_SLOTS, 2 * NUM_SLOTS))}
    for idx in order:
        node = nodes[idx]
        me, peer = node.rank, 1
        slot = (base_off + node.chunk_id * chunk_size) % NUM_SLOTS
        if node.op_type in _COPY_LIKE:
            buf[me][slot] = buf[peer][slot]
        elif node.op_type in _REDUCE_LIKE:
            buf[me][slot] = buf[me][slot] + buf[peer][slot]
        elif node.op_type in _WRITE_REMOTE:
            buf[peer][slot] = buf[me][slot]
    return buf[0], buf[1]


def concrete_simulation_match(src_nodes, src_edges, repl_nodes, repl_edges) -> bool:
    for geometry in _TEST_PARAM_SETS:
        a = _simulate(src_nodes, src_edges, geometry["chunk_size"], geometry["base_off"])
        b = _simulate(repl_nodes, repl_edges, geometry["chunk_size"], geometry["base_off"])
        if a is None or b is None or a != b:
            return False
    return True


def concrete_fingerprint(nodes, edges) -> Optional[str]:
    outcome = _simulate(nodes, edges, 4096, 0)
    return None if outcome is None else hashlib.md5(str(outcome).encode()).hexdigest()


def _count(nodes: Sequence[PatternNode], family) -> int:
    return sum(1 for n in nodes if n.op_type in family)


def signatures_compatible(src_nodes: Sequence[PatternNode],
                          repl_nodes: Sequence[PatternNode]) -> bool:
    """Necessary conditions for equivalence that cost nothing to test."""
    if _count(src_nodes, _REDUCE_LIKE) != _count(repl_nodes, _REDUCE_LIKE):
        return False
    if len({n.chunk_id for n in src_nodes}) != len({n.chunk_id for n in repl_nodes}):
        return False
    if bool(_count(src_nodes, _WRITE_REMOTE)) != bool(_count(repl_nodes, _WRITE_REMOTE)):
        return False
    if all(n.op_type in _SYNC_OPS for n in src_nodes) or \
            all(n.op_type in _SYNC_OPS for n in repl_nodes):
        return False
    both_multi = (len({n.channel for n in src_nodes}) > 1
                  and len({n.channel for n in repl_nodes}) > 1)
    if both_multi and _count(src_nodes, _COPY_LIKE) != _count(repl_nodes, _COPY_LIKE):
        return False
    return True


# -- z3 slot proof ------------------------------------------------------------

def _slot_for_chunk(chunk_id: int) -> int:
    return chunk_id % NUM_SLOTS


def _slot_based_check(src_nodes, src_edges, repl_nodes, repl_edges, timeout: float = 2.0) -> bool:
    """Prove both skeletons leave every (rank, slot) with the same 64-bit value
    for all initial contents (addition is bit-vector addition)."""
    try:
        import z3
    except ImportError as err:  # pragma: no cover
        raise ImportError("rule verification needs the 'z3-solver' package") from err

    orders = (_topo_sort(len(src_nodes), src_edges), _topo_sort(len(repl_nodes), repl_edges))
    if orders[0] is None or orders[1] is None:
        return False
    chunks = {n.chunk_id for n in (*src_nodes, *repl_nodes)}
    initial = {(r, _slot_for_chunk(c)): z3.BitVec(f"init_r{r}_s{_slot_for_chunk(c)}", 64)
               for r in range(2) for c in range(max(chunks, default=0) + 1)}
    zero = z3.BitVecVal(0, 64)

    def run(nodes, order):
        state = dict(initial)
        for idx in order:
            node = nodes[idx]
            me, peer, slot = node.rank, 1 - node.rank, _slot_for_chunk(node.chunk_id)
            if node.op_type in _COPY_LIKE:
                state[(me, slot)] = state.get((peer, slot), zero)
            elif node.op_type in _REDUCE_LIKE:
                state[(me, slot)] = state.get((me, slot), zero) + state.get((peer, slot), zero)
            elif node.op_type in _WRITE_REMOTE:
                state[(peer, slot)] = state.get((me, slot), zero)
        return state

    left, right = run(src_nodes, orders[0]), run(repl_nodes, orders[1])
    differs = [left.get(k, initial.get(k, zero)) != right.get(k, initial.get(k, zero))
               for k in set(left) | set(right)]
    if not differs:
        return True
    solver = z3.Solver()
    solver.set("timeout", int(timeout * 1000))
    solver.add(z3.Or(*differs))
    return solver.check() == z3.unsat


def _is_trivially_identical(src_nodes, src_edges, repl_nodes, repl_edges) -> bool:
    if len(src_nodes) != len(repl_nodes) or len(src_edges) != len(repl_edges):
        return False
    key = lambda n: (n.op_type, n.rank, n.chunk_id, n.channel)
    if any(key(a) != key(b) for a, b in zip(src_nodes, repl_nodes)):
        return False
    pairs = lambda es: {(e.src_idx, e.dst_idx) for e in es}
    return pairs(src_edges) == pairs(repl_edges)


def check_equivalence(src_nodes: List[PatternNode], src_edges: List[PatternEdge],
                      repl_nodes: List[PatternNode], repl_edges: List[PatternEdge],
                      timeout: float = 2.0) -> Optional[RewriteRule]:
    """A ``RewriteRule`` if the two skeletons are provably equivalent and not
    the same skeleton, else None."""
    if _is_trivially_identical(src_nodes, src_edges, repl_nodes, repl_edges):
        return None
    if not concrete_simulation_match(src_nodes, src_edges, repl_nodes, repl_edges):
        return None
    if not _slot_based_check(src_nodes, src_edges, repl_nodes, repl_edges, timeout):
        return None
    return RewriteRule(source_nodes=src_nodes, source_edges=src_edges,
                       replacement_nodes=repl_nodes, replacement_edges=repl_edges,
                       param_constraints=[], rule_id=f"rule_{uuid.uuid4().hex[:8]}")
