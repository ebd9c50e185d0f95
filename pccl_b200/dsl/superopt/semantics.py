"""Symbolic semantics of the plan primitives as z3 state transformers.

State: one z3 array per rank (32-bit element index -> 64-bit value) and a map
of posted signals.  Every primitive is modelled on a single representative
element of the region it touches (offset granularity), which is enough to
distinguish data-flow; reductions are an uninterpreted binary function made
commutative and associative by axioms (reference:
pccl/dsl/superopt/semantics.py:17-218).

z3 is required here; everything else in the package imports without it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

try:
    import z3
except ImportError as _err:  # pragma: no cover - exercised only without z3
    raise ImportError(
        "pccl.dsl.superopt.semantics needs the 'z3-solver' package; the DSL, compiler, "
        "algorithms and OCS layers work without it") from _err

from ..nodes import PrimitiveOpType as Op

_IDX = z3.BitVecSort(32)
_VAL = z3.BitVecSort(64)


@dataclass
class SymbolicState:
    bufs: Dict[int, "z3.ArrayRef"]
    signals: Dict[Tuple[int, int, int], "z3.BoolRef"] = field(default_factory=dict)
    constraints: List["z3.BoolRef"] = field(default_factory=list)

    def copy(self) -> "SymbolicState":
        return SymbolicState(dict(self.bufs), dict(self.signals), list(self.constraints))


_reduce_fn_cache: Dict[str, "z3.FuncDeclRef"] = {}


def _get_reduce_fn(reduce_op: str) -> "z3.FuncDeclRef":
    fn = _reduce_fn_cache.get(reduce_op)
    if fn is None:
        fn = _reduce_fn_cache[reduce_op] = z3.Function(f"reduce_{reduce_op}", _VAL, _VAL, _VAL)
    return fn


def get_reduce_axioms(reduce_op: str) -> List["z3.BoolRef"]:
    """Commutativity + associativity for sum/max/min; nothing for avg (which is
    sum followed by a scale and is not associative element-wise)."""
    if reduce_op not in ("sum", "max", "min"):
        return []
    f = _get_reduce_fn(reduce_op)
    a, b, c = (z3.BitVec(f"_ax_{n}", 64) for n in "abc")
    return [z3.ForAll([a, b], f(a, b) == f(b, a)),
            z3.ForAll([a, b, c], f(f(a, b), c) == f(a, f(b, c)))]


def make_initial_state(num_ranks: int = 2, prefix: str = "init") -> SymbolicState:
    return SymbolicState({r: z3.Array(f"{prefix}_buf_r{r}", _IDX, _VAL) for r in range(num_ranks)})


def _read_peer(state: SymbolicState, rank_expr, offset):
    """Value at ``offset`` in the buffer of a concrete or symbolic rank (2-rank model)."""
    if isinstance(rank_expr, int):
        return z3.Select(state.bufs[rank_expr], offset)
    return z3.If(rank_expr == z3.BitVecVal(0, 32),
                 z3.Select(state.bufs[0], offset), z3.Select(state.bufs[1], offset))


def _pull(state: SymbolicState, me: int, p: Dict) -> None:
    value = _read_peer(state, p["source_rank"], p["src_offset"])
    state.bufs[me] = z3.Store(state.bufs[me], p["dst_offset"], value)


def _reduce(state: SymbolicState, me: int, p: Dict) -> None:
    name = p.get("reduce_op", "sum")
    f = _get_reduce_fn(name if isinstance(name, str) else "sum")
    mine = z3.Select(state.bufs[me], p["dst_offset"])
    theirs = _read_peer(state, p["source_rank"], p["remote_offset"])
    state.bufs[me] = z3.Store(state.bufs[me], p["dst_offset"], f(mine, theirs))


def _push(state: SymbolicState, me: int, p: Dict) -> None:
    value = z3.Select(state.bufs[me], p["src_offset"])
    target, dst = p["target_rank"], p["dst_offset"]
    if isinstance(target, int):
        state.bufs[target] = z3.Store(state.bufs[target], dst, value)
        return
    for r in list(state.bufs):
        if r != me:
            state.bufs[r] = z3.If(target == z3.BitVecVal(r, 32),
                                  z3.Store(state.bufs[r], dst, value), state.bufs[r])


def _notify(state: SymbolicState, me: int, p: Dict) -> None:
    target, sig = p["target_rank"], p["signal_id"]
    if isinstance(target, int) and isinstance(sig, int):
        state.signals[(me, target, sig)] = z3.BoolVal(True)
    else:
        state.signals[(me, -1, -1)] = z3.Bool(f"sig_{me}_to_{target}_{sig}")


def _wait(state: SymbolicState, me: int, p: Dict) -> None:
    source, sig = p["source_rank"], p["signal_id"]
    if isinstance(source, int) and isinstance(sig, int):
        posted = state.signals.get((source, me, sig))
        # Waiting on a signal nobody posted is unsatisfiable (a deadlock).
        state.constraints.append(z3.BoolVal(False) if posted is None
                                 else posted == z3.BoolVal(True))


_ENCODERS = {
    Op.SM_COPY: _pull, Op.TMA_COPY: _pull, Op.CE_COPY: _pull, Op.MULTIMEM_STORE: _pull,
    Op.RDMA_READ: _pull,
    Op.SM_REDUCE: _reduce, Op.TMA_REDUCE: _reduce, Op.MULTIMEM_REDUCE: _reduce,
    Op.RDMA_WRITE: _push, Op.SM_PUT: _push,
    Op.NOTIFY: _notify, Op.WAIT_NOTIFY: _wait,
    Op.NOOP: lambda state, me, p: None,
}


def encode_op(op_type: Op, self_rank: int, params: Dict, state: SymbolicState) -> SymbolicState:
    """Return the state after ``self_rank`` executes one primitive."""
    try:
        apply = _ENCODERS[op_type]
    except KeyError:
        raise ValueError(f"Unknown op type: {op_type}") from None
    after = state.copy()
    apply(after, self_rank, params)
    return after


def encode_ordering(edges: List[Tuple[int, int]]) -> List["z3.BoolRef"]:
    """Happens-before constraints over integer timestamps ``t_i``."""
    stamps: Dict[int, "z3.ArithRef"] = {}
    out = []
    for src, dst in edges:
        for idx in (src, dst):
            stamps.setdefault(idx, z3.Int(f"t_{idx}"))
        out.append(stamps[src] < stamps[dst])
    out.extend(t >= 0 for t in stamps.values())
    return out
