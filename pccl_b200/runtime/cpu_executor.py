"""CPU reference executor for version-2 plans — the correctness oracle.

Two front ends share one interpreter:

* ``simulate(plans, inputs)`` runs all ranks of a collective inside one process.
  Ranks are cooperative coroutines over their operation DAG: an operation runs
  once its dependencies ran, ``wait_notify`` blocks until the semaphore is
  positive, and a round in which no rank advances is reported as a deadlock
  together with each rank's blocked operations.
* ``GlooPlanExecutor`` replays the same plans across real processes over a
  ``gloo`` group.  Peer memory is not addressable between processes, so every
  rank first derives the *global schedule* with the in-process simulator (on
  dummy data; the schedule depends only on the plans) and then walks it in
  lock step: when the schedule says "rank r pulls from rank p", p sends the
  slice and r receives it.  Signals need no messages because the schedule
  already honours them.

Primitive semantics (element offsets into each rank's working buffer; they are
the engine's semantics, reference: csrc/plugins/cuda/channels/sm_channel.h:15-97
for the parameter mapping and csrc/engine_c.cc:468-548 for the I/O placement):

    copy        self[dst:dst+size]   = peer[source_rank][src:src+size]
    reduce      self[dst:dst+count]  = peer[source_rank][remote:+count] (op) self[src:+count]
    put/write   peer[target_rank][dst:dst+size] = self[src:src+size]
    reduce_multi self[dst:+count]    = (op) over r in source_ranks of buf[r][remote:+count]
    multimem.reduce self[dst:+count] = (op) over all ranks r of buf[r][remote:+count]
    multimem.store  buf[r][dst:+size] = self[src:+size] for every rank r
    multimem.allreduce buf[r][off:+count] = (op) over all ranks s of buf[s][off:+count], for every r
    notify      signals[target_rank][signal_id] += 1
    wait_notify block until signals[self][signal_id] > 0, then -= 1

``avg`` is carried as ``sum`` through the primitives and applied once, as a
division by the world size, when the output is copied out.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch

Plan = Dict[str, Any]

_PULL = {"sm.copy", "tma.copy", "ce.copy", "rdma.read"}
_REDUCE = {"sm.reduce", "tma.reduce"}
_PUSH = {"sm.put", "rdma.write"}

_TORCH_DTYPE = {
    "float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
    "float8_e4m3": getattr(torch, "float8_e4m3fn", None),
    "float8_e5m2": getattr(torch, "float8_e5m2", None),
}


class PlanDeadlock(RuntimeError):
    """No rank can make progress; the message lists what each rank waits for."""


def _as_plan(plan: Union[str, Plan]) -> Plan:
    plan = json.loads(plan) if isinstance(plan, str) else plan
    if "operations" not in plan:
        raise ValueError("not a version-2 device plan: no top-level 'operations'")
    return plan


def _combine(kind: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if kind in ("sum", "avg"):
        return a + b
    if kind == "max":
        return torch.maximum(a, b)
    if kind == "min":
        return torch.minimum(a, b)
    raise ValueError(f"unknown reduce_op '{kind}'")


def plan_numel(plan: Plan) -> int:
    total = 1
    for extent in plan["tensor_info"]["shape"]:
        total *= extent
    return total


def plan_uses_avg(plan: Plan) -> bool:
    return any(op.get("params", {}).get("reduce_op") == "avg" for op in plan["operations"])


# ---------------------------------------------------------------------------
# I/O placement per collective type
# ---------------------------------------------------------------------------

def place_input(kind: str, buf: torch.Tensor, x: torch.Tensor, rank: int, world: int, n: int) -> None:
    flat = x.reshape(-1)
    if kind == "allgather":
        shard = n // world
        buf[rank * shard:rank * shard + flat.numel()] = flat[:shard] if flat.numel() > shard else flat
    else:
        buf[:flat.numel()] = flat


def take_output(kind: str, buf: torch.Tensor, rank: int, world: int, n: int) -> torch.Tensor:
    if kind == "reduce_scatter":
        shard = n // world
        return buf[rank * shard:(rank + 1) * shard].clone()
    if kind == "alltoall":
        chunk = n // world
        out = torch.empty(n, dtype=buf.dtype)
        for p in range(world):
            src = rank * chunk if p == rank else n + p * chunk
            out[p * chunk:(p + 1) * chunk] = buf[src:src + chunk]
        return out
    return buf[:n].clone()


# ---------------------------------------------------------------------------
# The interpreter
# ---------------------------------------------------------------------------

@dataclass
class _Rank:
    ops: List[Dict[str, Any]]
    missing: List[int]                    # unmet dependency count per op
    done: List[bool]
    signals: Dict[int, int] = field(default_factory=dict)
    ready: List[int] = field(default_factory=list)


Transfer = Callable[[int, int, int, int], torch.Tensor]


class _World:
    """State of all ranks plus the rules for running one operation."""

    def __init__(self, plans: Sequence[Plan], buffers: Sequence[torch.Tensor],
                 accumulate: torch.dtype):
        self.world = len(plans)
        self.buffers = list(buffers)
        self.accumulate = accumulate
        self.ranks: List[_Rank] = []
        for plan in plans:
            ops = plan["operations"]
            missing = [len(op.get("dependencies", [])) for op in ops]
            rank = _Rank(ops=ops, missing=missing, done=[False] * len(ops))
            rank.ready = [i for i, m in enumerate(missing) if m == 0]
            self.ranks.append(rank)
        self.trace: List[Tuple[int, int]] = []

    # data access -----------------------------------------------------------
    def _read(self, rank: int, off: int, count: int) -> torch.Tensor:
        return self.buffers[rank][off:off + count]

    def _check(self, rank: int, off: int, count: int, what: str) -> None:
        size = self.buffers[rank].numel()
        if off < 0 or count < 0 or off + count > size:
            raise IndexError(f"{what}: range [{off}, {off + count}) outside rank {rank}'s "
                             f"buffer of {size} elements")

    def _peer(self, value: int, what: str) -> int:
        if not 0 <= value < self.world:
            raise IndexError(f"{what}: rank {value} outside world of {self.world}")
        return value

    def _fold(self, kind: str, parts: List[torch.Tensor], like: torch.Tensor) -> torch.Tensor:
        acc = parts[0].to(self.accumulate)
        for part in parts[1:]:
            acc = _combine(kind, acc, part.to(self.accumulate))
        return acc.to(like.dtype)

    # one operation -----------------------------------------------------------
    def blocked(self, r: int, op: Dict[str, Any]) -> bool:
        if op["primitive"] != "wait_notify":
            return False
        return self.ranks[r].signals.get(op["params"]["signal_id"], 0) <= 0

    def run(self, r: int, op: Dict[str, Any]) -> None:
        name, p = op["primitive"], op.get("params", {})
        tag = f"rank {r} op {op.get('index')} {name}"
        me = self.buffers[r]
        if name in _PULL:
            src = self._peer(p["source_rank"], tag)
            self._check(src, p["src_offset"], p["size"], tag)
            self._check(r, p["dst_offset"], p["size"], tag)
            me[p["dst_offset"]:p["dst_offset"] + p["size"]] = \
                self._read(src, p["src_offset"], p["size"]).clone()
        elif name in _REDUCE:
            src = self._peer(p["source_rank"], tag)
            n = p["count"]
            self._check(src, p["remote_offset"], n, tag)
            self._check(r, p["src_offset"], n, tag)
            self._check(r, p["dst_offset"], n, tag)
            parts = [self._read(src, p["remote_offset"], n), self._read(r, p["src_offset"], n)]
            me[p["dst_offset"]:p["dst_offset"] + n] = self._fold(p.get("reduce_op", "sum"), parts, me)
        elif name in _PUSH:
            dst = self._peer(p["target_rank"], tag)
            self._check(r, p["src_offset"], p["size"], tag)
            self._check(dst, p["dst_offset"], p["size"], tag)
            self.buffers[dst][p["dst_offset"]:p["dst_offset"] + p["size"]] = \
                self._read(r, p["src_offset"], p["size"]).clone()
        elif name in ("sm.reduce_multi", "multimem.reduce"):
            sources = p["source_ranks"] if name == "sm.reduce_multi" else list(range(self.world))
            n = p["count"]
            parts = []
            for s in sources:
                self._check(self._peer(s, tag), p["remote_offset"], n, tag)
                parts.append(self._read(s, p["remote_offset"], n))
            self._check(r, p["dst_offset"], n, tag)
            me[p["dst_offset"]:p["dst_offset"] + n] = self._fold(p.get("reduce_op", "sum"), parts, me)
        elif name == "multimem.store":
            self._check(r, p["src_offset"], p["size"], tag)
            value = self._read(r, p["src_offset"], p["size"]).clone()
            for dst in range(self.world):
                self._check(dst, p["dst_offset"], p["size"], tag)
                self.buffers[dst][p["dst_offset"]:p["dst_offset"] + p["size"]] = value
        elif name == "multimem.allreduce":
            n, off = p["count"], p["offset"]
            for s in range(self.world):
                self._check(s, off, n, tag)
            value = self._fold(p.get("reduce_op", "sum"), [self._read(s, off, n) for s in range(self.world)], me)
            for dst in range(self.world):
                self.buffers[dst][off:off + n] = value
        elif name == "notify":
            target = self.ranks[self._peer(p["target_rank"], tag)]
            target.signals[p["signal_id"]] = target.signals.get(p["signal_id"], 0) + 1
        elif name == "wait_notify":
            self.ranks[r].signals[p["signal_id"]] -= 1
        elif name == "noop":
            pass
        else:
            raise ValueError(f"{tag}: primitive not executable on the CPU executor")

    # scheduling ----------------------------------------------------------------
    def run_to_completion(self) -> None:
        while True:
            progressed = False
            for r, rank in enumerate(self.ranks):
                while True:
                    runnable = next((i for i in rank.ready if not self.blocked(r, rank.ops[i])), None)
                    if runnable is None:
                        break
                    rank.ready.remove(runnable)
                    op = rank.ops[runnable]
                    self.run(r, op)
                    self.trace.append((r, runnable))
                    rank.done[runnable] = True
                    for nxt in op.get("next_ops", []):
                        rank.missing[nxt] -= 1
                        if rank.missing[nxt] == 0:
                            rank.ready.append(nxt)
                    rank.ready.sort()
                    progressed = True
            if all(all(rank.done) for rank in self.ranks):
                return
            if not progressed:
                stuck = {r: [(i, rank.ops[i]["primitive"], rank.ops[i].get("params"))
                             for i in rank.ready] for r, rank in enumerate(self.ranks)
                         if not all(rank.done)}
                raise PlanDeadlock(f"no rank can progress; blocked operations: {stuck}")

    def leftover_signals(self) -> Dict[int, Dict[int, int]]:
        return {r: {k: v for k, v in rank.signals.items() if v}
                for r, rank in enumerate(self.ranks) if any(rank.signals.values())}


def _accumulate_dtype(dtype: torch.dtype, exact: bool) -> torch.dtype:
    if exact:
        return torch.float64
    return torch.float32 if dtype in (torch.float16, torch.bfloat16) or dtype.itemsize == 1 else dtype


def simulate(plans: Sequence[Union[str, Plan]], inputs: Sequence[torch.Tensor],
             buffer_elems: Optional[int] = None, exact: bool = False,
             return_world: bool = False):
    """Run every rank's plan in-process and return each rank's output tensor.

    ``inputs[r]`` is rank r's input (full tensor, or its shard for allgather).
    ``exact=True`` keeps the working buffers in float64 — use it to obtain a
    reference value rather than to mimic device rounding.
    """
    plans = [_as_plan(p) for p in plans]
    world = len(plans)
    if len(inputs) != world:
        raise ValueError(f"{world} plans but {len(inputs)} inputs")
    kind = plans[0].get("collective_type", "")
    n = plan_numel(plans[0])
    dtype = torch.float64 if exact else inputs[0].dtype
    size = buffer_elems or 2 * n
    buffers = [torch.zeros(size, dtype=dtype) for _ in range(world)]
    for r, x in enumerate(inputs):
        place_input(kind, buffers[r], x.to(dtype), r, world, n)
    sim = _World(plans, buffers, _accumulate_dtype(dtype, exact))
    sim.run_to_completion()
    scale = world if plan_uses_avg(plans[0]) else 1
    outputs = []
    for r in range(world):
        out = take_output(kind, buffers[r], r, world, n)
        if scale != 1:
            out = (out.to(sim.accumulate) / scale).to(out.dtype)
        outputs.append(out.to(inputs[r].dtype) if not exact else out)
    return (outputs, sim) if return_world else outputs


def global_schedule(plans: Sequence[Union[str, Plan]]) -> List[Tuple[int, int]]:
    """A valid interleaving ``[(rank, op index), ...]`` of all ranks' plans."""
    plans = [_as_plan(p) for p in plans]
    n = plan_numel(plans[0])
    sim = _World(plans, [torch.zeros(2 * n, dtype=torch.float32) for _ in plans], torch.float32)
    sim.run_to_completion()
    return sim.trace


class GlooPlanExecutor:
    """Replay plans across the processes of a (CPU) ``torch.distributed`` group.

    The plans may describe more ranks than the group has processes: with W
    plans on G processes, process g hosts the W/G consecutive plan ranks
    ``[g*W/G, (g+1)*W/G)`` — an 8-rank plan can be replayed on two processes.
    """

    def __init__(self, group=None):
        import torch.distributed as dist
        self._dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def hosted_ranks(self, plan_world: int) -> List[int]:
        if plan_world % self.world:
            raise ValueError(f"{plan_world} plan ranks do not divide over {self.world} processes")
        per = plan_world // self.world
        return list(range(self.rank * per, (self.rank + 1) * per))

    def _fetch(self, owner: int, off: int, count: int, reader: int, per: int,
               bufs: Dict[int, torch.Tensor]) -> Optional[torch.Tensor]:
        """Slice ``[off, off+count)`` of plan rank ``owner``'s buffer, delivered
        to the process hosting plan rank ``reader`` (None on other processes)."""
        dist = self._dist
        src_proc, dst_proc = owner // per, reader // per
        if src_proc == dst_proc:
            return bufs[owner][off:off + count].clone() if self.rank == dst_proc else None
        if self.rank == src_proc:
            dist.send(bufs[owner][off:off + count].contiguous(), dst=dst_proc, group=self.group)
            return None
        if self.rank == dst_proc:
            box = torch.empty(count, dtype=next(iter(bufs.values())).dtype)
            dist.recv(box, src=src_proc, group=self.group)
            return box
        return None

    def execute(self, plans: Sequence[Union[str, Plan]],
                inputs: Union[torch.Tensor, Dict[int, torch.Tensor]]) -> Union[torch.Tensor, Dict[int, torch.Tensor]]:
        """``plans`` are all plan ranks' plans (every process passes the same
        list); ``inputs`` maps each hosted plan rank to its input (or is a single
        tensor when one rank is hosted).  Returns outputs in the same form."""
        plans = [_as_plan(p) for p in plans]
        hosted = self.hosted_ranks(len(plans))
        per = len(hosted)
        single = isinstance(inputs, torch.Tensor)
        if single:
            inputs = {hosted[0]: inputs}
        world = len(plans)
        kind = plans[0].get("collective_type", "")
        n = plan_numel(plans[0])
        dtype = next(iter(inputs.values())).dtype
        acc = _accumulate_dtype(dtype, False)
        bufs = {v: torch.zeros(2 * n, dtype=dtype) for v in hosted}
        for v in hosted:
            place_input(kind, bufs[v], inputs[v], v, world, n)

        def put(v: int, off: int, value: torch.Tensor) -> None:
            bufs[v][off:off + value.numel()] = value.to(dtype)

        for r, index in global_schedule(plans):
            op = plans[r]["operations"][index]
            name, p = op["primitive"], op.get("params", {})
            here = r in bufs
            if name in _PULL:
                got = self._fetch(p["source_rank"], p["src_offset"], p["size"], r, per, bufs)
                if here:
                    put(r, p["dst_offset"], got)
            elif name in _REDUCE:
                got = self._fetch(p["source_rank"], p["remote_offset"], p["count"], r, per, bufs)
                if here:
                    local = bufs[r][p["src_offset"]:p["src_offset"] + p["count"]]
                    put(r, p["dst_offset"],
                        _combine(p.get("reduce_op", "sum"), got.to(acc), local.to(acc)))
            elif name in _PUSH:
                # A push is a pull seen from the other side.
                got = self._fetch(r, p["src_offset"], p["size"], p["target_rank"], per, bufs)
                if p["target_rank"] in bufs:
                    put(p["target_rank"], p["dst_offset"], got)
            elif name in ("sm.reduce_multi", "multimem.reduce"):
                sources = p["source_ranks"] if name == "sm.reduce_multi" else range(world)
                total = None
                for s in sources:
                    got = self._fetch(s, p["remote_offset"], p["count"], r, per, bufs)
                    if here:
                        total = got.to(acc) if total is None else _combine(
                            p.get("reduce_op", "sum"), total, got.to(acc))
                if here:
                    put(r, p["dst_offset"], total)
            elif name == "multimem.store":
                for dst in range(world):
                    got = self._fetch(r, p["src_offset"], p["size"], dst, per, bufs)
                    if dst in bufs:
                        put(dst, p["dst_offset"], got)
            elif name == "multimem.allreduce":
                total = None
                for s in range(world):
                    got = self._fetch(s, p["offset"], p["count"], r, per, bufs)
                    if here:
                        total = got.to(acc) if total is None else _combine(
                            p.get("reduce_op", "sum"), total, got.to(acc))
                if here:
                    put(r, p["offset"], total)
                for dst in range(world):
                    if dst == r:
                        continue
                    got = self._fetch(r, p["offset"], p["count"], dst, per, bufs)
                    if dst in bufs:
                        put(dst, p["offset"], got)
            # notify / wait_notify / noop: ordering is already in the schedule

        outputs = {}
        for v in hosted:
            out = take_output(kind, bufs[v], v, world, n)
            if plan_uses_avg(plans[0]):
                out = (out.to(acc) / world).to(out.dtype)
            outputs[v] = out
        return outputs[hosted[0]] if single else outputs
