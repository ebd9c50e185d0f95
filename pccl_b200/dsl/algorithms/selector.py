"""Choice of algorithm per (world size, message size, fabric, device).

``select_algorithm`` is a table lookup.  For the H100 / NVLink 4 profile it
reproduces the reference's rule (reference:
pccl/dsl/algorithms/selector.py:23-54): ring unless the world is a power of two
>= 4 and the message is under 1 MiB, then recursive halving-doubling.  For a
switched fabric (NVLink 5 + NVSwitch) the crossovers come from the B200 sweep:
one-shot for latency-bound sizes, two-shot in the middle, NVLS (or two-shot
when the fabric cannot reduce in-switch) for bandwidth-bound sizes.

``select_algorithm_cost_based`` builds every candidate's plan and prices its
critical path with the cost model (reference: selector.py:57-114).
"""

from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

from ..nodes import PrimitiveOpType
from ..superopt.cost_model import (GpuProfile, H100_PROFILE, NVLINK_TOPOLOGY, TopologyProfile,
                                   critical_path_cost, plan_cost)
from ..superopt.rule import PatternEdge, PatternNode
from .base import CollectiveAlgorithm, is_power_of_two
from .direct import NvlsAllreduce, OneShotAllreduce, TwoShotAllreduce
from .recursive_hd import RecursiveHalvingDoubling
from .ring import RingAllreduce
from .tree import TreeAllreduce

_is_power_of_2 = is_power_of_two

#: message-size crossovers (bytes) on a switched fabric, by world size, used when no tuning file
#: covers the world size: (one-shot up to, in-switch reduction from, in-switch reduction up to);
#: two-shot elsewhere.  With two ranks the in-switch all-reduce moves 1.5x the bytes of two-shot
#: per link direction and never wins; from four ranks on it moves fewer ((W+1)/W against 2(W-1)/W
#: of the message) and wins wherever bandwidth matters.
_NEVER = 1 << 62
SWITCHED_CROSSOVERS: Dict[int, tuple] = {
    2: (4 * 1024 * 1024, _NEVER, _NEVER),
    4: (2 * 1024 * 1024, 2 * 1024 * 1024, _NEVER),
    8: (128 * 1024, 4 * 1024 * 1024, _NEVER),
}


_PACKAGED_TUNING = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuning_b200.json")
_tuning_cache: Dict[str, dict] = {}


def tuning_path(path: Optional[str] = None) -> str:
    """Where measured choices are read from: the argument, ``PCCL_TUNING_FILE``,
    ``~/.pccl/tuning_b200.json`` if it exists, else the table shipped with the package
    (written by ``bench/collective_sweep.py --write-tuning`` on 8 x B200)."""
    if path:
        return path
    env = os.environ.get("PCCL_TUNING_FILE")
    if env:
        return env
    home = os.path.expanduser("~/.pccl/tuning_b200.json")
    return home if os.path.exists(home) else _PACKAGED_TUNING


def load_tuning(path: Optional[str] = None) -> dict:
    """The tuning document (cached per path); ``{}`` when there is none or it is unreadable."""
    path = tuning_path(path)
    if path not in _tuning_cache:
        try:
            with open(path) as handle:
                _tuning_cache[path] = json.load(handle)
        except (OSError, ValueError):
            _tuning_cache[path] = {}
    return _tuning_cache[path]


def clear_tuning_cache() -> None:
    _tuning_cache.clear()


def tuned_route(kind: str, world_size: int, data_bytes: int, path: Optional[str] = None) -> Optional[dict]:
    """The measured best way to run ``kind`` at this world size and message size, or ``None``.

    The tuning file holds, per collective and world size, break points sorted by size:
    ``{"routes": {"allreduce": {"8": [{"max_bytes": 524288, "algorithm": "ll"}, {"max_bytes": 33554432,
    "algorithm": "push"}, {"max_bytes": null, "algorithm": "nvls", "channels": 16}]}}}``; the first
    entry whose ``max_bytes`` covers the message applies (``null`` = no upper bound)."""
    table = load_tuning(path).get("routes", {}).get(kind, {}).get(str(world_size))
    if not table:
        return None
    for entry in table:
        limit = entry.get("max_bytes")
        if limit is None or data_bytes <= limit:
            return entry
    return table[-1]


def load_tuned_crossovers(path: Optional[str] = None) -> Dict[int, tuple]:
    """All-reduce crossovers ``{world: (one-shot up to, in-switch from, in-switch up to)}`` from the
    tuning file's ``allreduce_crossovers``, else the built-in table."""
    raw = load_tuning(path)
    return {int(k): tuple(v) for k, v in raw.get("allreduce_crossovers", {}).items()} or SWITCHED_CROSSOVERS


def select_algorithm(world_size: int, data_bytes: int,
                     topology: TopologyProfile = NVLINK_TOPOLOGY,
                     device: GpuProfile = H100_PROFILE) -> CollectiveAlgorithm:
    forced = os.environ.get("PCCL_ALGO")
    if forced:
        from . import ALGORITHMS
        if forced in ALGORITHMS:
            return ALGORITHMS[forced]()

    if getattr(topology, "uniform_all_to_all", False):
        from . import ALGORITHMS
        route = tuned_route("allreduce", world_size, data_bytes)
        if route is not None and route.get("plan_algorithm", route.get("algorithm")) in ALGORITHMS:
            name = route.get("plan_algorithm", route["algorithm"])
            if name not in ("nvls", "hybrid", "nvls_twopass") or topology.in_switch_reduction:
                return ALGORITHMS[name]()
        table = load_tuned_crossovers()
        nearest = min(table, key=lambda w: abs(w - world_size))
        entry = tuple(table[nearest])
        if len(entry) == 2:                      # older tuning files: (one-shot up to, two-shot up to)
            entry = (entry[0], entry[1], _NEVER)
        one_shot_max, nvls_from, nvls_to = entry
        if data_bytes <= one_shot_max:
            return OneShotAllreduce()
        if topology.in_switch_reduction and nvls_from < data_bytes <= nvls_to:
            return NvlsAllreduce()
        return TwoShotAllreduce()

    if not is_power_of_two(world_size) or world_size <= 2:
        return RingAllreduce()
    if data_bytes >= 1024 * 1024:
        return RingAllreduce()
    return RecursiveHalvingDoubling()


def _as_pattern(graph) -> tuple:
    index = {nid: i for i, nid in enumerate(graph.nodes)}
    nodes = [PatternNode(op_type=n.op_type or PrimitiveOpType.NOOP, rank=0, channel=n.channel)
             for n in graph.nodes.values()]
    edges = [PatternEdge(index[nid], index[nxt]) for nid, n in graph.nodes.items()
             for nxt in n.next_ops if nxt in index]
    return nodes, edges


def select_algorithm_cost_based(rank: int, world_size: int, tensor_size: int, data_bytes: int,
                                topology: TopologyProfile = NVLINK_TOPOLOGY,
                                device: GpuProfile = H100_PROFILE, dtype: str = "bfloat16",
                                executor: str = "tma") -> CollectiveAlgorithm:
    candidates: List[CollectiveAlgorithm] = [RingAllreduce()]
    if is_power_of_two(world_size) and world_size >= 2:
        candidates += [RecursiveHalvingDoubling(), TreeAllreduce()]
    if getattr(topology, "uniform_all_to_all", False) and tensor_size % world_size == 0:
        candidates += [OneShotAllreduce(), TwoShotAllreduce()]
        if topology.in_switch_reduction:
            candidates.append(NvlsAllreduce())
    if len(candidates) == 1:
        return candidates[0]

    switched = getattr(topology, "uniform_all_to_all", False)
    elem_bytes = max(1, data_bytes // max(1, tensor_size))
    best, best_cost = candidates[0], float("inf")
    for algorithm in candidates:
        try:
            native = algorithm.name in ("oneshot", "twoshot", "nvls")
            graph = algorithm.build_allreduce(rank=rank, world_size=world_size,
                                              tensor_size=tensor_size, dtype=dtype,
                                              executor="sm" if native else executor)
            if switched:
                # Whole-plan pricing, node by node, with fabric-aware signal costs.
                cost = plan_cost(graph, device, topology, elem_bytes, world_size)
            else:
                # The reference's pricing: every primitive at the full message size.
                cost = critical_path_cost(*_as_pattern(graph), device, data_bytes)
        except Exception:
            continue
        if cost < best_cost:
            best, best_cost = algorithm, cost
    return best
