"""``OCSPlan``: what an external switch controller hands the runtime for one barrier.

The runtime never computes topologies; it checks that every participant holds
the *same* plan before the next collective is released
(reference: pccl/ocs/plan.py:10-131).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, replace
from typing import Any, Dict, Iterable, Optional, Tuple

SUPPORTED_ALGORITHMS = {"ring", "rhd", "tree", "auto", "torch_native"}
SUPPORTED_BACKENDS = {"torch", "pccl"}
KNOWN_ROUTE_MODES = {"STATIC_PLAN", "ID_ROUTE", "SEGMENT_ROUTE", "USER_PLAN"}

#: fields every participant must agree on (participant set is compared as a bitmap)
_IDENTITY = ("job_id", "group_id", "barrier_id", "epoch_id", "next_epoch_id")
_ROUTING = ("topology_id", "route_mode", "route_plan_id", "algorithm", "backend")


def _time_us() -> int:
    return time.time_ns() // 1000


def _one_of(value: Any, allowed: set, what: str) -> str:
    if value.__class__ is str and value in allowed:       # the common case, without a conversion
        return value
    text = str(value)
    if text not in allowed:
        raise ValueError(f"unsupported {what} '{text}', expected one of {sorted(allowed)}")
    return text


@dataclass(frozen=True)
class OCSPlan:
    job_id: str = "default"
    group_id: int = 0
    barrier_id: int = 0
    epoch_id: int = 0
    next_epoch_id: int = 1
    participant_ranks: Tuple[int, ...] = ()
    topology_id: int = 0
    route_mode: str = "STATIC_PLAN"
    route_plan_id: int = 0
    algorithm: str = "torch_native"
    backend: str = "torch"
    payload: bytes = b""

    def __post_init__(self) -> None:
        put = lambda name, value: object.__setattr__(self, name, value)
        put("algorithm", _one_of(self.algorithm, SUPPORTED_ALGORITHMS, "OCS algorithm"))
        put("backend", _one_of(self.backend, SUPPORTED_BACKENDS, "OCS backend"))
        put("route_mode", _one_of(self.route_mode, KNOWN_ROUTE_MODES, "route_mode"))

        ranks = tuple(int(r) for r in self.participant_ranks)
        if ranks:
            if min(ranks) < 0:
                raise ValueError("participant_ranks must be non-negative")
            if len(set(ranks)) != len(ranks):
                raise ValueError("participant_ranks must not contain duplicates")
        put("participant_ranks", ranks)

        if self.payload is None:
            put("payload", b"")
        elif isinstance(self.payload, (bytes, bytearray, memoryview)):
            put("payload", bytes(self.payload))
        else:
            raise TypeError("payload must be bytes-like")

    @property
    def participant_bitmap(self) -> int:
        bits = 0
        for rank in self.participant_ranks:
            bits |= 1 << rank
        return bits

    def with_default_participants(self, world_size: int) -> "OCSPlan":
        """An empty participant list means "the whole group"."""
        if self.participant_ranks:
            return self
        # Every other field was validated when `self` was built: copy instead of re-validating.
        clone = object.__new__(OCSPlan)
        clone.__dict__.update(self.__dict__)
        clone.__dict__.pop("_consistency", None)
        object.__setattr__(clone, "participant_ranks", tuple(range(int(world_size))))
        return clone

    def consistency_fields(self) -> Dict[str, Any]:
        cached = self.__dict__.get("_consistency")       # the plan is immutable: computed once
        if cached is None:
            cached = {name: getattr(self, name) for name in _IDENTITY}
            cached["participant_bitmap"] = self.participant_bitmap
            cached.update((name, getattr(self, name)) for name in _ROUTING)
            object.__setattr__(self, "_consistency", cached)
        return dict(cached)

    def ready_record(self, src_rank: int, world_size: int, arrive_seq: int = 0,
                     arrival_time_us: Optional[int] = None) -> Dict[str, Any]:
        """The READY record this rank contributes to the barrier."""
        plan = self.with_default_participants(world_size)
        record: Dict[str, Any] = {
            "msg_type": "OCS_BARRIER_READY",
            "version": 1,
            "src_rank": int(src_rank),
            "src_gpu_id": int(src_rank),
            "arrive_seq": int(arrive_seq),
            "payload_len": len(plan.payload),
            "arrival_time_us": _time_us() if arrival_time_us is None else int(arrival_time_us),
        }
        record.update(plan.consistency_fields())
        return record


def normalize_plan_sequence(plans: Iterable[OCSPlan]) -> Tuple[OCSPlan, ...]:
    out = tuple(plans)
    if any(not isinstance(plan, OCSPlan) for plan in out):
        raise TypeError("all static plans must be OCSPlan instances")
    return out
