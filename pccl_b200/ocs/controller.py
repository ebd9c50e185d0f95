"""Plan providers: the northbound side of the OCS runtime
(reference: pccl/ocs/controller.py:14-71)."""

from __future__ import annotations

from dataclasses import replace
from itertools import count
from typing import Dict, Iterable, Mapping, Optional, Protocol, Tuple, Union, runtime_checkable

from .plan import OCSPlan, normalize_plan_sequence

PlanInput = Union[Iterable[OCSPlan], Mapping[str, Iterable[OCSPlan]]]


@runtime_checkable
class OCSPlanController(Protocol):
    def next_plan(self, event_key: str, rank: int, world_size: int) -> OCSPlan:
        """The precomputed plan for the next occurrence of ``event_key``."""


class StaticPlanController:
    """Replays fixed plan lists, one list per event key, cyclically.

    A bare iterable is filed under ``"all_reduce"``.  Events without a list get
    a synthesized plan whose barrier / epoch ids count occurrences.
    """

    def __init__(self, plans: Optional[PlanInput] = None,
                 default_algorithm: str = "torch_native", default_backend: str = "torch") -> None:
        self.default_algorithm = default_algorithm
        self.default_backend = default_backend
        self._plans: Dict[str, Tuple[OCSPlan, ...]] = {}
        self._cursors: Dict[str, "count[int]"] = {}
        if plans is None:
            return
        if isinstance(plans, Mapping):
            for key, sequence in plans.items():
                self._plans[str(key)] = normalize_plan_sequence(sequence)
        else:
            self._plans["all_reduce"] = normalize_plan_sequence(plans)

    def next_plan(self, event_key: str, rank: int, world_size: int) -> OCSPlan:
        event = str(event_key)
        occurrence = next(self._cursors.setdefault(event, count()))
        listed = self._plans.get(event)
        if listed:
            plan = listed[occurrence % len(listed)]
        else:
            plan = OCSPlan(barrier_id=occurrence, epoch_id=occurrence,
                           next_epoch_id=occurrence + 1,
                           participant_ranks=tuple(range(int(world_size))),
                           algorithm=self.default_algorithm, backend=self.default_backend)
        return replace(plan.with_default_participants(world_size))
