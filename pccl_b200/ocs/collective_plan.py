"""Sequences of *different* collectives separated by OCS barriers.

Where ``OcsPhaseRunner`` cuts one graph, a collective plan strings together
independently built graphs (each with its own ``collective_type``), e.g.
all-reduce on topology 1, all-to-all on topology 2, all-reduce again
(reference: pccl/ocs/collective_plan.py:23-253).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..dsl.algorithms import RingAllreduce
from ..dsl.codegen import RuntimeGraphGenerator
from ..dsl.compiler import Compiler
from ..dsl.graph import PrimitiveIRGraph
from ._phases import EngineBackedRunner, discard_dir
from .plan import OCSPlan
from .runtime import OCSRuntime


def _check_barrier_layout(phases, what: str) -> None:
    """Every phase but the last is followed by a barrier; the last is not."""
    if not phases:
        raise ValueError(f"{what} plan must contain at least one phase")
    if phases[-1].barrier_after is not None:
        raise ValueError(f"the final {what} phase must not have a following barrier")
    if any(phase.barrier_after is None for phase in phases[:-1]):
        raise ValueError(f"every non-final {what} phase requires an OCS barrier")


@dataclass(frozen=True)
class OCSCollectivePhase:
    name: str
    graph: PrimitiveIRGraph
    barrier_after: Optional[OCSPlan] = None

    def __post_init__(self) -> None:
        if not self.name:
            raise ValueError("OCS collective phase name must not be empty")
        if self.graph.has_ocs_barriers():
            raise ValueError("an OCS collective phase must not contain an OCS barrier node")
        if not self.graph.collective_type:
            raise ValueError("an OCS collective phase must declare collective_type")


@dataclass(frozen=True)
class OCSCollectivePlan:
    phases: Tuple[OCSCollectivePhase, ...]

    def __post_init__(self) -> None:
        _check_barrier_layout(self.phases, "collective")


@dataclass
class PreparedOcsCollectivePlan:
    operation_names: Tuple[str, ...]
    phase_files: Tuple[Path, ...]
    barriers_after_phase: Tuple[Optional[OCSPlan], ...]
    collective_types: Tuple[str, ...]
    json_dir: Path
    owns_json_dir: bool
    closed: bool = False

    def close(self) -> None:
        if not self.closed:
            discard_dir(self.json_dir, self.owns_json_dir)
        self.closed = True


class OcsCollectivePlanRunner(EngineBackedRunner):
    _tmp_prefix = "pccl-ocs-plan-"

    def __init__(self, engine: Any = None, runtime: Optional[OCSRuntime] = None,
                 compiler: Optional[Compiler] = None, json_dir: Optional[str] = None) -> None:
        super().__init__(engine, runtime, compiler, json_dir)

    def prepare(self, plan: OCSCollectivePlan,
                operation_name: str = "ocs_collective_plan") -> PreparedOcsCollectivePlan:
        """Compile every phase to its own version-2 plan file (registration
        happens at execution time, one live operation at a time)."""
        json_dir, owned = self._create_json_dir()
        names: List[str] = []
        files: List[Path] = []
        try:
            for index, phase in enumerate(plan.phases):
                document = RuntimeGraphGenerator().generate(self.compiler.compile(phase.graph))
                if document.get("version") != 2:
                    raise RuntimeError(
                        f"collective phase '{phase.name}' did not compile to JSON v2")
                name = f"{operation_name}_{index}_{phase.name}"
                path = json_dir / f"{name}.json"
                path.write_text(json.dumps(document, indent=2), encoding="utf-8")
                names.append(name)
                files.append(path)
        except Exception:
            discard_dir(json_dir, owned)
            raise
        return PreparedOcsCollectivePlan(
            operation_names=tuple(names), phase_files=tuple(files),
            barriers_after_phase=tuple(p.barrier_after for p in plan.phases),
            collective_types=tuple(p.graph.collective_type for p in plan.phases),
            json_dir=json_dir, owns_json_dir=owned)

    def execute(self, prepared: PreparedOcsCollectivePlan, input_tensor: torch.Tensor,
                output_tensor: Optional[torch.Tensor] = None,
                group: Optional[dist.ProcessGroup] = None, timeout: Optional[float] = None,
                async_op: bool = False) -> torch.Tensor:
        if async_op:
            raise NotImplementedError("OCS collective plans only support blocking execution")
        if prepared.closed:
            raise RuntimeError("prepared OCS collective plan has been closed")
        return self._run_phases(prepared.operation_names, prepared.phase_files,
                                prepared.barriers_after_phase, input_tensor, output_tensor,
                                group, timeout, "collective phase")


def barrier_sequence(world_size: int, job_id: str, group_id: int, first_barrier_id: int,
                     first_epoch_id: int, algorithm: str, backend: str):
    """Factory for the i-th barrier of a fixed plan (ids count up from the firsts)."""
    everyone = tuple(range(world_size))

    def barrier(offset: int, topology_id: int) -> OCSPlan:
        return OCSPlan(job_id=job_id, group_id=group_id, barrier_id=first_barrier_id + offset,
                       epoch_id=first_epoch_id + offset, next_epoch_id=first_epoch_id + offset + 1,
                       participant_ranks=everyone, topology_id=topology_id,
                       route_plan_id=first_barrier_id + offset, algorithm=algorithm,
                       backend=backend)
    return barrier


def build_ring_allreduce_alltoall_plan(rank: int, world_size: int, tensor_size: int,
                                       dtype: str = "float32", executor: str = "sm",
                                       job_id: str = "ocs_collective_plan", group_id: int = 0,
                                       first_barrier_id: int = 0,
                                       first_epoch_id: int = 0) -> OCSCollectivePlan:
    """all-reduce -> barrier(topology 1) -> all-to-all -> barrier(topology 2) -> all-reduce."""
    if world_size < 2:
        raise ValueError("the fixed collective plan requires at least two ranks")
    if tensor_size <= 0 or tensor_size % world_size:
        raise ValueError("tensor_size must be positive and divisible by world_size")
    ring = RingAllreduce()
    barrier = barrier_sequence(world_size, job_id, group_id, first_barrier_id, first_epoch_id,
                               algorithm="ring", backend="pccl")
    args = (rank, world_size, tensor_size, dtype, executor)
    return OCSCollectivePlan(phases=(
        OCSCollectivePhase("allreduce_0", ring.build_allreduce(*args), barrier(0, 1)),
        OCSCollectivePhase("alltoall_1", ring.build_alltoall(*args), barrier(1, 2)),
        OCSCollectivePhase("allreduce_2", ring.build_allreduce(*args)),
    ))


def build_switched_allreduce_alltoall_plan(rank: int, world_size: int, tensor_size: int,
                                           dtype: str = "float32", executor: str = "sm",
                                           job_id: str = "ocs_collective_plan", group_id: int = 0,
                                           first_barrier_id: int = 0,
                                           first_epoch_id: int = 0) -> OCSCollectivePlan:
    """The same three phases with the templates made for a switched fabric, where every peer is one
    hop away: two-shot all-reduce (direct reduce-scatter, then direct all-gather) and a direct
    all-to-all, instead of W - 1 ring steps each."""
    from ..dsl.algorithms import TwoShotAllreduce
    if world_size < 2:
        raise ValueError("the fixed collective plan requires at least two ranks")
    if tensor_size <= 0 or tensor_size % world_size:
        raise ValueError("tensor_size must be positive and divisible by world_size")
    direct = TwoShotAllreduce()
    barrier = barrier_sequence(world_size, job_id, group_id, first_barrier_id, first_epoch_id,
                               algorithm="auto", backend="pccl")
    args = (rank, world_size, tensor_size, dtype, executor)
    return OCSCollectivePlan(phases=(
        OCSCollectivePhase("allreduce_0", direct.build_allreduce(*args), barrier(0, 1)),
        OCSCollectivePhase("alltoall_1", direct.build_alltoall(*args), barrier(1, 2)),
        OCSCollectivePhase("allreduce_2", direct.build_allreduce(*args)),
    ))
