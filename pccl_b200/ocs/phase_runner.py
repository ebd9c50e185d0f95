"""Runner for one graph that contains OCS barriers (a JSON v3 manifest).

The manifest's phases are written out as ordinary version-2 plans, one per
phase, and executed with a controller release between them
(reference: pccl/ocs/phase_runner.py:22-214).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..dsl.codegen import RuntimeGraphGenerator
from ..dsl.compiler import Compiler
from ..dsl.graph import PrimitiveIRGraph
from ._phases import EngineBackedRunner, discard_dir
from .plan import OCSPlan
from .runtime import OCSRuntime


@dataclass
class PreparedOcsGraph:
    """Per phase: operation name and plan file (None for an empty phase) and
    the barrier that follows it (None after the last phase)."""

    operation_names: Tuple[Optional[str], ...]
    phase_files: Tuple[Optional[Path], ...]
    barriers_after_phase: Tuple[Optional[OCSPlan], ...]
    manifest: Dict[str, Any]
    json_dir: Path
    owns_json_dir: bool
    closed: bool = False

    def close(self) -> None:
        if not self.closed:
            discard_dir(self.json_dir, self.owns_json_dir)
        self.closed = True


class OcsPhaseRunner(EngineBackedRunner):
    _tmp_prefix = "pccl-ocs-"

    def __init__(self, engine: Any = None, runtime: Optional[OCSRuntime] = None,
                 compiler: Optional[Compiler] = None, json_dir: Optional[str] = None) -> None:
        super().__init__(engine, runtime, compiler, json_dir)

    def prepare(self, graph: PrimitiveIRGraph, operation_name: Optional[str] = None) -> PreparedOcsGraph:
        """Compile ``graph`` and write one plan file per non-empty phase.
        Registration is left to ``execute``: all operations share one signal
        space, so only the running phase may be registered."""
        compiled = self.compiler.compile(graph)
        manifest = RuntimeGraphGenerator().generate(compiled)
        if manifest.get("execution_model") != "phased_ocs":
            raise ValueError("OcsPhaseRunner requires a graph containing an OCS barrier")
        phases = compiled.split_ocs_phases()
        if len(phases) != len(manifest["phases"]):
            raise RuntimeError("OCS phase manifest does not match the compiled IR graph")

        json_dir, owned = self._create_json_dir()
        stem = operation_name or compiled.graph_id
        names: List[Optional[str]] = []
        files: List[Optional[Path]] = []
        try:
            for phase, entry in zip(phases, manifest["phases"]):
                if not entry["operations"]:
                    names.append(None)
                    files.append(None)
                    continue
                name = f"{stem}_phase_{phase.index}"
                path = json_dir / f"{name}.json"
                path.write_text(json.dumps(self._to_runtime_v2(manifest, entry), indent=2),
                                encoding="utf-8")
                names.append(name)
                files.append(path)
        except Exception:
            discard_dir(json_dir, owned)
            raise
        barriers = tuple(p.barrier.to_ocs_plan() if p.barrier is not None else None
                         for p in phases)
        return PreparedOcsGraph(tuple(names), tuple(files), barriers, manifest, json_dir, owned)

    def execute(self, prepared: PreparedOcsGraph, input_tensor: torch.Tensor,
                output_tensor: Optional[torch.Tensor] = None,
                group: Optional[dist.ProcessGroup] = None, timeout: Optional[float] = None,
                async_op: bool = False) -> torch.Tensor:
        if async_op:
            raise NotImplementedError("OcsPhaseRunner only supports blocking execution")
        if prepared.closed:
            raise RuntimeError("prepared OCS graph has been closed")
        if all(name is None for name in prepared.operation_names):
            # Barriers only: the data passes through untouched.
            if output_tensor is not None:
                output_tensor.copy_(input_tensor)
            for barrier in prepared.barriers_after_phase:
                if barrier is not None:
                    self.runtime.barrier_switch(barrier, group=group, timeout=timeout)
            return input_tensor if output_tensor is None else output_tensor
        return self._run_phases(prepared.operation_names, prepared.phase_files,
                                prepared.barriers_after_phase, input_tensor, output_tensor,
                                group, timeout, "OCS phase")

    @staticmethod
    def _to_runtime_v2(manifest: Dict[str, Any], phase_manifest: Dict[str, Any]) -> Dict[str, Any]:
        plan = {"version": 2, "executors": phase_manifest["executors"],
                "operations": phase_manifest["operations"]}
        for key in ("tensor_info", "collective_type"):
            if key in manifest:
                plan[key] = manifest[key]
        return plan
