"""Plan JSON writer and reader.

Two document kinds exist (reference: pccl/dsl/codegen/json_generator.py:24-119):

* **version 2** — one device plan: ``tensor_info``, optional
  ``collective_type``, ``executors`` and a topologically ordered ``operations``
  list whose entries carry ``index / executor / primitive / channel /
  dependencies / next_ops / params``.
* **version 3** (``execution_model: "phased_ocs"``) — emitted when the graph
  holds OCS barriers: per-phase operation lists plus ``control_operations`` for
  the host barriers, and deliberately *no* top-level ``operations`` so a plain
  device-plan loader rejects it.

``load_plan_graph`` is the inverse for version-2 documents; the CPU executor
and the round-trip tests use it.
"""

from __future__ import annotations

import json
from typing import Any, Dict, List, Sequence, Union

from ..graph import PrimitiveIRGraph
from ..nodes import (IRNodeVariant, PrimitiveOpType, TensorInfo, DeviceType,
                     node_from_params)
from .mapping import EXECUTOR_FROM_NAME, get_executor_name, get_primitive_name


class RuntimeGraphGenerator:
    def __init__(self, indent: int = 2):
        self.indent = indent

    # -- public ------------------------------------------------------------
    def generate(self, graph: PrimitiveIRGraph) -> Dict[str, Any]:
        if graph.is_empty():
            raise ValueError("Cannot generate JSON from empty graph")
        graph.validate()
        if graph.has_ocs_barriers():
            return self._phased_manifest(graph)
        document: Dict[str, Any] = {"version": 2}
        document.update(self._header(graph))
        document.update(self._operation_table(graph.topological_sort()))
        return document

    def generate_string(self, graph: PrimitiveIRGraph) -> str:
        return json.dumps(self.generate(graph), indent=self.indent)

    def generate_to_file(self, graph: PrimitiveIRGraph, filename: str) -> str:
        text = self.generate_string(graph)
        with open(filename, "w") as handle:
            handle.write(text)
        return text

    # -- pieces ------------------------------------------------------------
    @staticmethod
    def _header(graph: PrimitiveIRGraph) -> Dict[str, Any]:
        header: Dict[str, Any] = {}
        info = next((n.tensor_info for n in graph.nodes.values()
                     if n.tensor_info is not None), None)
        if info is not None:
            header["tensor_info"] = {"dtype": str(info.dtype), "shape": list(info.shape)}
        if graph.collective_type:
            header["collective_type"] = graph.collective_type
        if getattr(graph, "algorithm", ""):
            header["algorithm"] = graph.algorithm     # additive hint for the engine
        return header

    @staticmethod
    def _operation_table(nodes: Sequence[IRNodeVariant]) -> Dict[str, Any]:
        """Operations of one phase; edges leaving the phase are dropped."""
        index_of = {node.op_id: i for i, node in enumerate(nodes)}
        executors: Dict[str, None] = {}
        operations: List[Dict[str, Any]] = []
        for i, node in enumerate(nodes):
            executor = get_executor_name(node)
            executors.setdefault(executor)
            operations.append({
                "index": i,
                "executor": executor,
                "primitive": get_primitive_name(node),
                "channel": node.channel,
                "dependencies": [index_of[d] for d in node.dependencies if d in index_of],
                "next_ops": [index_of[s] for s in node.next_ops if s in index_of],
                "params": node.to_params(),
            })
        return {"executors": list(executors), "operations": operations}

    def _phased_manifest(self, graph: PrimitiveIRGraph) -> Dict[str, Any]:
        executors: Dict[str, None] = {}
        phases: List[Dict[str, Any]] = []
        controls: List[Dict[str, Any]] = []
        for phase in graph.split_ocs_phases():
            table = self._operation_table(phase.nodes)
            for name in table["executors"]:
                executors.setdefault(name)
            phases.append({"index": phase.index, **table})
            if phase.barrier is not None:
                controls.append({
                    "index": len(controls),
                    "primitive": get_primitive_name(phase.barrier),
                    "executor": get_executor_name(phase.barrier),
                    "after_phase": phase.index,
                    "before_phase": phase.index + 1,
                    "params": phase.barrier.to_params(),
                })
        manifest: Dict[str, Any] = {
            "version": 3,
            "execution_model": "phased_ocs",
            "executors": list(executors),
            "phases": phases,
            "control_operations": controls,
        }
        manifest.update(self._header(graph))
        return manifest


def load_plan_graph(plan: Union[str, Dict[str, Any]], name: str = "loaded_plan") -> PrimitiveIRGraph:
    """Rebuild a ``PrimitiveIRGraph`` from a version-2 plan (dict or JSON text).

    Node ids become ``op{index}``; dependencies, channels, executors and params
    are restored, so ``RuntimeGraphGenerator().generate(load_plan_graph(p)) == p``
    for plans this library wrote.
    """
    if isinstance(plan, str):
        plan = json.loads(plan)
    if "operations" not in plan:
        raise ValueError("not a version-2 device plan: no top-level 'operations'")
    info = None
    if "tensor_info" in plan:
        info = TensorInfo(plan["tensor_info"]["dtype"], tuple(plan["tensor_info"]["shape"]))
    graph = PrimitiveIRGraph(graph_name=name, collective_type=plan.get("collective_type", ""))
    graph.algorithm = plan.get("algorithm", "")
    for op in plan["operations"]:
        op_type = PrimitiveOpType(op["primitive"])
        executor = EXECUTOR_FROM_NAME.get(op.get("executor", "cuda_sm"))
        device = DeviceType.CPU if op.get("executor") == "host" else DeviceType.CUDA
        node = node_from_params(op_type, op.get("params", {}), op_id=f"op{op['index']}",
                                device=device, executor=executor)
        node.tensor_info = info
        node.channel = op.get("channel", 0)
        node.dependencies = [f"op{d}" for d in op.get("dependencies", [])]
        graph.add_node(node)
    for nid, node in graph.nodes.items():
        for dep in node.dependencies:
            graph.nodes[dep].add_next_op(nid)
    graph._update_boundary_points()
    return graph
