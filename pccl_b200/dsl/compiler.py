"""Compiler driver: analysis -> DCE -> [superopt] -> [channelize] -> analysis -> JSON.

Mirrors the reference pipeline (reference: pccl/dsl/compiler.py:12-77) with two
additions: ``gpu_profile`` actually selects the device cost profile
("h100" or "b200"), and the README calling convention
``compile_to_json_string(graph, compiler)`` is accepted next to
``compile_to_json_string(graph, indent=2)``.
"""

from __future__ import annotations

from typing import Any, Dict, Optional, Union

from .codegen import RuntimeGraphGenerator
from .graph import PrimitiveIRGraph
from .passes import ChannelizePass, DeadCodeEliminationPass, DependencyAnalysisPass


class Compiler:
    def __init__(self, enable_dce: bool = True, enable_superopt: bool = False,
                 enable_channelize: bool = False, num_channels: int = 2,
                 gpu_profile: str = "h100", data_size_hint: int = 0,
                 topology: object = None, device_profile: object = None):
        self.enable_dce = enable_dce
        self.enable_superopt = enable_superopt
        self.enable_channelize = enable_channelize
        self.num_channels = num_channels
        self.gpu_profile = gpu_profile
        self.data_size_hint = data_size_hint
        self.topology = topology
        self.device_profile = device_profile

    def _profiles(self):
        """(device profile, topology) chosen by explicit objects, else by name."""
        from .superopt.cost_model import profile_by_name, topology_for_profile
        device = self.device_profile or profile_by_name(self.gpu_profile)
        topology = self.topology or topology_for_profile(self.gpu_profile)
        return device, topology

    def compile(self, graph: PrimitiveIRGraph) -> PrimitiveIRGraph:
        DependencyAnalysisPass().run(graph)
        if self.enable_dce:
            DeadCodeEliminationPass().run(graph)
        if self.enable_superopt:
            if graph.has_ocs_barriers():
                raise ValueError(
                    "Superoptimization across OCS barriers is unsupported; "
                    "compile the generated OCS phases independently")
            from .superopt.pass_ import SuperoptPass
            device, topology = self._profiles()
            SuperoptPass(device_profile=device, topology=topology,
                         data_size_hint=self.data_size_hint).run(graph)
        if self.enable_channelize:
            device, _ = self._profiles()
            ChannelizePass(num_channels=self.num_channels, profile=device).run(graph)
        DependencyAnalysisPass().run(graph)
        return graph

    def compile_to_dict(self, graph: PrimitiveIRGraph) -> Dict[str, Any]:
        return RuntimeGraphGenerator().generate(self.compile(graph))

    def compile_to_json(self, graph: PrimitiveIRGraph, output_file: Optional[str] = None) -> str:
        generator = RuntimeGraphGenerator()
        compiled = self.compile(graph)
        if output_file:
            return generator.generate_to_file(compiled, output_file)
        return generator.generate_string(compiled)


def _split_second_arg(arg: Union[int, Compiler, None]):
    if isinstance(arg, Compiler):
        return arg, 2
    return Compiler(), (2 if arg is None else arg)


def compile_to_json_string(graph: PrimitiveIRGraph,
                           indent: Union[int, Compiler, None] = 2) -> str:
    compiler, indent = _split_second_arg(indent)
    return RuntimeGraphGenerator(indent=indent).generate_string(compiler.compile(graph))


def compile_to_json_file(graph: PrimitiveIRGraph, output_file: str,
                         indent: Union[int, Compiler, None] = 2) -> str:
    compiler, indent = _split_second_arg(indent)
    return RuntimeGraphGenerator(indent=indent).generate_to_file(
        compiler.compile(graph), output_file)
