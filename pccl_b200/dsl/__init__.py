"""The plan DSL: IR nodes, graph, builder, compiler, algorithm templates, superoptimizer.

Importing this package needs only the standard library; z3 is loaded on first
use of rule verification.
"""

from .nodes import (
    DeviceType, ExecutorType, PrimitiveOpType, TensorInfo, ReduceOp, IRNode, IRNodeVariant,
    SmReduceNode, SmCopyNode, TmaCopyNode, TmaReduceNode, MultimemReduceNode, MultimemStoreNode,
    CeCopyNode, RdmaWriteNode, RdmaReadNode, NotifyNode, WaitNotifyNode, OcsBarrierNode,
    SmPutNode, SmReduceMultiNode,
)
from .graph import OcsPhase, PrimitiveIRGraph
from .decorators import build_graph, Stream, CommunicationOp
from .pipeline import Pipeline
from .compiler import Compiler, compile_to_json_string, compile_to_json_file
from .superopt import discover_rules, load_rules

__all__ = [
    "DeviceType", "ExecutorType", "PrimitiveOpType", "TensorInfo", "ReduceOp",
    "IRNode", "IRNodeVariant",
    "SmReduceNode", "SmCopyNode", "TmaCopyNode", "TmaReduceNode",
    "MultimemReduceNode", "MultimemStoreNode",
    "CeCopyNode", "RdmaWriteNode", "RdmaReadNode",
    "NotifyNode", "WaitNotifyNode", "OcsBarrierNode", "SmPutNode", "SmReduceMultiNode",
    "OcsPhase", "PrimitiveIRGraph",
    "build_graph", "Stream", "CommunicationOp", "Pipeline",
    "Compiler", "compile_to_json_string", "compile_to_json_file",
    "discover_rules", "load_rules",
]
