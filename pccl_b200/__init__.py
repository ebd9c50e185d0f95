"""pccl_b200 — Blackwell-native collective communication and fused compute.

Layers (each importable on its own):

* ``pccl_b200.dsl``      plan DSL, compiler, algorithm templates, superoptimizer
* ``pccl_b200.ocs``      optical-circuit-switch aware host runtime
* ``pccl_b200.runtime``  CPU reference executor for plans (the test oracle)
* ``pccl_b200.engine``   Python face of the native engine (loaded on first use)
* ``pccl_b200.parallel`` collectives API on top of the engine
* ``pccl_b200.ops``      fused compute + collective operators (tcgen05 kernels)
* ``pccl_b200.models``   tensor-/expert-parallel reference blocks built on the ops

Importing the package loads neither the CUDA extension nor z3.  The engine
entry points below are resolved lazily.
"""

__version__ = "0.3.0"

from .dsl import (
    DeviceType, ExecutorType, PrimitiveOpType, TensorInfo, ReduceOp,
    IRNode, IRNodeVariant,
    SmReduceNode, SmCopyNode, TmaCopyNode, TmaReduceNode, MultimemReduceNode, MultimemStoreNode,
    CeCopyNode, RdmaWriteNode, RdmaReadNode, NotifyNode, WaitNotifyNode, OcsBarrierNode,
    SmPutNode, SmReduceMultiNode,
    OcsPhase, PrimitiveIRGraph, build_graph, Stream, CommunicationOp, Pipeline,
    Compiler, compile_to_json_string, compile_to_json_file,
)
from .ocs import (
    OCSError, OCSBarrierTimeout, OCSLinkNotReady, OCSPlan, OCSPlanMismatchError, OCSProtocolError,
    OCSBarrierState, OCSLinkState, OCSPlanController, OCSRuntime, OCSSwitchResult,
    OCSCollectivePhase, OCSCollectivePlan, OcsCollectivePlanRunner, OcsPhaseRunner,
    PreparedOcsCollectivePlan, PreparedOcsGraph,
    StaticPlanController, SwitchConnector, TorchDistributedSwitchConnector, TensorSwitchConnector,
    OcsTorchPlanRunner, TorchCollectivePhase, TorchCollectivePlan,
    build_ring_allreduce_alltoall_plan, build_torch_allreduce_alltoall_plan,
    OCS_CONTROL_MAGIC, OCS_CONTROL_MAX_PAYLOAD_BYTES, OCS_CONTROL_VERSION,
    OCSControlMessage, OCSControlMessageKey, OCSControlMessageType, OCSControlStatus,
    ack_target, build_ack, build_ready, build_release, ocs_all_reduce, ocs_barrier_switch,
    plan_digest,
)

_ENGINE_API = (
    "get_engine", "register_operation", "execute_operation", "execute_operation_async",
    "sync_operation", "reset_signals", "get_endpoint", "initialize_engine",
    "empty_symmetric", "PCCLTimeoutError", "PCCLError",
)


def __getattr__(name):
    if name in _ENGINE_API:
        from . import engine
        return getattr(engine, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = [
    "__version__",
    "DeviceType", "ExecutorType", "PrimitiveOpType", "TensorInfo", "ReduceOp",
    "IRNode", "IRNodeVariant",
    "SmReduceNode", "SmCopyNode", "TmaCopyNode", "TmaReduceNode",
    "MultimemReduceNode", "MultimemStoreNode",
    "CeCopyNode", "RdmaWriteNode", "RdmaReadNode",
    "NotifyNode", "WaitNotifyNode", "OcsBarrierNode", "SmPutNode", "SmReduceMultiNode",
    "OcsPhase", "PrimitiveIRGraph",
    "build_graph", "Stream", "CommunicationOp", "Pipeline",
    "Compiler", "compile_to_json_string", "compile_to_json_file",
    "OCSError", "OCSBarrierTimeout", "OCSLinkNotReady", "OCSPlan", "OCSPlanMismatchError",
    "OCSProtocolError",
    "OCSBarrierState", "OCSLinkState", "OCSPlanController", "OCSRuntime",
    "OCSSwitchResult", "OCSCollectivePhase", "OCSCollectivePlan",
    "OcsCollectivePlanRunner", "OcsPhaseRunner", "PreparedOcsCollectivePlan", "PreparedOcsGraph",
    "StaticPlanController", "SwitchConnector", "TorchDistributedSwitchConnector",
    "TensorSwitchConnector",
    "OcsTorchPlanRunner", "TorchCollectivePhase", "TorchCollectivePlan",
    "build_ring_allreduce_alltoall_plan", "build_torch_allreduce_alltoall_plan",
    "OCS_CONTROL_MAGIC", "OCS_CONTROL_MAX_PAYLOAD_BYTES", "OCS_CONTROL_VERSION",
    "OCSControlMessage", "OCSControlMessageKey", "OCSControlMessageType", "OCSControlStatus",
    "ack_target", "build_ack", "build_ready", "build_release", "ocs_all_reduce",
    "ocs_barrier_switch", "plan_digest",
    *_ENGINE_API,
]
