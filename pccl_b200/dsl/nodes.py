"""IR node types of the plan DSL.

Every primitive a plan can contain is a small dataclass whose ``to_params()``
dictionary is, verbatim, the ``params`` object of the JSON plan.  The field
names are therefore a wire contract shared with the reference implementation
(reference: pccl/dsl/nodes.py:24-37 for the primitive names, :131-430 for the
per-primitive parameter sets, :432-538 for the OCS barrier node).

Unlike the reference, the twelve data/signal node classes are not written out
by hand: they are stamped from four *parameter shapes* (reduce, pull-copy,
push-copy, signal) by ``_make_node_class`` so that validation and
serialisation live in one place.  Two primitives are additions of this
library: ``sm.put`` (a push-style copy used by one-shot / two-shot plans) and
``sm.reduce_multi`` (reduce one slice from several peers at once, the natural
primitive on an NVSwitch fabric where every peer is one hop away).
"""

from __future__ import annotations

import dataclasses
import uuid
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional, Tuple, Union


class DeviceType(Enum):
    CPU = "cpu"
    CUDA = "cuda"
    RDMA = "rdma"
    # README-style spelling accepted as an alias of CUDA.
    GPU = "cuda"


class ExecutorType(Enum):
    SM = "sm"
    TMA = "tma"
    CE = "ce"
    HOST = "host"
    RDMA = "rdma"
    MULTIMEM = "multimem"


class PrimitiveOpType(Enum):
    SM_REDUCE = "sm.reduce"
    SM_COPY = "sm.copy"
    TMA_COPY = "tma.copy"
    TMA_REDUCE = "tma.reduce"
    CE_COPY = "ce.copy"
    MULTIMEM_REDUCE = "multimem.reduce"
    MULTIMEM_STORE = "multimem.store"
    RDMA_WRITE = "rdma.write"
    RDMA_READ = "rdma.read"
    NOTIFY = "notify"
    WAIT_NOTIFY = "wait_notify"
    OCS_BARRIER = "ocs.barrier"
    NOOP = "noop"
    # Additions of this library (additive to the plan format).
    SM_PUT = "sm.put"
    SM_REDUCE_MULTI = "sm.reduce_multi"
    MULTIMEM_ALLREDUCE = "multimem.allreduce"


class ReduceOp(Enum):
    SUM = "sum"
    MAX = "max"
    MIN = "min"
    AVG = "avg"


_EXECUTOR_OF: Dict[PrimitiveOpType, ExecutorType] = {
    PrimitiveOpType.SM_REDUCE: ExecutorType.SM,
    PrimitiveOpType.SM_COPY: ExecutorType.SM,
    PrimitiveOpType.SM_PUT: ExecutorType.SM,
    PrimitiveOpType.SM_REDUCE_MULTI: ExecutorType.SM,
    PrimitiveOpType.TMA_COPY: ExecutorType.TMA,
    PrimitiveOpType.TMA_REDUCE: ExecutorType.TMA,
    PrimitiveOpType.CE_COPY: ExecutorType.CE,
    PrimitiveOpType.MULTIMEM_REDUCE: ExecutorType.MULTIMEM,
    PrimitiveOpType.MULTIMEM_STORE: ExecutorType.MULTIMEM,
    PrimitiveOpType.MULTIMEM_ALLREDUCE: ExecutorType.MULTIMEM,
    PrimitiveOpType.RDMA_WRITE: ExecutorType.RDMA,
    PrimitiveOpType.RDMA_READ: ExecutorType.RDMA,
    PrimitiveOpType.OCS_BARRIER: ExecutorType.HOST,
    PrimitiveOpType.NOOP: ExecutorType.SM,
}


def infer_executor(op_type: PrimitiveOpType) -> Optional[ExecutorType]:
    """Executor implied by a primitive name; ``None`` for notify/wait, whose
    executor depends on the device the node is placed on."""
    return _EXECUTOR_OF.get(op_type)


VALID_DTYPES = {"float32", "float16", "bfloat16", "float8_e4m3", "float8_e5m2"}
DTYPE_BYTES = {"float32": 4, "float16": 2, "bfloat16": 2, "float8_e4m3": 1, "float8_e5m2": 1}
OCS_ALGORITHMS = {"ring", "rhd", "tree", "auto", "torch_native"}
OCS_BACKENDS = {"torch", "pccl"}
OCS_ROUTE_MODES = {"STATIC_PLAN", "ID_ROUTE", "SEGMENT_ROUTE", "USER_PLAN"}
_REDUCE_NAMES = tuple(m.value for m in ReduceOp)


@dataclass(init=False)
class TensorInfo:
    """dtype name + shape of the tensor a plan operates on.

    Accepts the positional form ``TensorInfo(dtype, shape)`` as well as the
    keyword form with an ignored ``device=`` argument.
    """

    dtype: Any
    shape: tuple

    def __init__(self, dtype: Any = None, shape: tuple = None, device: Any = None):
        if not isinstance(shape, tuple):
            raise ValueError(f"shape must be a tuple, got {type(shape)}")
        name = _dtype_name(dtype)
        if name not in VALID_DTYPES:
            raise ValueError(
                f"unsupported dtype '{name}', must be one of {sorted(VALID_DTYPES)}")
        self.dtype = dtype
        self.shape = shape

    def numel(self) -> int:
        total = 1
        for extent in self.shape:
            total *= extent
        return total

    def nbytes(self) -> int:
        return self.numel() * DTYPE_BYTES[_dtype_name(self.dtype)]


def _dtype_name(dtype: Any) -> str:
    text = str(dtype)
    # torch.float32 -> "float32"; torch.float8_e4m3fn -> "float8_e4m3".
    if text.startswith("torch."):
        text = text[len("torch."):]
        if text.endswith("fn"):
            text = text[:-2]
    return text


@dataclass(repr=False)
class IRNode:
    op_id: str = ""
    op_type: Optional[PrimitiveOpType] = None
    device: DeviceType = DeviceType.CUDA
    executor: Optional[ExecutorType] = None
    tensor_info: Optional[TensorInfo] = None
    dependencies: List[str] = field(default_factory=list)
    next_ops: List[str] = field(default_factory=list)
    channel: int = 0

    def __post_init__(self):
        self._finish_identity()

    def _finish_identity(self) -> None:
        if self.op_type is not None:
            if not self.op_id:
                stem = self.op_type.value.replace(".", "_")
                self.op_id = f"{stem}_{uuid.uuid4().hex[:8]}"
            if self.executor is None:
                self.executor = infer_executor(self.op_type)

    def add_dependency(self, dep_id: str) -> None:
        if dep_id not in self.dependencies:
            self.dependencies.append(dep_id)

    def add_next_op(self, next_id: str) -> None:
        if next_id not in self.next_ops:
            self.next_ops.append(next_id)

    def to_params(self) -> Dict[str, Any]:
        return {}

    def validate(self) -> bool:
        return True

    def __repr__(self) -> str:
        kind = self.op_type.value if self.op_type else "none"
        where = self.executor.value if self.executor else "none"
        return f"IRNode(id={self.op_id}, type={kind}, executor={where})"


# ---------------------------------------------------------------------------
# Parameter shapes.  (field name, default) in the order they are serialised.
# ---------------------------------------------------------------------------

_SHAPE_REDUCE = (("reduce_op", "sum"), ("source_rank", -1), ("src_offset", 0),
                 ("dst_offset", 0), ("remote_offset", 0), ("count", 0))
_SHAPE_PULL = (("source_rank", -1), ("src_offset", 0), ("dst_offset", 0), ("size", 0))
_SHAPE_PUSH = (("target_rank", -1), ("src_offset", 0), ("dst_offset", 0), ("size", 0))
_SHAPE_NOTIFY = (("signal_id", 0), ("target_rank", -1))
_SHAPE_WAIT = (("signal_id", 0), ("source_rank", -1))


def _make_node_class(cls_name: str, op_type: PrimitiveOpType, shape, doc: str):
    """Stamp one node dataclass from a parameter shape."""
    names = [n for n, _ in shape]
    peer_field = "source_rank" if "source_rank" in names else "target_rank"
    extent_field = "count" if "count" in names else ("size" if "size" in names else None)
    has_reduce = "reduce_op" in names
    is_signal = extent_field is None

    def __post_init__(self):
        if self.op_type is None:
            self.op_type = op_type
        self._finish_identity()
        if is_signal and self.executor is None:
            on_gpu = self.device == DeviceType.CUDA
            self.executor = ExecutorType.SM if on_gpu else ExecutorType.HOST

    def validate(self) -> bool:
        if has_reduce and self.reduce_op not in _REDUCE_NAMES:
            raise ValueError(f"{cls_name}: invalid reduce_op '{self.reduce_op}'")
        peer = getattr(self, peer_field)
        if peer < 0:
            raise ValueError(f"{cls_name}: {peer_field} must be non-negative, got {peer}")
        if extent_field is not None:
            extent = getattr(self, extent_field)
            if extent < 0:
                raise ValueError(
                    f"{cls_name}: {extent_field} must be non-negative, got {extent}")
        return True

    def to_params(self) -> Dict[str, Any]:
        return {n: getattr(self, n) for n in names}

    namespace = {"__post_init__": __post_init__, "validate": validate,
                 "to_params": to_params, "__doc__": doc, "PARAM_NAMES": tuple(names)}
    fields = [(n, type(d), field(default=d)) for n, d in shape]
    cls = dataclasses.make_dataclass(cls_name, fields, bases=(IRNode,), namespace=namespace)
    cls.__module__ = __name__
    return cls


SmReduceNode = _make_node_class(
    "SmReduceNode", PrimitiveOpType.SM_REDUCE, _SHAPE_REDUCE,
    "self[dst:dst+count] = peer[source_rank][remote:remote+count] (op) self[src:src+count], by SM threads.")
SmCopyNode = _make_node_class(
    "SmCopyNode", PrimitiveOpType.SM_COPY, _SHAPE_PULL,
    "self[dst:dst+size] = peer[source_rank][src:src+size], pulled by SM threads.")
TmaCopyNode = _make_node_class(
    "TmaCopyNode", PrimitiveOpType.TMA_COPY, _SHAPE_PULL,
    "Same semantics as sm.copy; the executor may stage local tiles with TMA.")
TmaReduceNode = _make_node_class(
    "TmaReduceNode", PrimitiveOpType.TMA_REDUCE, _SHAPE_REDUCE,
    "Same semantics as sm.reduce; the executor may stage local tiles with TMA.")
MultimemReduceNode = _make_node_class(
    "MultimemReduceNode", PrimitiveOpType.MULTIMEM_REDUCE, _SHAPE_REDUCE,
    "In-switch reduction: multimem.ld_reduce over all ranks' copies of a slice.")
MultimemStoreNode = _make_node_class(
    "MultimemStoreNode", PrimitiveOpType.MULTIMEM_STORE, _SHAPE_PULL,
    "In-switch broadcast: multimem.st of a local slice to every rank.")
CeCopyNode = _make_node_class(
    "CeCopyNode", PrimitiveOpType.CE_COPY, _SHAPE_PULL,
    "Pull copy executed by a copy engine (cudaMemcpyPeerAsync).")
RdmaWriteNode = _make_node_class(
    "RdmaWriteNode", PrimitiveOpType.RDMA_WRITE, _SHAPE_PUSH,
    "peer[target_rank][dst:dst+size] = self[src:src+size] over RDMA.")
RdmaReadNode = _make_node_class(
    "RdmaReadNode", PrimitiveOpType.RDMA_READ, _SHAPE_PULL,
    "self[dst:dst+size] = peer[source_rank][src:src+size] over RDMA.")
NotifyNode = _make_node_class(
    "NotifyNode", PrimitiveOpType.NOTIFY, _SHAPE_NOTIFY,
    "signals[target_rank][signal_id] += 1 (counting-semaphore post).")
WaitNotifyNode = _make_node_class(
    "WaitNotifyNode", PrimitiveOpType.WAIT_NOTIFY, _SHAPE_WAIT,
    "Block until signals[self][signal_id] > 0, then decrement it.")
SmPutNode = _make_node_class(
    "SmPutNode", PrimitiveOpType.SM_PUT, _SHAPE_PUSH,
    "peer[target_rank][dst:dst+size] = self[src:src+size], pushed by SM threads.")


@dataclass
class SmReduceMultiNode(IRNode):
    """self[dst:dst+count] = (op) over r in source_ranks of buffer_r[remote:remote+count].

    ``source_ranks`` may include the executing rank itself.  One node replaces
    the N-1 chained ``sm.reduce`` nodes of a direct reduce-scatter step.
    """

    reduce_op: str = "sum"
    source_ranks: Tuple[int, ...] = ()
    dst_offset: int = 0
    remote_offset: int = 0
    count: int = 0

    def __post_init__(self):
        if self.op_type is None:
            self.op_type = PrimitiveOpType.SM_REDUCE_MULTI
        self.source_ranks = tuple(int(r) for r in self.source_ranks)
        self._finish_identity()

    def validate(self) -> bool:
        if self.reduce_op not in _REDUCE_NAMES:
            raise ValueError(f"SmReduceMultiNode: invalid reduce_op '{self.reduce_op}'")
        if not self.source_ranks or any(r < 0 for r in self.source_ranks):
            raise ValueError("SmReduceMultiNode: source_ranks must be non-empty and non-negative")
        if self.count < 0:
            raise ValueError(f"SmReduceMultiNode: count must be non-negative, got {self.count}")
        return True

    def to_params(self) -> Dict[str, Any]:
        return {"reduce_op": self.reduce_op, "source_ranks": list(self.source_ranks),
                "dst_offset": self.dst_offset, "remote_offset": self.remote_offset,
                "count": self.count}


@dataclass
class MultimemAllreduceNode(IRNode):
    """buffer_r[offset:offset+count] = (op) over all ranks s of buffer_s[offset:offset+count], for every r.

    One pass through the switch: each 16-byte vector is fetched with ``multimem.ld_reduce``
    (the switch folds every rank's copy) and written straight back with ``multimem.st`` (the
    switch delivers it to every rank), so the reduce traffic (outbound) and the broadcast
    traffic (inbound) share the link at the same time instead of one after the other.  Ranks
    must run it on disjoint ranges between two barriers.
    """

    reduce_op: str = "sum"
    offset: int = 0
    count: int = 0

    def __post_init__(self):
        if self.op_type is None:
            self.op_type = PrimitiveOpType.MULTIMEM_ALLREDUCE
        self._finish_identity()

    def validate(self) -> bool:
        if self.reduce_op not in _REDUCE_NAMES:
            raise ValueError(f"MultimemAllreduceNode: invalid reduce_op '{self.reduce_op}'")
        if self.offset < 0 or self.count < 0:
            raise ValueError("MultimemAllreduceNode: offset and count must be non-negative")
        return True

    def to_params(self) -> Dict[str, Any]:
        return {"reduce_op": self.reduce_op, "offset": self.offset, "count": self.count}


@dataclass
class OcsBarrierNode(IRNode):
    """Host-side control point at which the optical-circuit-switch topology may change.

    It never becomes device work: a graph containing one is emitted as a phased
    manifest and the host obtains a controller release between phases.
    """

    group_id: int = 0
    barrier_id: int = 0
    epoch_id: int = 0
    next_epoch_id: int = 1
    participant_ranks: Tuple[int, ...] = ()
    topology_id: int = 0
    route_mode: str = "STATIC_PLAN"
    route_plan_id: int = 0
    algorithm: str = "auto"
    backend: str = "pccl"
    payload: bytes = b""
    timeout_ms: int = 0

    def __post_init__(self):
        if self.op_type is None:
            self.op_type = PrimitiveOpType.OCS_BARRIER
        if self.device == DeviceType.CUDA:
            self.device = DeviceType.CPU
        self._finish_identity()
        if self.executor is None:
            self.executor = ExecutorType.HOST
        self.participant_ranks = tuple(int(r) for r in self.participant_ranks)
        if self.payload is None:
            self.payload = b""
        elif isinstance(self.payload, (bytes, bytearray, memoryview)):
            self.payload = bytes(self.payload)
        else:
            raise TypeError("OcsBarrierNode: payload must be bytes-like")

    @property
    def participant_bitmap(self) -> int:
        bits = 0
        for rank in self.participant_ranks:
            bits |= 1 << rank
        return bits

    def validate(self) -> bool:
        def bad(msg: str):
            raise ValueError(f"OcsBarrierNode: {msg}")

        if self.group_id < 0:
            bad(f"group_id must be non-negative, got {self.group_id}")
        if self.barrier_id < 0:
            bad(f"barrier_id must be non-negative, got {self.barrier_id}")
        if self.epoch_id < 0 or self.next_epoch_id <= self.epoch_id:
            bad("next_epoch_id must be greater than a non-negative epoch_id")
        if not self.participant_ranks:
            bad("participant_ranks must not be empty")
        if min(self.participant_ranks) < 0:
            bad("participant_ranks must be non-negative")
        if len(set(self.participant_ranks)) != len(self.participant_ranks):
            bad("participant_ranks must not contain duplicates")
        if self.topology_id < 0 or self.route_plan_id < 0:
            bad("topology_id and route_plan_id must be non-negative")
        if self.route_mode not in OCS_ROUTE_MODES:
            bad(f"unsupported route_mode '{self.route_mode}'")
        if self.algorithm not in OCS_ALGORITHMS:
            bad(f"unsupported algorithm '{self.algorithm}'")
        if self.backend not in OCS_BACKENDS:
            bad(f"unsupported backend '{self.backend}'")
        if self.timeout_ms < 0:
            bad("timeout_ms must be non-negative")
        return True

    def to_params(self) -> Dict[str, Any]:
        return {
            "group_id": self.group_id,
            "barrier_id": self.barrier_id,
            "epoch_id": self.epoch_id,
            "next_epoch_id": self.next_epoch_id,
            "participant_ranks": list(self.participant_ranks),
            "participant_bitmap": self.participant_bitmap,
            "topology_id": self.topology_id,
            "route_mode": self.route_mode,
            "route_plan_id": self.route_plan_id,
            "algorithm": self.algorithm,
            "backend": self.backend,
            "payload_hex": self.payload.hex(),
            "timeout_ms": self.timeout_ms,
        }

    def to_ocs_plan(self):
        """The runtime plan object equivalent to this barrier."""
        from ..ocs.plan import OCSPlan  # late import: the DSL does not depend on OCS

        keys = ("group_id", "barrier_id", "epoch_id", "next_epoch_id", "participant_ranks",
                "topology_id", "route_mode", "route_plan_id", "algorithm", "backend", "payload")
        return OCSPlan(**{k: getattr(self, k) for k in keys})


IRNodeVariant = Union[
    SmReduceNode, SmCopyNode, TmaCopyNode, TmaReduceNode,
    MultimemReduceNode, MultimemStoreNode,
    CeCopyNode, RdmaWriteNode, RdmaReadNode,
    NotifyNode, WaitNotifyNode, OcsBarrierNode,
    SmPutNode, SmReduceMultiNode, MultimemAllreduceNode,
]

#: primitive name -> node class, for code that rebuilds nodes from plan JSON.
NODE_CLASS_BY_OP: Dict[PrimitiveOpType, type] = {
    PrimitiveOpType.SM_REDUCE: SmReduceNode,
    PrimitiveOpType.SM_COPY: SmCopyNode,
    PrimitiveOpType.TMA_COPY: TmaCopyNode,
    PrimitiveOpType.TMA_REDUCE: TmaReduceNode,
    PrimitiveOpType.MULTIMEM_REDUCE: MultimemReduceNode,
    PrimitiveOpType.MULTIMEM_STORE: MultimemStoreNode,
    PrimitiveOpType.CE_COPY: CeCopyNode,
    PrimitiveOpType.RDMA_WRITE: RdmaWriteNode,
    PrimitiveOpType.RDMA_READ: RdmaReadNode,
    PrimitiveOpType.NOTIFY: NotifyNode,
    PrimitiveOpType.WAIT_NOTIFY: WaitNotifyNode,
    PrimitiveOpType.SM_PUT: SmPutNode,
    PrimitiveOpType.SM_REDUCE_MULTI: SmReduceMultiNode,
    PrimitiveOpType.MULTIMEM_ALLREDUCE: MultimemAllreduceNode,
    PrimitiveOpType.OCS_BARRIER: OcsBarrierNode,
}


def node_from_params(op_type: PrimitiveOpType, params: Dict[str, Any], **common) -> IRNode:
    """Build the node class for ``op_type`` from a plan ``params`` dictionary,
    ignoring keys the class does not know (forward compatibility)."""
    cls = NODE_CLASS_BY_OP[op_type]
    accepted = {f.name for f in dataclasses.fields(cls)}
    kwargs = {k: v for k, v in params.items() if k in accepted}
    if cls is OcsBarrierNode and "payload_hex" in params:
        kwargs["payload"] = bytes.fromhex(params["payload_hex"])
    kwargs.update(common)
    return cls(**kwargs)
