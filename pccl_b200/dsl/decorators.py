"""Builder front-end: ``CommunicationOp``, ``Stream`` and ``build_graph``.

``CommunicationOp`` is a context manager that records primitives into a
``PrimitiveIRGraph``.  Ordering is implicit: every primitive depends on the
previous primitive of the *stream* it was issued in, streams are independent
chains, and ``wait()`` / ``wait_for()`` add cross-stream edges (reference:
pccl/dsl/decorators.py:38-57 for Stream, :60-329 for CommunicationOp).

Internally each stream (and the implicit default stream) is a ``_Frontier``:
the id of its newest node plus the extra dependencies queued for its next
node.  All primitive methods funnel through ``_emit``.

Two calling conventions are accepted.  The context-manager form above is the
real one.  The README of the reference also shows a descriptor form,
``CommunicationOp(op_type="allreduce", tensor=TensorInfo(...), reduce_op=...)``
added to a stream with ``stream.add_op``; that form is accepted too and is
expanded by ``Compiler`` into a concrete algorithm template.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

from . import nodes as N
from .graph import PrimitiveIRGraph
from .nodes import DeviceType, IRNodeVariant, TensorInfo


class _Frontier:
    """Tail of one dependency chain."""

    __slots__ = ("name", "last_node_id", "pending_dependencies")

    def __init__(self, name: str):
        self.name = name
        self.last_node_id: Optional[str] = None
        self.pending_dependencies: List[str] = []

    def take_pending_dependencies(self) -> List[str]:
        taken, self.pending_dependencies = self.pending_dependencies, []
        return taken


# Kept under its historical name for code that introspects stream state.
_StreamState = _Frontier


class Stream:
    """Named, independent dependency chain inside a ``CommunicationOp``.

    Re-entering a stream with the same name continues its chain.  The README
    form ``Stream(channel=0)`` + ``add_op`` builds a descriptor list instead.
    """

    _active_comm_op: Optional["CommunicationOp"] = None

    def __init__(self, name: Optional[str] = None, channel: Optional[int] = None):
        if name is None:
            name = f"ch{0 if channel is None else channel}"
        self.name = name
        self.channel = channel
        self.ops: List["CommunicationOp"] = []
        self._comm_op: Optional["CommunicationOp"] = None
        self._outer: Optional[str] = None

    def add_op(self, op: "CommunicationOp") -> "Stream":
        self.ops.append(op)
        return self

    def __enter__(self) -> "Stream":
        owner = Stream._active_comm_op
        if owner is None:
            raise RuntimeError("Stream must be used within a CommunicationOp context")
        self._comm_op = owner
        self._outer = owner._active_stream_name
        owner._get_or_create_stream(self.name)
        owner._active_stream_name = self.name
        return self

    def __exit__(self, exc_type, exc, tb):
        if self._comm_op is not None:
            self._comm_op._active_stream_name = self._outer
        return False


class CommunicationOp:
    def __init__(self, name: Optional[str] = None, device: DeviceType = DeviceType.CUDA,
                 auto_dependency: bool = True, *, op_type: Optional[str] = None,
                 tensor: Optional[TensorInfo] = None, reduce_op: Any = None,
                 peer: Optional[int] = None):
        if name is None:
            name = op_type or "unnamed_op"
        self.name = name
        self.default_device = device
        self.auto_dependency = auto_dependency
        # Descriptor-form fields (None in the builder form).
        self.op_type = op_type
        self.reduce_op = reduce_op
        self.peer = peer

        self.graph = PrimitiveIRGraph(graph_name=name)
        self.current_tensor_info: Optional[TensorInfo] = tensor
        self._current_channel = 0
        self._default = _Frontier("")
        self._streams: Dict[str, _Frontier] = {}
        self._active_stream_name: Optional[str] = None
        self._nodes_in_order: List[str] = []
        self._ocs_phase_root_id: Optional[str] = None

    # -- bookkeeping exposed for compatibility ------------------------------
    @property
    def last_node_id(self) -> Optional[str]:
        return self._default.last_node_id

    @last_node_id.setter
    def last_node_id(self, value: Optional[str]) -> None:
        self._default.last_node_id = value

    @property
    def _pending_dependencies(self) -> List[str]:
        return self._default.pending_dependencies

    @property
    def active_stream(self) -> Optional[_Frontier]:
        if self._active_stream_name:
            return self._streams.get(self._active_stream_name)
        return None

    def _get_or_create_stream(self, name: str) -> _Frontier:
        frontier = self._streams.get(name)
        if frontier is None:
            frontier = self._streams[name] = _Frontier(name)
            if self._ocs_phase_root_id is not None:
                frontier.pending_dependencies.append(self._ocs_phase_root_id)
        return frontier

    # -- context manager ----------------------------------------------------
    def __enter__(self) -> "CommunicationOp":
        Stream._active_comm_op = self
        return self

    def __exit__(self, exc_type, exc, tb):
        Stream._active_comm_op = None
        if exc_type is None:
            self._finalize_dependencies()
        return False

    def tensor(self, dtype: Any, shape: tuple) -> "CommunicationOp":
        self.current_tensor_info = TensorInfo(dtype=dtype, shape=shape)
        return self

    def set_channel(self, channel: int) -> "CommunicationOp":
        self._current_channel = channel
        return self

    def get_graph(self) -> PrimitiveIRGraph:
        return self.graph

    # -- the single emission path ---------------------------------------------
    def _emit(self, cls, **params) -> IRNodeVariant:
        return self._add_node(cls(device=self.default_device, **params))

    def _add_node(self, node: IRNodeVariant) -> IRNodeVariant:
        if self.current_tensor_info:
            node.tensor_info = self.current_tensor_info
        node.channel = self._current_channel
        frontier = self.active_stream
        chain = frontier if frontier is not None else self._default
        if self.auto_dependency:
            if frontier is not None:
                for dep in frontier.take_pending_dependencies():
                    node.add_dependency(dep)
            if chain.last_node_id:
                node.add_dependency(chain.last_node_id)
        self.graph.add_node(node)
        chain.last_node_id = node.op_id
        if frontier is None:
            self._nodes_in_order.append(node.op_id)
        return node

    def _track_node(self, node_id: str) -> None:
        self._default.last_node_id = node_id
        self._nodes_in_order.append(node_id)

    # -- data primitives ------------------------------------------------------
    def sm_reduce(self, source_rank: int, src_offset: int, dst_offset: int,
                  remote_offset: int, count: int, reduce_op: str = "sum"):
        return self._emit(N.SmReduceNode, reduce_op=reduce_op, source_rank=source_rank,
                          src_offset=src_offset, dst_offset=dst_offset,
                          remote_offset=remote_offset, count=count)

    def tma_reduce(self, source_rank: int, src_offset: int, dst_offset: int,
                   remote_offset: int, count: int, reduce_op: str = "sum"):
        return self._emit(N.TmaReduceNode, reduce_op=reduce_op, source_rank=source_rank,
                          src_offset=src_offset, dst_offset=dst_offset,
                          remote_offset=remote_offset, count=count)

    def multimem_reduce(self, source_rank: int, src_offset: int, dst_offset: int,
                        remote_offset: int, count: int, reduce_op: str = "sum"):
        return self._emit(N.MultimemReduceNode, reduce_op=reduce_op, source_rank=source_rank,
                          src_offset=src_offset, dst_offset=dst_offset,
                          remote_offset=remote_offset, count=count)

    def sm_reduce_multi(self, source_ranks, dst_offset: int, remote_offset: int,
                        count: int, reduce_op: str = "sum"):
        return self._emit(N.SmReduceMultiNode, reduce_op=reduce_op,
                          source_ranks=tuple(source_ranks), dst_offset=dst_offset,
                          remote_offset=remote_offset, count=count)

    def sm_copy(self, source_rank: int, src_offset: int, dst_offset: int, size: int):
        return self._emit(N.SmCopyNode, source_rank=source_rank, src_offset=src_offset,
                          dst_offset=dst_offset, size=size)

    def tma_copy(self, source_rank: int, src_offset: int, dst_offset: int, size: int):
        return self._emit(N.TmaCopyNode, source_rank=source_rank, src_offset=src_offset,
                          dst_offset=dst_offset, size=size)

    def ce_copy(self, source_rank: int, src_offset: int, dst_offset: int, size: int):
        return self._emit(N.CeCopyNode, source_rank=source_rank, src_offset=src_offset,
                          dst_offset=dst_offset, size=size)

    def multimem_store(self, source_rank: int, src_offset: int, dst_offset: int, size: int):
        return self._emit(N.MultimemStoreNode, source_rank=source_rank, src_offset=src_offset,
                          dst_offset=dst_offset, size=size)

    def multimem_allreduce(self, offset: int, count: int, reduce_op: str = "sum"):
        return self._emit(N.MultimemAllreduceNode, reduce_op=reduce_op, offset=offset, count=count)

    def sm_put(self, target_rank: int, src_offset: int, dst_offset: int, size: int):
        return self._emit(N.SmPutNode, target_rank=target_rank, src_offset=src_offset,
                          dst_offset=dst_offset, size=size)

    def rdma_write(self, target_rank: int, src_offset: int, dst_offset: int, size: int):
        return self._emit(N.RdmaWriteNode, target_rank=target_rank, src_offset=src_offset,
                          dst_offset=dst_offset, size=size)

    def rdma_read(self, source_rank: int, src_offset: int, dst_offset: int, size: int):
        return self._emit(N.RdmaReadNode, source_rank=source_rank, src_offset=src_offset,
                          dst_offset=dst_offset, size=size)

    # -- signals --------------------------------------------------------------
    def notify(self, signal_id: int, target_rank: int):
        return self._emit(N.NotifyNode, signal_id=signal_id, target_rank=target_rank)

    def wait_notify(self, signal_id: int, source_rank: int):
        return self._emit(N.WaitNotifyNode, signal_id=signal_id, source_rank=source_rank)

    def ocs_barrier(self, barrier_id: int, epoch_id: int, next_epoch_id: int,
                    participant_ranks: tuple, topology_id: int, route_plan_id: int,
                    group_id: int = 0, route_mode: str = "STATIC_PLAN",
                    algorithm: str = "auto", backend: str = "pccl",
                    payload: bytes = b"", timeout_ms: int = 0) -> N.OcsBarrierNode:
        """Insert a graph-wide host barrier.

        The barrier joins *every* node emitted so far (not only the active
        stream) and becomes the root every later node hangs from, which is what
        makes the graph splittable into phases.
        """
        node = N.OcsBarrierNode(
            group_id=group_id, barrier_id=barrier_id, epoch_id=epoch_id,
            next_epoch_id=next_epoch_id, participant_ranks=participant_ranks,
            topology_id=topology_id, route_mode=route_mode, route_plan_id=route_plan_id,
            algorithm=algorithm, backend=backend, payload=payload, timeout_ms=timeout_ms,
            device=DeviceType.CPU)
        for earlier in self.graph.nodes.values():
            node.add_dependency(earlier.op_id)
            earlier.add_next_op(node.op_id)
        self.graph.add_node(node)

        self._ocs_phase_root_id = node.op_id
        self._nodes_in_order.append(node.op_id)
        for frontier in (self._default, *self._streams.values()):
            frontier.last_node_id = node.op_id
            frontier.pending_dependencies.clear()
        return node

    # -- cross-stream ordering ------------------------------------------------
    def _queue_dependency(self, node_id: str) -> None:
        (self.active_stream or self._default).pending_dependencies.append(node_id)

    def wait(self, stream_name: str) -> None:
        other = self._streams.get(stream_name)
        if other is None:
            raise ValueError(f"Stream '{stream_name}' not found")
        if not other.last_node_id:
            raise ValueError(f"Stream '{stream_name}' has no operations to wait for")
        self._queue_dependency(other.last_node_id)

    def wait_for(self, node: IRNodeVariant) -> None:
        if not node or not node.op_id:
            raise ValueError("Invalid node reference")
        self._queue_dependency(node.op_id)

    # -- finalisation -----------------------------------------------------------
    def _finalize_dependencies(self) -> None:
        if self.graph.is_empty():
            return
        # A wait() issued after a chain's last primitive attaches to that primitive.
        for frontier in (*self._streams.values(), self._default):
            leftover = frontier.take_pending_dependencies()
            if leftover and frontier.last_node_id:
                tail = self.graph.get_node(frontier.last_node_id)
                for dep in leftover:
                    tail.add_dependency(dep)
        for nid, node in self.graph.nodes.items():
            for dep in node.dependencies:
                producer = self.graph.nodes.get(dep)
                if producer is not None:
                    producer.add_next_op(nid)
        try:
            self.graph.validate()
        except ValueError as err:
            raise ValueError(f"Graph validation failed: {err}")


def build_graph(name: str, builder_func: Callable[[CommunicationOp], None],
                device: DeviceType = DeviceType.CUDA) -> PrimitiveIRGraph:
    with CommunicationOp(name=name, device=device) as op:
        builder_func(op)
        return op.get_graph()
