"""Python face of the native engine.

The module-level functions are the public runtime API (reference:
pccl/engine.py:52-115): ``get_engine``, ``register_operation(name, file)``,
``execute_operation(name, input, output=None)``, ``execute_operation_async``,
``sync_operation``, ``reset_signals``, ``get_endpoint`` and
``initialize_engine(group)``.  They are also re-exported lazily from the package
root (``pccl.get_engine`` ...).

Two engines implement the same surface:

* ``Engine`` wraps the CUDA extension ``pccl_b200.engine_c`` (one process per GPU).
  ``initialize_engine`` exchanges endpoint records over the given process group
  (any backend), maps every peer's symmetric heap and brings NVLS multicast up
  when all ranks support it.
* ``CpuEngine`` is used when no CUDA device is present (or ``PCCL_EXECUTOR=cpu``):
  plans are replayed over the group's CPU backend (gloo) by the reference
  executor, so the whole stack above the engine runs on a CPU-only box.

Additions: ``working_buffer`` (tensor view of the plan working buffer — a
collective whose input *is* that view runs without staging copies),
``empty_symmetric`` (symmetric allocation for the fused operators),
``reset_engine`` and the ``PCCLError`` / ``PCCLTimeoutError`` exceptions.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


class PCCLError(RuntimeError):
    """Engine failure (bad plan, missing peer, CUDA error)."""


class PCCLTimeoutError(PCCLError):
    """A device-side wait ran out of its time budget; the engine must be reset."""


_native = None


def load_native():
    """Import the CUDA extension, with a loud error when it is missing on a GPU box."""
    global _native, PCCLError, PCCLTimeoutError
    if _native is None:
        try:
            from . import engine_c
        except ImportError as err:
            raise ImportError(
                "pccl_b200.engine_c is not built; run `python setup.py build_ext --inplace` "
                "(or `python -c 'import __graft_entry__ as g; g.build()'`) in the repository root") from err
        _native = engine_c
        PCCLError = engine_c.PCCLError
        PCCLTimeoutError = engine_c.PCCLTimeoutError
    return _native


def _debug_endpoint_init(stage: str) -> None:
    if os.environ.get("PCCL_DEBUG_ENDPOINT_INIT") == "1":
        rank = dist.get_rank() if dist.is_initialized() else -1
        print(f"PCCL_ENDPOINT_INIT rank={rank} {stage}", flush=True)


class Engine:
    """One process, one GPU.  Thin wrapper over ``engine_c.Engine``."""

    def __init__(self):
        self._engine = load_native().Engine.get_instance()

    # -- reference verbs ------------------------------------------------------------------
    def register_operation(self, name: str, filename: str) -> bool:
        """``filename``: path of a plan file (the reference's contract) or the plan JSON text itself."""
        if str(filename).lstrip().startswith("{"):
            return self.register_operation_from_string(name, str(filename))
        return self._engine.regOp(name, str(filename))

    def register_operation_from_string(self, name: str, plan_json: str) -> bool:
        return self._engine.regOpFromString(name, plan_json)

    def execute_operation(self, name, input_tensor, output_tensor=None):
        if output_tensor is None:
            output_tensor = torch.empty_like(input_tensor)
        self._engine.exeOp(name, input_tensor, output_tensor)
        return output_tensor

    def execute_operation_async(self, name, input_tensor, output_tensor=None):
        if output_tensor is None:
            output_tensor = torch.empty_like(input_tensor)
        self._engine.exeOpAsync(name, input_tensor, output_tensor)
        return output_tensor

    def sync_operation(self, name) -> None:
        self._engine.syncOp(name)

    def reset_signals(self, name) -> None:
        self._engine.resetSignals(name)

    def get_endpoint(self) -> str:
        return self._engine.exportEndpoint()

    def update_endpoint(self, rank: int, endpoint: str) -> bool:
        return self._engine.updateEndpoint(rank, endpoint)

    # -- additions --------------------------------------------------------------------------
    def reset(self) -> None:
        """Zero signals / counters / status after an error.  Collective: call on
        every rank between two barriers."""
        self._engine.reset()

    def working_buffer(self, shape, dtype=torch.float32, offset_bytes: int = 0) -> torch.Tensor:
        return self._engine.workingBuffer(list(shape) if not isinstance(shape, int) else [shape],
                                          dtype, offset_bytes)

    def empty_symmetric(self, shape, dtype=torch.bfloat16):
        shape = [shape] if isinstance(shape, int) else list(shape)
        tensor, offset = self._engine.allocSymmetric(shape, dtype)
        tensor.heap_offset = offset
        return tensor

    def stats(self) -> Dict[str, Any]:
        return json.loads(self._engine.stats())

    def nvls_active(self) -> bool:
        return self._engine.nvlsActive()

    def set_timeout_ms(self, ms: int) -> None:
        self._engine.setTimeoutMs(int(ms))

    def set_trace(self, on: bool = True) -> None:
        """Device timeline on / off (also ``PCCL_TRACE=1``): while on, every step of a plan stamps
        ``%globaltimer`` when it is reached, when its data movement starts and ends and when its
        signals are posted.  The next launch after a change rebuilds the operation's tables."""
        self._engine.setTrace(bool(on))

    def trace(self, name: str) -> List[Dict[str, Any]]:
        """Steps of the most recent launch of ``name`` (after a synchronize): chain, step, kind,
        CTAs, bytes and the four stamps in nanoseconds since the launch's first stamp.
        ``pccl_b200.utils.trace.summarize`` turns it into a per-phase table."""
        return list(self._engine.trace(name))

    @property
    def rank(self) -> int:
        return self._engine.rank()

    @property
    def world(self) -> int:
        return self._engine.world()

    @property
    def native(self):
        return self._engine


class CpuEngine:
    """Engine surface on top of the CPU plan executor and a gloo group."""

    def __init__(self):
        self._plans: Dict[str, Dict[str, Any]] = {}
        self._all_plans: Dict[str, List[Dict[str, Any]]] = {}
        self.group = None

    def register_operation(self, name: str, filename: str) -> bool:
        if str(filename).lstrip().startswith("{"):
            return self.register_operation_from_string(name, str(filename))
        try:
            with open(filename) as handle:
                return self.register_operation_from_string(name, handle.read())
        except OSError:
            return False

    def register_operation_from_string(self, name: str, plan_json: str) -> bool:
        try:
            plan = json.loads(plan_json)
        except ValueError:
            return False
        if "operations" not in plan:          # phased manifests are split by the OCS runners
            return False
        self._plans[name] = plan
        self._all_plans.pop(name, None)
        return True

    def _gathered(self, name: str) -> List[Dict[str, Any]]:
        if name not in self._all_plans:
            if dist.is_initialized() and dist.get_world_size(self.group) > 1:
                box: List[Optional[Dict[str, Any]]] = [None] * dist.get_world_size(self.group)
                dist.all_gather_object(box, self._plans[name], group=self.group)
                self._all_plans[name] = box
            else:
                self._all_plans[name] = [self._plans[name]]
        return self._all_plans[name]

    def execute_operation(self, name, input_tensor, output_tensor=None):
        from .runtime.cpu_executor import GlooPlanExecutor, simulate
        if name not in self._plans:
            raise PCCLError(f"operation '{name}' is not registered")
        plans = self._gathered(name)
        flat = input_tensor.detach().reshape(-1).cpu()
        if len(plans) == 1:
            result = simulate(plans, [flat])[0]
        else:
            result = GlooPlanExecutor(self.group).execute(plans, flat)
        if output_tensor is None:
            output_tensor = torch.empty(result.numel(), dtype=input_tensor.dtype)
        output_tensor.reshape(-1)[:result.numel()].copy_(result)
        return output_tensor

    execute_operation_async = execute_operation

    def sync_operation(self, name) -> None:
        pass

    def reset_signals(self, name) -> None:
        pass

    def reset(self) -> None:
        pass

    def get_endpoint(self) -> str:
        rank = dist.get_rank() if dist.is_initialized() else 0
        return json.dumps({"version": 1, "rank": rank, "executor": "cpu"})

    def update_endpoint(self, rank: int, endpoint: str) -> bool:
        return True

    def stats(self) -> Dict[str, Any]:
        return {name: {"executor": "cpu"} for name in self._plans}

    def nvls_active(self) -> bool:
        return False


_engine_instance = None


def _use_cpu() -> bool:
    return os.environ.get("PCCL_EXECUTOR", "").lower() == "cpu" or not torch.cuda.is_available()


def get_engine():
    global _engine_instance
    if _engine_instance is None:
        _engine_instance = CpuEngine() if _use_cpu() else Engine()
    return _engine_instance


def register_operation(name, filename):
    return get_engine().register_operation(name, filename)


def execute_operation(name, input_tensor, output_tensor=None):
    return get_engine().execute_operation(name, input_tensor, output_tensor)


def execute_operation_async(name, input_tensor, output_tensor=None):
    return get_engine().execute_operation_async(name, input_tensor, output_tensor)


def sync_operation(name):
    return get_engine().sync_operation(name)


def reset_signals(name):
    return get_engine().reset_signals(name)


def get_endpoint():
    return get_engine().get_endpoint()


def reset_engine():
    return get_engine().reset()


def working_buffer(shape, dtype=torch.float32, offset_bytes: int = 0):
    return get_engine().working_buffer(shape, dtype, offset_bytes)


def empty_symmetric(shape, dtype=torch.bfloat16):
    return get_engine().empty_symmetric(shape, dtype)


def _all_agree(flag: bool, group) -> bool:
    """Logical AND of ``flag`` over the group (works on any backend)."""
    votes: List[Optional[bool]] = [None] * dist.get_world_size(group)
    dist.all_gather_object(votes, bool(flag), group=group)
    return all(votes)


def initialize_engine(group: Optional[dist.ProcessGroup] = None):
    """Connect the ranks of ``group``: exchange endpoints, map peers, bring up NVLS."""
    engine = get_engine()
    _debug_endpoint_init("engine_ready")
    if isinstance(engine, CpuEngine):
        engine.group = group
        if dist.is_initialized():
            dist.barrier(group=group)
        return engine

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    endpoint = engine.get_endpoint()
    _debug_endpoint_init("endpoint_exported")
    endpoints: List[Optional[str]] = [None] * world
    dist.all_gather_object(endpoints, endpoint, group=group)
    _debug_endpoint_init("endpoint_payloads_gathered")
    ok = True
    for peer, text in enumerate(endpoints):
        if peer != rank:
            ok &= bool(engine.update_endpoint(peer, text))
    _debug_endpoint_init("remote_endpoints_updated")
    if not _all_agree(ok, group):
        raise PCCLError("endpoint exchange failed on at least one rank (see PCCL_LOG_LEVEL=INFO output)")

    # NVLS: three stages separated by agreement rounds, which double as barriers.
    native = engine.native
    staged = True
    for stage in range(3):
        staged = _all_agree(staged and native.nvlsStage(stage), group)
        if not staged:
            break
    if not staged:
        native.nvlsDisable()
    dist.barrier(group=group)
    _debug_endpoint_init("barrier_complete")
    return engine
