"""Shared machinery of the two engine-backed OCS runners.

Both runners materialise a list of (operation name, plan file, barrier after)
triples and then run the same loop: register the phase's plan, fence the ranks,
execute, commit the barrier, reset the signal space (reference:
pccl/ocs/phase_runner.py:120-176 and pccl/ocs/collective_plan.py:137-172 hold
two copies of this loop).
"""

from __future__ import annotations

import shutil
import tempfile
from pathlib import Path
from typing import Any, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .plan import OCSPlan
from .runtime import OCSRuntime


class EngineBackedRunner:
    """Holds the engine (any object with ``register_operation`` /
    ``execute_operation`` / optional ``reset_signals``), the OCS runtime, the
    compiler and the directory plan files are written to."""

    _tmp_prefix = "pccl-ocs-"

    def __init__(self, engine: Any = None, runtime: Optional[OCSRuntime] = None,
                 compiler: Any = None, json_dir: Optional[str] = None) -> None:
        from ..dsl.compiler import Compiler
        self.engine = engine
        self.runtime = runtime if runtime is not None else OCSRuntime()
        self.compiler = compiler if compiler is not None else Compiler()
        self.json_dir = Path(json_dir) if json_dir is not None else None
        #: a prepared plan that is executed again keeps its operations registered: the second and later
        #: executions skip the registration and the host barrier that orders it (set False to register
        #: at every execution)
        self.reuse_registrations = True
        self._live: dict = {}

    def _create_json_dir(self) -> Tuple[Path, bool]:
        """(directory, whether this runner owns and may delete it)."""
        if self.json_dir is not None:
            self.json_dir.mkdir(parents=True, exist_ok=True)
            return self.json_dir, False
        return Path(tempfile.mkdtemp(prefix=self._tmp_prefix)), True

    def _engine(self) -> Any:
        if self.engine is None:
            from .. import engine as default_engine
            self.engine = default_engine
        return self.engine

    def _reset_signals(self, operation_name: str) -> None:
        reset = getattr(self._engine(), "reset_signals", None)
        if callable(reset):
            reset(operation_name)

    @staticmethod
    def _synchronize_phase_registration(group: Optional[dist.ProcessGroup]) -> None:
        """All ranks must have registered before any rank's kernel posts a
        signal into a peer."""
        if dist.is_initialized():
            dist.barrier(group=group)

    def _run_phases(self, names: Sequence[Optional[str]], files: Sequence[Optional[Path]],
                    barriers: Sequence[Optional[OCSPlan]], input_tensor: torch.Tensor,
                    output_tensor: Optional[torch.Tensor], group, timeout,
                    what: str) -> torch.Tensor:
        data_phases = [i for i, name in enumerate(names) if name is not None]
        last = data_phases[-1] if data_phases else -1
        current = input_tensor
        # A signal reset must never run while a peer may already post the next phase's signals.
        # First execution (the reference's order): execute, barrier, reset, and the host barrier that
        # follows the next registration orders the reset before any peer's next kernel.  Reused
        # registrations have no such host barrier, so there the reset moves in front of the OCS
        # barrier: execute_operation is blocking and plans are balanced, hence every signal posted to
        # this rank in the phase has been consumed when it returns, and the OCS barrier then separates
        # the reset from the peers' next phase.
        reset_unfenced = False
        for i, (name, path) in enumerate(zip(names, files)):
            reused = False
            if name is not None:
                if path is None:
                    raise RuntimeError("data phase is missing its generated JSON")
                target = output_tensor if (i == last and output_tensor is not None) \
                    else torch.empty_like(current)
                reused = self.reuse_registrations and self._live.get(name) == str(path)
                if not reused:
                    self._live.pop(name, None)
                    if not self._engine().register_operation(name, str(path)):
                        raise RuntimeError(f"failed to register {what} '{name}'")
                    self._synchronize_phase_registration(group)
                    self._live[name] = str(path)
                elif reset_unfenced:
                    self._synchronize_phase_registration(group)
                reset_unfenced = False
                # execute_operation is blocking, so the host barrier below
                # cannot overtake this phase's device work.
                self._engine().execute_operation(name, current, target)
                current = target
            if barriers[i] is not None:
                if name is not None and reused:
                    self._reset_signals(name)
                self.runtime.barrier_switch(barriers[i], group=group, timeout=timeout)
                if name is not None and not reused:
                    self._reset_signals(name)
                    reset_unfenced = True
        return current


def discard_dir(path: Path, owned: bool) -> None:
    if owned:
        shutil.rmtree(path, ignore_errors=True)
