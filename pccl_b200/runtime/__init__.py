"""Reference executors that need no GPU."""

from .cpu_executor import GlooPlanExecutor, PlanDeadlock, global_schedule, simulate

__all__ = ["simulate", "global_schedule", "GlooPlanExecutor", "PlanDeadlock"]
