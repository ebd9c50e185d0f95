"""Parallelism layer: collectives API and tensor-/expert-parallel building blocks."""

from .collectives import (all_gather, all_reduce, all_to_all, check_errors, default_channels, ensure_lean_push,
                          ensure_plan, init,
                          reduce_scatter, registered_plans, reset, synchronize, working_tensor)

__all__ = ["init", "all_reduce", "all_gather", "reduce_scatter", "all_to_all", "working_tensor",
           "ensure_plan", "ensure_lean_push", "default_channels", "registered_plans", "synchronize", "reset", "check_errors"]


def __getattr__(name):
    if name in ("ColumnParallelLinear", "RowParallelLinear", "ExpertParallelMoE", "GradientBuckets"):
        from . import layers
        return getattr(layers, name)
    raise AttributeError(name)
