"""Names used in plan JSON (reference: pccl/dsl/codegen/mapping.py:7-26)."""

from __future__ import annotations

from typing import Dict

from ..nodes import ExecutorType, IRNodeVariant

_EXECUTOR_NAME_MAP: Dict[ExecutorType, str] = {
    ExecutorType.SM: "cuda_sm",
    ExecutorType.TMA: "cuda_tma",
    ExecutorType.CE: "cuda_ce",
    ExecutorType.HOST: "host",
    ExecutorType.RDMA: "cuda_rdma",
    ExecutorType.MULTIMEM: "cuda_multimem",
}

EXECUTOR_FROM_NAME: Dict[str, ExecutorType] = {v: k for k, v in _EXECUTOR_NAME_MAP.items()}


def get_primitive_name(node: IRNodeVariant) -> str:
    """The ``primitive`` string of an operation: the op type's value."""
    return node.op_type.value


def get_executor_name(node: IRNodeVariant) -> str:
    """The ``executor`` string of an operation; nodes without one run on the host."""
    return _EXECUTOR_NAME_MAP.get(node.executor, "host") if node.executor else "host"
