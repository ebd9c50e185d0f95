"""Small helpers."""

from .to_tensor import to_str, to_tensor

__all__ = ["to_tensor", "to_str"]
