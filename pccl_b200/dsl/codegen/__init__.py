"""Plan serialisation (JSON v2 device plans, JSON v3 phased manifests)."""

from .mapping import get_executor_name, get_primitive_name
from .json_generator import RuntimeGraphGenerator, load_plan_graph

__all__ = ["get_primitive_name", "get_executor_name", "RuntimeGraphGenerator", "load_plan_graph"]
