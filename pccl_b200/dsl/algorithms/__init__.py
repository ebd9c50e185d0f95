"""Collective algorithm templates and their selector."""

from .base import CollectiveAlgorithm
from .ring import RingAllreduce
from .recursive_hd import RecursiveHalvingDoubling
from .tree import TreeAllreduce
from .direct import (DirectCollectives, HybridAllreduce, NvlsAllreduce, NvlsTwoPassAllreduce, OneShotAllreduce,
                     TwoShotAllreduce)
from .selector import select_algorithm, select_algorithm_cost_based

ALGORITHMS = {
    "ring": RingAllreduce,
    "rhd": RecursiveHalvingDoubling,
    "tree": TreeAllreduce,
    "oneshot": OneShotAllreduce,
    "twoshot": TwoShotAllreduce,
    "nvls": NvlsAllreduce,
    "nvls_twopass": NvlsTwoPassAllreduce,
    "hybrid": HybridAllreduce,
}

__all__ = [
    "CollectiveAlgorithm", "RingAllreduce", "RecursiveHalvingDoubling", "TreeAllreduce",
    "OneShotAllreduce", "TwoShotAllreduce", "NvlsAllreduce", "NvlsTwoPassAllreduce", "HybridAllreduce",
    "DirectCollectives",
    "ALGORITHMS", "select_algorithm", "select_algorithm_cost_based",
]
