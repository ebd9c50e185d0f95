"""Collective algorithm templates and their selector."""

from .base import CollectiveAlgorithm
from .ring import RingAllreduce
from .recursive_hd import RecursiveHalvingDoubling
from .tree import TreeAllreduce
from .direct import DirectCollectives, NvlsAllreduce, OneShotAllreduce, TwoShotAllreduce
from .selector import select_algorithm, select_algorithm_cost_based

ALGORITHMS = {
    "ring": RingAllreduce,
    "rhd": RecursiveHalvingDoubling,
    "tree": TreeAllreduce,
    "oneshot": OneShotAllreduce,
    "twoshot": TwoShotAllreduce,
    "nvls": NvlsAllreduce,
}

__all__ = [
    "CollectiveAlgorithm", "RingAllreduce", "RecursiveHalvingDoubling", "TreeAllreduce",
    "OneShotAllreduce", "TwoShotAllreduce", "NvlsAllreduce", "DirectCollectives",
    "ALGORITHMS", "select_algorithm", "select_algorithm_cost_based",
]
