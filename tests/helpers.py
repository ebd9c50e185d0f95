"""Helpers shared by the CPU-side tests."""

import socket

import torch

from pccl_b200.dsl.compiler import Compiler


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def build_plans(algorithm, kind, world, n, dtype="float32", executor="sm", channels=1, **compiler_kw):
    return [Compiler(**compiler_kw).compile_to_dict(
        getattr(algorithm, "build_" + kind)(r, world, n, dtype, executor, channels))
        for r in range(world)]


def make_inputs(kind, world, n, dtype=torch.float32):
    xs = []
    for r in range(world):
        g = torch.Generator().manual_seed(r)
        xs.append(torch.randn(n // world if kind == "allgather" else n, generator=g).to(dtype))
    return xs


def expected(kind, xs, world, n):
    """float64 reference result per rank."""
    xd = [x.double() for x in xs]
    if kind == "allreduce":
        return [sum(xd)] * world
    if kind == "reduce_scatter":
        s, c = sum(xd), n // world
        return [s[r * c:(r + 1) * c] for r in range(world)]
    if kind == "allgather":
        return [torch.cat(xd)] * world
    if kind == "alltoall":
        c = n // world
        return [torch.cat([xd[p][r * c:(r + 1) * c] for p in range(world)]) for r in range(world)]
    raise ValueError(kind)
