"""Helpers of the GPU tests: run plans on a LocalCluster (N virtual ranks, one GPU)."""

import torch

from helpers import build_plans, expected, make_inputs

TOL = {torch.float32: dict(atol=1e-5, rtol=1e-5), torch.bfloat16: dict(atol=0.08, rtol=2 ** -6),
       torch.float16: dict(atol=0.01, rtol=2 ** -9)}
DTYPE_NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16"}


def new_cluster(world, buffer_bytes=32 << 20, timeout_ms=4000):
    from pccl_b200 import engine_c
    cluster = engine_c.LocalCluster(world, 0, buffer_bytes)
    cluster.setTimeoutMs(timeout_ms)
    return cluster


def run_on_cluster(cluster, name, plans, xs, out_numel):
    import json
    texts = [p if isinstance(p, str) else json.dumps(p) for p in plans]
    cluster.regOp(name, texts)
    dev_in = [x.cuda() for x in xs]
    # Outputs sit between guard elements that must come back untouched: a kernel that writes one vector
    # too far (odd sizes, clamped tails) is caught here instead of corrupting a neighbour silently.
    guard = 64
    padded = [torch.full((out_numel + 2 * guard,), float("nan"), device="cuda", dtype=xs[0].dtype) for _ in xs]
    for buf in padded:
        buf[:guard] = 12345.0
        buf[guard + out_numel:] = 12345.0
    dev_out = [buf[guard:guard + out_numel] for buf in padded]
    cluster.exeOp(name, dev_in, dev_out)
    torch.cuda.synchronize()
    for r, buf in enumerate(padded):
        assert bool((buf[:guard] == 12345.0).all()) and bool((buf[guard + out_numel:] == 12345.0).all()), \
            f"{name}: rank {r} wrote outside its output"
    return [o.cpu() for o in dev_out]


def check_collective(cluster, algorithm, kind, world, n, dtype=torch.float32, channels=1, repeats=1, tag=""):
    plans = build_plans(algorithm, kind, world, n, DTYPE_NAME[dtype], "sm", channels)
    xs = make_inputs(kind, world, n, dtype)
    out_numel = n // world if kind == "reduce_scatter" else n
    name = f"{algorithm.name}_{kind}_{world}_{n}_{DTYPE_NAME[dtype]}_{channels}{tag}"
    refs = expected(kind, xs, world, n)
    for _ in range(repeats):
        outs = run_on_cluster(cluster, name, plans, xs, out_numel)
        for r, (out, ref) in enumerate(zip(outs, refs)):
            torch.testing.assert_close(out.double(), ref, msg=lambda m: f"{name} rank {r}: {m}", **TOL[dtype])
