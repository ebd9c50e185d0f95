"""Latency of the OCS barrier-and-switch state machine and of one small collective call.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/ocs_barrier_bench.py \
        --iters 10000 [--backend gloo|nccl]

Part 1: `OCSRuntime.barrier_switch` with the object connector (pickled READY records through
`all_gather_object`, the reference's mechanism: pccl/ocs/runtime.py:150-199) and with the tensor
connector (one fixed-size all-gather + one 4-word broadcast).  Per-rank wall-clock latencies,
p50 / p99 of the slowest rank.
Part 2 (nccl backend only): host overhead and device time of one 4 KB all-reduce through
`execute_operation` against `dist.all_reduce`.
One JSON line per measurement on rank 0.
"""

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def percentiles(samples_us):
    t = torch.tensor(sorted(samples_us), dtype=torch.float64)
    pick = lambda q: float(t[min(len(t) - 1, int(q * len(t)))])
    return pick(0.5), pick(0.99), float(t.mean())


def max_over_ranks(values, device):
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10000)
    ap.add_argument("--backend", default=None)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    backend = args.backend or ("nccl" if torch.cuda.is_available() else "gloo")
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    else:
        dist.init_process_group("gloo")
    device = torch.device("cuda") if backend == "nccl" else torch.device("cpu")

    from pccl_b200.ocs import OCSPlan, OCSRuntime
    from pccl_b200.ocs.runtime import TensorSwitchConnector, TorchDistributedSwitchConnector

    for label, connector in (("object_connector", TorchDistributedSwitchConnector()),
                             ("tensor_connector", TensorSwitchConnector())):
        runtime = OCSRuntime(connector=connector)
        lat = []
        for i in range(args.iters + 20):
            plan = OCSPlan(job_id="bench", group_id=0, barrier_id=i, epoch_id=i, next_epoch_id=i + 1,
                           topology_id=i % 2)
            t0 = time.perf_counter_ns()
            runtime.barrier_switch(plan)
            if i >= 20:
                lat.append((time.perf_counter_ns() - t0) / 1e3)
            runtime.history.clear()
        p50, p99, mean = max_over_ranks(list(percentiles(lat)), device)
        if rank == 0:
            print(json.dumps({"bench": "ocs_barrier_switch", "connector": label, "backend": backend, "world": world,
                              "iters": args.iters, "p50_us": round(p50, 1), "p99_us": round(p99, 1),
                              "mean_us": round(mean, 1), "clock": "host perf_counter, max over ranks"}), flush=True)

    if backend == "nccl":
        import pccl_b200.parallel as pp
        pp.init()
        numel = 1024                                   # 4 KB of fp32
        x = pp.working_tensor(numel, torch.float32)
        y = torch.zeros(numel, device="cuda")
        name = pp.ensure_plan("allreduce", numel, torch.float32)

        def measure(fn, sync):
            for _ in range(20):
                fn()
            sync()
            dist.barrier()
            host0 = time.perf_counter_ns()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(1000):
                fn()
            b.record()
            host_us = (time.perf_counter_ns() - host0) / 1e3 / 1000
            sync()
            return host_us, a.elapsed_time(b)

        ours = measure(lambda: pp.all_reduce(x, async_op=True), lambda: pp.synchronize(name))
        nccl = measure(lambda: dist.all_reduce(y), torch.cuda.synchronize)
        vals = max_over_ranks([ours[0], ours[1], nccl[0], nccl[1]], device)
        if rank == 0:
            print(json.dumps({"bench": "allreduce_4KB_call", "world": world,
                              "ours_host_us_per_call": round(vals[0], 2), "ours_device_us_per_call": round(vals[1], 2),
                              "nccl_host_us_per_call": round(vals[2], 2), "nccl_device_us_per_call": round(vals[3], 2),
                              "note": "1000 back-to-back calls; device = CUDA events / 1000, max over ranks"}),
                  flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
