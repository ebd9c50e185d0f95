"""Latency of the OCS barrier-and-switch state machine and of one small collective call.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/ocs_barrier_bench.py \
        --iters 10000 [--connectors object,tensor,nvlink,board] [--backend gloo|nccl]

Part 1: `OCSRuntime.barrier_switch`, back to back, with
  object   pickled READY records through `all_gather_object` + `broadcast_object_list`
           (the reference's mechanism: pccl/ocs/runtime.py:139-203; its bench is
           tests/bench_ocs_barrier_latency.py:84-165),
  tensor   one fixed-size tensor all-gather + one 4-word broadcast on the process group,
  nvlink   `NvlinkSwitchConnector`: both rounds as single-CTA kernels that signal through the
           peers' symmetric memory, results read from mapped pinned memory,
  board    the signal board's bare barrier (one round, no state machine), the floor of `nvlink`.
Every rank times every barrier on its host clock; per barrier the slowest rank counts, and the
p50 / p99 / mean of that maximum are reported (the statistic of the reference's bench, lines 43-66).
Part 2 (nccl backend only): host overhead and device time of one 4 KB all-reduce through
`pccl.execute_operation` on a registered plan (in-heap tensor and ordinary tensor), through
`pccl_b200.parallel.all_reduce` (packet kernel) and through `dist.all_reduce`.
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


def slowest_rank_stats(samples_us, device):
    """p50 / p99 / mean over barriers of the per-barrier maximum over ranks."""
    mine = torch.tensor(samples_us, dtype=torch.float64, device=device)
    dist.all_reduce(mine, op=dist.ReduceOp.MAX)
    t = mine.sort().values
    pick = lambda q: float(t[min(len(t) - 1, int(q * len(t)))])
    return pick(0.5), pick(0.99), float(t.mean())


def max_over_ranks(values, device):
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10000)
    ap.add_argument("--slow-iters", type=int, default=0, help="iterations of the object connector (default: --iters)")
    ap.add_argument("--connectors", default="object,tensor,nvlink,board")
    ap.add_argument("--backend", default=None)
    ap.add_argument("--calls", type=int, default=1000, help="back-to-back calls of part 2")
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
    from pccl_b200.ocs.runtime import (NvlinkSwitchConnector, TensorSwitchConnector,
                                       TorchDistributedSwitchConnector)

    wanted = [c for c in args.connectors.split(",") if c]
    native_ok = backend == "nccl" and world > 1
    if native_ok and any(c in ("nvlink", "board") for c in wanted):
        import pccl_b200.parallel as pp
        pp.init()
    nvlink = NvlinkSwitchConnector() if native_ok and any(c in ("nvlink", "board") for c in wanted) else None

    for label in wanted:
        if label in ("nvlink", "board") and nvlink is None:
            continue
        iters = (args.slow_iters or args.iters) if label == "object" else args.iters
        lat = []
        if label == "board":
            for i in range(iters + 50):
                t0 = time.perf_counter_ns()
                ok, missing, _ = nvlink.board.barrier(2_000_000)
                if not ok:
                    raise RuntimeError(f"signal board barrier {i}: rank {missing} missing")
                if i >= 50:
                    lat.append((time.perf_counter_ns() - t0) / 1e3)
        else:
            connector = {"object": TorchDistributedSwitchConnector, "tensor": TensorSwitchConnector}.get(label)
            runtime = OCSRuntime(connector=nvlink if label == "nvlink" else connector())
            for i in range(iters + 50):
                plan = OCSPlan(job_id="bench", group_id=0, barrier_id=i, epoch_id=i, next_epoch_id=i + 1,
                               topology_id=i % 2)
                t0 = time.perf_counter_ns()
                runtime.barrier_switch(plan)
                if i >= 50:
                    lat.append((time.perf_counter_ns() - t0) / 1e3)
                runtime.history.clear()
        p50, p99, mean = slowest_rank_stats(lat, device)
        if rank == 0:
            print(json.dumps({"bench": "ocs_barrier_switch", "connector": label, "backend": backend, "world": world,
                              "iters": iters, "p50_us": round(p50, 1), "p99_us": round(p99, 1),
                              "mean_us": round(mean, 1),
                              "clock": "host perf_counter per barrier, max over ranks per barrier"}), flush=True)

    if backend == "nccl" and world > 1:
        import pccl_b200 as pccl
        import pccl_b200.parallel as pp
        pp.init()
        numel = 1024                                   # 4 KB of fp32
        x = pp.working_tensor(numel, torch.float32)
        y = torch.zeros(numel, device="cuda")
        z = torch.zeros(numel, device="cuda")
        name = pp.ensure_plan("allreduce", numel, torch.float32, "oneshot", 1)

        def measure(fn, sync):
            for _ in range(20):
                fn()
            sync()
            dist.barrier()
            host0 = time.perf_counter_ns()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.calls):
                fn()
            b.record()
            host_us = (time.perf_counter_ns() - host0) / 1e3 / args.calls
            sync()
            return host_us, a.elapsed_time(b) * 1e3 / args.calls

        rows = {
            "execute_operation_in_heap": measure(lambda: pccl.execute_operation_async(name, x, x),
                                                 lambda: pccl.sync_operation(name)),
            "execute_operation_staged": measure(lambda: pccl.execute_operation_async(name, y, z),
                                                lambda: pccl.sync_operation(name)),
            "parallel_all_reduce_packet_kernel": measure(lambda: pp.all_reduce(y), lambda: pp.synchronize(name)),
            "nccl_all_reduce": measure(lambda: dist.all_reduce(y), torch.cuda.synchronize),
        }
        flat = max_over_ranks([v for pair in rows.values() for v in pair], device)
        if rank == 0:
            out = {"bench": "allreduce_4KB_call", "world": world, "calls": args.calls,
                   "note": "back-to-back calls; host = wall clock of the issuing loop / calls, device = CUDA events "
                           "/ calls, max over ranks; execute_operation runs the registered one-shot plan"}
            for i, key in enumerate(rows):
                out[key] = {"host_us": round(flat[2 * i], 2), "device_us": round(flat[2 * i + 1], 2)}
            print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
