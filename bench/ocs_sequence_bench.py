"""What the OCS control boundaries cost on top of the collectives they separate.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench/ocs_sequence_bench.py \
        [--elements 1048576] [--iterations 50] [--connectors tensor,nvlink]

The sequence all-reduce -> all-to-all -> all-reduce is run five ways on the same input:
  native            three `torch.distributed` (NCCL) calls, no boundaries;
  torch_plan        `OcsTorchPlanRunner`: the same calls with an OCS barrier-and-switch after the
                    first and the second (the comparison of the reference's
                    tests/bench_ocs_torch_overhead.py:105-200);
  engine_plan       `OcsCollectivePlanRunner` over this library's engine: every phase is a compiled
                    ring plan, registered (once; later executions reuse the registration) and
                    executed through register_operation / execute_operation, with the same barriers
                    and a signal reset after each;
  engine_plan_switched  the same runner over two-shot all-reduce and direct all-to-all plans, the
                    templates made for a switched fabric;
  engine_native     the three engine plans run back to back without barriers.
Each iteration is timed on the host between two device synchronisations; per iteration the
slowest rank counts; median and p95 over iterations.  Results of all four are checked against the
closed form.  One JSON line per variant and connector on rank 0.
"""

import argparse
import json
import os
import statistics
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def summary(per_iteration_us):
    ordered = sorted(per_iteration_us)
    return {"median_us": round(statistics.median(ordered), 1),
            "p95_us": round(ordered[int(round((len(ordered) - 1) * 0.95))], 1)}


def slowest_rank(samples_us):
    t = torch.tensor(samples_us, dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--elements", type=int, default=1 << 20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iterations", type=int, default=50)
    ap.add_argument("--connectors", default="tensor,nvlink")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    if args.elements % world:
        raise SystemExit("--elements must be divisible by the world size")

    import pccl_b200 as pccl
    import pccl_b200.parallel as pp
    from pccl_b200.ocs import (NvlinkSwitchConnector, OcsCollectivePlanRunner, OCSRuntime, OcsTorchPlanRunner,
                               TensorSwitchConnector, TorchDistributedSwitchConnector,
                               build_ring_allreduce_alltoall_plan, build_switched_allreduce_alltoall_plan,
                               build_torch_allreduce_alltoall_plan)
    pp.init()
    x = torch.full((args.elements,), float(rank + 1), device="cuda")
    # every element: sum of ranks' values, exchanged (unchanged: all equal), summed again
    expected = float(sum(range(1, world + 1)) * world)
    total = args.warmup + args.iterations

    def timed(run_once):
        out, lat = None, []
        for i in range(total):
            torch.cuda.synchronize()
            dist.barrier()
            t0 = time.perf_counter_ns()
            out = run_once(i)
            torch.cuda.synchronize()
            if i >= args.warmup:
                lat.append((time.perf_counter_ns() - t0) / 1e3)
        if not torch.equal(out, torch.full_like(out, expected)):
            raise RuntimeError("sequence produced an unexpected result")
        return slowest_rank(lat)

    def native(_):
        a = x.clone()
        dist.all_reduce(a)
        b = torch.empty_like(a)
        dist.all_to_all_single(b, a)
        dist.all_reduce(b)
        return b

    results = [("native", None, timed(native), None)]

    connectors = {"object": TorchDistributedSwitchConnector, "tensor": TensorSwitchConnector,
                  "nvlink": NvlinkSwitchConnector}
    engine_files = None
    for label in [c for c in args.connectors.split(",") if c]:
        connector = connectors[label]()
        runtime = OCSRuntime(connector=connector)
        torch_runner = OcsTorchPlanRunner(runtime=runtime)
        torch_plans = [build_torch_allreduce_alltoall_plan(world, first_barrier_id=2 * i, first_epoch_id=2 * i)
                       for i in range(total)]
        lat = timed(lambda i: torch_runner.execute(torch_plans[i], x))
        barriers = [float(r["latency_us"]) for r in runtime.history[2 * args.warmup:]]
        results.append(("torch_plan", label, lat, slowest_rank(barriers)))

        runtime = OCSRuntime(connector=connector)
        engine_runner = OcsCollectivePlanRunner(engine=pccl.engine, runtime=runtime)
        prepared = [engine_runner.prepare(
            build_ring_allreduce_alltoall_plan(rank, world, args.elements, "float32", "sm",
                                               first_barrier_id=2 * i, first_epoch_id=2 * i), f"seq{label}")
            for i in range(1)]
        # One prepared plan serves every iteration: barrier ids only have to agree between ranks.
        lat = timed(lambda i: engine_runner.execute(prepared[0], x))
        barriers = [float(r["latency_us"]) for r in runtime.history[2 * args.warmup:]]
        results.append(("engine_plan", label, lat, slowest_rank(barriers)))
        engine_files = prepared[0]

        # The same sequence with the templates made for a switched fabric (two-shot, direct all-to-all).
        runtime = OCSRuntime(connector=connector)
        switched_runner = OcsCollectivePlanRunner(engine=pccl.engine, runtime=runtime)
        switched = switched_runner.prepare(
            build_switched_allreduce_alltoall_plan(rank, world, args.elements, "float32", "sm"), f"sw{label}")
        lat = timed(lambda i: switched_runner.execute(switched, x))
        barriers = [float(r["latency_us"]) for r in runtime.history[2 * args.warmup:]]
        results.append(("engine_plan_switched", label, lat, slowest_rank(barriers)))

    if engine_files is not None:
        names = list(engine_files.operation_names)
        for name, path in zip(names, engine_files.phase_files):
            pccl.register_operation(name + "_nb", str(path))
        dist.barrier()

        def engine_native(_):
            cur = x
            for name in names:
                nxt = torch.empty_like(cur)
                pccl.execute_operation_async(name + "_nb", cur, nxt)
                cur = nxt
            return cur
        results.append(("engine_native", None, timed(engine_native), None))

    if rank == 0:
        for variant, label, lat, barriers in results:
            row = {"bench": "ocs_sequence", "variant": variant, "connector": label, "world": world,
                   "elements": args.elements, "iterations": args.iterations, "completion": summary(lat)}
            if barriers:
                row["barrier_completion"] = summary(barriers)
                row["barriers_per_iteration"] = 2
            print(json.dumps(row), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
