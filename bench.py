"""Headline benchmark: AllReduce (SUM) bus bandwidth at 512 MB fp32.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

Prints one JSON line (rank 0).  ``value`` is the bus bandwidth in GB/s,
``algbw * 2(N-1)/N``, of an in-place all-reduce on the engine's symmetric working
buffer, timed on the device with CUDA events (K back-to-back steps between two
barriers, max over ranks).  The 512 MB message is four times the 126 MB L2, so
no explicit L2 flush is needed between iterations.

N = 1 has no peer to reduce with.  It runs the same kernels as two *virtual*
ranks on the one GPU (one cooperative launch, peer copies through HBM instead of
NVLink) and reports the two-rank bus-bandwidth formula; ``config.parallelism``
says so.

``e2e`` repeats the measurement through the public API including, per step, the
host-to-device copy of the step's input from pinned memory and a device-to-host
read of a slice of the result.

``--impl reference`` runs the unmodified reference from ``baseline/_ref`` for the
same metric, or prints why it cannot.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MESSAGE_BYTES = 512 << 20
PUBLISHED = {2: 246.4, 4: 274.8, 8: 282.0}     # the reference's published 512 MB bus GB/s (bf16, H100; its README.md:97-99)


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs.

    Reads NVML from a polling thread (about one sample per millisecond, so that even a
    timed region of a few milliseconds is covered); read-only, nothing is set.
    """

    def __init__(self, index: int):
        self.index, self.samples, self.stop_flag, self.thread, self.max_mhz = index, [], False, None, None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._poll, args=(handle,), daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001 - no NVML: report "unsampled"
            self.thread = None
        return self

    def _poll(self, handle):
        nv = self.nvml
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except AttributeError:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((mhz, int(reasons)))
            except Exception:  # noqa: BLE001
                break
            time.sleep(0.001)

    def __exit__(self, *exc):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        seen = 0
        for _, r in self.samples:
            seen |= r
        reasons = [name for name, bit in bits.items() if seen & bit]
        return {"sm_mhz": statistics.median(m for m, _ in self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.samples)}


def bus_factor(n: int) -> float:
    return 2.0 * (n - 1) / n


def run_ours(args):
    import torch
    import torch.distributed as dist

    n_gpus = args.gpus
    numel = args.bytes // 4
    if n_gpus == 1:
        return run_single_gpu(args, numel)

    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    os.environ.setdefault("PCCL_BUFFER_SIZE", str(max(1 << 30, 2 * args.bytes)))
    os.environ.setdefault("PCCL_WAIT_TIMEOUT_MS", "4000")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import pccl_b200.parallel as pp
    engine = pp.init()

    x = pp.working_tensor(numel, torch.float32)
    host_in = torch.randn(numel, generator=torch.Generator().manual_seed(rank)).pin_memory()
    host_out = torch.empty(1024, dtype=torch.float32).pin_memory()
    x.copy_(host_in, non_blocking=True)
    ref = sum(torch.randn(numel, generator=torch.Generator().manual_seed(r))[:4096].double() for r in range(world))

    # Pick the algorithm outside the timed region: unless one is forced, the selector's choice and the
    # other large-message templates are each run once for correctness (first 4096 elements against a
    # float64 sum of every rank's input) and three times for speed; all ranks agree on the outcome
    # through NCCL, a candidate that fails or is wrong on any rank is dropped.
    from pccl_b200 import engine as _eng
    candidates = [args.algo] if args.algo else [None, "twoshot", "ring"] + (["nvls"] if engine.nvls_active() else [])
    best, tried = None, {}
    for algo in candidates:
        ok, err, t_ms, plan = 1, float("inf"), float("inf"), None
        try:
            plan = pp.ensure_plan("allreduce", numel, torch.float32, algo, args.channels)
            x.copy_(host_in, non_blocking=True)
            pp.all_reduce(x, algorithm=algo, channels=args.channels)
            err = float((x[:4096].double().cpu() - ref).abs().max())
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(3):
                pp.all_reduce(x, algorithm=algo, channels=args.channels, async_op=True)
            b.record()
            pp.synchronize(plan)
            t_ms = a.elapsed_time(b) / 3
        except Exception as failure:  # noqa: BLE001 - a failing candidate is skipped, not fatal
            ok = 0
            sys.stderr.write(f"[bench] rank {rank}: candidate {algo or 'auto'} failed: {failure}\n")
        verdict = torch.tensor([float(ok and err < 1e-3), -t_ms if t_ms != float("inf") else -1e9],
                               device="cuda", dtype=torch.float64)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
        good, t_all = bool(verdict[0].item() > 0.5), -float(verdict[1].item())
        if not good:
            torch.cuda.synchronize()
            dist.barrier()
            if plan is not None:
                _eng.reset_signals(plan)
            dist.barrier()
            continue
        tried[algo or "auto"] = round(t_all, 4)
        if best is None or t_all < best[1]:
            best = (algo, t_all, plan, err)
    if best is None:
        raise RuntimeError("no all-reduce algorithm produced a correct result on every rank")
    chosen, _, name, max_err = best

    def step():
        pp.all_reduce(x, algorithm=chosen, channels=args.channels, async_op=True)

    for _ in range(args.warmup):
        step()
    pp.synchronize(name)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        torch.cuda.synchronize()
        dist.barrier()
    pp.synchronize(name)
    ms = start.elapsed_time(stop) / args.steps

    # end to end: H2D of the input, all-reduce, D2H of a slice of the result, every step
    def e2e_step():
        x.copy_(host_in, non_blocking=True)
        pp.all_reduce(x, algorithm=chosen, channels=args.channels, async_op=True)
        host_out.copy_(x[:1024], non_blocking=True)

    for _ in range(min(2, args.warmup)):
        e2e_step()
    pp.synchronize(name)
    dist.barrier()
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.steps):
        e2e_step()
    stop.record()
    torch.cuda.synchronize()
    dist.barrier()
    e2e_ms = start.elapsed_time(stop) / args.steps

    times = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()
    stats = engine.stats().get(name, {})
    result = None
    if rank == 0:
        value = args.bytes / (ms * 1e-3) / 1e9 * bus_factor(world)
        e2e = args.bytes / (e2e_ms * 1e-3) / 1e9 * bus_factor(world)
        kind, algorithm, channels = pp.registered_plans()[name]
        result = {
            "metric": "allreduce_bus_bandwidth_512MB_fp32", "value": round(value, 2), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / PUBLISHED[world], 3) if world in PUBLISHED else None,
            "dtype": "fp32", "data": "synthetic randn(seed=rank)",
            "config": {"model": "allreduce_sum", "global_batch": args.bytes, "seq_len": numel,
                       "parallelism": f"dp{world}", "algorithm": algorithm, "channels": channels,
                       "nvls": bool(engine.nvls_active()), "ctas": stats.get("ctas"),
                       "in_place": True, "l2": "message (512 MB) exceeds the 126 MB L2; no flush needed",
                       "max_abs_err_first_4096": max_err,
                       "candidates_ms": tried},
            "clocks": clocks.summary(),
            "e2e": {"value": round(e2e, 2), "unit": "GB/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": args.bytes, "d2h_bytes_per_step": 4096},
            "gpu_launches": args.steps,
        }
        print(json.dumps(result), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return result


def run_single_gpu(args, numel):
    """Two virtual ranks on one GPU through the same interpreter kernel."""
    import torch
    from pccl_b200 import Compiler, engine_c
    from pccl_b200.dsl.algorithms import ALGORITHMS

    torch.cuda.set_device(0)
    world = 2
    algorithm = args.algo or "twoshot"
    channels = args.channels or 8
    cluster = engine_c.LocalCluster(world, 0, args.bytes + (64 << 20))
    plans = [Compiler().compile_to_json(
        ALGORITHMS[algorithm]().build_allreduce(r, world, numel, "float32", "sm", channels)) for r in range(world)]
    cluster.regOp("bench_ar", plans)
    host_in = [torch.randn(numel, generator=torch.Generator().manual_seed(r)).pin_memory() for r in range(world)]
    host_out = torch.empty(1024, dtype=torch.float32).pin_memory()
    xs = [torch.empty(numel, device="cuda") for _ in range(world)]
    outs = [torch.empty(numel, device="cuda") for _ in range(world)]
    for x, h in zip(xs, host_in):
        x.copy_(h)

    def step():
        cluster.exeOp("bench_ar", xs, outs)

    step()
    ref = host_in[0][:4096].double() + host_in[1][:4096].double()
    max_err = float((outs[0][:4096].double().cpu() - ref).abs().max())
    for _ in range(args.warmup):
        step()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    with ClockSampler(0) as clocks:
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / args.steps

    def e2e_step():
        for x, h in zip(xs, host_in):
            x.copy_(h, non_blocking=True)
        cluster.exeOp("bench_ar", xs, outs)
        host_out.copy_(outs[0][:1024], non_blocking=True)

    e2e_step()
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.steps):
        e2e_step()
    stop.record()
    torch.cuda.synchronize()
    e2e_ms = start.elapsed_time(stop) / args.steps

    value = args.bytes / (ms * 1e-3) / 1e9 * bus_factor(world)
    e2e = args.bytes / (e2e_ms * 1e-3) / 1e9 * bus_factor(world)
    info = cluster.opInfo("bench_ar", 0)
    result = {
        "metric": "allreduce_bus_bandwidth_512MB_fp32", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic randn(seed=rank)",
        "config": {"model": "allreduce_sum", "global_batch": args.bytes, "seq_len": numel,
                   "parallelism": "2 virtual ranks on 1 GPU (peer copies through HBM, staged in/out copies timed)",
                   "algorithm": algorithm, "channels": channels, "ctas_per_rank": int(info["ctas"]),
                   "l2": "message (512 MB) exceeds the 126 MB L2; no flush needed",
                   "max_abs_err_first_4096": max_err},
        "clocks": clocks.summary(),
        "e2e": {"value": round(e2e, 2), "unit": "GB/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": 2 * args.bytes, "d2h_bytes_per_step": 4096},
        "gpu_launches": args.steps,
    }
    print(json.dumps(result), flush=True)
    return result


def run_reference(args):
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_bench
    except Exception as err:  # noqa: BLE001 - any failure means the arm is unavailable
        print(json.dumps({"impl": "reference", "unavailable": f"reference harness not importable: {err}"}))
        return
    reference_bench.main(args)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bytes", type=int, default=MESSAGE_BYTES)
    ap.add_argument("--algo", default=None)
    ap.add_argument("--channels", type=int, default=None)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
