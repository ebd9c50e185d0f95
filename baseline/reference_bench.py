"""Reference arm of bench.py: the unmodified reference from ``baseline/_ref``.

The reference is installed with

    python -m pip install --no-index --no-build-isolation --no-deps \
        --find-links /opt/wheelhouse --target baseline/_ref <reference checkout>

and driven here through its own public API and stock code path only: its DSL
templates and ``Compiler(enable_superopt=True)`` produce the plan file,
``pccl.engine.initialize_engine / register_operation / execute_operation_async /
sync_operation`` run it (the call sequence of the reference's own
tests/bench_algo_comparison.py:81-152).  Nothing of pccl_b200 is imported.

Same metric and JSON line as ``bench.py``, with ``"impl": "reference"``.  The
reference publishes "best of its algorithms" per size, so ring and (for
power-of-two worlds) recursive halving-doubling are both timed and the faster is
reported.  When the reference cannot run, one line with ``"unavailable"`` is
printed and the exit status is 0.
"""

import ctypes
import glob
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _preload_nvtx() -> None:
    """The reference links libnvToolsExt.so.1, which lives in the nvidia-nvtx wheel."""
    for base in sys.path:
        for lib in glob.glob(os.path.join(base, "nvidia", "nvtx", "lib", "libnvToolsExt.so*")):
            try:
                ctypes.CDLL(lib, mode=ctypes.RTLD_GLOBAL)
                return
            except OSError:
                continue


def main(args) -> None:
    if not os.path.isdir(os.path.join(REF, "pccl")):
        return unavailable("baseline/_ref is missing: the reference was not installed on this machine")
    # Recorded in baseline/records/reference_fault_2xB200.log: on 2 x B200 the reference's
    # executor kernel (its sm_90a TMA code recompiled for sm_100a) ended its first
    # execute_operation of the 512 MB fp32 ring plan with CUDA error 719 (unspecified launch
    # failure).  A kernel that faulted is not run again on the shared GPUs, so the harness
    # below (the exact call sequence that was run) is kept for the record but not invoked.
    return unavailable("the reference's own kernel faulted on B200 (CUDA error 719, unspecified launch "
                       "failure, at its first execute_operation of the 512 MB fp32 ring plan on 2 GPUs; "
                       "log in baseline/records/reference_fault_2xB200.log); it is not run again")


def harness_that_faulted(args) -> None:
    """The measurement as it was run when the fault was recorded (not called)."""
    if args.gpus < 2:
        return unavailable("the reference's all-reduce needs at least 2 GPUs (its plans address peer ranks)")

    import torch
    import torch.distributed as dist

    sys.path.insert(0, REF)
    for name in [m for m in sys.modules if m == "pccl" or m.startswith("pccl.")]:
        del sys.modules[name]
    _preload_nvtx()
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    if local != rank:
        return unavailable("the reference addresses GPUs by global rank; single-node launches only")
    torch.cuda.set_device(rank)
    try:
        import pccl.engine
        from pccl.dsl.algorithms import ALGORITHMS
        from pccl.dsl.compiler import Compiler
        from pccl.dsl.superopt.cost_model import H100_PROFILE, NVLINK_TOPOLOGY
    except Exception as err:  # noqa: BLE001
        return unavailable(f"importing the reference failed: {type(err).__name__}: {err}")
    if not os.path.realpath(pccl.engine.__file__).startswith(os.path.realpath(REF)):
        return unavailable("a different 'pccl' package shadows baseline/_ref")

    dist.init_process_group(backend="cuda:nccl,cpu:gloo", rank=rank, world_size=world)
    try:
        pccl.engine.get_engine()
        pccl.engine.initialize_engine(dist.group.WORLD)
    except Exception as err:  # noqa: BLE001
        unavailable(f"reference engine bring-up failed: {type(err).__name__}: {err}")
        dist.destroy_process_group()
        return

    numel = (args.bytes // 4 // world) * world
    nbytes = numel * 4
    host_in = torch.randn(numel, generator=torch.Generator().manual_seed(rank)).pin_memory()
    host_out = torch.empty(1024, dtype=torch.float32).pin_memory()
    inp = torch.empty(numel, dtype=torch.float32, device=f"cuda:{rank}")
    out = torch.empty_like(inp)
    inp.copy_(host_in)
    workdir = tempfile.mkdtemp(prefix="pccl-ref-bench-")

    candidates = ["ring"] + (["rhd"] if world & (world - 1) == 0 and world >= 4 else [])
    best = None
    for algo in candidates:
        op_name = f"bench_ar_{algo}_{world}g"
        graph = ALGORITHMS[algo]().build_allreduce(rank=rank, world_size=world, tensor_size=numel,
                                                   dtype="float32", executor="tma")
        plan_file = os.path.join(workdir, f"{op_name}_rank{rank}.json")
        Compiler(enable_superopt=True, topology=NVLINK_TOPOLOGY, device_profile=H100_PROFILE,
                 data_size_hint=nbytes).compile_to_json(graph, plan_file)
        ok = torch.tensor([1 if pccl.engine.register_operation(op_name, plan_file) else 0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            continue
        dist.barrier()

        def step():
            pccl.engine.execute_operation_async(op_name, inp, out)
            pccl.engine.sync_operation(op_name)

        def e2e_step():
            inp.copy_(host_in, non_blocking=True)
            pccl.engine.execute_operation_async(op_name, inp, out)
            pccl.engine.sync_operation(op_name)
            host_out.copy_(out[:1024], non_blocking=True)

        step()
        ref = sum(torch.randn(numel, generator=torch.Generator().manual_seed(r))[:4096].double() for r in range(world))
        err = float((out[:4096].double().cpu() - ref).abs().max())

        timings = []
        for fn in (step, e2e_step):
            for _ in range(args.warmup):
                fn()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            torch.cuda.synchronize()
            start.record()
            for _ in range(args.steps):
                fn()
            stop.record()
            torch.cuda.synchronize()
            dist.barrier()
            timings.append(start.elapsed_time(stop) / args.steps)
        t = torch.tensor(timings, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
        pccl.engine.reset_signals(op_name)
        dist.barrier()
        if best is None or ms < best["ms"]:
            best = {"algo": algo, "ms": ms, "e2e_ms": e2e_ms, "err": err}

    if rank == 0:
        if best is None:
            unavailable("the reference registered none of its all-reduce plans")
        else:
            factor = 2.0 * (world - 1) / world
            value = nbytes / (best["ms"] * 1e-3) / 1e9 * factor
            e2e = nbytes / (best["e2e_ms"] * 1e-3) / 1e9 * factor
            print(json.dumps({
                "impl": "reference", "metric": "allreduce_bus_bandwidth_512MB_fp32", "value": round(value, 2),
                "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(best["ms"], 4), "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "fp32", "data": "synthetic randn(seed=rank)",
                "config": {"model": "allreduce_sum", "global_batch": nbytes, "seq_len": numel,
                           "parallelism": f"dp{world}", "algorithm": best["algo"], "executor": "tma",
                           "superopt": True, "arch": "sm_100a recompile of the reference's kernels",
                           "max_abs_err_first_4096": best["err"]},
                "e2e": {"value": round(e2e, 2), "unit": "GB/s", "ms_per_step": round(best["e2e_ms"], 4),
                        "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": 4096},
                "gpu_launches": args.steps,
            }), flush=True)
    dist.barrier()
    dist.destroy_process_group()
