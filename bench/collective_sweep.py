"""Collective bandwidth / latency sweep against NCCL.

Multi-GPU (one process per GPU):

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench/collective_sweep.py \
        --collectives allreduce,allgather,reduce_scatter --dtypes fp32,bf16 \
        --min-bytes 1K --max-bytes 1G --algos auto,ring,rhd,tree,oneshot,twoshot,nvls --channels auto

Single GPU (N virtual ranks in one cooperative launch, peer traffic through HBM):

    python bench/collective_sweep.py --virtual-ranks 2 --max-bytes 256M --algos twoshot

Per (collective, dtype, size, algorithm, channels) one JSON line: device time (CUDA events around
`--iters` back-to-back calls, max over ranks), algorithm and bus bandwidth
(bus = alg * 2(N-1)/N for all-reduce, alg * (N-1)/N otherwise), the NCCL time for the same call
(defaults, NVLS allowed, no clone in the timed region), and the ratio.  `--check` verifies every
all-reduce configuration first (float64 host sum of randn(seed=rank) inputs up to --check-bytes,
NCCL above), `--out` keeps all rows as JSON, `--write-tuning` merges the winners per size into the
tuning file that `select_algorithm` and `pccl_b200.parallel` read.  Messages smaller than
the 126 MB L2 are timed L2-warm (like NCCL's own tests); the JSON says so.
The reference's sweep is tests/bench_algo_comparison.py (rank-0 timing, host sync per call).
"""

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def parse_size(text: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(text[:-1]) * mult[text[-1].upper()] if text[-1].upper() in mult else int(text)


def sizes(lo: int, hi: int):
    s = lo
    while s <= hi:
        yield s
        s *= 2


def bus_factor(kind: str, n: int) -> float:
    return 2.0 * (n - 1) / n if kind == "allreduce" else (n - 1) / n


def timed_loop(fn, iters, sync, barrier=None):
    for _ in range(3):
        fn()
    sync()
    if barrier:
        barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    sync()
    return start.elapsed_time(stop) / iters


def run_multi(args):
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    os.environ.setdefault("PCCL_BUFFER_SIZE", str(max(2 << 30, 2 * args.max_bytes)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import pccl_b200.parallel as pp
    engine = pp.init()

    def reduce_max(ms):
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    rows = []

    def allreduce_error(call, full, numel, dtype):
        """max |result - float64 host sum of every rank's randn(seed=rank)| for messages up to
        --check-bytes (every rank regenerates all inputs on the host); larger ones are compared with
        NCCL's all-reduce of the same input on the device.  Max over ranks."""
        esize = torch.empty((), dtype=dtype).element_size()
        if numel * esize <= args.check_bytes:
            parts = [torch.randn(numel, generator=torch.Generator().manual_seed(r)).to(dtype) for r in range(world)]
            full.copy_(parts[rank])
            ref = sum(p.double() for p in parts)
            call()
            torch.cuda.synchronize()
            err = float((full.double().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
        else:
            full.normal_()
            ref = full.clone()
            dist.all_reduce(ref)
            call()
            torch.cuda.synchronize()
            err = float(((full.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-30)))
        t = torch.tensor([err], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    for kind in args.collectives:
        for dname in args.dtypes:
            dtype = DTYPES[dname]
            esize = torch.empty((), dtype=dtype).element_size()
            for nbytes in (args.sizes or sizes(args.min_bytes, args.max_bytes)):
                numel = max(world * 8, nbytes // esize // (world * 8) * (world * 8))
                full = pp.working_tensor(numel, dtype)
                shard = numel // world
                x_shard = torch.randn(shard, device="cuda").to(dtype)
                out_shard = torch.empty(shard, device="cuda", dtype=dtype)
                nccl_buf = torch.randn(numel, device="cuda").to(dtype)
                nccl_out = torch.empty_like(nccl_buf)
                iters = args.iters if nbytes <= (64 << 20) else max(3, args.iters // 4)

                def nccl_call():
                    if kind == "allreduce":
                        dist.all_reduce(nccl_buf)
                    elif kind == "allgather":
                        dist.all_gather_into_tensor(nccl_out, x_shard)
                    elif kind == "reduce_scatter":
                        dist.reduce_scatter_tensor(out_shard, nccl_buf)
                    else:
                        dist.all_to_all_single(nccl_out, nccl_buf)

                nccl_ms = reduce_max(timed_loop(nccl_call, iters, torch.cuda.synchronize, dist.barrier))
                for algo in args.algos:
                    allowed = {"allreduce": ("auto", "ll", "push", "ring", "rhd", "tree", "oneshot", "twoshot", "nvls",
                                             "nvls_twopass", "hybrid", "nvls_kernel"),
                               "allgather": ("auto", "ll", "push", "ring", "rhd", "twoshot", "nvls"),
                               "reduce_scatter": ("auto", "ll", "push", "ring", "rhd", "twoshot", "nvls"),
                               "alltoall": ("auto", "ll", "push", "ring", "twoshot")}[kind]
                    if algo not in allowed:
                        continue
                    if algo == "oneshot" and nbytes > (4 << 20):
                        continue
                    if algo == "ll" and (nbytes if kind == "allreduce" else nbytes // world) > pp.collectives.LL_MAX_BYTES:
                        continue
                    if algo == "push" and nbytes > pp.collectives.PUSH_MAX_BYTES:
                        continue
                    if algo in ("rhd", "tree") and world & (world - 1):
                        continue
                    if algo == "nvls_kernel" and not pp.collectives._nvls_kernel_ok(full, "sum"):
                        continue
                    for ch in args.channels:
                        forced_algo = None if algo == "auto" else algo
                        forced_ch = None if ch == "auto" else int(ch)
                        plan_algo = None if forced_algo in ("push", "ll") else forced_algo   # plan registered for reporting
                        try:
                            uses_ll = kind == "allreduce" and algo in ("auto", "ll") and \
                                pp.collectives._ll_eligible(full, "sum", forced_algo)
                            uses_push = kind == "allreduce" and not uses_ll and algo in ("auto", "push") and \
                                pp.collectives._push_eligible(full, "sum", forced_algo)
                            if kind == "allreduce" and algo == "nvls_kernel":
                                name = ""                       # a kernel, not a plan
                                call = lambda: pp.all_reduce(full, algorithm="nvls_kernel", async_op=True)
                            elif kind == "allreduce":
                                name = pp.ensure_plan(kind, numel, dtype, None if (uses_ll or uses_push) else plan_algo,
                                                      forced_ch)
                                call = lambda: pp.all_reduce(full, algorithm=forced_algo, channels=forced_ch, async_op=True)
                            elif kind == "allgather":
                                name = pp.ensure_plan(kind, numel, dtype, plan_algo, forced_ch)
                                mine = full[rank * shard:(rank + 1) * shard]
                                uses_ll = pp.collectives._ll_part_ok(mine, full, forced_algo)
                                uses_push = not uses_ll and pp.collectives._push_ok(full, mine, forced_algo)
                                call = lambda: pp.all_gather(full, mine, algorithm=forced_algo, channels=forced_ch, async_op=True)
                            elif kind == "reduce_scatter":
                                name = pp.ensure_plan(kind, numel, dtype, plan_algo, forced_ch)
                                mine = full[rank * shard:(rank + 1) * shard]
                                uses_ll = pp.collectives._ll_part_ok(mine, full, forced_algo)
                                uses_push = not uses_ll and pp.collectives._push_ok(full, mine, forced_algo)
                                call = lambda: pp.reduce_scatter(mine, full, algorithm=forced_algo, channels=forced_ch, async_op=True)
                            else:
                                name = pp.ensure_plan(kind, numel, dtype, plan_algo or "twoshot", forced_ch)
                                uses_ll = pp.collectives._ll_part_ok(full[:shard], nccl_out, forced_algo)
                                uses_push = not uses_ll and pp.collectives._push_ok(full, nccl_out, forced_algo)
                                call = lambda: pp.all_to_all(nccl_out, full, algorithm=forced_algo, channels=forced_ch,
                                                            async_op=True)
                        except Exception as err:  # noqa: BLE001
                            if rank == 0:
                                print(json.dumps({"collective": kind, "algo": algo, "bytes": nbytes, "skipped": str(err)[:120]}))
                            continue
                        rel_err = None
                        if kind == "allreduce" and args.check:
                            rel_err = allreduce_error(call, full, numel, dtype)
                        ms = reduce_max(timed_loop(call, iters, lambda: pp.synchronize(name), dist.barrier))
                        if rank == 0:
                            _, real_algo, real_ch = pp.registered_plans()[name] if name else (kind, algo, 0)
                            if uses_ll:
                                real_algo, real_ch = "ll", 0
                            elif uses_push:
                                real_algo, real_ch = "push", 0
                            alg = numel * esize / (ms * 1e-3) / 1e9
                            row = {
                                "collective": kind, "dtype": dname, "bytes": numel * esize, "world": world,
                                "algo": real_algo, "requested": algo, "channels": real_ch,
                                "nvls": bool(engine.nvls_active()), "us": round(ms * 1e3, 2),
                                "algbw_gbs": round(alg, 2), "busbw_gbs": round(alg * bus_factor(kind, world), 2),
                                "nccl_us": round(nccl_ms * 1e3, 2), "vs_nccl": round(nccl_ms / ms, 3),
                                "l2": "cold (message > L2)" if numel * esize > (126 << 20) else "warm",
                                "in_place": kind != "alltoall"}
                            if rel_err is not None:
                                row["max_rel_err"] = rel_err
                                row["checked_against"] = "float64 host sum" if numel * esize <= args.check_bytes \
                                    else "NCCL all-reduce of the same input"
                            rows.append(row)
                            print(json.dumps(row), flush=True)
    if rank == 0:
        if args.out:
            with open(args.out, "w") as handle:
                json.dump({"world": world, "iters": args.iters, "rows": rows}, handle, indent=1)
        if args.write_tuning:
            write_tuning(args.write_tuning, world, rows)
    dist.barrier()
    dist.destroy_process_group()


_KERNEL_ROUTES = ("ll", "push", "nvls_kernel")


def write_tuning(path, world, rows):
    """Merge this sweep's winners into the tuning file: per collective, break points
    [{"max_bytes", "algorithm", "channels", "us"}] where consecutive sizes with the same winner are
    merged (a winner is kept while it stays within 3 % of the best) and the last entry is open-ended.  Only sizes that were measured with at least two
    algorithms count (a lone "auto" row says nothing about the alternatives)."""
    try:
        with open(path) as handle:
            doc = json.load(handle)
    except (OSError, ValueError):
        doc = {}
    doc.setdefault("routes", {})
    for kind in sorted({r["collective"] for r in rows}):
        by_size = {}
        for r in rows:
            if r["collective"] != kind or r.get("requested") == "auto":
                continue
            by_size.setdefault(r["bytes"], []).append(r)
        table = []
        for nbytes in sorted(by_size):
            cands = by_size[nbytes]
            if len(cands) < 2:
                continue
            best = min(cands, key=lambda r: r["us"])
            # Hysteresis: the previous size's winner stays unless another one beats it by more than 3 %
            # (timer noise otherwise flips the table between equals).
            if table:
                same = [r for r in cands if r["algo"] == table[-1]["algorithm"]
                        and (r["channels"] or None) == table[-1].get("channels")]
                if same and min(r["us"] for r in same) <= 1.03 * best["us"]:
                    best = min(same, key=lambda r: r["us"])
            entry = {"max_bytes": nbytes, "algorithm": best["algo"], "us": best["us"]}
            if best["channels"]:
                entry["channels"] = best["channels"]
            if best["algo"] in _KERNEL_ROUTES:
                # a kernel won: also name the best plan, for callers the kernel does not take
                plans = [r for r in cands if r["algo"] not in _KERNEL_ROUTES]
                if plans:
                    best_plan = min(plans, key=lambda r: r["us"])
                    kept = [r for r in plans if table and r["algo"] == table[-1].get("plan_algorithm")]
                    if kept and min(r["us"] for r in kept) <= 1.05 * best_plan["us"]:
                        best_plan = kept[0]
                    entry["plan_algorithm"] = best_plan["algo"]
            if table and all(table[-1].get(k) == entry.get(k) for k in ("algorithm", "channels", "plan_algorithm")):
                table[-1].update(max_bytes=nbytes, us=best["us"])
            else:
                table.append(entry)
        if table:
            table[-1]["max_bytes"] = None
            doc["routes"].setdefault(kind, {})[str(world)] = table
    doc["source"] = "bench/collective_sweep.py --write-tuning"
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as handle:
        json.dump(doc, handle, indent=1)


def run_virtual(args):
    from pccl_b200 import Compiler, engine_c
    from pccl_b200.dsl.algorithms import ALGORITHMS
    torch.cuda.set_device(0)
    world = args.virtual_ranks
    cluster = engine_c.LocalCluster(world, 0, 2 * args.max_bytes + (16 << 20))
    names = {"fp32": "float32", "bf16": "bfloat16", "fp16": "float16"}
    for kind in args.collectives:
        for dname in args.dtypes:
            dtype = DTYPES[dname]
            esize = torch.empty((), dtype=dtype).element_size()
            for nbytes in sizes(args.min_bytes, args.max_bytes):
                numel = max(world * 8, nbytes // esize // (world * 8) * (world * 8))
                for algo in args.algos:
                    if algo == "auto":
                        algo = "twoshot"
                    for ch in args.channels:
                        channels = 1 if ch == "auto" else int(ch)
                        try:
                            plans = [Compiler().compile_to_json(getattr(ALGORITHMS[algo](), "build_" + kind)(
                                r, world, numel, names[dname], "sm", channels)) for r in range(world)]
                            name = f"{kind}_{algo}_{dname}_{numel}_{channels}"
                            cluster.regOp(name, plans)
                        except Exception as err:  # noqa: BLE001
                            print(json.dumps({"collective": kind, "algo": algo, "bytes": nbytes, "skipped": str(err)[:120]}))
                            continue
                        in_n = numel // world if kind == "allgather" else numel
                        out_n = numel // world if kind == "reduce_scatter" else numel
                        xs = [torch.randn(in_n, device="cuda").to(dtype) for _ in range(world)]
                        outs = [torch.empty(out_n, device="cuda", dtype=dtype) for _ in range(world)]
                        iters = args.iters if nbytes <= (64 << 20) else max(3, args.iters // 4)
                        ms = timed_loop(lambda: cluster.exeOp(name, xs, outs), iters, torch.cuda.synchronize)
                        alg = numel * esize / (ms * 1e-3) / 1e9
                        print(json.dumps({"collective": kind, "dtype": dname, "bytes": numel * esize,
                                          "virtual_ranks": world, "algo": algo, "channels": channels,
                                          "ctas_per_rank": int(cluster.opInfo(name, 0)["ctas"]),
                                          "us": round(ms * 1e3, 2), "algbw_gbs": round(alg, 2),
                                          "busbw_gbs": round(alg * bus_factor(kind, world), 2),
                                          "note": "one GPU, staged in/out copies included"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--collectives", default="allreduce")
    ap.add_argument("--dtypes", default="fp32")
    ap.add_argument("--min-bytes", default="1K")
    ap.add_argument("--max-bytes", default="512M")
    ap.add_argument("--algos", default="auto")
    ap.add_argument("--channels", default="auto")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--virtual-ranks", type=int, default=0)
    ap.add_argument("--sizes", default=None, help="explicit list of sizes (e.g. 256K,16M,512M) instead of powers of two")
    ap.add_argument("--out", default=None, help="write every row to this JSON file (rank 0)")
    ap.add_argument("--write-tuning", default=None,
                    help="merge the fastest algorithm per size into this tuning file (the selector reads it)")
    ap.add_argument("--tuning-from", nargs="+", default=None, metavar="SWEEP_JSON",
                    help="no measurement: rebuild --write-tuning from saved --out files (any worlds, any collectives)")
    ap.add_argument("--check", action="store_true", help="verify every all-reduce configuration before timing it")
    ap.add_argument("--check-bytes", default="16M",
                    help="up to this size the check is against a float64 host sum, above it against NCCL")
    args = ap.parse_args()
    if args.tuning_from:
        if not args.write_tuning:
            ap.error("--tuning-from needs --write-tuning")
        for path in args.tuning_from:
            with open(path) as handle:
                saved = json.load(handle)
            write_tuning(args.write_tuning, saved["world"], saved["rows"])
        return
    args.collectives = args.collectives.split(",")
    args.dtypes = args.dtypes.split(",")
    args.algos = args.algos.split(",")
    args.channels = args.channels.split(",")
    args.min_bytes, args.max_bytes = parse_size(args.min_bytes), parse_size(args.max_bytes)
    args.check_bytes = parse_size(args.check_bytes)
    args.sizes = [parse_size(x) for x in args.sizes.split(",")] if args.sizes else None
    if args.sizes:
        args.max_bytes = max(args.max_bytes, max(args.sizes))
    if args.virtual_ranks:
        run_virtual(args)
    else:
        run_multi(args)


if __name__ == "__main__":
    main()
