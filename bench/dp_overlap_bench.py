"""How much of the data-parallel gradient all-reduce hides under backward.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench/dp_overlap_bench.py \
        [--layers 8] [--hidden 4096] [--tokens 8192] [--bucket-mb 32]

A stack of bf16 linear layers runs forward + backward three ways: alone (no reduction), followed by
the bucketed reduction after backward has finished (`GradientBuckets.reduce`), and with the
reduction driven by autograd hooks on a side stream while backward still computes
(`GradientBuckets.attach` / `finish`).  Device time per step (CUDA events, max over ranks):

    overlap = (t_backward_alone + t_reduce_alone - t_hooked) / t_reduce_alone

The same with `torch.nn.parallel.DistributedDataParallel` (NCCL, its own buckets) is printed beside it.
One JSON line on rank 0.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--bucket-mb", type=int, default=32)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import pccl_b200.parallel as pp
    from pccl_b200.parallel.layers import GradientBuckets
    pp.init()

    torch.manual_seed(3)
    model = torch.nn.Sequential(*[torch.nn.Linear(args.hidden, args.hidden, bias=False)
                                  for _ in range(args.layers)]).cuda().bfloat16()
    x = torch.randn(args.tokens, args.hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rank)
                    ).bfloat16()
    buckets = GradientBuckets(model.parameters(), bucket_bytes=args.bucket_mb << 20)

    def fwd_bwd(module=model):
        module.zero_grad(set_to_none=True)
        module(x).float().pow(2).mean().backward()

    def timed(step):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.iters):
            step()
        stop.record()
        torch.cuda.synchronize()
        t = torch.tensor([start.elapsed_time(stop) / args.iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    t_alone = timed(fwd_bwd)

    def after():
        fwd_bwd()
        buckets.reduce()
    t_after = timed(after)

    buckets.attach()

    def hooked():
        fwd_bwd()
        buckets.finish()
    t_hooked = timed(hooked)
    buckets.detach()
    pp.check_errors()

    ddp = torch.nn.parallel.DistributedDataParallel(model, bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
    t_ddp = timed(lambda: fwd_bwd(ddp))

    if rank == 0:
        t_reduce = t_after - t_alone
        grad_mb = sum(p.numel() for p in model.parameters()) * 2 / 2 ** 20
        print(json.dumps({
            "bench": "dp_overlap", "world": world, "layers": args.layers, "hidden": args.hidden, "tokens": args.tokens,
            "gradient_mb": round(grad_mb, 1), "bucket_mb": args.bucket_mb,
            "fwd_bwd_alone_ms": round(t_alone, 3), "reduce_after_backward_ms": round(t_after, 3),
            "reduce_alone_ms": round(t_reduce, 3), "hooked_ms": round(t_hooked, 3),
            "overlap_fraction": round((t_alone + t_reduce - t_hooked) / t_reduce, 3) if t_reduce > 0 else None,
            "torch_ddp_nccl_ms": round(t_ddp, 3),
            "hooked_vs_ddp": round(t_ddp / t_hooked, 3)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
