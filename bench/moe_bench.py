"""Expert-parallel MoE feed-forward: fused kernels against an unfused PyTorch / NCCL baseline.

    python bench/moe_bench.py                                   # one GPU, all experts local
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench/moe_bench.py

Default shape: 4096 tokens per rank, hidden 4096, ffn 14336, 8 experts, top-2 (Mixtral-8x7B's
layer).  The baseline routes with torch, exchanges rows with all_to_all_single (NCCL), runs the
experts with cuBLAS and returns the rows the same way.  Device time with CUDA events, L2
flushed between iterations, max over ranks; one JSON line from rank 0.  FLOPs count the rows
actually routed (2 per token) times 3 weight matrices.
"""

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def baseline_layer(x, wg, w1, w3, w2, world, rank, dist):
    """Unfused expert-parallel MoE: torch routing + NCCL all-to-all + cuBLAS experts."""
    tokens, hidden = x.shape
    experts = wg.shape[0]
    le = experts // world
    logits = x.float() @ wg.float().t()
    top, idx = logits.topk(2, dim=-1)
    gates = torch.softmax(top, dim=-1)
    flat_e = idx.flatten()
    order = flat_e.argsort(stable=True)
    rows = x[order // 2]
    counts = torch.bincount(flat_e, minlength=experts)
    if world > 1:
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts)
        send_split = counts.view(world, le).sum(1).tolist()
        recv_split = recv_counts.view(world, le).sum(1).tolist()
        got = torch.empty(sum(recv_split), hidden, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(got, rows, recv_split, send_split)
        per_src = recv_counts.view(world, le)
        # rows arrive grouped by source, then by local expert: regroup by expert
        expert_of = torch.repeat_interleave(torch.arange(le, device=x.device).repeat(world), per_src.flatten())
        regroup = expert_of.argsort(stable=True)
        got = got[regroup]
        per_expert = per_src.sum(0).tolist()
    else:
        got, per_expert, regroup = rows, counts.tolist(), None
    outs, start = [], 0
    for e in range(le):
        xe = got[start:start + per_expert[e]]
        start += per_expert[e]
        outs.append((F.silu(xe @ w1[e].t()) * (xe @ w3[e].t())) @ w2[e].t())
    y = torch.cat(outs)
    if world > 1:
        back = torch.empty_like(y)
        back[regroup] = y
        ret = torch.empty(2 * tokens, hidden, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(ret, back, send_split, recv_split)
    else:
        ret = y
    out = torch.zeros(tokens, hidden, dtype=torch.float32, device=x.device)
    out.index_add_(0, order // 2, ret.float() * gates.flatten()[order, None])
    return out.to(x.dtype)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-baseline", action="store_true")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist = None
    from pccl_b200.ops import moe
    le = args.experts // world
    if world > 1:
        import torch.distributed as dist
        need = le * world * args.tokens * args.hidden * 2 + args.tokens * 2 * args.hidden * 2 + (64 << 20)
        os.environ.setdefault("PCCL_ARENA_SIZE", str(max(1 << 30, need)))
        os.environ.setdefault("PCCL_BUFFER_SIZE", str(64 << 20))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        import pccl_b200.parallel as pp
        pp.init()
    gen = torch.Generator(device="cuda").manual_seed(3)
    h, f = args.hidden, args.ffn
    wg = (torch.randn(args.experts, h, device="cuda", generator=gen) * 0.5).to(torch.bfloat16)
    w1 = (torch.randn(le, f, h, device="cuda", generator=gen) * h ** -0.5).to(torch.bfloat16)
    w3 = (torch.randn(le, f, h, device="cuda", generator=gen) * h ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(le, h, f, device="cuda", generator=gen) * f ** -0.5).to(torch.bfloat16)
    layer = moe.FusedMoE(args.tokens, h, f, args.experts, local=world == 1)
    layer.set_weights(wg, w1, w3, w2)
    xs = [torch.randn(args.tokens, h, device="cuda", generator=torch.Generator(device="cuda").manual_seed(50 + rank + 8 * i))
          .to(torch.bfloat16) for i in range(4)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    native = __import__("pccl_b200.engine", fromlist=["load_native"]).load_native().fused

    def timed(fn):
        for i in range(3):
            fn(xs[i % 4])
        torch.cuda.synchronize()
        total = 0.0
        for i in range(args.iters):
            flush.zero_()
            if dist:
                dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn(xs[i % 4])
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        ms = total / args.iters
        if dist:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms

    fused_ms = timed(lambda x: layer(x))
    err = native.read_error()
    base_ms = None
    max_err = None
    if not args.no_baseline:
        base_ms = timed(lambda x: baseline_layer(x, wg, w1, w3, w2, world, rank, dist))
        ref = baseline_layer(xs[0], wg, w1, w3, w2, world, rank, dist)
        out = layer(xs[0])
        torch.cuda.synchronize()
        max_err = (out.float() - ref.float()).abs().max().item() / max(ref.float().abs().max().item(), 1e-6)
    flops = 2.0 * args.tokens * 2 * 3 * h * f          # per rank: 2 routed rows per token, 3 matrices
    if rank == 0:
        print(json.dumps({
            "op": "moe_ffn_top2", "world": world, "tokens_per_rank": args.tokens, "hidden": h, "ffn": f,
            "experts": args.experts, "fused_ms": round(fused_ms, 4),
            "fused_tflops_per_gpu": round(flops / (fused_ms * 1e-3) / 1e12, 1),
            "baseline_ms": None if base_ms is None else round(base_ms, 4),
            "speedup": None if base_ms is None else round(base_ms / fused_ms, 3),
            "rel_max_diff_vs_baseline": max_err, "error_word": err,
            "timing": "CUDA events, L2 flushed, max over ranks"}), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
