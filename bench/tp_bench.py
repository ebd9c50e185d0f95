"""Fused tensor-parallel GEMMs against the unfused cuBLAS + NCCL sequence.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench/tp_bench.py [--iters 20]

Llama-3-8B shapes at TP = N scaled from the TP = 8 configuration (tokens 1024 per rank):
  GEMM -> reduce-scatter   X[1024*N, 14336/8] x W[14336/8, 4096]   (row-parallel down projection)
  all-gather -> GEMM       X shard [1024, 4096] -> [1024*N, 4096] x W[4096, 14336/8]
  all-reduce + residual + RMSNorm at 1 / 128 / 8192 tokens, and the whole SwiGLU feed-forward block
Times are device times (CUDA events), max over ranks, median of the iterations; a 256 MB
buffer is rewritten between iterations so operands leave the L2.  The roofline time is the
slower of FLOPs / measured bf16 peak and NVLink bytes / 770 GB/s (measured peer-copy rate).
One JSON line per operator on rank 0.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.add_(1)
        dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        t = torch.tensor([start.elapsed_time(stop)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t))
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens-per-rank", type=int, default=1024)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--k-local", type=int, default=1792)
    ap.add_argument("--copy-ctas", type=int, default=0)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    os.environ.setdefault("PCCL_ARENA_SIZE", str(2 << 30))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import pccl_b200.parallel as pp
    from pccl_b200.ops import AllGatherGemm, GemmReduceScatter, gemm
    pp.init()
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peak_tflops = json.load(open(peaks_path))["bf16_tflops"] if os.path.exists(peaks_path) else 1590.0
    link_gbs = 770.0
    flush = torch.zeros(64 << 20, device="cuda")
    m, h, kl = args.tokens_per_rank * world, args.hidden, args.k_local
    results = []

    # GEMM -> reduce-scatter
    x = torch.randn(m, kl, device="cuda").to(torch.bfloat16)
    w = (torch.randn(h, kl, device="cuda") * 0.02).to(torch.bfloat16)
    fused = GemmReduceScatter(m, h, kl)
    out = torch.empty(m // world, h, device="cuda", dtype=torch.bfloat16)
    partial = torch.empty(m, h, device="cuda", dtype=torch.bfloat16)

    def unfused():
        torch.matmul(x, w.t(), out=partial)
        dist.reduce_scatter_tensor(out, partial)

    t_fused = timed(lambda: fused(x, w, out), args.iters, flush)
    gemm.check()
    t_unfused = timed(unfused, args.iters, flush)
    t_gemm = timed(lambda: torch.matmul(x, w.t(), out=partial), args.iters, flush)
    t_ours_gemm = timed(lambda: gemm.matmul_nt(x, w, partial), args.iters, flush)
    flops = 2.0 * m * h * kl
    link_bytes = (world - 1) / world * m * h * 2
    roof_ms = max(flops / (peak_tflops * 1e12), link_bytes / (link_gbs * 1e9)) * 1e3
    results.append({"op": "gemm_reduce_scatter", "shape": [m, h, kl], "world": world,
                    "fused_ms": round(t_fused, 4), "unfused_cublas_nccl_ms": round(t_unfused, 4),
                    "cublas_gemm_only_ms": round(t_gemm, 4), "our_gemm_only_ms": round(t_ours_gemm, 4),
                    "speedup_vs_unfused": round(t_unfused / t_fused, 3),
                    "roofline_ms": round(roof_ms, 4), "fraction_of_roofline": round(roof_ms / t_fused, 3),
                    "roofline_terms": {"compute_ms": round(flops / (peak_tflops * 1e9), 4),
                                       "nvlink_ms": round(link_bytes / (link_gbs * 1e6), 4),
                                       "peak": "measured cuBLAS burst, 770 GB/s measured peer copy"}})

    # all-gather -> GEMM
    xs = torch.randn(m // world, h, device="cuda").to(torch.bfloat16)
    wl = (torch.randn(kl, h, device="cuda") * 0.02).to(torch.bfloat16)
    ag = AllGatherGemm(m, kl, h, copy_ctas=args.copy_ctas)
    ag.local_shard.copy_(xs)
    y = torch.empty(m, kl, device="cuda", dtype=torch.bfloat16)
    gathered = torch.empty(m, h, device="cuda", dtype=torch.bfloat16)

    def unfused_ag():
        dist.all_gather_into_tensor(gathered, xs)
        torch.matmul(gathered, wl.t(), out=y)

    t_fused = timed(lambda: ag(ag.local_shard, wl, y), args.iters, flush)
    gemm.check()
    t_unfused = timed(unfused_ag, args.iters, flush)
    t_gemm = timed(lambda: torch.matmul(gathered, wl.t(), out=y), args.iters, flush)
    link_bytes = (world - 1) / world * m * h * 2
    roof_ms = max(flops / (peak_tflops * 1e12), link_bytes / (link_gbs * 1e9)) * 1e3
    results.append({"op": "all_gather_gemm", "shape": [m, kl, h], "world": world, "copy_ctas": args.copy_ctas,
                    "fused_ms": round(t_fused, 4), "unfused_nccl_cublas_ms": round(t_unfused, 4),
                    "cublas_gemm_only_ms": round(t_gemm, 4), "speedup_vs_unfused": round(t_unfused / t_fused, 3),
                    "roofline_ms": round(roof_ms, 4), "fraction_of_roofline": round(roof_ms / t_fused, 3)})
    # all-reduce + residual + RMSNorm (decode, small prefill, large prefill token counts)
    from pccl_b200.ops import AllReduceResidualRMSNorm
    hbm_gbs = json.load(open(peaks_path))["hbm_gbs"] if os.path.exists(peaks_path) else 6650.0
    for tokens in (1, 128, 8192):
        gamma = torch.ones(h, device="cuda", dtype=torch.bfloat16)
        part = torch.randn(tokens, h, device="cuda").to(torch.bfloat16)
        res = torch.randn(tokens, h, device="cuda").to(torch.bfloat16)
        for use_nvls in ("force", False):
            op = AllReduceResidualRMSNorm(tokens, h, use_nvls=use_nvls)
            op.x.copy_(part)
            op.residual.copy_(res)
            t_fused = timed(lambda: op(gamma), args.iters, flush)
            gemm.check()
            buf, resid = part.clone(), res.clone()

            def unfused_norm():
                dist.all_reduce(buf)
                resid.add_(buf)
                return torch.nn.functional.rms_norm(resid, (h,), gamma, 1e-5)

            t_unfused = timed(unfused_norm, args.iters, flush)
            # bytes that must cross NVLink per GPU and direction: (W-1)/W of x for the reduction and (W-1)/W of
            # h for the delivery (y is computed where it is used); the local pass reads x, the residual and
            # h once and writes h and y
            link_bytes = (world - 1) / world * tokens * h * 2 * 2
            local_bytes = tokens * h * 2 * (3 / world + 3)
            roof_ms = (link_bytes / (link_gbs * 1e9) + local_bytes / (hbm_gbs * 1e9)) * 1e3
            results.append({"op": "ar_residual_rmsnorm", "tokens": tokens, "hidden": h, "world": world,
                            "path": "nvls" if use_nvls else "peer", "fused_ms": round(t_fused, 4),
                            "unfused_nccl_torch_ms": round(t_unfused, 4),
                            "speedup_vs_unfused": round(t_unfused / t_fused, 3),
                            "roofline_ms": round(roof_ms, 5), "fraction_of_roofline": round(roof_ms / t_fused, 3)})
    # The whole tensor + sequence parallel SwiGLU feed-forward: two fused kernels against the
    # unfused block (NCCL all-gather, cuBLAS, silu * up, cuBLAS, NCCL reduce-scatter).
    from pccl_b200.models import TensorParallelMLP
    f_local = kl
    w_gu = (torch.randn(2 * f_local, h, device="cuda") * 0.02).to(torch.bfloat16)
    w_dn = (torch.randn(h, f_local, device="cuda") * 0.02).to(torch.bfloat16)
    mlp = TensorParallelMLP(m, h, f_local, w_gu, w_dn)
    x_shard = torch.randn(m // world, h, device="cuda").to(torch.bfloat16)
    mlp.up.input_shard.copy_(x_shard)
    full = torch.empty(m, h, device="cuda", dtype=torch.bfloat16)
    gu = torch.empty(m, 2 * f_local, device="cuda", dtype=torch.bfloat16)
    act = torch.empty(m, f_local, device="cuda", dtype=torch.bfloat16)
    part_out = torch.empty(m, h, device="cuda", dtype=torch.bfloat16)
    y_shard = torch.empty(m // world, h, device="cuda", dtype=torch.bfloat16)

    def unfused_mlp():
        dist.all_gather_into_tensor(full, x_shard)
        torch.matmul(full, w_gu.t(), out=gu)
        torch.mul(torch.nn.functional.silu(gu[:, :f_local]), gu[:, f_local:], out=act)
        torch.matmul(act, w_dn.t(), out=part_out)
        dist.reduce_scatter_tensor(y_shard, part_out)

    t_fused = timed(lambda: mlp(mlp.up.input_shard), args.iters, flush)
    gemm.check()
    t_unfused = timed(unfused_mlp, args.iters, flush)
    mlp_flops = 2.0 * m * h * 2 * f_local + 2.0 * m * f_local * h
    mlp_link = 2 * (world - 1) / world * m * h * 2
    roof_ms = max(mlp_flops / (peak_tflops * 1e12), mlp_link / 2 / (link_gbs * 1e9)) * 1e3
    results.append({"op": "tp_swiglu_mlp_block", "tokens": m, "hidden": h, "ffn_local": f_local, "world": world,
                    "fused_ms": round(t_fused, 4), "unfused_nccl_cublas_ms": round(t_unfused, 4),
                    "speedup_vs_unfused": round(t_unfused / t_fused, 3), "kernels_fused": 2,
                    "roofline_ms": round(roof_ms, 4), "fraction_of_roofline": round(roof_ms / t_fused, 3),
                    "note": "all-gather + gate/up GEMM + SwiGLU in one kernel, down GEMM + reduce-scatter in one"})
    if rank == 0:
        for r in results:
            print(json.dumps(r), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
