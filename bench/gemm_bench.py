"""Time the tcgen05 GEMM against torch.matmul (cuBLAS) on one GPU.

    python bench/gemm_bench.py [--shapes 8192x4096x1792,8192x1792x4096] [--iters 20]

Device timing with CUDA events; a 256 MB buffer is rewritten between iterations
so that operands do not stay in the 126 MB L2.  Prints one JSON line per shape with
TFLOP/s of the paired-SM kernel ("ours": tcgen05.mma.cta_group::2 on 256 x 256 tiles), of the
one-SM-per-tile kernel and of cuBLAS, and the fraction of the measured cuBLAS peak in
MEASURED_PEAKS.json.
"""

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters, flush):
    start = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    stop = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    for i in range(iters):
        flush.add_(1)
        start[i].record()
        fn()
        stop[i].record()
    torch.cuda.synchronize()
    times = sorted(s.elapsed_time(e) for s, e in zip(start, stop))
    return times[len(times) // 2], times[0]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="8192x4096x1792,8192x1792x4096,8192x8192x8192")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    from pccl_b200.ops import gemm
    peaks = {}
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peaks = json.load(open(path))
    peak = peaks.get("bf16_tflops", 1590.0)
    flush = torch.zeros(64 << 20, device="cuda", dtype=torch.float32)
    for spec in args.shapes.split(","):
        m, n, k = (int(x) for x in spec.split("x"))
        a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        b = torch.randn(n, k, device="cuda").to(torch.bfloat16)
        c = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        one_med, _ = timed(lambda: gemm.matmul_nt(a, b, c, sms_per_tile=1), args.iters, flush)
        ours_med, ours_min = timed(lambda: gemm.matmul_nt(a, b, c, sms_per_tile=2), args.iters, flush)
        gemm.check()
        lib_med, lib_min = timed(lambda: torch.matmul(a, b.t(), out=c), args.iters, flush)
        flops = 2.0 * m * n * k
        print(json.dumps({
            "shape": [m, n, k], "ours_ms": round(ours_med, 4), "cublas_ms": round(lib_med, 4),
            "ours_tflops": round(flops / ours_med / 1e9, 1), "cublas_tflops": round(flops / lib_med / 1e9, 1),
            "one_sm_per_tile_tflops": round(flops / one_med / 1e9, 1),
            "ours_best_tflops": round(flops / ours_min / 1e9, 1),
            "frac_of_measured_peak": round(flops / ours_med / 1e9 / peak, 3),
            "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback"}), flush=True)


if __name__ == "__main__":
    main()
