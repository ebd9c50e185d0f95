"""Small single-GPU runs of the fused kernels (world 1), sized for a profiler capture.

With one rank the collective half of each kernel degenerates (the only "peer" is this GPU), so a
capture shows the compute half and the kernel's own memory traffic: the GEMM main loop with the
reduce-scatter / all-gather epilogue, reducer warps and copier CTAs, and the RMSNorm pass.  (The
packet and push kernels need a peer and have no one-rank form.)  Each case checks its result against a PyTorch fp32 reference and
prints one JSON line with the CUDA-event time.

    python bench/single_gpu_cases.py --case gemm_rs
    ncu --set full --clock-control none -k regex:umma_gemm2 -c 1 -o prof python bench/single_gpu_cases.py --case gemm_rs
"""

import argparse
import json
import os
import sys

os.environ.setdefault("RANK", "0")
os.environ.setdefault("WORLD_SIZE", "1")
os.environ.setdefault("PCCL_BUFFER_SIZE", str(256 << 20))
os.environ.setdefault("PCCL_ARENA_SIZE", str(1 << 30))

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters * 1e3


def _close(got, ref, tol):
    err = (got.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    if not err <= tol * scale + 1e-3:
        raise SystemExit(f"mismatch: max error {err} against magnitude {scale}")
    return err


def case_gemm_rs(iters):
    from pccl_b200.ops.tensor_parallel import GemmReduceScatter
    m, n, k = 8192, 4096, 1792
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    op = GemmReduceScatter(m, n, k)
    out = op(x, w)
    torch.cuda.synchronize()
    _close(out, x.float() @ w.float().t(), 2e-2)
    return dict(shape=[m, n, k], us=_time(lambda: op(x, w, out), iters))


def case_ag_gemm(iters, swiglu=False):
    from pccl_b200.ops.tensor_parallel import AllGatherGemm
    m, n, k = 8192, 1792 * (2 if swiglu else 1), 4096
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    op = AllGatherGemm(m, n, k, swiglu=swiglu)
    op.local_shard.copy_(x)
    out = op(op.local_shard, w)
    torch.cuda.synchronize()
    ref = x.float() @ w.float().t()
    if swiglu:
        groups = ref.view(m, n // 32, 2, 16)
        ref = (torch.nn.functional.silu(groups[:, :, 0]) * groups[:, :, 1]).reshape(m, n // 2)
    _close(out, ref, 3e-2)
    return dict(shape=[m, n, k], swiglu=swiglu, us=_time(lambda: op(op.local_shard, w, out), iters))


def case_ar_rmsnorm(iters):
    from pccl_b200.ops.tensor_parallel import AllReduceResidualRMSNorm
    tokens, hidden = 16384, 4096                       # 3 x 128 MB of traffic: larger than L2
    op = AllReduceResidualRMSNorm(tokens, hidden, use_nvls=False)
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda")).to(torch.bfloat16)
    x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    res = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    y, h = op(gamma, x, res)
    torch.cuda.synchronize()
    href = (x.float() + res.float()).to(torch.bfloat16).float()
    ref = href * torch.rsqrt(href.pow(2).mean(-1, keepdim=True) + op.eps) * gamma.float()
    _close(y, ref, 2e-2)
    us = _time(lambda: op(gamma), iters)
    return dict(tokens=tokens, hidden=hidden, us=us, gbs=round(4 * tokens * hidden * 2 / us / 1e3, 1))


def case_bucket_pack(iters):
    """64 gradients of mixed sizes (256 MB in all) gathered into one bucket and scattered back."""
    import pccl_b200 as pccl
    fused = pccl.engine.load_native().fused
    sizes = [(4 << 20) + 1024 * (i % 5) for i in range(48)] + [65536 + 8 * i for i in range(16)]     # bf16 elements
    grads = [torch.randn(n, device="cuda").to(torch.bfloat16) for n in sizes]
    offsets, at = [], 0
    for n in sizes:
        offsets.append(at * 2)
        at += n
    bucket = torch.zeros(at, device="cuda", dtype=torch.bfloat16)
    fused.bucket_pack(grads, offsets, bucket, False)
    torch.cuda.synchronize()
    if not torch.equal(bucket, torch.cat(grads)):
        raise SystemExit("pack mismatch")
    back = [torch.zeros_like(g) for g in grads]
    fused.bucket_pack(back, offsets, bucket, True)
    torch.cuda.synchronize()
    if not all(torch.equal(a, b) for a, b in zip(back, grads)):
        raise SystemExit("unpack mismatch")
    us = _time(lambda: fused.bucket_pack(grads, offsets, bucket, False), iters)
    return dict(tensors=len(sizes), bytes=at * 2, us=us, gbs=round(2 * at * 2 / us / 1e3, 1))


CASES = {
    "bucket_pack": case_bucket_pack,
    "gemm_rs": case_gemm_rs,
    "ag_gemm": case_ag_gemm,
    "ag_gemm_swiglu": lambda iters: case_ag_gemm(iters, swiglu=True),
    "ar_rmsnorm": case_ar_rmsnorm,
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    import pccl_b200 as pccl
    pccl.get_engine()
    row = CASES[args.case](args.iters)
    native = pccl.engine.load_native().fused
    if native.read_error() != 0:
        raise SystemExit(f"device error flag {native.read_error()}")
    print(json.dumps(dict(case=args.case, world=1, **row)))


if __name__ == "__main__":
    main()
