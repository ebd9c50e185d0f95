"""Per-CTA timeline of the fused GEMM kernels: when the MMAs, the epilogue and the reducers finish.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench/trace_fused_gemm.py \
        [--tokens-per-rank 1024] [--hidden 4096] [--k-local 1792]

For GEMM->reduce-scatter, all-gather->GEMM and the plain GEMM of the same shapes, every CTA stamps
`%globaltimer` when it enters, when its last MMA is issued, when its epilogue is done, when its first
accumulator is complete, when its reducer warps saw their first / last block complete and when they
finished, and when it leaves.  Rank 0 prints min / median / max over CTAs in microseconds since the
first CTA entered (one launch each, after warm-up).
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

STAMPS = ["enter", "mma_done", "epilogue_done", "reducers_done", "leave", "first_accumulator",
          "reducer_first_block_ready", "reducer_last_block_ready"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens-per-rank", type=int, default=1024)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--k-local", type=int, default=1792)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    os.environ.setdefault("PCCL_ARENA_SIZE", str(2 << 30))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import pccl_b200.parallel as pp
    from pccl_b200 import engine as _engine
    from pccl_b200.ops import AllGatherGemm, GemmReduceScatter, gemm
    pp.init()
    fused = _engine.load_native().fused
    m, h, kl = args.tokens_per_rank * world, args.hidden, args.k_local

    def report(tag):
        t = torch.tensor(fused.gemm_trace_read(), dtype=torch.int64).view(-1, len(STAMPS))
        t = t[t[:, 0] > 0]
        rel = (t - t[:, 0].min()).float() / 1e3
        row = {}
        for i, name in enumerate(STAMPS):
            seen = t[:, i] > 0
            if seen.any():
                v = rel[:, i][seen]
                row[name] = [round(float(v.min()), 1), round(float(v.median()), 1), round(float(v.max()), 1)]
        if rank == 0:
            print(tag, json.dumps(row), flush=True)

    def traced(tag, call, warm=3):
        for _ in range(warm):
            call()
        torch.cuda.synchronize()
        dist.barrier()
        fused.gemm_trace_enable(True)                    # clears the stamps
        call()
        torch.cuda.synchronize()
        report(tag)

    x = torch.randn(m, kl, device="cuda").to(torch.bfloat16)
    w = (torch.randn(h, kl, device="cuda") * 0.02).to(torch.bfloat16)
    rs = GemmReduceScatter(m, h, kl)
    out = torch.empty(m // world, h, device="cuda", dtype=torch.bfloat16)
    traced(f"gemm_reduce_scatter [{m},{kl}]x[{kl},{h}] min/median/max us", lambda: rs(x, w, out))
    part = torch.empty(m, h, device="cuda", dtype=torch.bfloat16)
    traced("plain gemm of that shape", lambda: gemm.matmul_nt(x, w, part))

    xs = torch.randn(m // world, h, device="cuda").to(torch.bfloat16)
    wl = (torch.randn(kl, h, device="cuda") * 0.02).to(torch.bfloat16)
    ag = AllGatherGemm(m, kl, h)
    ag.local_shard.copy_(xs)
    y = torch.empty(m, kl, device="cuda", dtype=torch.bfloat16)
    traced(f"all_gather_gemm [{m},{h}]x[{h},{kl}] min/median/max us", lambda: ag(ag.local_shard, wl, y))
    traced("plain gemm of that shape", lambda: gemm.matmul_nt(ag.gathered, wl, y))
    fused.gemm_trace_enable(False)
    gemm.check()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
