"""Device timeline of one all-reduce plan: where the time of a launch goes, per phase.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench/trace_allreduce.py \
        [--algo nvls] [--bytes 536870912] [--steps]

Turns the engine's per-step `%globaltimer` stamps on (PCCL_TRACE), runs the plan a few times on the
symmetric working buffer and prints rank 0's summary of the last launch: per phase the bytes, the
span, the per-direction NVLink rate, and per chain the time spent waiting, moving and posting.
`--steps` also lists every step of chain 0 with its four stamps (for small plans).
"""

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--algo", default="nvls")
    ap.add_argument("--bytes", type=int, default=512 << 20)
    ap.add_argument("--steps", action="store_true")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    os.environ.setdefault("PCCL_BUFFER_SIZE", str(max(1 << 30, 2 * args.bytes)))
    os.environ["PCCL_TRACE"] = "1"
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import pccl_b200.parallel as pp
    from pccl_b200.utils.trace import summarize
    engine = pp.init()
    n = args.bytes // 4
    x = pp.working_tensor(n, torch.float32)
    x.normal_()
    for _ in range(4):
        pp.all_reduce(x, algorithm=args.algo, async_op=True)
    torch.cuda.synchronize()
    name = [k for k, v in pp.registered_plans().items() if v[1] == args.algo][0]
    trace = engine.trace(name)
    if rank == 0:
        print(f"plan {name} on {world} GPUs")
        print(summarize(trace, world))
        if args.steps:
            t0 = min(s["t_reached_ns"] for s in trace if s["t_reached_ns"])
            for s in trace[:40]:
                print({k: (v - t0 if k.startswith("t_") and v else v) for k, v in s.items()})
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
