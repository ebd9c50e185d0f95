"""Worker of the multi-GPU tests (one process per GPU, launched by torchrun).

Runs every collective through the public API on the engine's multi-process path
(VMM heap + fd passing + NVLS when available) and checks it against NCCL on the
same inputs.  Prints ``MULTI_GPU_PASS {json}`` on rank 0 when everything matched.
"""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    os.environ.setdefault("PCCL_BUFFER_SIZE", str(256 << 20))
    os.environ.setdefault("PCCL_ARENA_SIZE", str(1 << 30))
    os.environ.setdefault("PCCL_WAIT_TIMEOUT_MS", "5000")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import pccl_b200.parallel as pp
    engine = pp.init()
    report = {"world": world, "nvls": bool(engine.nvls_active()), "checked": 0}

    def tol(dtype):
        return dict(atol=1e-4, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.1, rtol=2 ** -6)

    algos = ["ring", "twoshot", "oneshot", "nvls", "nvls_twopass", "hybrid"] + \
        (["rhd", "tree"] if world & (world - 1) == 0 else [])
    for dtype in (torch.float32, torch.bfloat16):
        for numel in (world * 1024, world * 100003, 4 << 20):
            gen = torch.Generator(device="cuda").manual_seed(1000 + rank)
            x = torch.randn(numel, device="cuda", generator=gen).to(dtype)
            ref = x.float().clone()
            dist.all_reduce(ref)
            for algo in algos:
                if algo == "oneshot" and numel > (1 << 20):
                    continue
                for channels in (1, 4):
                    if numel % (channels * world) and algo != "hybrid":   # hybrid reduces the ragged tail itself
                        continue
                    y = x.clone()
                    pp.all_reduce(y, algorithm=algo, channels=channels)
                    torch.testing.assert_close(y.float(), ref, msg=lambda m: f"allreduce {algo} c{channels} "
                                               f"{dtype} n={numel} rank {rank}: {m}", **tol(dtype))
                    report["checked"] += 1
            # zero-copy: the tensor is the working buffer itself
            w = pp.working_tensor(numel, dtype)
            w.copy_(x)
            pp.all_reduce(w)
            torch.testing.assert_close(w.float(), ref, **tol(dtype))

            shard = numel // world
            # reduce-scatter
            out = torch.empty(shard, device="cuda", dtype=dtype)
            for algo in ("ring", "twoshot", "nvls"):
                pp.reduce_scatter(out, x, algorithm=algo)
                torch.testing.assert_close(out.float(), ref[rank * shard:(rank + 1) * shard], **tol(dtype))
                report["checked"] += 1
            # all-gather
            full = torch.empty(numel, device="cuda", dtype=dtype)
            expect = torch.empty(numel, device="cuda", dtype=dtype)
            dist.all_gather_into_tensor(expect, x[:shard].contiguous())
            for algo in ("ring", "twoshot", "nvls"):
                full.zero_()
                pp.all_gather(full, x[:shard].contiguous(), algorithm=algo)
                assert torch.equal(full, expect), f"allgather {algo} {dtype} n={numel}"
                report["checked"] += 1
            # all-to-all
            got = torch.empty(numel, device="cuda", dtype=dtype)
            want = torch.empty(numel, device="cuda", dtype=dtype)
            dist.all_to_all_single(want, x)
            for algo in ("ring", "twoshot"):
                pp.all_to_all(got, x, algorithm=algo)
                assert torch.equal(got, want), f"alltoall {algo} {dtype} n={numel}"
                report["checked"] += 1

    # copy-engine executor: same results, data moved by cudaMemcpyAsync on per-channel streams
    numel = world * (1 << 18)
    x = torch.randn(numel, device="cuda", generator=torch.Generator(device="cuda").manual_seed(50 + rank))
    shard = numel // world
    expect = torch.empty(numel, device="cuda")
    dist.all_gather_into_tensor(expect, x[:shard].contiguous())
    full = torch.zeros(numel, device="cuda")
    for channels in (1, 4):
        full.zero_()
        pp.all_gather(full, x[:shard].contiguous(), channels=channels, executor="ce")
        assert torch.equal(full, expect), f"ce allgather c{channels}"
    want = torch.empty(numel, device="cuda")
    dist.all_to_all_single(want, x)
    got = torch.empty(numel, device="cuda")
    pp.all_to_all(got, x, channels=2, executor="ce")
    assert torch.equal(got, want), "ce alltoall"
    ce_ops = [n for n, st in engine.stats().items() if st.get("copy_engine")]
    assert len(ce_ops) >= 3, f"copy-engine executor not used: {ce_ops}"
    report["copy_engine_ops"] = len(ce_ops)

    # packet-protocol small-message all-reduce: ordinary (non-symmetric) tensors, in place, many calls
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for numel in (4, 1024, 20000, 65536):
            for call in range(3):
                gen = torch.Generator(device="cuda").manual_seed(1000 * call + 17 * rank + numel)
                x = torch.randn(numel, device="cuda", generator=gen).to(dtype)
                ref = x.float().clone()
                dist.all_reduce(ref)
                y = pp.all_reduce(x.clone(), algorithm="ll")
                torch.cuda.synchronize()
                gemm_mod = __import__("pccl_b200.ops.gemm", fromlist=["check"])
                gemm_mod.check()
                atol = 1e-5 if dtype == torch.float32 else 0.06
                torch.testing.assert_close(y.float(), ref, atol=atol, rtol=2e-2,
                                           msg=lambda t: f"ll allreduce {dtype} n={numel} call {call} rank {rank}: {t}")
        report["checked"] += 1
    # fused push all-reduce: ordinary tensors, in place, sizes that do not divide evenly over the ranks
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for numel in (8, 4096 + 8, 300000, 1 << 21):
            for call in range(3):
                gen = torch.Generator(device="cuda").manual_seed(2000 * call + 31 * rank + numel)
                x = torch.randn(numel, device="cuda", generator=gen).to(dtype)
                ref = x.float().clone()
                dist.all_reduce(ref)
                y = pp.all_reduce(x.clone(), algorithm="push")
                torch.cuda.synchronize()
                __import__("pccl_b200.ops.gemm", fromlist=["check"]).check()
                atol = 1e-5 if dtype == torch.float32 else 0.06
                torch.testing.assert_close(y.float(), ref, atol=atol, rtol=2e-2,
                                           msg=lambda t: f"push allreduce {dtype} n={numel} call {call} rank {rank}: {t}")
        report["checked"] += 1
    x = torch.randn(100000, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9 + rank))
    y = pp.all_reduce(x.clone(), algorithm="push")
    gathered = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(gathered, y)
    assert all(torch.equal(gathered[0], g) for g in gathered), "push allreduce differs between ranks"

    # push reduce-scatter / all-gather / all-to-all on ordinary tensors, against NCCL
    for dtype in (torch.float32, torch.bfloat16):
        for shard in (8, 1000 * 8, 1 << 18):
            n = shard * world
            gen = torch.Generator(device="cuda").manual_seed(77 + rank + shard)
            full_in = torch.randn(n, device="cuda", generator=gen).to(dtype)
            mine = torch.randn(shard, device="cuda", generator=gen).to(dtype)
            for call in range(2):
                ref = torch.empty(shard, device="cuda", dtype=torch.float32)
                dist.reduce_scatter_tensor(ref, full_in.float())
                got = pp.reduce_scatter(torch.empty(shard, device="cuda", dtype=dtype), full_in, algorithm="push")
                ref_g = torch.empty(n, device="cuda", dtype=dtype)
                dist.all_gather_into_tensor(ref_g, mine)
                got_g = pp.all_gather(torch.empty(n, device="cuda", dtype=dtype), mine, algorithm="push")
                ref_a = torch.empty(n, device="cuda", dtype=dtype)
                dist.all_to_all_single(ref_a, full_in)
                got_a = pp.all_to_all(torch.empty(n, device="cuda", dtype=dtype), full_in, algorithm="push")
                torch.cuda.synchronize()
                __import__("pccl_b200.ops.gemm", fromlist=["check"]).check()
                atol = 1e-5 if dtype == torch.float32 else 0.06
                torch.testing.assert_close(got.float(), ref, atol=atol, rtol=2e-2,
                                           msg=lambda t: f"push reduce_scatter {dtype} shard={shard} rank {rank}: {t}")
                assert torch.equal(got_g, ref_g), f"push all_gather {dtype} shard={shard} rank {rank}"
                assert torch.equal(got_a, ref_a), f"push all_to_all {dtype} shard={shard} rank {rank}"
        report["checked"] += 1

    # every rank must hold bit-identical results (sums are taken in rank order)
    x = torch.randn(4096, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5 + rank))
    y = pp.all_reduce(x.clone(), algorithm="ll")
    gathered = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(gathered, y)
    assert all(torch.equal(gathered[0], g) for g in gathered), "ll allreduce differs between ranks"

    # max / avg through the API
    x = torch.randn(world * 4096, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rank))
    ref = x.clone(); dist.all_reduce(ref, op=dist.ReduceOp.MAX)
    y = x.clone(); pp.all_reduce(y, op="max", algorithm="twoshot")
    torch.testing.assert_close(y, ref)
    ref = x.clone(); dist.all_reduce(ref); ref /= world
    y = x.clone(); pp.all_reduce(y, op="avg", algorithm="twoshot")
    torch.testing.assert_close(y, ref, atol=1e-5, rtol=1e-5)

    # ---- fused tensor-parallel GEMMs (tcgen05 kernels with the collective in the epilogue) ----
    from pccl_b200.ops import AllGatherGemm, GemmReduceScatter, gemm
    for (m, n, k) in ((world * 256, 512, 192), (world * 1024, 4096, 1792)):
        gen = torch.Generator(device="cuda").manual_seed(7 + rank)
        x = torch.randn(m, k, device="cuda", generator=gen).to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
        full = x.float() @ w.float().t()
        ref = torch.empty(m // world, n, device="cuda")
        dist.reduce_scatter_tensor(ref, full)
        op = GemmReduceScatter(m, n, k)
        for call in range(3):          # several calls: epoch counting and slot parity
            y = op(x, w)
            torch.cuda.synchronize()
            gemm.check()
            torch.testing.assert_close(y.float(), ref, atol=0.03, rtol=3e-2,
                                       msg=lambda t: f"gemm_rs {m}x{n}x{k} call {call} rank {rank}: {t}")
        report["checked"] += 1

        rows = m // world
        xs = torch.randn(rows, k, device="cuda", generator=gen).to(torch.bfloat16)
        wl = (torch.randn(n, k, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
        gathered = torch.empty(m, k, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(gathered, xs)
        ref = gathered.float() @ wl.float().t()
        ag = AllGatherGemm(m, n, k)
        for call in range(3):
            y = ag(xs, wl)
            torch.cuda.synchronize()
            gemm.check()
            torch.testing.assert_close(y.float(), ref, atol=0.03, rtol=3e-2,
                                       msg=lambda t: f"ag_gemm {m}x{n}x{k} call {call} rank {rank}: {t}")
        report["checked"] += 1

    # ---- all-reduce + residual + RMSNorm (one-shot for tiny token counts, two-shot otherwise) ----
    from pccl_b200.ops import AllReduceResidualRMSNorm
    hidden = 4096
    for tokens in (1, 128, 1024):
        for use_nvls in ("force", False):
            gen = torch.Generator(device="cuda").manual_seed(100 + rank)
            xp = torch.randn(tokens, hidden, device="cuda", generator=gen).to(torch.bfloat16)
            gen0 = torch.Generator(device="cuda").manual_seed(5)          # identical on every rank
            res0 = torch.randn(tokens, hidden, device="cuda", generator=gen0).to(torch.bfloat16)
            gamma = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=gen0)).to(torch.bfloat16)
            total = xp.float().clone()
            dist.all_reduce(total)
            h_ref = total + res0.float()
            y_ref = h_ref * torch.rsqrt(h_ref.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()
            op = AllReduceResidualRMSNorm(tokens, hidden, use_nvls=use_nvls)
            for call in range(2):
                op.x.copy_(xp)
                op.residual.copy_(res0)
                y, h = op(gamma)
                torch.cuda.synchronize()
                gemm.check()
                torch.testing.assert_close(h.float(), h_ref, atol=0.06, rtol=2e-2,
                                           msg=lambda t: f"ar_rmsnorm h T={tokens} nvls={use_nvls} rank {rank}: {t}")
                torch.testing.assert_close(y.float(), y_ref, atol=0.06, rtol=2e-2,
                                           msg=lambda t: f"ar_rmsnorm y T={tokens} nvls={use_nvls} rank {rank}: {t}")
            report["checked"] += 1

    # ---- expert-parallel MoE: route + dispatch, grouped expert GEMMs, gate-weighted return + combine ----
    from pccl_b200.ops import moe
    for (tokens, hidden_m, ffn, experts) in ((512, 512, 1024, 8), (300, 1024, 2048, 8)):
        gen0 = torch.Generator(device="cuda").manual_seed(11)             # identical on every rank
        wg = (torch.randn(experts, hidden_m, device="cuda", generator=gen0) * 0.5).to(torch.bfloat16)
        w1 = (torch.randn(experts, ffn, hidden_m, device="cuda", generator=gen0) * hidden_m ** -0.5).to(torch.bfloat16)
        w3 = (torch.randn(experts, ffn, hidden_m, device="cuda", generator=gen0) * hidden_m ** -0.5).to(torch.bfloat16)
        w2 = (torch.randn(experts, hidden_m, ffn, device="cuda", generator=gen0) * ffn ** -0.5).to(torch.bfloat16)
        layer = moe.FusedMoE(tokens, hidden_m, ffn, experts)
        le = experts // world
        mine = slice(rank * le, (rank + 1) * le)
        layer.set_weights(wg, w1[mine], w3[mine], w2[mine])
        gen = torch.Generator(device="cuda").manual_seed(200 + rank)
        for call in range(3):
            xt = torch.randn(tokens, hidden_m, device="cuda", generator=gen).to(torch.bfloat16)
            out = layer(xt)
            torch.cuda.synchronize()
            gemm.check()
            ref, ref_idx, _ = moe.moe_reference(xt, wg, w1, w3, w2)
            same = (layer.topk_idx.long() == ref_idx).all(dim=-1)
            assert same.float().mean() > 0.95, f"moe routing differs on rank {rank}"
            err = (out.float() - ref)[same].abs().max().item()
            scale = ref[same].abs().max().item()
            assert err <= 2e-2 * scale + 1e-3, f"moe T={tokens} call {call} rank {rank}: error {err} vs {scale}"
        report["checked"] += 1

    # ---- model blocks and data-parallel gradient buckets ----
    from pccl_b200.models import TensorParallelMLP
    from pccl_b200.parallel.layers import GradientBuckets
    tokens, hid, f_local = world * 128, 512, 256
    gen0 = torch.Generator(device="cuda").manual_seed(21)                 # identical on every rank
    wgu_all = [(torch.randn(2 * f_local, hid, device="cuda", generator=gen0) * hid ** -0.5).to(torch.bfloat16)
               for _ in range(world)]
    wd_all = [(torch.randn(hid, f_local, device="cuda", generator=gen0) * f_local ** -0.5).to(torch.bfloat16)
              for _ in range(world)]
    x_full = torch.randn(tokens, hid, device="cuda", generator=gen0).to(torch.bfloat16)
    mlp = TensorParallelMLP(tokens, hid, f_local, wgu_all[rank], wd_all[rank])
    rows = tokens // world
    y = mlp(x_full[rank * rows:(rank + 1) * rows].contiguous())
    torch.cuda.synchronize()
    gemm.check()
    ref = TensorParallelMLP.reference(x_full, wgu_all, wd_all)[rank * rows:(rank + 1) * rows]
    err = (y.float() - ref).abs().max().item()
    assert err <= 3e-2 * ref.abs().max().item() + 1e-2, f"tp mlp rank {rank}: error {err}"
    report["checked"] += 1

    params = [torch.nn.Parameter(torch.zeros(n, device="cuda", dtype=torch.bfloat16)) for n in (1000, 333, 70000, 8)]
    expect = []
    for i, prm in enumerate(params):
        gen = torch.Generator(device="cuda").manual_seed(300 + 10 * rank + i)
        prm.grad = torch.randn(prm.shape, device="cuda", generator=gen).to(torch.bfloat16)
        total = prm.grad.float().clone()
        dist.all_reduce(total)
        expect.append(total / world)
    GradientBuckets(params, bucket_bytes=64 << 10).reduce()
    torch.cuda.synchronize()
    for prm, want in zip(params, expect):
        torch.testing.assert_close(prm.grad.float(), want, atol=0.03, rtol=2e-2)
    report["checked"] += 1

    # Hook-driven reduction during a real backward, next to GEMMs that keep the SMs busy: the buckets'
    # collectives are launched while backward still computes (all their CTAs resident at once, so the
    # matmuls delay them but cannot starve them).
    torch.manual_seed(77)                                                 # identical weights on every rank
    layers = torch.nn.Sequential(*[torch.nn.Linear(2048, 2048, bias=False) for _ in range(4)]).cuda().bfloat16()
    buckets = GradientBuckets(layers.parameters(), bucket_bytes=2048 * 2048 * 2).attach()
    for step in range(2):
        layers.zero_grad(set_to_none=True)
        xb = torch.randn(4096, 2048, device="cuda", generator=torch.Generator(device="cuda").manual_seed(40 + rank + step)
                         ).bfloat16()
        layers(xb).float().pow(2).mean().backward()
        buckets.finish()
        torch.cuda.synchronize()
        pp.check_errors()
    # reference: the same backward without hooks, averaged with NCCL
    buckets.detach()
    layers.zero_grad(set_to_none=True)
    layers(xb).float().pow(2).mean().backward()
    for prm in layers.parameters():
        want = prm.grad.float().clone()
        dist.all_reduce(want)
        prm.expected = want / world
    layers.zero_grad(set_to_none=True)
    buckets.attach()
    layers(xb).float().pow(2).mean().backward()
    buckets.finish()
    torch.cuda.synchronize()
    for prm in layers.parameters():
        torch.testing.assert_close(prm.grad.float(), prm.expected, atol=2e-3, rtol=5e-2)
    buckets.detach()
    report["checked"] += 1

    # ---- OCS layer over the real engine, the NVLink connector, rank-uniform path choice ----
    from pccl_b200 import selfcheck
    ocs = selfcheck.run(only=["misaligned_view_same_path", "ocs_barrier_nvlink_connector",
                              "ocs_collective_plan_over_engine", "ocs_phase_runner_over_engine"])
    assert not ocs["failed"] and ocs["passed"] == 4, f"OCS / path-choice cases: {ocs}"
    report["checked"] += ocs["passed"]

    # A rank that never joins a barrier: the others' wait runs out (a short limit), they get a
    # timeout naming the missing rank, and after a collective reset the board works again.
    from pccl_b200.ocs import OCSBarrierTimeout, OCSPlan, OCSRuntime
    connector = selfcheck._nvlink_connector()
    runtime = OCSRuntime(connector=connector)
    if rank != world - 1:
        try:
            runtime.barrier_switch(OCSPlan(job_id="absent", barrier_id=50, epoch_id=50, next_epoch_id=51), timeout=0.3)
        except OCSBarrierTimeout as err:
            assert str(world - 1) in str(err), f"timeout does not name the missing rank: {err}"
        else:
            raise AssertionError("a barrier completed without one of its ranks")
    torch.cuda.synchronize()
    dist.barrier()
    connector.board.reset()
    dist.barrier()
    release = runtime.barrier_switch(OCSPlan(job_id="absent", barrier_id=51, epoch_id=51, next_epoch_id=52))
    assert release["status"] == "OK"
    report["checked"] += 1

    # A push collective whose peer never calls: bounded wait, error surfaced by synchronize(), reset, then correct.
    if os.environ.get("PCCL_TEST_PUSH_TIMEOUT", "1") == "1":
        probe = torch.ones(4096, device="cuda")
        if rank == 0:
            pp.all_reduce(probe, algorithm="push")
            try:
                pp.synchronize()
            except Exception as err:  # noqa: BLE001
                assert "push collective" in str(err), f"unexpected error text: {err}"
            else:
                raise AssertionError("a push all-reduce without its peers reported no timeout")
        pp.reset()
        probe = torch.full((4096,), float(rank + 1), device="cuda")
        pp.all_reduce(probe, algorithm="push")
        pp.synchronize()
        assert torch.equal(probe, torch.full_like(probe, world * (world + 1) / 2)), "push all-reduce wrong after reset"
        report["checked"] += 1

    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_PASS " + json.dumps(report), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except Exception as err:  # one greppable line per failing rank, then the usual traceback
        print(f"MULTI_GPU_FAIL rank {os.environ.get('RANK')}: {type(err).__name__}: "
              + " | ".join(str(err).splitlines()[:12]), flush=True)
        raise
