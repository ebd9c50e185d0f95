"""A fast multi-GPU self-check: one small case of every multi-rank path, against NCCL.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m pccl_b200.selfcheck

or, from a program that already initialised the process group and the engine::

    from pccl_b200 import selfcheck
    report = selfcheck.run()          # {"passed": 17, "failed": [], "skipped": [...], "seconds": 2.1}

Every case runs on every rank; a case counts as passed only if it passed on all of them (the
ranks agree through one small NCCL reduction per case), and after a failed case the collective
state is reset so that later cases are still meaningful.  Cases are small (a few MB at most) and
every device wait inside the library is bounded, so a broken path shows up as a named failure,
not as a hang.  The thorough versions of these cases (all dtypes, odd sizes, repeated calls) are
in tests/multi_gpu_worker.py; the reference checks its collectives with a manual script only
(tests/test_correctness.py:140-289).
"""

from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


def _tol(dtype):
    return dict(atol=1e-4, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.1, rtol=2 ** -6)


def _randn(n, seed, dtype=torch.float32):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(n, device="cuda", generator=gen).to(dtype)


class _Ctx:
    def __init__(self):
        import pccl_b200.parallel as pp
        self.pp = pp
        self.engine = pp.init()
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.nvls = bool(self.engine.nvls_active())


# ---- cases -----------------------------------------------------------------------------------

def _allreduce_plan(algorithm: str, dtype=torch.float32, numel_per_rank: int = 65536, channels: int = 2):
    def case(c: _Ctx):
        n = c.world * numel_per_rank
        x = _randn(n, 100 + c.rank, dtype)
        ref = x.float().clone()
        dist.all_reduce(ref)
        y = x.clone()
        c.pp.all_reduce(y, algorithm=algorithm, channels=channels)
        torch.testing.assert_close(y.float(), ref, **_tol(dtype))
    return case


def _switch_kernel_allreduce(c: _Ctx):
    """The in-switch all-reduce kernel: in place on a symmetric tensor and staged on an ordinary one,
    twice each (call counting)."""
    for dtype in (torch.float32, torch.bfloat16):
        n = c.world * 98304
        x = _randn(n, 300 + c.rank, dtype)
        ref = x.float().clone()
        dist.all_reduce(ref)
        sym = c.pp.working_tensor(n, dtype)
        for _ in range(2):
            sym.copy_(x)
            c.pp.all_reduce(sym, algorithm="nvls_kernel")
            c.pp.synchronize()
            torch.testing.assert_close(sym.float(), ref, **_tol(dtype))
            y = c.pp.all_reduce(x.clone(), algorithm="nvls_kernel")
            c.pp.synchronize()
            torch.testing.assert_close(y.float(), ref, **_tol(dtype))


def _packet_allreduce(c: _Ctx):
    for dtype in (torch.float32, torch.bfloat16):
        x = _randn(16384, 7 + c.rank, dtype)
        ref = x.float().clone()
        dist.all_reduce(ref)
        y = c.pp.all_reduce(x.clone(), algorithm="ll")
        c.pp.synchronize()
        torch.testing.assert_close(y.float(), ref, atol=1e-5 if dtype == torch.float32 else 0.06, rtol=2e-2)


def _push_mode(mode: str):
    def case(c: _Ctx):
        pp, world, rank = c.pp, c.world, c.rank
        shard = 32768
        n = shard * world
        full = _randn(n, 31 + rank, torch.bfloat16)
        mine = _randn(shard, 57 + rank, torch.bfloat16)
        if mode == "allreduce":
            ref = full.float().clone()
            dist.all_reduce(ref)
            got = pp.all_reduce(full.clone(), algorithm="push")
            pp.synchronize()
            torch.testing.assert_close(got.float(), ref, atol=0.06, rtol=2e-2)
        elif mode == "reduce_scatter":
            ref = torch.empty(shard, device="cuda")
            dist.reduce_scatter_tensor(ref, full.float())
            got = pp.reduce_scatter(torch.empty(shard, device="cuda", dtype=torch.bfloat16), full, algorithm="push")
            pp.synchronize()
            torch.testing.assert_close(got.float(), ref, atol=0.06, rtol=2e-2)
        elif mode == "all_gather":
            ref = torch.empty(n, device="cuda", dtype=torch.bfloat16)
            dist.all_gather_into_tensor(ref, mine)
            got = pp.all_gather(torch.empty(n, device="cuda", dtype=torch.bfloat16), mine, algorithm="push")
            pp.synchronize()
            assert torch.equal(got, ref), "push all_gather differs from NCCL"
        else:
            ref = torch.empty(n, device="cuda", dtype=torch.bfloat16)
            dist.all_to_all_single(ref, full)
            got = pp.all_to_all(torch.empty(n, device="cuda", dtype=torch.bfloat16), full, algorithm="push")
            pp.synchronize()
            assert torch.equal(got, ref), "push all_to_all differs from NCCL"
    return case


def _packet_shard_collectives(c: _Ctx):
    """Reduce-scatter, all-gather (also with the input inside the output) and all-to-all through the packet
    kernel, interleaved with packet all-reduces (they share the buffer and the call counter)."""
    pp, world, rank = c.pp, c.world, c.rank
    for dtype, shard in ((torch.float32, 4096), (torch.bfloat16, 10240)):
        n = shard * world
        full = _randn(n, 41 + rank, dtype)
        mine = _randn(shard, 67 + rank, dtype)
        tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.06, rtol=2e-2)
        ref = torch.empty(shard, device="cuda")
        dist.reduce_scatter_tensor(ref, full.float())
        got = pp.reduce_scatter(torch.empty(shard, device="cuda", dtype=dtype), full, algorithm="ll")
        torch.testing.assert_close(got.float(), ref, **tol)
        ref = torch.empty(n, device="cuda", dtype=dtype)
        dist.all_gather_into_tensor(ref, mine)
        got = pp.all_gather(torch.empty(n, device="cuda", dtype=dtype), mine, algorithm="ll")
        assert torch.equal(got, ref), "packet all_gather differs from NCCL"
        inplace = torch.zeros(n, device="cuda", dtype=dtype)
        inplace[rank * shard:(rank + 1) * shard] = mine
        pp.all_gather(inplace, inplace[rank * shard:(rank + 1) * shard])     # unforced: small parts take this path
        assert torch.equal(inplace, ref), "in-place packet all_gather differs from NCCL"
        x = _randn(2048, 5 + rank, dtype)
        want = x.float().clone()
        dist.all_reduce(want)
        torch.testing.assert_close(pp.all_reduce(x.clone(), algorithm="ll").float(), want, **tol)
        ref = torch.empty(n, device="cuda", dtype=dtype)
        dist.all_to_all_single(ref, full)
        got = pp.all_to_all(torch.empty(n, device="cuda", dtype=dtype), full, algorithm="ll")
        assert torch.equal(got, ref), "packet all_to_all differs from NCCL"
    pp.synchronize()


def _misaligned_views_take_the_same_path(c: _Ctx):
    """One rank passes a view that is not 16-byte (nor 8-byte) aligned: every rank must still run the
    same kernel, and the reduction must land in that view."""
    n = 4096
    for algorithm in ("ll", "push"):
        base = _randn(n + 3, 900 + c.rank)
        view = base[3:3 + n] if c.rank == 0 else base[:n]      # rank 0 starts 12 bytes into the allocation
        ref = view.clone()
        dist.all_reduce(ref)
        c.pp.all_reduce(view, algorithm=algorithm)
        c.pp.synchronize()
        torch.testing.assert_close(view, ref, atol=1e-5, rtol=1e-5)


def _plan_shards(algorithm: str):
    def case(c: _Ctx):
        pp, world, rank = c.pp, c.world, c.rank
        n = world * 262144
        shard = n // world
        x = _randn(n, 300 + rank)
        ref = x.clone()
        dist.all_reduce(ref)
        out = torch.empty(shard, device="cuda")
        pp.reduce_scatter(out, x, algorithm=algorithm)
        torch.testing.assert_close(out, ref[rank * shard:(rank + 1) * shard], atol=1e-4, rtol=1e-5)
        expect = torch.empty(n, device="cuda")
        dist.all_gather_into_tensor(expect, x[:shard].contiguous())
        full = torch.zeros(n, device="cuda")
        pp.all_gather(full, x[:shard].contiguous(), algorithm=algorithm)
        assert torch.equal(full, expect), f"{algorithm} all_gather differs from NCCL"
    return case


def _copy_engine_all_gather(c: _Ctx):
    n = c.world * 262144
    shard = n // c.world
    x = _randn(n, 400 + c.rank)
    expect = torch.empty(n, device="cuda")
    dist.all_gather_into_tensor(expect, x[:shard].contiguous())
    full = torch.zeros(n, device="cuda")
    c.pp.all_gather(full, x[:shard].contiguous(), channels=2, executor="ce")
    assert torch.equal(full, expect), "copy-engine all_gather differs from NCCL"
    assert any(st.get("copy_engine") for st in c.engine.stats().values()), "copy-engine executor not used"


def _ar_rmsnorm(use_nvls):
    def case(c: _Ctx):
        from pccl_b200.ops import AllReduceResidualRMSNorm, gemm
        tokens, hidden = 128, 4096
        xp = _randn(tokens * hidden, 500 + c.rank, torch.bfloat16).view(tokens, hidden)
        res0 = _randn(tokens * hidden, 5, torch.bfloat16).view(tokens, hidden)
        gamma = (1 + 0.1 * _randn(hidden, 6)).to(torch.bfloat16)
        total = xp.float().clone()
        dist.all_reduce(total)
        h_ref = total + res0.float()
        y_ref = h_ref * torch.rsqrt(h_ref.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()
        op = AllReduceResidualRMSNorm(tokens, hidden, use_nvls=use_nvls)
        op.x.copy_(xp)
        op.residual.copy_(res0)
        y, h = op(gamma)
        torch.cuda.synchronize()
        gemm.check()
        torch.testing.assert_close(h.float(), h_ref, atol=0.06, rtol=2e-2)
        torch.testing.assert_close(y.float(), y_ref, atol=0.06, rtol=2e-2)
    return case


def _gemm_reduce_scatter(c: _Ctx):
    from pccl_b200.ops import GemmReduceScatter, gemm
    m, n, k = c.world * 256, 512, 192
    x = _randn(m * k, 600 + c.rank, torch.bfloat16).view(m, k)
    w = (_randn(n * k, 650 + c.rank) * 0.02).to(torch.bfloat16).view(n, k)
    ref = torch.empty(m // c.world, n, device="cuda")
    dist.reduce_scatter_tensor(ref, x.float() @ w.float().t())
    op = GemmReduceScatter(m, n, k)
    for _ in range(2):
        y = op(x, w)
        torch.cuda.synchronize()
        gemm.check()
        torch.testing.assert_close(y.float(), ref, atol=0.03, rtol=3e-2)


def _all_gather_gemm(c: _Ctx):
    from pccl_b200.ops import AllGatherGemm, gemm
    m, n, k = c.world * 256, 512, 192
    xs = _randn(m // c.world * k, 700 + c.rank, torch.bfloat16).view(m // c.world, k)
    w = (_randn(n * k, 750 + c.rank) * 0.02).to(torch.bfloat16).view(n, k)
    gathered = torch.empty(m, k, device="cuda", dtype=torch.bfloat16)
    dist.all_gather_into_tensor(gathered, xs)
    ref = gathered.float() @ w.float().t()
    op = AllGatherGemm(m, n, k)
    for _ in range(2):
        y = op(xs, w)
        torch.cuda.synchronize()
        gemm.check()
        torch.testing.assert_close(y.float(), ref, atol=0.03, rtol=3e-2)


def _expert_parallel_moe(c: _Ctx):
    from pccl_b200.ops import gemm, moe
    tokens, hidden, ffn, experts = 256, 512, 1024, 8
    if experts % c.world:
        raise _Skip(f"{experts} experts do not divide over {c.world} ranks")
    wg = (_randn(experts * hidden, 11) * 0.5).to(torch.bfloat16).view(experts, hidden)
    w1 = (_randn(experts * ffn * hidden, 12) * hidden ** -0.5).to(torch.bfloat16).view(experts, ffn, hidden)
    w3 = (_randn(experts * ffn * hidden, 13) * hidden ** -0.5).to(torch.bfloat16).view(experts, ffn, hidden)
    w2 = (_randn(experts * hidden * ffn, 14) * ffn ** -0.5).to(torch.bfloat16).view(experts, hidden, ffn)
    layer = moe.FusedMoE(tokens, hidden, ffn, experts)
    le = experts // c.world
    mine = slice(c.rank * le, (c.rank + 1) * le)
    layer.set_weights(wg, w1[mine], w3[mine], w2[mine])
    xt = _randn(tokens * hidden, 800 + c.rank, torch.bfloat16).view(tokens, hidden)
    out = layer(xt)
    torch.cuda.synchronize()
    gemm.check()
    ref, ref_idx, _ = moe.moe_reference(xt, wg, w1, w3, w2)
    same = (layer.topk_idx.long() == ref_idx).all(dim=-1)
    assert same.float().mean() > 0.95, "MoE routing differs from the reference"
    err = (out.float() - ref)[same].abs().max().item()
    assert err <= 2e-2 * ref[same].abs().max().item() + 1e-3, f"MoE error {err}"


_connector = None


def _nvlink_connector():
    """One board per process (its slots come from the arena, which is never handed back)."""
    global _connector
    if _connector is None:
        from pccl_b200.ocs import NvlinkSwitchConnector
        _connector = NvlinkSwitchConnector()
    return _connector


def _ocs_barrier_over_nvlink(c: _Ctx):
    from pccl_b200.ocs import OCSPlan, OCSPlanMismatchError, OCSRuntime
    runtime = OCSRuntime(connector=_nvlink_connector())
    for i in range(5):
        release = runtime.barrier_switch(OCSPlan(job_id="selfcheck", barrier_id=i, epoch_id=i, next_epoch_id=i + 1,
                                                 topology_id=i % 2))
        assert release["status"] == "OK" and len(release["ready_records"]) == c.world
        assert sorted(r["src_rank"] for r in release["ready_records"]) == list(range(c.world))
    # One rank arrives with another topology: every rank must see the mismatch.
    odd = OCSPlan(job_id="selfcheck", barrier_id=9, epoch_id=9, next_epoch_id=10,
                  topology_id=7 if c.rank == c.world - 1 else 1)
    try:
        runtime.barrier_switch(odd)
    except OCSPlanMismatchError:
        pass
    else:
        raise AssertionError("a plan mismatch went unnoticed")
    # Validation failed before the commit round on every rank alike, so the board stays in step.
    release = runtime.barrier_switch(OCSPlan(job_id="selfcheck", barrier_id=10, epoch_id=10, next_epoch_id=11))
    assert release["status"] == "OK"


def _ocs_collective_plan_over_engine(c: _Ctx):
    """all-reduce -> barrier -> all-to-all -> barrier -> all-reduce as engine plans."""
    import pccl_b200 as pccl
    from pccl_b200.ocs import OcsCollectivePlanRunner, OCSRuntime, build_ring_allreduce_alltoall_plan
    n = c.world * 4096
    runtime = OCSRuntime(connector=_nvlink_connector())
    runner = OcsCollectivePlanRunner(engine=pccl.engine, runtime=runtime)
    prepared = runner.prepare(build_ring_allreduce_alltoall_plan(c.rank, c.world, n, "float32", "sm",
                                                                 job_id="selfcheck_plan"), "selfcheck_seq")
    try:
        x = _randn(n, 1000 + c.rank)
        ref = x.clone()
        dist.all_reduce(ref)
        swapped = torch.empty_like(ref)
        dist.all_to_all_single(swapped, ref)
        dist.all_reduce(swapped)
        out = runner.execute(prepared, x)
        torch.testing.assert_close(out, swapped, atol=1e-3, rtol=1e-5)
        assert len([r for r in runtime.history if r["msg_type"] == "OCS_BARRIER_RELEASE"]) == 2
    finally:
        prepared.close()


def _ocs_phase_runner_over_engine(c: _Ctx):
    """One graph cut by an ocs_barrier (a version-3 manifest): direct reduce-scatter, barrier, all-gather."""
    import pccl_b200 as pccl
    from pccl_b200.dsl.algorithms.base import all_pairs_barrier
    from pccl_b200.dsl.decorators import build_graph
    from pccl_b200.ocs import OcsPhaseRunner, OCSRuntime
    rank, world = c.rank, c.world
    n = world * 8192
    piece = n // world

    def build(op):
        op.tensor("float32", (n,))
        all_pairs_barrier(op, rank, world, 200)
        op.sm_reduce_multi(source_ranks=list(range(world)), remote_offset=rank * piece, dst_offset=rank * piece,
                           count=piece)
        all_pairs_barrier(op, rank, world, 300)
        op.ocs_barrier(barrier_id=1, epoch_id=0, next_epoch_id=1, participant_ranks=tuple(range(world)),
                       topology_id=1, route_plan_id=1)
        all_pairs_barrier(op, rank, world, 400)
        for i in range(1, world):
            peer = (rank + i) % world
            op.sm_copy(source_rank=peer, src_offset=peer * piece, dst_offset=peer * piece, size=piece)
        all_pairs_barrier(op, rank, world, 500)

    graph = build_graph(f"selfcheck_phased_rank{rank}", build)
    graph.collective_type = "allreduce"
    runtime = OCSRuntime(connector=_nvlink_connector())
    runner = OcsPhaseRunner(engine=pccl.engine, runtime=runtime)
    prepared = runner.prepare(graph, "selfcheck_phased")
    try:
        assert prepared.manifest["version"] == 3 and len(prepared.operation_names) == 2
        x = _randn(n, 1100 + rank)
        ref = x.clone()
        dist.all_reduce(ref)
        out = runner.execute(prepared, x)
        torch.testing.assert_close(out, ref, atol=1e-4, rtol=1e-5)
    finally:
        prepared.close()


class _Skip(Exception):
    pass


def cases(nvls: bool) -> List[Tuple[str, Callable[[_Ctx], None]]]:
    out: List[Tuple[str, Callable[[_Ctx], None]]] = [
        ("packet_allreduce", _packet_allreduce),
        ("push_allreduce", _push_mode("allreduce")),
        ("push_reduce_scatter", _push_mode("reduce_scatter")),
        ("push_all_gather", _push_mode("all_gather")),
        ("push_all_to_all", _push_mode("all_to_all")),
        ("misaligned_view_same_path", _misaligned_views_take_the_same_path),
        ("plan_twoshot_allreduce", _allreduce_plan("twoshot")),
        ("plan_ring_allreduce_bf16", _allreduce_plan("ring", torch.bfloat16)),
        ("plan_twoshot_rs_ag", _plan_shards("twoshot")),
        ("copy_engine_all_gather", _copy_engine_all_gather),
        ("ar_residual_rmsnorm_peer", _ar_rmsnorm(False)),
        ("packet_shard_collectives", _packet_shard_collectives),
        ("gemm_reduce_scatter", _gemm_reduce_scatter),
        ("all_gather_gemm", _all_gather_gemm),
        ("expert_parallel_moe", _expert_parallel_moe),
        ("ocs_barrier_nvlink_connector", _ocs_barrier_over_nvlink),
        ("ocs_collective_plan_over_engine", _ocs_collective_plan_over_engine),
        ("ocs_phase_runner_over_engine", _ocs_phase_runner_over_engine),
    ]
    if nvls:
        out += [
            ("plan_nvls_allreduce", _allreduce_plan("nvls")),
            ("plan_nvls_allreduce_bf16", _allreduce_plan("nvls", torch.bfloat16)),
            ("plan_hybrid_allreduce", _allreduce_plan("hybrid", channels=4)),
            ("switch_kernel_allreduce", _switch_kernel_allreduce),
            ("plan_nvls_rs_ag", _plan_shards("nvls")),
            ("ar_residual_rmsnorm_nvls", _ar_rmsnorm("force")),
        ]
    return out


def run(only: Optional[List[str]] = None, verbose: bool = False) -> Dict[str, object]:
    """Run the cases (all, or those named in ``only``).  Collective; needs an initialised NCCL group."""
    ctx = _Ctx()
    t0 = time.perf_counter()
    passed, failed, skipped = 0, [], []
    for name, fn in cases(ctx.nvls):
        if only and name not in only:
            continue
        ok, note = 1, ""
        try:
            fn(ctx)
            torch.cuda.synchronize()
        except _Skip as why:
            ok, note = 2, str(why)
        except Exception as err:  # noqa: BLE001 - every failure becomes a named entry of the report
            ok, note = 0, f"{type(err).__name__}: {str(err).splitlines()[0][:200] if str(err) else ''}"
        verdict = torch.tensor([ok], device="cuda", dtype=torch.int32)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
        agreed = int(verdict.item())
        if agreed == 0:
            failed.append(name if not note else f"{name} ({note})" if ok == 0 else name)
            ctx.pp.reset()
            global _connector
            if _connector is not None:
                _connector.board.reset()
                dist.barrier()
        elif agreed == 2:
            skipped.append(name)
        else:
            passed += 1
        if verbose and ctx.rank == 0:
            print(f"[selfcheck] {name}: {'ok' if agreed == 1 else 'skipped' if agreed == 2 else 'FAILED ' + note}",
                  flush=True)
    if not ctx.nvls:
        skipped.append("nvls cases (no multicast on this box)")
    return {"passed": passed, "failed": failed, "skipped": skipped, "world": ctx.world,
            "seconds": round(time.perf_counter() - t0, 2)}


def main() -> None:
    import json
    import os
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    os.environ.setdefault("PCCL_BUFFER_SIZE", str(256 << 20))
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    report = run(verbose=True)
    if rank == 0:
        print("SELFCHECK " + json.dumps(report), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if report["failed"]:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
