"""Multi-process paths on CPU (gloo, world_size 2): plan replay, the OCS barrier
over real collectives, torch collective plans, and a rank that fails on the host."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from helpers import free_port  # noqa: E402


def _run(worker, world, *args, timeout=120):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(worker, r, world, port, queue, args)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, payload = queue.get(timeout=timeout)
            results[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    for rank, payload in results.items():
        if isinstance(payload, str) and payload.startswith("ERROR"):
            raise AssertionError(f"rank {rank}: {payload}")
    return results


def _entry(worker, rank, world, port, queue, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        import datetime
        dist.init_process_group("gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=60))
        queue.put((rank, worker(rank, world, *args)))
    except Exception as err:  # pragma: no cover - surfaced through the queue
        import traceback
        queue.put((rank, "ERROR " + traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


# -- config 1: 8-rank ring plan, superopt, JSON, replay on 2 gloo processes ----------------

def _replay_worker(rank, world, plan_world, n, algorithm):
    import json
    from pccl_b200 import Compiler
    from pccl_b200.dsl.algorithms import ALGORITHMS
    from pccl_b200.runtime import GlooPlanExecutor
    texts = [Compiler(enable_superopt=True).compile_to_json(
        ALGORITHMS[algorithm]().build_allreduce(r, plan_world, n, "float32", "sm"))
        for r in range(plan_world)]
    for text in texts:                                   # JSON round trip
        assert json.dumps(json.loads(text), indent=2) == text
    ex = GlooPlanExecutor()
    hosted = ex.hosted_ranks(plan_world)
    inputs = {v: torch.randn(n, generator=torch.Generator().manual_seed(v)) for v in hosted}
    outs = ex.execute(texts, inputs)
    total = sum(torch.randn(n, generator=torch.Generator().manual_seed(v)) for v in range(plan_world))
    return max(float((outs[v] - total).abs().max()) for v in hosted)


def test_eight_rank_ring_plan_replayed_on_two_gloo_processes():
    errors = _run(_replay_worker, 2, 8, 1024 * 1024, "ring")
    assert max(errors.values()) <= 1e-5


def test_twoshot_plan_one_rank_per_process():
    errors = _run(_replay_worker, 2, 2, 4096, "twoshot")
    assert max(errors.values()) <= 1e-5


# -- OCS barrier over real object / tensor collectives -------------------------------------

def _barrier_worker(rank, world, connector_name, link_ready):
    from pccl_b200.ocs import (OCSLinkNotReady, OCSPlan, OCSRuntime, TensorSwitchConnector,
                               TorchDistributedSwitchConnector)
    cls = {"object": TorchDistributedSwitchConnector, "tensor": TensorSwitchConnector}[connector_name]
    rt = OCSRuntime(connector=cls(link_ready=link_ready))
    plan = OCSPlan(barrier_id=1, participant_ranks=(0, 1), topology_id=4)
    try:
        out = rt.barrier_switch(plan)
    except OCSLinkNotReady:
        return "aborted:" + rt.history[-1]["msg_type"]
    return "released:%d:%s" % (len(out["ready_records"]), out["link_state"])


@pytest.mark.parametrize("connector", ["object", "tensor"])
def test_barrier_over_gloo(connector):
    assert set(_run(_barrier_worker, 2, connector, True).values()) == {"released:2:LINK_ALIGNED"}
    assert set(_run(_barrier_worker, 2, connector, False).values()) == {"aborted:OCS_BARRIER_ABORT"}


def _mismatch_worker(rank, world, connector_name):
    from pccl_b200.ocs import (OCSPlan, OCSPlanMismatchError, OCSRuntime, TensorSwitchConnector,
                               TorchDistributedSwitchConnector)
    cls = {"object": TorchDistributedSwitchConnector, "tensor": TensorSwitchConnector}[connector_name]
    plan = OCSPlan(barrier_id=1, participant_ranks=(0, 1), topology_id=4 + rank)   # ranks disagree
    try:
        OCSRuntime(connector=cls()).barrier_switch(plan)
    except OCSPlanMismatchError as err:
        return "mismatch" if "topology_id" in str(err) else "other"
    return "released"


@pytest.mark.parametrize("connector", ["object", "tensor"])
def test_plan_mismatch_detected_on_every_rank(connector):
    assert set(_run(_mismatch_worker, 2, connector).values()) == {"mismatch"}


def _torch_plan_worker(rank, world):
    from pccl_b200.ocs import OcsTorchPlanRunner, build_torch_allreduce_alltoall_plan, ocs_all_reduce
    x = torch.arange(4, dtype=torch.float32) + 10 * rank
    out = OcsTorchPlanRunner().execute(build_torch_allreduce_alltoall_plan(world), x)
    y = ocs_all_reduce(torch.ones(2) * (rank + 1))
    return out.tolist(), y.tolist()


def test_torch_collective_plan_over_gloo():
    res = _run(_torch_plan_worker, 2)
    # AR: [10,12,14,16] on both; A2A: rank0 keeps [10,12 | 10,12], rank1 [14,16 | 14,16]; AR sums them.
    assert res[0][0] == res[1][0] == [24.0, 28.0, 24.0, 28.0]
    assert res[0][1] == [3.0, 3.0]


# -- a rank that dies on the host: the survivor gets an error, not a hang --------------------

def _failing_worker(rank, world):
    import datetime
    from pccl_b200.ocs import OCSPlan, OCSRuntime
    group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=3))
    if rank == 1:
        return "left before the barrier"                # never sends READY
    try:
        OCSRuntime().barrier_switch(OCSPlan(participant_ranks=(0, 1)), group=group)
    except Exception as err:
        return "error:" + type(err).__name__
    return "released"


def test_missing_rank_ends_the_barrier_with_an_error():
    res = _run(_failing_worker, 2)
    assert res[1] == "left before the barrier" and res[0].startswith("error:")
