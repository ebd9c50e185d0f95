"""The plan-interpreter kernel on a real GPU: every template, dtype and odd size,
run as N virtual ranks in one cooperative launch and compared with a float64
host reference; bounded-wait failure path; reference-emitted plans."""

import copy
import gzip
import json
import os

import pytest
import torch

from gpu_helpers import TOL, check_collective, new_cluster, run_on_cluster
from helpers import build_plans, expected, make_inputs
from pccl_b200.dsl.algorithms import (ALGORITHMS, NvlsAllreduce, OneShotAllreduce, RingAllreduce,
                                      TwoShotAllreduce)

pytestmark = pytest.mark.gpu

KINDS = ("allreduce", "reduce_scatter", "allgather", "alltoall")


def _supported():
    for name, cls in ALGORITHMS.items():
        for kind in KINDS:
            try:
                getattr(cls(), "build_" + kind)(0, 2, 64, "float32", "sm")
            except NotImplementedError:
                continue
            yield name, kind


@pytest.fixture(scope="module")
def clusters():
    made = {}

    def get(world):
        if world not in made:
            made[world] = new_cluster(world)
        return made[world]
    yield get
    made.clear()


@pytest.mark.parametrize("name,kind", list(_supported()))
@pytest.mark.parametrize("world", [2, 4, 8])
def test_templates_fp32(clusters, name, kind, world):
    # 4 KiB per rank: vector path, aligned.
    check_collective(clusters(world), ALGORITHMS[name](), kind, world, 1024 * world, repeats=2)


@pytest.mark.parametrize("name", ["ring", "twoshot", "oneshot", "nvls", "rhd"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_allreduce_16bit_accumulates_in_fp32(clusters, name, dtype):
    check_collective(clusters(8), ALGORITHMS[name](), "allreduce", 8, 8 * 4096, dtype)


@pytest.mark.parametrize("per_rank", [1, 3, 17, 1001, 4097])
@pytest.mark.parametrize("name", ["ring", "twoshot"])
def test_odd_sizes_keep_every_element(clusters, name, per_rank):
    # Chunks that are not multiples of 16 bytes and offsets that are misaligned.
    for dtype in (torch.float32, torch.bfloat16):
        check_collective(clusters(4), ALGORITHMS[name](), "allreduce", 4, 4 * per_rank, dtype)


def test_large_message_multi_cta(clusters):
    check_collective(clusters(2), TwoShotAllreduce(), "allreduce", 2, 4 << 20, channels=4)
    check_collective(clusters(2), RingAllreduce(), "allreduce", 2, 4 << 20, channels=2)
    check_collective(clusters(4), OneShotAllreduce(), "allreduce", 4, 1 << 18)


@pytest.mark.parametrize("channels", [2, 8, 32])
def test_multichannel(clusters, channels):
    check_collective(clusters(4), RingAllreduce(), "allreduce", 4, 4 * 32 * 64, channels=channels)
    check_collective(clusters(4), TwoShotAllreduce(), "allreduce", 4, 4 * 32 * 64, channels=channels)


@pytest.mark.parametrize("op", ["max", "min", "avg"])
def test_reduce_ops(clusters, op):
    world, n = 4, 4 * 1000
    for dtype in (torch.float32, torch.bfloat16):
        name = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
        plans = build_plans(TwoShotAllreduce(), "allreduce", world, n, name)
        for plan in plans:
            for o in plan["operations"]:
                if "reduce_op" in o["params"]:
                    o["params"]["reduce_op"] = op
        xs = make_inputs("allreduce", world, n, dtype)
        xd = torch.stack([x.double() for x in xs])
        ref = {"max": xd.max(0).values, "min": xd.min(0).values, "avg": xd.mean(0)}[op]
        for out in run_on_cluster(clusters(world), f"redop_{op}_{name}", plans, xs, n):
            torch.testing.assert_close(out.double(), ref, **TOL[dtype])


def test_fp8_copy_and_reduce(clusters):
    if not hasattr(torch, "float8_e4m3fn"):
        pytest.skip("no fp8 dtypes in this torch")
    world, n = 2, 2 * 4096
    plans = build_plans(TwoShotAllreduce(), "allreduce", world, n, "float8_e4m3")
    xs = [(torch.randn(n, generator=torch.Generator().manual_seed(r)) * 0.5).to(torch.float8_e4m3fn)
          for r in range(world)]
    raw = [x.view(torch.uint8) for x in xs]
    cluster = clusters(world)
    cluster.regOp("fp8_ar", [json.dumps(p) for p in plans])
    outs = [torch.zeros(n, dtype=torch.uint8, device="cuda") for _ in range(world)]
    cluster.exeOp("fp8_ar", [r.cuda() for r in raw], outs)
    got = outs[0].cpu().view(torch.float8_e4m3fn).float()
    ref = (xs[0].float() + xs[1].float()).to(torch.float8_e4m3fn).float()
    torch.testing.assert_close(got, ref, atol=0.0, rtol=0.0)


def _golden():
    path = os.path.join(os.path.dirname(__file__), "golden", "reference_plans.json.gz")
    with gzip.open(path, "rt") as handle:
        return json.load(handle)


@pytest.mark.parametrize("tag", sorted(_golden()))
def test_reference_emitted_plans_run_unchanged(clusters, tag):
    plans = _golden()[tag]
    kind, world = plans[0]["collective_type"], len(plans)
    n = plans[0]["tensor_info"]["shape"][0]
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[plans[0]["tensor_info"]["dtype"]]
    xs = make_inputs(kind, world, n, dtype)
    out_numel = n // world if kind == "reduce_scatter" else n
    outs = run_on_cluster(clusters(world), "golden_" + tag, plans, xs, out_numel)
    for out, ref in zip(outs, expected(kind, xs, world, n)):
        torch.testing.assert_close(out.double(), ref, **TOL[dtype])


def test_lost_notify_times_out_with_status_and_engine_recovers():
    """A wait that nothing satisfies must end with an error status, not a hang."""
    from pccl_b200 import engine_c
    cluster = new_cluster(2, timeout_ms=300)
    plans = build_plans(RingAllreduce(), "allreduce", 2, 2048)
    broken = copy.deepcopy(plans)
    victim = next(o for o in broken[1]["operations"] if o["primitive"] == "notify")
    victim["primitive"] = "noop"
    victim["params"] = {}
    xs = make_inputs("allreduce", 2, 2048)
    # Registration sees all ranks' plans and refuses this set before anything is launched ...
    with pytest.raises(engine_c.PCCLError, match="would deadlock"):
        run_on_cluster(cluster, "broken", broken, xs, 2048)
    # ... so the device-side wait limit is reached with that check switched off.
    cluster.setProtocolCheck(False)
    with pytest.raises(engine_c.PCCLTimeoutError, match="timed out waiting for a signal"):
        run_on_cluster(cluster, "broken", broken, xs, 2048)
    cluster.setProtocolCheck(True)
    status = cluster.lastStatus()
    assert any(s["code"] == 1 for s in status)
    cluster.reset()
    outs = run_on_cluster(cluster, "healthy", plans, xs, 2048)
    torch.testing.assert_close(outs[0].double(), xs[0].double() + xs[1].double(), atol=1e-5, rtol=1e-5)


def test_device_timeline_of_a_launch():
    """Tracing on: every step of the last launch carries four ordered %globaltimer stamps."""
    from pccl_b200 import engine_c
    from pccl_b200.utils.trace import phases, summarize
    world, n = 2, 1 << 20
    cluster = engine_c.LocalCluster(world, 0, 32 << 20)
    cluster.setTrace(True)
    plans = build_plans(TwoShotAllreduce(), "allreduce", world, n, channels=2)
    xs = make_inputs("allreduce", world, n)
    outs = run_on_cluster(cluster, "traced", plans, xs, n)
    torch.testing.assert_close(outs[0].double(), xs[0].double() + xs[1].double(), atol=1e-5, rtol=1e-5)
    trace = cluster.trace("traced", 0)
    assert len(trace) == cluster.opInfo("traced", 0)["steps"]
    for step in trace:
        assert step["t_reached_ns"] <= step["t_data_ns"] <= step["t_done_ns"] <= step["t_posted_ns"]
    rows = {r["kind"]: r for r in phases(trace, world)}
    assert rows["reduce_multi"]["bytes"] == n * 4 // world and rows["reduce_multi"]["span_us"] > 0
    assert "copy" in rows and "launch span" in summarize(trace, world)


def test_single_rank_engine_round_trip(tmp_path):
    """The process-level Engine (world 1): register from a file, run, zero-copy view."""
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("PCCL_BUFFER_SIZE", str(64 << 20))
    os.environ.setdefault("PCCL_ARENA_SIZE", str(64 << 20))
    import pccl_b200 as pccl
    from pccl_b200 import Compiler
    engine = pccl.get_engine()
    n = 4096
    path = tmp_path / "ar.json"
    # (A one-rank ring would wait for a post nobody sends; the switch-native templates degrade cleanly.)
    Compiler().compile_to_json(TwoShotAllreduce().build_allreduce(0, 1, n, "float32", "sm"), str(path))
    assert pccl.register_operation("ar_w1", str(path))
    x = torch.randn(n, device="cuda")
    y = pccl.execute_operation("ar_w1", x)
    torch.testing.assert_close(y, x)
    w = engine.working_buffer(n, torch.float32)
    w.copy_(x)
    pccl.execute_operation("ar_w1", w, w)
    torch.testing.assert_close(w, x)
    assert not pccl.register_operation("bad", str(tmp_path / "missing.json"))
    assert engine.stats()["ar_w1"]["calls"] == 2
