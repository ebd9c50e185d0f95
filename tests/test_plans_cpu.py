"""Every algorithm template, replayed on the CPU executor against float64 sums;
reference-emitted golden plans; deadlock and bounds diagnostics."""

import copy
import gzip
import json
import os

import pytest
import torch

from helpers import build_plans, expected, make_inputs
from pccl_b200.dsl.algorithms import (ALGORITHMS, NvlsAllreduce, OneShotAllreduce,
                                      RecursiveHalvingDoubling, RingAllreduce, TreeAllreduce,
                                      TwoShotAllreduce)
from pccl_b200.runtime import PlanDeadlock, simulate

KINDS = ("allreduce", "reduce_scatter", "allgather", "alltoall")


def _supported():
    for name, cls in ALGORITHMS.items():
        for kind in KINDS:
            try:
                getattr(cls(), "build_" + kind)(0, 2, 64, "float32", "sm")
            except NotImplementedError:
                continue
            yield name, kind


@pytest.mark.parametrize("name,kind", list(_supported()))
@pytest.mark.parametrize("world", [2, 4, 8])
def test_template_matches_float64_reference(name, kind, world):
    n = 48 * world
    plans = build_plans(ALGORITHMS[name](), kind, world, n)
    xs = make_inputs(kind, world, n)
    outs, sim = simulate(plans, xs, return_world=True)
    for out, ref in zip(outs, expected(kind, xs, world, n)):
        torch.testing.assert_close(out.double(), ref, atol=1e-5, rtol=1e-5)
    assert sim.leftover_signals() == {}, "plans must be re-runnable without a signal reset"


@pytest.mark.parametrize("channels", [1, 2, 4, 8, 16, 32])
def test_multichannel_ring_and_twoshot(channels):
    world, n = 4, 4 * 32 * 8
    for algorithm in (RingAllreduce(), TwoShotAllreduce(), OneShotAllreduce(), NvlsAllreduce()):
        plans = build_plans(algorithm, "allreduce", world, n, channels=channels)
        assert max(op["channel"] for op in plans[0]["operations"]) == channels - 1
        xs = make_inputs("allreduce", world, n)
        for out in simulate(plans, xs):
            torch.testing.assert_close(out.double(), sum(x.double() for x in xs), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("kind", ["reduce_scatter", "allgather", "alltoall"])
@pytest.mark.parametrize("name", ["twoshot", "nvls"])
def test_multichannel_sharded_collectives_keep_contiguous_shards(name, kind):
    world, n, channels = 4, 4 * 8 * 16, 8
    if name == "nvls" and kind == "alltoall":
        pytest.skip("no in-switch all-to-all")
    plans = build_plans(ALGORITHMS[name](), kind, world, n, channels=channels)
    xs = make_inputs(kind, world, n)
    for out, ref in zip(simulate(plans, xs), expected(kind, xs, world, n)):
        torch.testing.assert_close(out.double(), ref, atol=1e-5, rtol=1e-5)


def test_bf16_accumulates_in_fp32():
    world, n = 8, 64 * 8
    plans = build_plans(TwoShotAllreduce(), "allreduce", world, n, dtype="bfloat16")
    xs = make_inputs("allreduce", world, n, torch.bfloat16)
    ref = sum(x.double() for x in xs)
    for out in simulate(plans, xs):
        assert out.dtype == torch.bfloat16
        torch.testing.assert_close(out.double(), ref, atol=0.05, rtol=2 ** -7)


@pytest.mark.parametrize("op,fold", [("max", torch.maximum), ("min", torch.minimum)])
def test_max_min_reduce_ops(op, fold):
    world, n = 4, 64
    plans = build_plans(RingAllreduce(), "allreduce", world, n)
    for plan in plans:
        for o in plan["operations"]:
            if "reduce_op" in o["params"]:
                o["params"]["reduce_op"] = op
    xs = make_inputs("allreduce", world, n)
    ref = xs[0]
    for x in xs[1:]:
        ref = fold(ref, x)
    for out in simulate(plans, xs):
        torch.testing.assert_close(out, ref)


def test_avg_is_sum_scaled_once():
    world, n = 4, 64
    plans = build_plans(TwoShotAllreduce(), "allreduce", world, n)
    for plan in plans:
        for o in plan["operations"]:
            if "reduce_op" in o["params"]:
                o["params"]["reduce_op"] = "avg"
    xs = make_inputs("allreduce", world, n)
    for out in simulate(plans, xs):
        torch.testing.assert_close(out.double(), sum(x.double() for x in xs) / world,
                                   atol=1e-6, rtol=1e-6)


def _golden():
    path = os.path.join(os.path.dirname(__file__), "golden", "reference_plans.json.gz")
    with gzip.open(path, "rt") as handle:
        return json.load(handle)


@pytest.mark.parametrize("tag", sorted(_golden()))
def test_reference_emitted_plans_replay_unchanged(tag):
    plans = _golden()[tag]
    kind, world = plans[0]["collective_type"], len(plans)
    n = plans[0]["tensor_info"]["shape"][0]
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[plans[0]["tensor_info"]["dtype"]]
    xs = make_inputs(kind, world, n, dtype)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype is torch.float32 else dict(atol=0.1, rtol=2 ** -6)
    for out, ref in zip(simulate(plans, xs), expected(kind, xs, world, n)):
        torch.testing.assert_close(out.double(), ref, **tol)


def test_our_templates_emit_the_reference_primitive_sequences():
    """Plan compatibility in the other direction: same ops, same params."""
    golden = _golden()
    cases = {
        "ring_ar_w8_sm": (RingAllreduce(), "allreduce", 8, 8192, "bfloat16", "sm", 1),
        "ring_ar_w2_c2": (RingAllreduce(), "allreduce", 2, 4096, "float32", "tma", 2),
        "rhd_ar_w8": (RecursiveHalvingDoubling(), "allreduce", 8, 8192, "float32", "tma", 1),
        "tree_ar_w8": (TreeAllreduce(), "allreduce", 8, 1024, "float32", "sm", 1),
        "ring_rs_w4": (RingAllreduce(), "reduce_scatter", 4, 4096, "float32", "sm", 1),
        "ring_ag_w4": (RingAllreduce(), "allgather", 4, 4096, "float32", "sm", 1),
        "ring_a2a_w4": (RingAllreduce(), "alltoall", 4, 4096, "float32", "sm", 1),
    }
    for tag, (alg, kind, world, n, dtype, ex, ch) in cases.items():
        ours = build_plans(alg, kind, world, n, dtype, ex, ch)
        for mine, theirs in zip(ours, golden[tag]):
            mine = copy.deepcopy(mine)
            mine.pop("algorithm")                     # additive field of this library
            assert mine == theirs, tag


def test_missing_notify_is_reported_as_deadlock():
    plans = build_plans(RingAllreduce(), "allreduce", 2, 64)
    victim = next(i for i, o in enumerate(plans[1]["operations"]) if o["primitive"] == "notify")
    plans[1]["operations"][victim]["primitive"] = "noop"
    with pytest.raises(PlanDeadlock, match="wait_notify"):
        simulate(plans, make_inputs("allreduce", 2, 64))


def test_out_of_range_access_is_reported():
    plans = build_plans(RingAllreduce(), "allreduce", 2, 64)
    data = next(o for o in plans[0]["operations"] if "count" in o["params"])
    data["params"]["remote_offset"] = 10 ** 6
    with pytest.raises(IndexError, match="outside rank"):
        simulate(plans, make_inputs("allreduce", 2, 64))


def test_switched_fabric_selector_built_in_crossovers(tmp_path, monkeypatch):
    """Without a tuning file: two ranks never take the in-switch path (it moves 1.5x the bytes of
    two-shot there); from four ranks on it takes over once bandwidth matters."""
    from pccl_b200.dsl.algorithms import selector
    from pccl_b200.dsl.superopt import B200_PROFILE, NVLINK5_TOPOLOGY
    monkeypatch.setenv("PCCL_TUNING_FILE", str(tmp_path / "none.json"))
    monkeypatch.delenv("PCCL_ALGO", raising=False)
    selector.clear_tuning_cache()
    pick = lambda w, b: type(selector.select_algorithm(w, b, NVLINK5_TOPOLOGY, B200_PROFILE)).__name__
    try:
        assert pick(2, 64 << 10) == "OneShotAllreduce"
        assert pick(2, 512 << 20) == "TwoShotAllreduce"
        assert pick(4, 1 << 20) == "OneShotAllreduce"
        assert pick(4, 8 << 20) == "NvlsAllreduce"
        assert pick(4, 512 << 20) == "NvlsAllreduce"
        assert pick(8, 1 << 20) == "TwoShotAllreduce"
        assert pick(8, 512 << 20) == "NvlsAllreduce"
    finally:
        selector.clear_tuning_cache()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fraction", [0.0, 0.3, 0.7, 1.0])
def test_hybrid_allreduce_covers_ragged_sizes(world, fraction):
    """In-switch channels, two-shot channels and the rounding tail together reduce every element."""
    from pccl_b200.dsl.algorithms import HybridAllreduce
    n = 5 * world * 16 * 4 + 24          # not a multiple of channels * world * 16
    plans = build_plans(HybridAllreduce(fraction), "allreduce", world, n, channels=4)
    kinds = {op["primitive"] for op in plans[0]["operations"]}
    if 0.0 < fraction < 1.0:
        assert {"multimem.allreduce", "sm.reduce_multi", "sm.copy"} <= kinds
    xs = make_inputs("allreduce", world, n)
    outs, sim = simulate(plans, xs, return_world=True)
    for out in outs:
        torch.testing.assert_close(out.double(), sum(x.double() for x in xs), atol=1e-5, rtol=1e-5)
    assert sim.leftover_signals() == {}


def test_nvls_allreduce_is_one_pass_and_two_pass_variant_remains():
    from pccl_b200.dsl.algorithms import NvlsTwoPassAllreduce
    one = build_plans(NvlsAllreduce(), "allreduce", 4, 256)[0]
    two = build_plans(NvlsTwoPassAllreduce(), "allreduce", 4, 256)[0]
    assert [op["primitive"] for op in one["operations"] if "multimem" in op["primitive"]] == ["multimem.allreduce"]
    assert [op["primitive"] for op in two["operations"] if "multimem" in op["primitive"]] == \
        ["multimem.reduce", "multimem.store"]


def _native():
    try:
        from pccl_b200 import engine_c
        return engine_c
    except ImportError:
        pytest.skip("native extension not built")


def test_native_world_check_accepts_templates_and_names_a_lost_notify():
    """The engine's own abstract replay of all ranks' signal protocols (no GPU involved)."""
    native = _native()
    for name in ("ring", "twoshot", "nvls", "hybrid", "rhd", "tree", "oneshot"):
        plans = build_plans(ALGORITHMS[name](), "allreduce", 4, 4 * 64 * 4, channels=2)
        report = native.check_world([json.dumps(p) for p in plans])
        assert not report["deadlock"] and report["leftover_signals"] == 0, (name, report)
        assert report["notifies"] == report["waits"] > 0
    broken = copy.deepcopy(build_plans(RingAllreduce(), "allreduce", 2, 2048))
    victim = next(o for o in broken[1]["operations"] if o["primitive"] == "notify")
    victim["primitive"], victim["params"] = "noop", {}
    report = native.check_world([json.dumps(p) for p in broken])
    assert report["deadlock"] and "blocked at" in report["detail"] and "wait_notify" in report["detail"]
    extra = copy.deepcopy(build_plans(RingAllreduce(), "allreduce", 2, 2048))
    extra[0]["operations"].append({"index": len(extra[0]["operations"]), "executor": "cuda_sm", "primitive": "notify",
                                   "channel": 0, "dependencies": [], "next_ops": [],
                                   "params": {"signal_id": 7, "target_rank": 1}})
    report = native.check_world([json.dumps(p) for p in extra])
    assert not report["deadlock"] and report["leftover_signals"] == 1 and "signal 7" in report["detail"]
    odd = build_plans(RingAllreduce(), "allreduce", 2, 2 * 1001)
    assert native.check_world([json.dumps(p) for p in odd])["misaligned_ops"] > 0


def test_coresident_clamp():
    """Grids of kernels whose CTAs wait on one another never exceed what is resident at once."""
    native = _native()
    assert native.coresident_limit(1, 148) == 148 and native.coresident_limit(2, 148) == 296
    assert native.clamp_coresident(128, 1, 148) == 128
    assert native.clamp_coresident(400, 2, 148) == 296
    assert native.clamp_coresident(0, 1, 148) == 1
    assert native.clamp_coresident(64, 0, 148) == 0      # the kernel does not fit at all
