"""IR nodes, graph container, builder front-end, pipeline, codegen."""

import json

import pytest

from pccl_b200 import (CommunicationOp, Compiler, DeviceType, ExecutorType, Pipeline,
                       PrimitiveIRGraph, PrimitiveOpType, Stream, TensorInfo, build_graph,
                       compile_to_json_string)
from pccl_b200.dsl import nodes as N
from pccl_b200.dsl.codegen import RuntimeGraphGenerator, load_plan_graph


def test_node_identity_and_executor_inference():
    n = N.SmReduceNode(source_rank=1, count=8)
    assert n.op_type is PrimitiveOpType.SM_REDUCE and n.executor is ExecutorType.SM
    assert n.op_id.startswith("sm_reduce_") and len(n.op_id) == len("sm_reduce_") + 8
    assert N.TmaCopyNode(source_rank=0).executor is ExecutorType.TMA
    assert N.MultimemStoreNode(source_rank=0).executor is ExecutorType.MULTIMEM
    assert N.NotifyNode(target_rank=0).executor is ExecutorType.SM
    assert N.NotifyNode(target_rank=0, device=DeviceType.CPU).executor is ExecutorType.HOST
    assert N.OcsBarrierNode(participant_ranks=(0, 1)).device is DeviceType.CPU
    assert DeviceType.GPU is DeviceType.CUDA


def test_param_dictionaries_are_the_json_contract():
    assert list(N.SmReduceNode(source_rank=1).to_params()) == [
        "reduce_op", "source_rank", "src_offset", "dst_offset", "remote_offset", "count"]
    assert list(N.CeCopyNode(source_rank=1).to_params()) == [
        "source_rank", "src_offset", "dst_offset", "size"]
    assert list(N.RdmaWriteNode(target_rank=1).to_params()) == [
        "target_rank", "src_offset", "dst_offset", "size"]
    assert N.NotifyNode(signal_id=7, target_rank=2).to_params() == {"signal_id": 7, "target_rank": 2}
    assert N.SmReduceMultiNode(source_ranks=[0, 1], count=4).to_params()["source_ranks"] == [0, 1]


@pytest.mark.parametrize("make, message", [
    (lambda: N.SmReduceNode(source_rank=0, reduce_op="xor"), "invalid reduce_op"),
    (lambda: N.SmCopyNode(), "source_rank must be non-negative"),
    (lambda: N.SmPutNode(), "target_rank must be non-negative"),
    (lambda: N.TmaCopyNode(source_rank=0, size=-1), "size must be non-negative"),
    (lambda: N.OcsBarrierNode(participant_ranks=()), "participant_ranks"),
    (lambda: N.OcsBarrierNode(participant_ranks=(0,), epoch_id=3, next_epoch_id=3), "next_epoch_id"),
])
def test_validation_messages(make, message):
    with pytest.raises(ValueError, match=message):
        make().validate()


def test_tensor_info_rules():
    assert TensorInfo("bfloat16", (4, 8)).numel() == 32
    assert TensorInfo(dtype="float32", shape=(3,), device="cuda").nbytes() == 12
    with pytest.raises(ValueError, match="shape must be a tuple"):
        TensorInfo("float32", [4])
    with pytest.raises(ValueError, match="unsupported dtype"):
        TensorInfo("int8", (4,))


def test_graph_edges_cycles_and_order():
    g = PrimitiveIRGraph(graph_name="g")
    a, b, c = (g.add_node(N.NotifyNode(op_id=i, target_rank=0)) for i in "abc")
    g.add_edge("a", "b"); g.add_edge("b", "c"); g.add_edge("a", "b")
    assert b.dependencies == ["a"] and a.next_ops == ["b"]
    with pytest.raises(ValueError, match="cycle"):
        g.add_edge("c", "a")
    assert c.next_ops == [] and "c" not in a.dependencies      # rolled back
    with pytest.raises(ValueError, match="already exists"):
        g.add_node(N.NotifyNode(op_id="a", target_rank=0))
    assert [n.op_id for n in g.topological_sort()] == ["a", "b", "c"]
    g.remove_node("b")
    assert a.next_ops == [] and c.dependencies == []
    with pytest.raises(ValueError, match="empty"):
        PrimitiveIRGraph().validate()


def test_deep_chain_does_not_recurse():
    g = PrimitiveIRGraph()
    prev = None
    for i in range(5000):
        g.add_node(N.NotifyNode(op_id=f"n{i}", target_rank=0))
        if prev:
            g.nodes[f"n{i}"].add_dependency(prev); g.nodes[prev].add_next_op(f"n{i}")
        prev = f"n{i}"
    assert g.validate() and len(g.topological_sort()) == 5000


def test_streams_are_independent_chains_and_wait_joins_them():
    with CommunicationOp("op") as op:
        op.tensor("float32", (64,))
        with Stream("a"):
            a1 = op.sm_copy(1, 0, 0, 8)
            a2 = op.notify(0, 1)
        with Stream("b"):
            b1 = op.sm_copy(1, 8, 8, 8)
            op.wait("a")
            b2 = op.notify(1, 1)
        with Stream("a"):
            a3 = op.wait_notify(0, 1)
    assert a2.dependencies == [a1.op_id] and b1.dependencies == []
    assert set(b2.dependencies) == {b1.op_id, a2.op_id}
    assert a3.dependencies == [a2.op_id]
    assert op.get_graph().entry_points == [a1.op_id, b1.op_id]
    with pytest.raises(RuntimeError):
        Stream("x").__enter__()


def test_pipeline_rotates_channels():
    with CommunicationOp("p") as op:
        op.tensor("bfloat16", (64,))
        with Pipeline(depth=2).bind(op) as pipe:
            made = []
            for i in range(4):
                with pipe.stage():
                    made.append(op.tma_copy(1, i * 8, i * 8, 8))
    assert [n.channel for n in made] == [0, 1, 0, 1]
    assert made[2].dependencies == [made[0].op_id] and made[1].dependencies == []
    with pytest.raises(ValueError):
        Pipeline(depth=0)


def _two_phase_graph():
    def build(op):
        op.tensor("float32", (16,))
        op.sm_copy(1, 0, 0, 8)
        op.ocs_barrier(barrier_id=3, epoch_id=0, next_epoch_id=1, participant_ranks=(0, 1),
                       topology_id=5, route_plan_id=9, payload=b"\x01\x02")
        with Stream("late"):
            op.sm_copy(1, 8, 8, 8)
    return build_graph("two_phase", build)


def test_v2_document_shape_and_round_trip():
    def build(op):
        op.tensor("float32", (16,))
        op.notify(100, 1); op.wait_notify(100, 1)
        op.sm_reduce(1, 0, 0, 0, 16)
    g = build_graph("g", build)
    g.collective_type = "allreduce"
    doc = json.loads(compile_to_json_string(g))
    assert list(doc) == ["version", "tensor_info", "collective_type", "executors", "operations"]
    assert doc["operations"][0] == {"index": 0, "executor": "cuda_sm", "primitive": "notify",
                                    "channel": 0, "dependencies": [], "next_ops": [1],
                                    "params": {"signal_id": 100, "target_rank": 1}}
    again = RuntimeGraphGenerator().generate(load_plan_graph(doc))
    assert again == doc
    assert json.loads(compile_to_json_string(build_graph("g", build), Compiler(enable_superopt=True)))[
        "operations"][2]["primitive"] == "tma.reduce"


def test_v3_manifest_for_barrier_graphs():
    doc = RuntimeGraphGenerator().generate(_two_phase_graph())
    assert doc["version"] == 3 and doc["execution_model"] == "phased_ocs"
    assert "operations" not in doc
    assert [len(p["operations"]) for p in doc["phases"]] == [1, 1]
    ctl = doc["control_operations"][0]
    assert ctl["primitive"] == "ocs.barrier" and ctl["executor"] == "host"
    assert (ctl["after_phase"], ctl["before_phase"]) == (0, 1)
    assert ctl["params"]["payload_hex"] == "0102" and ctl["params"]["participant_bitmap"] == 3
    with pytest.raises(ValueError, match="Superoptimization across OCS barriers"):
        Compiler(enable_superopt=True).compile(_two_phase_graph())


def test_barrier_must_cut_the_whole_graph():
    g = _two_phase_graph()
    stray = g.add_node(N.SmCopyNode(op_id="stray", source_rank=1, size=1))
    with pytest.raises(ValueError, match="must depend on every node"):
        g.validate()
    del stray


def test_trace_summary_reports_phase_rates():
    """The timeline reader: per-kind spans and per-direction link rates from raw stamps."""
    from pccl_b200.utils.trace import phases, summarize, waits
    mb = 1 << 20
    trace = [
        {"chain": 0, "step": 0, "kind": "noop", "ctas": 4, "bytes": 0,
         "t_reached_ns": 0, "t_data_ns": 2000, "t_done_ns": 2000, "t_posted_ns": 2500},
        {"chain": 0, "step": 1, "kind": "multimem.allreduce", "ctas": 4, "bytes": 8 * mb,
         "t_reached_ns": 2500, "t_data_ns": 3000, "t_done_ns": 103000, "t_posted_ns": 103500},
        {"chain": 1, "step": 0, "kind": "reduce_multi", "ctas": 4, "bytes": 4 * mb,
         "t_reached_ns": 0, "t_data_ns": 3000, "t_done_ns": 53000, "t_posted_ns": 53200},
    ]
    rows = {r["kind"]: r for r in phases(trace, world=8)}
    assert abs(rows["multimem.allreduce"]["span_us"] - 100.0) < 1e-6
    assert abs(rows["multimem.allreduce"]["tx_gbs"] - 8 * mb * 9 / 100000) < 1e-6      # (W + 1) slices per direction
    assert abs(rows["reduce_multi"]["rx_gbs"] - 4 * mb * 7 / 50000) < 1e-6
    w = waits(trace)
    assert w["chains"] == 2 and abs(w["total_us"] - 103.5) < 1e-6
    assert "multimem.allreduce" in summarize(trace, 8)


def test_selector_follows_a_tuning_file(tmp_path, monkeypatch):
    """`collective_sweep --write-tuning` output drives select_algorithm and the route lookup."""
    import importlib.util
    import json
    import os
    from pccl_b200.dsl.algorithms import selector
    from pccl_b200.dsl.superopt.cost_model import B200_PROFILE, NVLINK5_TOPOLOGY
    spec = importlib.util.spec_from_file_location(
        "collective_sweep", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench",
                                         "collective_sweep.py"))
    sweep = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sweep)
    rows = []
    for size, (ll, two, nvls) in {4096: (5, 9, 12), 1 << 20: (30, 25, 28), 1 << 24: (200, 150, 120),
                                  1 << 29: (3000, 1500, 1000)}.items():
        for algo, us in (("ll", ll), ("twoshot", two), ("nvls", nvls)):
            rows.append({"collective": "allreduce", "bytes": size, "algo": algo, "requested": algo,
                         "channels": 0 if algo == "ll" else 16, "us": us})
    path = tmp_path / "tuning.json"
    sweep.write_tuning(str(path), 8, rows)
    sweep.write_tuning(str(path), 4, [dict(r, us=r["us"] + (600 if r["algo"] == "nvls" else 0)) for r in rows])
    doc = json.loads(path.read_text())
    assert [e["algorithm"] for e in doc["routes"]["allreduce"]["8"]] == ["ll", "twoshot", "nvls"]
    assert doc["routes"]["allreduce"]["8"][-1]["max_bytes"] is None and "4" in doc["routes"]["allreduce"]
    # where a kernel wins, the best plan is named beside it (for callers the kernel does not take)
    assert doc["routes"]["allreduce"]["8"][0]["plan_algorithm"] == "twoshot"
    monkeypatch.setenv("PCCL_TUNING_FILE", str(path))
    monkeypatch.delenv("PCCL_ALGO", raising=False)
    selector.clear_tuning_cache()
    try:
        assert selector.tuned_route("allreduce", 8, 1000)["algorithm"] == "ll"
        assert selector.tuned_route("allreduce", 8, 1 << 30)["algorithm"] == "nvls"
        assert selector.tuned_route("allreduce", 2, 1 << 20) is None
        # every swept size: the selector's plan algorithm is the measured winner among the plan algorithms
        for size in (1 << 20, 1 << 24, 1 << 29):
            best = min((r for r in rows if r["bytes"] == size and r["algo"] != "ll"), key=lambda r: r["us"])["algo"]
            assert selector.select_algorithm(8, size, NVLINK5_TOPOLOGY, B200_PROFILE).name == best
        assert selector.select_algorithm(4, 1 << 29, NVLINK5_TOPOLOGY, B200_PROFILE).name == "twoshot"
    finally:
        selector.clear_tuning_cache()


def test_packaged_tuning_matches_the_saved_sweeps():
    """The table shipped with the package picks, at every swept size and world, a configuration whose
    measured time is within 5 % of the best one measured (bench/results/sweep_*gpu_*.json)."""
    import glob
    import json
    import os
    from pccl_b200.dsl.algorithms import selector
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    packaged = os.path.join(root, "pccl_b200", "dsl", "algorithms", "tuning_b200.json")
    files = sorted(glob.glob(os.path.join(root, "bench", "results", "sweep_*gpu_allreduce.json")) +
                   glob.glob(os.path.join(root, "bench", "results", "sweep_*gpu_shards.json")))
    assert files and os.path.exists(packaged)
    selector.clear_tuning_cache()
    checked = 0
    for path in files:
        saved = json.load(open(path))
        world = saved["world"]
        sizes = {}
        for row in saved["rows"]:
            if row.get("requested") != "auto":
                sizes.setdefault((row["collective"], row["bytes"]), []).append(row)
        for (kind, nbytes), rows in sizes.items():
            if len(rows) < 2:
                continue
            route = selector.tuned_route(kind, world, nbytes, path=packaged)
            assert route is not None, (kind, world, nbytes)
            mine = [r["us"] for r in rows if r["algo"] == route["algorithm"]
                    and (route.get("channels") is None or r["channels"] == route["channels"])]
            assert mine, (kind, world, nbytes, route)
            assert min(mine) <= 1.05 * min(r["us"] for r in rows), (kind, world, nbytes, route)
            checked += 1
    assert checked > 100
    selector.clear_tuning_cache()


def test_tuning_can_be_rebuilt_offline_from_saved_sweeps(tmp_path):
    """`collective_sweep.py --tuning-from` needs no GPU: it reproduces the packaged table from bench/results."""
    import glob
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = sorted(glob.glob(os.path.join(root, "bench", "results", "sweep_*gpu_allreduce.json")) +
                   glob.glob(os.path.join(root, "bench", "results", "sweep_*gpu_shards.json")))
    out = tmp_path / "tuning.json"
    subprocess.run([sys.executable, os.path.join(root, "bench", "collective_sweep.py"), "--tuning-from", *files,
                    "--write-tuning", str(out)], check=True, timeout=120)
    rebuilt = json.loads(out.read_text())["routes"]
    packaged = json.load(open(os.path.join(root, "pccl_b200", "dsl", "algorithms", "tuning_b200.json")))["routes"]
    assert rebuilt == packaged
    known = {"ll", "push", "nvls_kernel", "ring", "rhd", "tree", "oneshot", "twoshot", "nvls", "nvls_twopass", "hybrid"}
    for kind in ("allreduce", "allgather", "reduce_scatter"):
        assert {"2", "4", "8"} <= set(packaged[kind]), kind
        for table in packaged[kind].values():
            assert table[-1]["max_bytes"] is None
            assert all(e["algorithm"] in known and e.get("plan_algorithm", "ring") in known for e in table)
