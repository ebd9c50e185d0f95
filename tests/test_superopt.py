"""Cost model, e-graph, rule model/cache, enumerator, verifier, the pass, selector."""

import pytest
import torch

from pccl_b200.dsl import nodes as N
from pccl_b200.dsl.algorithms import (NvlsAllreduce, OneShotAllreduce, RecursiveHalvingDoubling,
                                      RingAllreduce, TwoShotAllreduce, select_algorithm,
                                      select_algorithm_cost_based)
from pccl_b200.dsl.compiler import Compiler
from pccl_b200.dsl.decorators import CommunicationOp
from pccl_b200.dsl.nodes import PrimitiveOpType as Op
from pccl_b200.dsl.passes.channelize import ChannelizePass
from pccl_b200.dsl.superopt import discover_rules, load_rules
from pccl_b200.dsl.superopt.cost_model import (B200_PROFILE, H100_PROFILE, NVLINK5_TOPOLOGY,
                                               NVLINK_TOPOLOGY, GpuProfile, TopologyProfile,
                                               cost_delta, critical_path_cost, op_latency,
                                               profile_by_name)
from pccl_b200.dsl.superopt.egraph import EGraph, ENode, PatternExpr
from pccl_b200.dsl.superopt.egraph_bridge import egraph_to_ir, ir_to_egraph
from pccl_b200.dsl.superopt.enumerator import LinkType, _bell_partitions, enumerate_skeletons
from pccl_b200.dsl.superopt.pass_ import SuperoptPass
from pccl_b200.dsl.superopt.rule import (ApplicabilityPredicate, PatternEdge, PatternNode,
                                         RewriteRule)
from pccl_b200.dsl.superopt.rule_db import clear_rules, save_rules
from pccl_b200.dsl.superopt.verifier import check_equivalence, signatures_compatible


def P(op, chunk=0, ch=0):
    return PatternNode(op_type=op, rank=0, chunk_id=chunk, channel=ch)


def test_reference_profiles_are_preserved_and_b200_added():
    assert NVLINK_TOPOLOGY.bandwidth_gb_s == 450.0 and H100_PROFILE.bandwidth_gb_s["tma"] == 60.0
    assert NVLINK5_TOPOLOGY.bandwidth_gb_s == 900.0 and NVLINK5_TOPOLOGY.in_switch_reduction
    assert B200_PROFILE.num_channels == 32
    assert profile_by_name("B200") is B200_PROFILE and profile_by_name("h100") is H100_PROFILE
    assert TopologyProfile.from_dict(NVLINK5_TOPOLOGY.to_dict()) == NVLINK5_TOPOLOGY
    assert GpuProfile.from_dict(B200_PROFILE.to_dict()) == B200_PROFILE


def test_latency_model():
    assert op_latency(Op.NOTIFY, H100_PROFILE, 1 << 20) == 1.0
    assert op_latency(Op.SM_COPY, H100_PROFILE, 50_000) == pytest.approx(2.0)
    assert op_latency(Op.TMA_COPY, H100_PROFILE, 1 << 20) < op_latency(Op.SM_COPY, H100_PROFILE, 1 << 20)
    # reduce is the slower of transfer and arithmetic
    assert op_latency(Op.SM_REDUCE, H100_PROFILE, 120_000) == pytest.approx(1 + 120_000 / 50e3)
    chain = [P(Op.SM_COPY), P(Op.SM_COPY)]
    serial = critical_path_cost(chain, [PatternEdge(0, 1)], H100_PROFILE, 1 << 20)
    spread = critical_path_cost([P(Op.SM_COPY, ch=0), P(Op.SM_COPY, ch=1)], [], H100_PROFILE, 1 << 20)
    assert spread < serial
    assert cost_delta(chain, [PatternEdge(0, 1)], [P(Op.TMA_COPY), P(Op.TMA_COPY)],
                      [PatternEdge(0, 1)], H100_PROFILE, 1 << 20) > 0
    assert critical_path_cost([], [], H100_PROFILE) == 0.0


def test_egraph_hashcons_merge_congruence_extract():
    eg = EGraph()
    x = eg.add(ENode("noop", 0))
    a = eg.add(ENode("sm.copy", 0, (x,), (("size", 8),)))
    assert eg.add(ENode("sm.copy", 0, (x,), (("size", 8),))) == a
    b = eg.add(ENode("tma.copy", 0, (x,), (("size", 8),)))
    pa, pb = eg.add(ENode("notify", 0, (a,))), eg.add(ENode("notify", 0, (b,)))
    assert eg.find(pa) != eg.find(pb)
    eg.merge(a, b); eg.rebuild()
    assert eg.find(pa) == eg.find(pb), "congruence closure"
    cost, best = eg.extract(a, lambda n, kids: {"sm.copy": 5, "tma.copy": 3}.get(n.op_type, 1)
                            + sum(kids.values()))
    assert best.op_type == "tma.copy" and cost == 4
    subs = eg.ematch(PatternExpr(op_category="copy", children=[PatternExpr(var="x")]))
    assert subs and all(s["x"] == eg.find(x) for s in subs)


def test_bridge_round_trip_keeps_structure():
    g = RingAllreduce().build_allreduce(0, 4, 4096, "float32", "sm")
    g.validate()
    eg, ids, roots = ir_to_egraph(g)
    assert len(ids) == g.size() and roots
    back = egraph_to_ir(eg, roots, lambda n, kids: 1 + max(kids.values(), default=0), g)
    assert [n.op_type for n in back.topological_sort()] == [n.op_type for n in g.topological_sort()]
    assert [n.to_params() for n in back.topological_sort()] == [n.to_params() for n in g.topological_sort()]


def test_pass_upgrades_executors_and_removes_duplicates():
    with CommunicationOp("dup") as op:
        op.tensor("float32", (64,))
        op.sm_copy(1, 0, 0, 32)
        op.sm_copy(1, 0, 0, 32)          # identical re-application
        op.notify(0, 1)
    g = op.get_graph()
    SuperoptPass(rules=[]).run(g)
    kinds = [n.op_type for n in g.topological_sort()]
    assert kinds == [Op.TMA_COPY, Op.NOTIFY]


def test_rule_model_cache_and_discovery(isolated_rule_cache):
    pred = ApplicabilityPredicate("size", ">=", 4096)
    assert pred.evaluate({"size": 4096}) and not pred.evaluate({"size": 1}) and pred.evaluate({})
    with pytest.raises(ValueError):
        ApplicabilityPredicate("size", "~", 1).evaluate({"size": 1})
    rule = RewriteRule([P(Op.SM_COPY)], [], [P(Op.TMA_COPY)], [], predicates=[pred], rule_id="r")
    assert RewriteRule.from_dict(rule.to_dict()) == rule
    save_rules(1, [rule])
    assert load_rules(1) == [rule]
    clear_rules(1)
    assert load_rules(1) == []

    rules = discover_rules(2, progress=False)
    assert any(r.rule_id.startswith("executor_upgrade_") for r in rules)
    shrinking = [r for r in rules if r.replacement_size() < r.source_size()]
    assert shrinking, "copy;copy on one chunk collapses to a single copy"
    assert load_rules(2) and (isolated_rule_cache / "rules_k2.json").exists()


def test_enumerator_counts_and_multichannel():
    assert [len(_bell_partitions(k)) for k in range(5)] == [1, 1, 2, 5, 15]
    one = list(enumerate_skeletons(1))
    assert len(one) == 5 and all(not e for _, e in one)
    assert len(list(enumerate_skeletons(1, LinkType.INTER))) == 2
    k2 = list(enumerate_skeletons(2))
    k2_mc = list(enumerate_skeletons(2, max_channels=2))
    assert len(k2_mc) > len(k2)
    assert any(len({n.channel for n in nodes}) == 2 for nodes, _ in k2_mc)


def test_verifier_accepts_equivalent_and_rejects_different():
    two = [P(Op.SM_COPY), P(Op.SM_COPY)]
    assert check_equivalence(two, [PatternEdge(0, 1)], [P(Op.SM_COPY)], []) is not None
    assert check_equivalence(two, [PatternEdge(0, 1)], two, [PatternEdge(0, 1)]) is None
    assert check_equivalence([P(Op.SM_REDUCE)], [], [P(Op.SM_COPY)], []) is None
    assert not signatures_compatible([P(Op.SM_REDUCE)], [P(Op.SM_COPY)])
    # copy chunk0 ; copy chunk1 commute
    ab = [P(Op.SM_COPY, 0), P(Op.CE_COPY, 1)]
    ba = [P(Op.CE_COPY, 1), P(Op.SM_COPY, 0)]
    assert check_equivalence(ab, [PatternEdge(0, 1)], ba, [PatternEdge(0, 1)]) is not None


def test_z3_semantics_copy_and_reduce():
    z3 = pytest.importorskip("z3")
    from pccl_b200.dsl.superopt.semantics import encode_op, get_reduce_axioms, make_initial_state
    s0 = make_initial_state()
    off = z3.BitVecVal(4, 32)
    s1 = encode_op(Op.SM_COPY, 0, {"source_rank": 1, "src_offset": off, "dst_offset": off, "size": 1}, s0)
    solver = z3.Solver()
    solver.add(z3.Select(s1.bufs[0], off) != z3.Select(s0.bufs[1], off))
    assert solver.check() == z3.unsat
    assert len(get_reduce_axioms("sum")) == 2 and get_reduce_axioms("avg") == []


def test_channelize_only_when_it_pays():
    def chain(count, size):
        with CommunicationOp("c") as op:
            op.tensor("float32", (count * size,))
            for i in range(count):
                op.sm_copy(1, i * size, i * size, size)
        return op.get_graph()
    g = chain(8, 1 << 20)
    ChannelizePass(num_channels=2).run(g)
    assert [n.channel for n in g.topological_sort()] == [0] * 4 + [1] * 4
    tiny = chain(8, 16)
    ChannelizePass(num_channels=2).run(tiny)
    assert {n.channel for n in tiny.nodes.values()} == {0}
    g32 = chain(64, 1 << 20)
    Compiler(enable_channelize=True, num_channels=32, gpu_profile="b200").compile(g32)
    assert max(n.channel for n in g32.nodes.values()) == 31


def test_selector_reference_rule_and_switched_fabric(monkeypatch, tmp_path):
    """The built-in rules (what applies when no measured table covers the world size)."""
    from pccl_b200.dsl.algorithms import selector
    monkeypatch.delenv("PCCL_ALGO", raising=False)
    monkeypatch.setenv("PCCL_TUNING_FILE", str(tmp_path / "no_table.json"))
    selector.clear_tuning_cache()
    assert isinstance(select_algorithm(2, 1 << 10), RingAllreduce)
    assert isinstance(select_algorithm(6, 1 << 10), RingAllreduce)
    assert isinstance(select_algorithm(8, 1 << 20), RingAllreduce)
    assert isinstance(select_algorithm(8, (1 << 20) - 1), RecursiveHalvingDoubling)
    kw = dict(topology=NVLINK5_TOPOLOGY, device=B200_PROFILE)
    assert isinstance(select_algorithm(8, 8 << 10, **kw), OneShotAllreduce)
    assert isinstance(select_algorithm(8, 1 << 20, **kw), TwoShotAllreduce)
    assert isinstance(select_algorithm(8, 512 << 20, **kw), NvlsAllreduce)
    no_nvls = TopologyProfile("nvlink5", 900.0, 0.7, uniform_all_to_all=True)
    assert isinstance(select_algorithm(8, 512 << 20, topology=no_nvls), TwoShotAllreduce)
    monkeypatch.setenv("PCCL_ALGO", "tree")
    assert select_algorithm(8, 1 << 30).name == "tree"
    selector.clear_tuning_cache()


def test_cost_based_selector_prefers_few_steps_for_small_and_bandwidth_for_large(monkeypatch):
    monkeypatch.delenv("PCCL_ALGO", raising=False)
    small = select_algorithm_cost_based(0, 8, 8 * 128, 8 * 128 * 4, NVLINK5_TOPOLOGY, B200_PROFILE,
                                        "float32", "sm")
    large = select_algorithm_cost_based(0, 8, 1 << 27, 1 << 29, NVLINK5_TOPOLOGY, B200_PROFILE,
                                        "float32", "sm")
    assert small.name == "oneshot"
    assert large.name in ("nvls", "twoshot") and large.bandwidth_optimal
    assert select_algorithm_cost_based(0, 6, 600, 2400).name == "ring"


# ---- structural rewrites for a switched fabric --------------------------------------------------

def _compile_with(graph, topology, size_hint=0):
    from pccl_b200 import Compiler
    return Compiler(enable_superopt=True, gpu_profile="b200", topology=topology,
                    data_size_hint=size_hint).compile_to_dict(graph)


def test_chain_of_reduces_becomes_one_multi_source_reduce():
    from pccl_b200.dsl.decorators import build_graph
    from pccl_b200.runtime import simulate
    world, n = 4, 256

    def plans(topology):
        out = []
        for rank in range(world):
            def build(op, rank=rank):
                from pccl_b200.dsl.algorithms.base import all_pairs_barrier
                op.tensor("float32", (n,))
                piece = n // world
                mine = rank * piece
                all_pairs_barrier(op, rank, world, 200)
                for i in range(1, world):
                    op.sm_reduce(source_rank=(rank + i) % world, src_offset=mine, dst_offset=mine,
                                 remote_offset=mine, count=piece)
                all_pairs_barrier(op, rank, world, 300)
            graph = build_graph(f"chain{rank}", build)
            graph.collective_type = "reduce_scatter"
            out.append(_compile_with(graph, topology))
        return out

    switched = TopologyProfile("nvlink5", 900.0, 0.7, uniform_all_to_all=True)
    fused = plans(switched)
    kinds = [op["primitive"] for op in fused[0]["operations"] if "reduce" in op["primitive"]]
    assert kinds == ["sm.reduce_multi"]
    assert sorted(next(op for op in fused[0]["operations"] if op["primitive"] == "sm.reduce_multi")
                  ["params"]["source_ranks"]) == [0, 1, 2, 3]
    xs = [torch.randn(n, generator=torch.Generator().manual_seed(r)) for r in range(world)]
    total = sum(x.double() for x in xs)
    for r, out in enumerate(simulate(fused, xs)):
        torch.testing.assert_close(out.double(), total[r * n // world:(r + 1) * n // world], atol=1e-5, rtol=1e-5)
    # A point-to-point fabric keeps the chain.
    kept = plans(NVLINK_TOPOLOGY)
    assert sum("reduce" in op["primitive"] for op in kept[0]["operations"]) == world - 1


@pytest.mark.parametrize("world", [4, 8])
def test_two_shot_becomes_in_switch_allreduce_when_the_fabric_reduces(world):
    from pccl_b200.dsl.algorithms import TwoShotAllreduce
    from pccl_b200.runtime import simulate
    n = world * 64 * 1024
    plans = [_compile_with(TwoShotAllreduce().build_allreduce(r, world, n, "float32", "sm", 2), NVLINK5_TOPOLOGY)
             for r in range(world)]
    kinds = {op["primitive"] for op in plans[0]["operations"]}
    assert "multimem.allreduce" in kinds and not kinds & {"sm.reduce_multi", "sm.copy", "tma.copy", "ce.copy"}
    # one barrier fewer per channel than the two-shot plan it came from
    before = TwoShotAllreduce().build_allreduce(0, world, n, "float32", "sm", 2)
    assert sum(op["primitive"] == "notify" for op in plans[0]["operations"]) == \
        sum(1 for node in before.nodes.values() if node.op_type.value == "notify") - 2 * (world - 1)
    xs = [torch.randn(n, generator=torch.Generator().manual_seed(r)) for r in range(world)]
    outs, sim = simulate(plans, xs, return_world=True)
    for out in outs:
        torch.testing.assert_close(out.double(), sum(x.double() for x in xs), atol=1e-4, rtol=1e-5)
    assert sim.leftover_signals() == {}


def test_two_shot_stays_on_peer_loads_where_the_switch_does_not_pay():
    from pccl_b200.dsl.algorithms import TwoShotAllreduce
    no_nvls = TopologyProfile("nvlink5", 900.0, 0.7, uniform_all_to_all=True)
    n = 8 * 64 * 1024
    kinds = {op["primitive"] for op in _compile_with(TwoShotAllreduce().build_allreduce(0, 8, n, "float32", "sm", 1),
                                                     no_nvls)["operations"]}
    assert "sm.reduce_multi" in kinds and not any(k.startswith("multimem") for k in kinds)
    # Two ranks: the in-switch path moves 1.5x the bytes of two-shot, so the price goes up and it is not taken.
    n = 2 * 1024 * 1024
    kinds = {op["primitive"] for op in _compile_with(TwoShotAllreduce().build_allreduce(0, 2, n, "float32", "sm", 1),
                                                     NVLINK5_TOPOLOGY)["operations"]}
    assert not any(k.startswith("multimem") for k in kinds)
    # fp8 has no in-switch arithmetic: the reduction stays on the SMs (the broadcast half may still move).
    kinds = {op["primitive"] for op in _compile_with(TwoShotAllreduce().build_allreduce(0, 8, n, "float8_e4m3", "sm", 1),
                                                     NVLINK5_TOPOLOGY)["operations"]}
    assert "sm.reduce_multi" in kinds and not kinds & {"multimem.reduce", "multimem.allreduce"}
