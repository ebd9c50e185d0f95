"""The superoptimization pass.

1. *Direct executor upgrades*: ``sm.copy -> tma.copy`` and
   ``sm.reduce -> tma.reduce`` in place (plan-compatible with the reference,
   whose engine prefers its TMA path; this library's engine runs both names on
   the same SM peer-load kernels, so the upgrade is free).
2. *Equality saturation*: IR -> e-graph, add executor alternatives, saturate
   with structural + cached SMT rules, extract the cheapest DAG under the
   device/topology cost model, and replace the graph's nodes
   (reference: pccl/dsl/superopt/pass_.py:52-159).
3. *Fabric rules* (switched fabrics only): runs of nodes are rewritten to multi-source
   reduces and to in-switch (multimem) reduction / broadcast where the cost model says the
   whole plan gets cheaper (`fabric_rules.py`).
"""

from __future__ import annotations

from functools import partial
from typing import List, Optional

from ..graph import PrimitiveIRGraph
from ..nodes import IRNodeVariant, PrimitiveOpType, node_from_params
from .cost_model import (GpuProfile, H100_PROFILE, NVLINK_TOPOLOGY, TopologyProfile,
                         egraph_node_cost)
from .domain_rules import add_executor_equivalences, smt_rules_to_egraph, structural_rules
from .egraph_bridge import egraph_to_ir, ir_to_egraph
from .enumerator import EXECUTOR_UPGRADES
from .rule import RewriteRule
from .rule_db import load_all_rules


class SuperoptPass:
    def __init__(self, device_profile: GpuProfile = H100_PROFILE,
                 topology: TopologyProfile = NVLINK_TOPOLOGY,
                 rules: Optional[List[RewriteRule]] = None, data_size_hint: int = 0,
                 max_k: int = 6, gpu_profile_name: str = "h100"):
        self.profile = device_profile
        self.topology = topology
        self.data_size_hint = data_size_hint
        self.rules = rules if rules is not None else load_all_rules(max_k=max_k)

    def run(self, graph: PrimitiveIRGraph) -> PrimitiveIRGraph:
        if graph.has_ocs_barriers():
            raise ValueError(
                "Superoptimization across OCS barriers is unsupported; "
                "split the graph into OCS phases first")
        self._apply_executor_upgrades(graph)
        self._apply_egraph_optimization(graph)
        self._apply_fabric_rules(graph)
        return graph

    # -- phase 1 ---------------------------------------------------------------
    def _apply_executor_upgrades(self, graph: PrimitiveIRGraph) -> bool:
        changed = False
        for nid, node in list(graph.nodes.items()):
            target = EXECUTOR_UPGRADES.get(node.op_type)
            if target is None:
                continue
            graph.nodes[nid] = self._clone_node_with_type(node, target)
            changed = True
        return changed

    @staticmethod
    def _clone_node_with_type(node: IRNodeVariant,
                              new_op_type: PrimitiveOpType) -> Optional[IRNodeVariant]:
        twin = node_from_params(new_op_type, node.to_params(), op_id=node.op_id,
                                device=node.device)
        twin.dependencies = list(node.dependencies)
        twin.next_ops = list(node.next_ops)
        twin.channel = node.channel
        twin.tensor_info = node.tensor_info
        return twin

    # -- phase 3 ---------------------------------------------------------------
    def _apply_fabric_rules(self, graph: PrimitiveIRGraph) -> bool:
        """Structural retargeting to a switched fabric (multi-source reduces, in-switch reduction
        and broadcast), each rewrite kept only if it lowers the plan's price."""
        from pccl_b200.dsl.superopt.fabric_rules import apply_fabric_rules
        self.fabric_rewrites = apply_fabric_rules(graph, self.profile, self.topology)
        return bool(self.fabric_rewrites)

    # -- phase 2 ---------------------------------------------------------------
    def _apply_egraph_optimization(self, graph: PrimitiveIRGraph) -> bool:
        if graph.size() < 2:
            return False
        if not graph.exit_points:
            graph._update_boundary_points()
        eg, _, roots = ir_to_egraph(graph)
        if not roots:
            return False
        add_executor_equivalences(eg)
        rules = structural_rules(eg) + smt_rules_to_egraph(eg, self.rules)
        if rules:
            eg.saturate(rules, limit=20)
        cost_fn = partial(egraph_node_cost, device=self.profile, topology=self.topology)
        rebuilt = egraph_to_ir(eg, roots, cost_fn, original_graph=graph)
        if rebuilt.size() == 0:
            return False
        graph.nodes.clear()
        graph.nodes.update(rebuilt.nodes)
        graph._update_boundary_points()
        return True
