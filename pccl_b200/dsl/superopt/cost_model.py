"""Latency model used by the superoptimizer, the channelize pass and the selector.

The model answers one question: how long does a small DAG of primitives take
on a given device and fabric?  Each primitive costs a fixed issue overhead plus
``bytes / bandwidth`` (reductions: the slower of transfer and arithmetic); a
pattern costs its critical path, where primitives on one channel serialise and
each extra channel adds a small launch overhead (reference:
pccl/dsl/superopt/cost_model.py:20-239).

The H100 / NVLink 4 objects keep the reference's numbers so cached rules and
profiles remain comparable.  ``B200_PROFILE`` / ``NVLINK5_TOPOLOGY`` price a
B200 on an NVSwitch fabric: 900 GB/s nominal (770 GB/s measured) per direction
to *any* peer, SM ld/st able to saturate it, and ``multimem`` primitives that
reduce inside the switch so a rank moves 1/N of the reduced bytes it would move
with peer loads.  On such a fabric a primitive that talks to many peers costs
the same as one that talks to a single peer, which is what makes one-shot and
two-shot algorithms win; ``op_latency`` accounts for that through
``TopologyProfile.uniform_all_to_all``.
"""

from __future__ import annotations

from collections import defaultdict, deque
from dataclasses import dataclass, field
from typing import Any, Dict, List

from ..nodes import PrimitiveOpType, infer_executor
from .rule import PatternEdge, PatternNode


@dataclass
class TopologyProfile:
    link_type: str = "nvlink"
    bandwidth_gb_s: float = 450.0
    latency_us: float = 1.0
    #: every peer reachable at full per-GPU bandwidth through a switch
    uniform_all_to_all: bool = False
    #: the switch can reduce / broadcast in the fabric (NVLS)
    in_switch_reduction: bool = False

    def to_dict(self) -> Dict[str, Any]:
        out = {"link_type": self.link_type, "bandwidth_gb_s": self.bandwidth_gb_s,
               "latency_us": self.latency_us}
        if self.uniform_all_to_all:
            out["uniform_all_to_all"] = True
        if self.in_switch_reduction:
            out["in_switch_reduction"] = True
        return out

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TopologyProfile":
        return cls(link_type=d.get("link_type", "nvlink"),
                   bandwidth_gb_s=d.get("bandwidth_gb_s", 450.0),
                   latency_us=d.get("latency_us", 1.0),
                   uniform_all_to_all=d.get("uniform_all_to_all", False),
                   in_switch_reduction=d.get("in_switch_reduction", False))


NVLINK_TOPOLOGY = TopologyProfile("nvlink", 450.0, 1.0)
RDMA_TOPOLOGY = TopologyProfile("rdma", 25.0, 5.0)
PCIE_TOPOLOGY = TopologyProfile("pcie", 32.0, 2.0)
#: NVLink 5 through NVSwitch: 900 GB/s per direction per GPU to any peer, NVLS capable.
NVLINK5_TOPOLOGY = TopologyProfile("nvlink5", 900.0, 0.7, uniform_all_to_all=True,
                                   in_switch_reduction=True)


def _h100_bandwidths() -> Dict[str, float]:
    return {"sm": 50.0, "tma": 60.0, "ce": 40.0, "rdma": 25.0, "multimem": 180.0, "host": 10.0}


def _h100_reduce() -> Dict[str, float]:
    return {"sm": 30.0, "tma": 35.0, "multimem": 100.0}


@dataclass
class GpuProfile:
    name: str = "h100"
    launch_overhead_us: float = 1.0
    bandwidth_gb_s: Dict[str, float] = field(default_factory=_h100_bandwidths)
    reduce_throughput_gops: Dict[str, float] = field(default_factory=_h100_reduce)
    num_channels: int = 4
    per_channel_bw_gb_s: Dict[str, float] = field(default_factory=_h100_bandwidths)
    channel_launch_overhead_us: float = 0.5

    def to_dict(self) -> Dict[str, Any]:
        return {
            "name": self.name,
            "launch_overhead_us": self.launch_overhead_us,
            "bandwidth_gb_s": self.bandwidth_gb_s,
            "reduce_throughput_gops": self.reduce_throughput_gops,
            "num_channels": self.num_channels,
            "per_channel_bw_gb_s": self.per_channel_bw_gb_s,
            "channel_launch_overhead_us": self.channel_launch_overhead_us,
        }

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GpuProfile":
        return cls(
            name=d.get("name", "custom"),
            launch_overhead_us=d.get("launch_overhead_us", 1.0),
            bandwidth_gb_s=d.get("bandwidth_gb_s", {}),
            reduce_throughput_gops=d.get("reduce_throughput_gops", {}),
            num_channels=d.get("num_channels", 4),
            per_channel_bw_gb_s=d.get("per_channel_bw_gb_s", {}),
            channel_launch_overhead_us=d.get("channel_launch_overhead_us", 0.5),
        )


H100_PROFILE = GpuProfile(name="h100")

# B200, calibrated on device timelines of 512 MB fp32 all-reduces (GB/s per NVLink direction actually
# sustained).  SM peer loads: the two-shot plan's pull-reduce and gather phases move 646-655 GB/s on
# 4 GPUs and 626 GB/s on 2 ("tma" plans execute on the same SM path: TMA never touches peer memory).
# In-switch: the one-pass multimem all-reduce moves (W+1)/W of the message per direction at 571-575 GB/s
# on 2, 4 and 8 GPUs alike.  Copy engines: 745 GB/s (cudaMemcpyPeer).  `plan_cost` multiplies a multimem
# step's slice by the number of slices that cross this GPU's links while every rank runs that step.
_B200_BW = {"sm": 640.0, "tma": 640.0, "ce": 745.0, "rdma": 50.0, "multimem": 572.0, "host": 25.0}
B200_PROFILE = GpuProfile(
    name="b200",
    launch_overhead_us=0.6,
    bandwidth_gb_s=dict(_B200_BW),
    reduce_throughput_gops={"sm": 600.0, "tma": 600.0, "multimem": 1600.0},
    num_channels=32,
    per_channel_bw_gb_s=dict(_B200_BW),
    channel_launch_overhead_us=0.05,
)

_PROFILES = {"h100": H100_PROFILE, "b200": B200_PROFILE}
_TOPOLOGIES = {"h100": NVLINK_TOPOLOGY, "b200": NVLINK5_TOPOLOGY}


def profile_by_name(name: str) -> GpuProfile:
    """Device profile for a ``Compiler(gpu_profile=...)`` string; unknown names
    fall back to a calibrated profile cached on disk, then to H100."""
    key = str(name).lower()
    if key in _PROFILES:
        return _PROFILES[key]
    from .rule_db import load_profile
    cached = load_profile(key)
    return GpuProfile.from_dict(cached) if cached else H100_PROFILE


def topology_for_profile(name: str) -> TopologyProfile:
    return _TOPOLOGIES.get(str(name).lower(), NVLINK_TOPOLOGY)


_COPY_OPS = frozenset({
    PrimitiveOpType.SM_COPY, PrimitiveOpType.TMA_COPY, PrimitiveOpType.CE_COPY,
    PrimitiveOpType.MULTIMEM_STORE, PrimitiveOpType.RDMA_WRITE, PrimitiveOpType.RDMA_READ,
    PrimitiveOpType.SM_PUT,
})
_REDUCE_OPS = frozenset({
    PrimitiveOpType.SM_REDUCE, PrimitiveOpType.TMA_REDUCE, PrimitiveOpType.MULTIMEM_REDUCE,
    PrimitiveOpType.SM_REDUCE_MULTI, PrimitiveOpType.MULTIMEM_ALLREDUCE,
})
_SYNC_OPS = frozenset({PrimitiveOpType.NOTIFY, PrimitiveOpType.WAIT_NOTIFY, PrimitiveOpType.NOOP})
_DEFAULT_BW = 10.0
_DEFAULT_GOPS = 30.0


def _us(amount: float, rate_g: float) -> float:
    """amount / (rate_g * 1e9) seconds, expressed in microseconds."""
    return amount / (rate_g * 1e3) if rate_g > 0 and amount > 0 else 0.0


def op_latency(op_type: PrimitiveOpType, profile: GpuProfile, data_size_bytes: int = 0) -> float:
    issue = profile.launch_overhead_us
    if op_type in _SYNC_OPS:
        return issue
    executor = infer_executor(op_type)
    key = executor.value if executor else "host"
    if op_type in _COPY_OPS:
        return issue + _us(data_size_bytes, profile.bandwidth_gb_s.get(key, _DEFAULT_BW))
    if op_type in _REDUCE_OPS:
        transfer = _us(data_size_bytes, profile.bandwidth_gb_s.get(key, _DEFAULT_BW))
        arithmetic = _us(data_size_bytes // 4,
                         profile.reduce_throughput_gops.get(key, _DEFAULT_GOPS))
        return issue + max(transfer, arithmetic)
    return issue


def critical_path_cost(nodes: List[PatternNode], edges: List[PatternEdge],
                       profile: GpuProfile, data_size_bytes: int = 0) -> float:
    """Longest path through the pattern in microseconds."""
    count = len(nodes)
    if count == 0:
        return 0.0
    channels = {node.channel for node in nodes}
    multi = len(channels) > 1

    successors: Dict[int, List[int]] = defaultdict(list)
    for edge in edges:
        successors[edge.src_idx].append(edge.dst_idx)
    if multi:
        # One channel is one in-order queue: chain its primitives.
        by_channel: Dict[int, List[int]] = defaultdict(list)
        for i, node in enumerate(nodes):
            by_channel[node.channel].append(i)
        for members in by_channel.values():
            for a, b in zip(members, members[1:]):
                if b not in successors[a]:
                    successors[a].append(b)

    cost = [op_latency(node.op_type, profile, data_size_bytes) for node in nodes]
    indegree = [0] * count
    for outs in successors.values():
        for v in outs:
            indegree[v] += 1
    finish = [0.0] * count
    ready = deque(i for i in range(count) if indegree[i] == 0)
    for i in ready:
        finish[i] = cost[i]
    while ready:
        u = ready.popleft()
        for v in successors[u]:
            finish[v] = max(finish[v], finish[u] + cost[v])
            indegree[v] -= 1
            if indegree[v] == 0:
                ready.append(v)

    total = max(finish)
    if multi:
        total += profile.channel_launch_overhead_us * (len(channels) - 1)
    return total


def egraph_node_cost(enode, child_costs: Dict[int, float], device: GpuProfile,
                     topology: TopologyProfile) -> float:
    """Extraction cost of one e-node: own cost + the slowest child.

    ``size`` / ``count`` parameters are element counts; they are priced at the
    executor's bandwidth, capped by the fabric's per-GPU link bandwidth.
    ``multimem`` e-nodes are only affordable on fabrics that reduce in-switch.
    """
    upstream = max(child_costs.values(), default=0.0)
    if enode.op_type in ("notify", "wait_notify", "noop"):
        return upstream + device.launch_overhead_us
    params = dict(enode.params)
    amount = params.get("size", params.get("count", 0))
    if not isinstance(amount, (int, float)):
        amount = 0
    key = enode.op_type.split(".", 1)[0]
    bandwidth = device.bandwidth_gb_s.get(key, _DEFAULT_BW)
    if key in ("sm", "tma", "ce", "multimem") and topology is not None:
        bandwidth = min(bandwidth, topology.bandwidth_gb_s)
    own = device.launch_overhead_us + _us(amount, bandwidth)
    if key == "multimem" and topology is not None and not topology.in_switch_reduction \
            and topology.uniform_all_to_all:
        own += 1e9  # a switched fabric without NVLS cannot run multimem primitives
    return upstream + own


def cost_delta(source_nodes: List[PatternNode], source_edges: List[PatternEdge],
               replacement_nodes: List[PatternNode], replacement_edges: List[PatternEdge],
               profile: GpuProfile, data_size_bytes: int = 0) -> float:
    """Microseconds saved by the replacement (positive = faster)."""
    return (critical_path_cost(source_nodes, source_edges, profile, data_size_bytes)
            - critical_path_cost(replacement_nodes, replacement_edges, profile, data_size_bytes))


def plan_cost(graph, profile: GpuProfile, topology: TopologyProfile, elem_bytes: int = 4,
              world_size: int = 1) -> float:
    """Critical-path time (µs) of a whole per-rank plan, priced node by node.

    Differences from ``critical_path_cost``, which prices every node of a small
    pattern at one common size: each data primitive is priced from its own
    ``size`` / ``count``; ``sm.reduce_multi`` moves one slice per remote source;
    a ``multimem`` primitive occupies the links with one slice per rank (the
    switch gathers from, or delivers to, all ``world_size`` ranks), at the
    profile's multimem rate, which already reflects that its reduce and
    broadcast halves use opposite link directions;
    transfers are capped by the fabric's per-GPU bandwidth; a ``wait_notify``
    costs one fabric latency; and on a switched fabric a run of consecutive
    notifies (or waits) on one chain costs a single step, because the engine
    issues them from parallel lanes.
    """
    order = graph.topological_sort()
    finish: Dict[str, float] = {}
    run_head: Dict[str, str] = {}          # node id -> first node of its signal run
    link = topology.bandwidth_gb_s if topology is not None else float("inf")
    parallel_signals = bool(topology is not None and topology.uniform_all_to_all)

    for node in order:
        op = node.op_type
        params = node.to_params()
        start = max((finish[d] for d in node.dependencies if d in finish), default=0.0)
        if op in _SYNC_OPS:
            own = topology.latency_us if (op == PrimitiveOpType.WAIT_NOTIFY and topology) \
                else profile.launch_overhead_us
            if parallel_signals and len(node.dependencies) == 1:
                prev = graph.nodes.get(node.dependencies[0])
                if prev is not None and prev.op_type == op:
                    own = 0.0                         # rides along with the run's first signal
        else:
            executor = infer_executor(op)
            key = executor.value if executor else "host"
            amount = params.get("size", params.get("count", 0)) * elem_bytes
            if op == PrimitiveOpType.SM_REDUCE_MULTI:
                amount *= max(1, len(params.get("source_ranks", ())) - 1)
            rate = profile.bandwidth_gb_s.get(key, _DEFAULT_BW)
            extra = 0.0
            if key == "multimem":
                # Slices on this GPU's busier link direction while all ranks run the step: a reduce
                # sends this rank's copy of all W slices, a store receives all W, the fused
                # all-reduce does both at once plus its own slice each way.
                amount *= max(1, world_size) + (1 if op == PrimitiveOpType.MULTIMEM_ALLREDUCE else 0)
                rate = min(rate, link)
                # A multimem access is answered by the switch after it has gathered (or delivered)
                # every rank's copy: two more fabric hops than a peer load before the first byte.
                extra = 2.0 * topology.latency_us if topology is not None else 0.0
            else:
                rate = min(rate, link)
            own = profile.launch_overhead_us + extra + _us(amount, rate)
        finish[node.op_id] = start + own
    return max(finish.values(), default=0.0)
