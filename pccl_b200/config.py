"""Run-time options in one place.

Every option is an environment variable read by the native engine or the Python
layers; ``PcclConfig.from_env()`` mirrors them in a dataclass and ``describe()``
prints the table.  Names shared with the reference keep their meaning
(reference: include/common/config.h:8-35, csrc/plugins/cuda/cuda_device.cc:290-298,
csrc/plugins/cuda/nvls_manager.h:29-31, csrc/engine_c.cc:87-104).
"""

from __future__ import annotations

import os
from dataclasses import dataclass, fields
from typing import Dict, Optional

_SIZES = {"k": 1 << 10, "m": 1 << 20, "g": 1 << 30}


def _size(text: str) -> int:
    text = text.strip()
    if text and text[-1].lower() in _SIZES:
        return int(text[:-1]) * _SIZES[text[-1].lower()]
    return int(text)


def _flag(text: str) -> bool:
    return text.strip().lower() not in ("0", "false", "off", "no", "")


OPTIONS: Dict[str, tuple] = {
    # name: (field, parser, default, description)
    "RANK": ("rank", int, None, "rank of this process (required by the native engine)"),
    "WORLD_SIZE": ("world_size", int, 1, "number of ranks"),
    "PCCL_BUFFER_SIZE": ("buffer_size", _size, 1 << 30, "bytes of the plan working buffer"),
    "PCCL_ARENA_SIZE": ("arena_size", _size, 1 << 30, "bytes of symmetric memory for fused operators"),
    "PCCL_NUM_BLOCKS": ("num_blocks", int, 128, "upper bound of CTAs per collective launch"),
    "PCCL_FORCE_BLOCKS": ("force_blocks", int, 0, "exact CTA count per launch (0 = heuristic)"),
    "PCCL_MIN_BYTES_PER_BLOCK": ("min_bytes_per_block", _size, 16 << 10, "smallest share worth another CTA"),
    "PCCL_WAIT_TIMEOUT_MS": ("wait_timeout_ms", int, 10000, "time budget of device-side waits per launch"),
    "PCCL_NVLS_ENABLE": ("nvls_enable", _flag, True, "use NVLS multicast when every rank supports it"),
    "PCCL_DISABLE_NVLS": ("disable_nvls", _flag, False, "turn NVLS off"),
    "PCCL_ALGO": ("algo", str, None, "force ring|rhd|tree|oneshot|twoshot|nvls|nvls_twopass|hybrid"),
    "PCCL_NVLS_FRACTION": ("nvls_fraction", float, 0.7,
                           "hybrid all-reduce: share of the message reduced in the switch, the rest goes two-shot"),
    "PCCL_CHANNELS": ("channels", int, None, "force the channel count of generated plans"),
    "PCCL_EXECUTOR": ("executor", str, None, "sm (default) | ce (copy engine) | cpu (gloo replay)"),
    "PCCL_LL_MAX_BYTES": ("ll_max_bytes", _size, 256 << 10,
                          "largest all-reduce taken by the packet-protocol kernel (0 = never)"),
    "PCCL_MOVER_TUNING": ("mover_tuning", int, 0,
                          "data-mover bits: 1 = two register tiles in flight, 2 = one tile in multimem steps"),
    "PCCL_CE_MIN_BYTES": ("ce_min_bytes", _size, 64 << 10, "copy-engine executor: smaller copies stay on the SM path"),
    "PCCL_CLOSING_BARRIER": ("closing_barrier", _flag, True,
                             "append an all-pairs barrier to pull-style plans (ring, rhd, tree, hand-built)"),
    "PCCL_RDMA": ("rdma", _flag, False, "build option: compile the verbs transport of the RDMA executor"),
    "PCCL_TUNING_FILE": ("tuning_file", str, None,
                         "JSON of measured routes per collective, world size and message size "
                         "(bench/collective_sweep.py --write-tuning)"),
    "PCCL_PLAN_CACHE": ("plan_cache", str, "~/.pccl/plans", "directory of compiled plans (off = compile every time)"),
    "PCCL_VALIDATE": ("validate", _flag, True,
                      "check all ranks' plans together (deadlock, leftover signals) when a plan is first compiled"),
    "PCCL_TRACE": ("trace", _flag, False, "stamp %globaltimer per plan step; read with Engine.trace(name)"),
    "PCCL_COOPERATIVE": ("cooperative", _flag, True,
                         "launch kernels whose CTAs wait on one another cooperatively (all CTAs resident)"),
    "PCCL_PUSH_MAX_BYTES": ("push_max_bytes", _size, 32 << 20,
                            "largest message taken by the fused push collectives (0 = never)"),
    "PCCL_PUSH_LEAN_CTAS": ("push_lean_ctas", int, 12,
                            "grid of the push kernel's second instance, used for collectives that overlap compute"),
    "PCCL_DP_TRANSPORT": ("dp_transport", str, "push",
                          "hooked gradient buckets: push (lean push kernel) | ce (copy-engine all-gather + local sum)"),
    "PCCL_GEMM_SMS_PER_TILE": ("gemm_sms_per_tile", int, 2,
                               "2 = pairs of SMs on 256x256 tiles (tcgen05.mma.cta_group::2), 1 = one SM per 128x256 tile"),
    "PCCL_GEMM_TILE_N": ("gemm_tile_n", int, 0, "tile width of the paired GEMM (multiple of 32; 0 = 256)"),
    "PCCL_GEMM_SPLIT_TAIL": ("gemm_split_tail", _flag, True,
                             "paired GEMM: cut the tiles of a sparsely filled last round along K"),
    "PCCL_GEMM_SPLIT_MIN_SLICES": ("gemm_split_min_slices", int, 3, "fewest K slices for which that split is used"),
    "PCCL_NVLS_CTAS": ("nvls_ctas", int, 64, "grid of the in-switch all-reduce kernel (algorithm \"nvls_kernel\")"),
    "PCCL_LOG_LEVEL": ("log_level", str, "WARN", "TRACE|DEBUG|INFO|WARN|ERROR|CRITICAL"),
    "PCCL_JOB_ID": ("job_id", str, None, "namespace of the fd-passing sockets"),
    "PCCL_DEBUG_ENDPOINT_INIT": ("debug_endpoint_init", _flag, False, "print bootstrap stages"),
}


@dataclass
class PcclConfig:
    rank: Optional[int] = None
    world_size: int = 1
    buffer_size: int = 1 << 30
    arena_size: int = 1 << 30
    num_blocks: int = 128
    force_blocks: int = 0
    min_bytes_per_block: int = 16 << 10
    wait_timeout_ms: int = 10000
    nvls_enable: bool = True
    disable_nvls: bool = False
    algo: Optional[str] = None
    nvls_fraction: float = 0.7
    channels: Optional[int] = None
    executor: Optional[str] = None
    ll_max_bytes: int = 256 << 10
    mover_tuning: int = 0
    ce_min_bytes: int = 64 << 10
    closing_barrier: bool = True
    rdma: bool = False
    tuning_file: Optional[str] = None
    plan_cache: str = "~/.pccl/plans"
    validate: bool = True
    trace: bool = False
    cooperative: bool = True
    push_max_bytes: int = 32 << 20
    push_lean_ctas: int = 12
    dp_transport: str = "push"
    gemm_sms_per_tile: int = 2
    gemm_tile_n: int = 0
    gemm_split_tail: bool = True
    gemm_split_min_slices: int = 3
    nvls_ctas: int = 64
    log_level: str = "WARN"
    job_id: Optional[str] = None
    debug_endpoint_init: bool = False

    @classmethod
    def from_env(cls, env=None) -> "PcclConfig":
        env = os.environ if env is None else env
        values = {}
        for name, (field, parse, default, _) in OPTIONS.items():
            raw = env.get(name)
            values[field] = default if raw in (None, "") else parse(raw)
        return cls(**values)

    def to_env(self) -> Dict[str, str]:
        """Environment assignments that reproduce this configuration."""
        out = {}
        for name, (field, _, default, _) in OPTIONS.items():
            value = getattr(self, field)
            if value is not None and value != default:
                out[name] = str(int(value)) if isinstance(value, bool) else str(value)
        return out


def describe() -> str:
    width = max(len(n) for n in OPTIONS)
    return "\n".join(f"{name.ljust(width)}  default={default!s:<12} {text}"
                     for name, (_, _, default, text) in OPTIONS.items())


assert {f.name for f in fields(PcclConfig)} == {v[0] for v in OPTIONS.values()}
