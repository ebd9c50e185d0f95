"""Expert-parallel Mixture-of-Experts feed-forward (top-2 routing, SwiGLU experts).

Three kernels per call, all on the caller's stream:

1. route + dispatch: router logits, softmax top-2 with renormalised gates, and each token row
   pushed straight into the receive buffer of the rank that owns its expert (NVLink stores);
2. expert GEMM 1 on the tcgen05 tensor cores over the filled rows only, SwiGLU in the epilogue;
3. expert GEMM 2 whose epilogue multiplies by the gate and stores each row into the combine
   buffer of the token's home rank, followed in the same kernel by the two-way sum per token.

Experts are spread evenly over the ranks (``experts % world == 0``); a region of ``cap`` rows
per (local expert, source rank) is reserved so that no token is ever dropped.  Without a
process group (one GPU) an ordinary CUDA buffer stands in for the symmetric heap.
Construction is collective.  The reference has no MoE operator; the workload is its
all-to-all template's target use (pccl/dsl/algorithms/ring.py, build_alltoall).
"""

from __future__ import annotations

import torch

from .. import engine as _engine
from .tensor_parallel import _fence

_BLOCK = 128


def interleave_gate_up(w1: torch.Tensor, w3: torch.Tensor) -> torch.Tensor:
    """Stack ``w1`` (gate) and ``w3`` (up), each ``[experts, ffn, hidden]``, as the kernel reads them.

    Per expert, rows alternate in groups of 16: 16 gate rows, then the 16 up rows of the same
    hidden units, so one 32-column slice of the accumulator holds both halves of SwiGLU.
    Returns ``[experts * 2 * ffn, hidden]``.
    """
    e, f, h = w1.shape
    if f % 16:
        raise ValueError("ffn must be a multiple of 16")
    g = w1.reshape(e, f // 16, 1, 16, h)
    u = w3.reshape(e, f // 16, 1, 16, h)
    return torch.cat([g, u], dim=2).reshape(e * 2 * f, h).contiguous()


def moe_reference(x, wg, w1, w3, w2):
    """Plain fp32 PyTorch statement of the layer (all experts local), for tests."""
    xf = x.float()
    logits = xf @ wg.float().t()
    top, idx = logits.topk(2, dim=-1)
    gates = torch.softmax(top, dim=-1)
    out = torch.zeros_like(xf)
    for e in range(wg.shape[0]):
        for k in range(2):
            rows = (idx[:, k] == e).nonzero().squeeze(-1)
            if rows.numel() == 0:
                continue
            xe = xf[rows]
            h = torch.nn.functional.silu(xe @ w1[e].float().t()) * (xe @ w3[e].float().t())
            out[rows] += gates[rows, k, None] * (h.to(torch.bfloat16).float() @ w2[e].float().t())
    return out, idx, gates


def _round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


class FusedMoE:
    """``out[tokens, hidden] = sum_k gate_k * expert_k(x)`` over the two routed experts of each token."""

    def __init__(self, tokens: int, hidden: int, ffn: int, experts: int, group=None, local: bool = False):
        self.tokens, self.hidden, self.ffn, self.experts = tokens, hidden, ffn, experts
        self.native = _engine.load_native().fused
        self.local = local
        if local:
            self.world, self.rank = 1, 0
        else:
            self.engine = _engine.get_engine()
            self.world, self.rank = self.engine.world, self.engine.rank
        if experts % self.world:
            raise ValueError(f"{experts} experts do not divide over {self.world} ranks")
        self.local_experts = experts // self.world
        self.cap = _round_up(tokens, _BLOCK)
        regions = self.local_experts * self.world
        sizes = [
            regions * self.cap * hidden * 2,        # recv
            regions * self.cap * 8,                 # meta
            _round_up(regions * 4, 256),            # counts
            256,                                    # ready flags
            256,                                    # done flags
            tokens * 2 * hidden * 2,                # combine
        ]
        if local:
            offsets, total = [], 0
            for s in sizes:
                offsets.append(total)
                total += _round_up(s, 256)
            self.heap = torch.zeros(total, dtype=torch.uint8, device="cuda")
            self.offsets = offsets
        else:
            self.heap = None
            self._buffers = [self.engine.empty_symmetric((_round_up(s, 256),), torch.uint8) for s in sizes]
            for b in self._buffers[2:5]:
                b.zero_()
            self.offsets = [b.heap_offset for b in self._buffers]
        self.h = torch.empty(regions * self.cap, ffn, dtype=torch.bfloat16, device="cuda")
        self.scratch = torch.zeros(experts + 1, dtype=torch.int32, device="cuda")
        self.cta_counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.topk_idx = torch.empty(tokens, 2, dtype=torch.int32, device="cuda")
        self.topk_gate = torch.empty(tokens, 2, dtype=torch.float32, device="cuda")
        self.epoch = 0
        self.wg = self.w13 = self.w2 = None
        if not local:
            _fence(group)

    def set_weights(self, wg: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor) -> None:
        """``wg [experts, hidden]`` (replicated); ``w1, w3 [local_experts, ffn, hidden]`` and
        ``w2 [local_experts, hidden, ffn]`` are this rank's experts."""
        le = self.local_experts
        if tuple(w1.shape) != (le, self.ffn, self.hidden) or tuple(w2.shape) != (le, self.hidden, self.ffn):
            raise ValueError("expert weights have the wrong shape")
        self.wg = wg.to(torch.bfloat16).contiguous()
        self.w13 = interleave_gate_up(w1.to(torch.bfloat16), w3.to(torch.bfloat16))
        self.w2 = w2.to(torch.bfloat16).reshape(le * self.hidden, self.ffn).contiguous()

    def __call__(self, x: torch.Tensor, out: torch.Tensor = None, ctas: int = 0, phases: int = 7) -> torch.Tensor:
        if self.wg is None:
            raise RuntimeError("set_weights() first")
        if tuple(x.shape) != (self.tokens, self.hidden) or x.dtype != torch.bfloat16:
            raise ValueError(f"x must be bf16 [{self.tokens}, {self.hidden}]")
        if out is None:
            out = torch.empty(self.tokens, self.hidden, dtype=torch.bfloat16, device=x.device)
        self.epoch += 1
        self.native.moe_forward(x.contiguous(), self.wg, self.w13, self.w2, self.h, out, self.scratch,
                                self.cta_counter, self.offsets, self.cap, self.epoch, self.heap, ctas, phases,
                                self.topk_idx, self.topk_gate)
        return out


def route(x: torch.Tensor, wg: torch.Tensor):
    """Router alone: ``(topk_idx [T,2] int32, gates [T,2] fp32, slots [T,2] int32, counts [E] int32)``."""
    native = _engine.load_native().fused
    tokens, experts = x.shape[0], wg.shape[0]
    scratch = torch.empty(experts + 1, dtype=torch.int32, device=x.device)
    idx = torch.empty(tokens, 2, dtype=torch.int32, device=x.device)
    gate = torch.empty(tokens, 2, dtype=torch.float32, device=x.device)
    slot = torch.empty(tokens, 2, dtype=torch.int32, device=x.device)
    counts = torch.empty(experts, dtype=torch.int32, device=x.device)
    native.moe_route(x.contiguous(), wg.contiguous(), scratch, idx, gate, slot, counts)
    return idx, gate, slot, counts
