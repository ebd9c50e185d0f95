"""Model blocks that exercise the fused operators end to end (inference forward).

``TensorParallelMLP``   Llama-style SwiGLU feed-forward under tensor + sequence parallelism:
    x[T/W, H] -(all-gather fused into the GEMM, SwiGLU in its epilogue)-> [T, F/W]
      -(GEMM with fused reduce-scatter)-> [T/W, H]: two kernels per block, no element-wise pass.
``MixtralMoEBlock``     residual + RMSNorm + expert-parallel top-2 MoE feed-forward.

Each block has a `reference()` in plain PyTorch (fp32) used by the tests.  The reference
framework has no model code; the shapes follow the Llama-3-8B / Mixtral-8x7B layers that its
benchmarks' collectives are sized for.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ..parallel.layers import ColumnParallelLinear, ExpertParallelMoE, RowParallelLinear


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()).to(x.dtype)


class TensorParallelMLP:
    def __init__(self, tokens: int, hidden: int, ffn_local: int, w_gate_up: torch.Tensor, w_down: torch.Tensor):
        """``w_gate_up [2 * ffn_local, hidden]`` (gate rows then up rows), ``w_down [hidden, ffn_local]``."""
        from ..ops.moe import interleave_gate_up
        self.tokens, self.hidden, self.ffn_local = tokens, hidden, ffn_local
        if ffn_local % 16:
            raise ValueError("ffn_local must be a multiple of 16")
        # Gate and up rows interleaved in groups of 16: one 32-column slice of the accumulator then
        # holds both halves of 16 outputs, which is what the fused epilogue combines.
        stacked = interleave_gate_up(w_gate_up[:ffn_local].unsqueeze(0), w_gate_up[ffn_local:].unsqueeze(0))
        self.up = ColumnParallelLinear(tokens, hidden, 2 * ffn_local, stacked, swiglu=True)
        self.down = RowParallelLinear(tokens, ffn_local, hidden, w_down)
        self.act = torch.empty(tokens, ffn_local, dtype=torch.bfloat16, device="cuda")

    def __call__(self, x_shard: torch.Tensor) -> torch.Tensor:
        self.up(x_shard, self.act)                                   # [T, F/W] = silu(gate) * up
        return self.down(self.act)                                   # [T/W, H]

    @staticmethod
    def reference(x_full: torch.Tensor, w_gate_up_all, w_down_all) -> torch.Tensor:
        """All ranks' weights (lists indexed by rank) applied to the gathered input, fp32."""
        out = torch.zeros(x_full.shape[0], w_down_all[0].shape[0], device=x_full.device)
        for wgu, wd in zip(w_gate_up_all, w_down_all):
            f = wgu.shape[0] // 2
            gu = x_full.float() @ wgu.float().t()
            act = (F.silu(gu[:, :f]) * gu[:, f:]).to(torch.bfloat16).float()
            out += act @ wd.float().t()
        return out


class MixtralMoEBlock:
    def __init__(self, tokens: int, hidden: int, ffn: int, experts: int, gamma: torch.Tensor, local: bool = False):
        self.gamma = gamma
        self.moe = ExpertParallelMoE(tokens, hidden, ffn, experts, local=local)

    def load(self, wg, w1, w3, w2) -> None:
        self.moe.load(wg, w1, w3, w2)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.moe(rms_norm(x, self.gamma))
