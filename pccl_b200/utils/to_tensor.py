"""String <-> uint8 tensor helpers used when endpoint records travel through
tensor collectives (reference: pccl/utils/to_tensor.py:4-14)."""

import torch


def to_tensor(s: str) -> torch.Tensor:
    return torch.tensor(list(s.encode("utf-8")), dtype=torch.uint8)


def to_str(t: torch.Tensor) -> str:
    return bytes(t.detach().cpu().to(torch.uint8).tolist()).decode("utf-8")
