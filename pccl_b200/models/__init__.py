"""Model blocks built from the fused operators (tensor-parallel MLP, expert-parallel MoE block)."""


def __getattr__(name):
    if name in ("TensorParallelMLP", "MixtralMoEBlock", "rms_norm"):
        from . import blocks
        return getattr(blocks, name)
    raise AttributeError(name)


__all__ = ["TensorParallelMLP", "MixtralMoEBlock", "rms_norm"]
