"""Host-side pieces of the fused operators that need no GPU."""

import torch


def test_interleave_gate_up_layout():
    from pccl_b200.ops.moe import interleave_gate_up
    e, f, h = 2, 48, 8
    w1 = torch.arange(e * f * h, dtype=torch.float32).reshape(e, f, h)
    w3 = -w1
    w13 = interleave_gate_up(w1, w3).reshape(e, 2 * f, h)
    for expert in range(e):
        for group in range(f // 16):
            rows = w13[expert, 32 * group:32 * (group + 1)]
            assert torch.equal(rows[:16], w1[expert, 16 * group:16 * (group + 1)])
            assert torch.equal(rows[16:], w3[expert, 16 * group:16 * (group + 1)])


def test_moe_reference_matches_dense_formulation():
    from pccl_b200.ops.moe import moe_reference
    torch.manual_seed(0)
    t, h, f, e = 32, 16, 32, 4
    x = torch.randn(t, h).to(torch.bfloat16)
    wg = torch.randn(e, h).to(torch.bfloat16)
    w1, w3 = torch.randn(e, f, h).to(torch.bfloat16), torch.randn(e, f, h).to(torch.bfloat16)
    w2 = torch.randn(e, h, f).to(torch.bfloat16)
    out, idx, gates = moe_reference(x, wg, w1, w3, w2)
    probs = torch.softmax(x.float() @ wg.float().t(), dim=-1)
    top, top_idx = probs.topk(2, dim=-1)
    assert torch.equal(top_idx, idx)
    torch.testing.assert_close(gates, top / top.sum(-1, keepdim=True), atol=1e-5, rtol=1e-5)
    dense = torch.zeros(t, h)
    for token in range(t):
        for k in range(2):
            ex = idx[token, k]
            hid = torch.nn.functional.silu(x[token].float() @ w1[ex].float().t()) * (x[token].float() @ w3[ex].float().t())
            dense[token] += gates[token, k] * (hid.to(torch.bfloat16).float() @ w2[ex].float().t())
    torch.testing.assert_close(out, dense, atol=1e-2, rtol=1e-2)


def test_config_describes_every_option():
    from pccl_b200 import config
    text = config.describe()
    for name in config.OPTIONS:
        assert name in text
    cfg = config.PcclConfig.from_env({"PCCL_LL_MAX_BYTES": "64K", "PCCL_NUM_BLOCKS": "64"})
    assert cfg.ll_max_bytes == 64 << 10 and cfg.num_blocks == 64
    assert config.PcclConfig.from_env(cfg.to_env()).num_blocks == 64


def test_lowering_runs_independent_gather_copies_without_barriers():
    """Two-shot's W-1 gather copies form one barrier-free run; the reduce before them keeps its barrier."""
    from pccl_b200 import Compiler, engine
    from pccl_b200.dsl.algorithms import TwoShotAllreduce
    native = engine.load_native()
    world, numel = 4, 1 << 20
    plan = Compiler().compile_to_json(TwoShotAllreduce().build_allreduce(1, world, numel, "float32", "sm", 1))
    summary = native.lower_plan_summary(plan, 1, world, 64 << 20, 16, False)
    steps = summary["chain_list"][0]["steps"]
    copies = [s for s in steps if s[0] == 1 and s[5] > 0]        # kind 1 = pull copy
    assert len(copies) == world - 1
    assert [s[6] for s in copies] == [1] * (world - 2) + [0]     # all but the last defer their barrier
    assert all(s[6] == 0 for s in steps if s[0] not in (1, 2))   # nothing else does


def test_gradient_bucket_partition():
    from pccl_b200.parallel.layers import partition_buckets
    assert partition_buckets([10, 10, 10, 50, 5], 25) == [[0, 1], [2], [3], [4]]
    assert partition_buckets([], 8) == []
    assert partition_buckets([100], 8) == [[0]]
    flat = [i for b in partition_buckets(list(range(1, 40)), 64) for i in b]
    assert flat == list(range(39))
