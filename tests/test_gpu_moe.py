"""MoE router and fused expert-parallel feed-forward on one GPU against plain PyTorch fp32."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _weights(experts, hidden, ffn, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    wg = (torch.randn(experts, hidden, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w1 = (torch.randn(experts, ffn, hidden, device="cuda", generator=g) * hidden ** -0.5).to(torch.bfloat16)
    w3 = (torch.randn(experts, ffn, hidden, device="cuda", generator=g) * hidden ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(experts, hidden, ffn, device="cuda", generator=g) * ffn ** -0.5).to(torch.bfloat16)
    return wg, w1, w3, w2


@pytest.mark.parametrize("tokens,hidden,experts", [(1000, 512, 8), (257, 1024, 4), (64, 256, 64), (4096, 4096, 8)])
def test_router_matches_torch(tokens, hidden, experts):
    from pccl_b200.ops import moe
    x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    wg = (torch.randn(experts, hidden, device="cuda") * 0.5).to(torch.bfloat16)
    idx, gate, slot, counts = moe.route(x, wg)
    torch.cuda.synchronize()
    logits = x.float() @ wg.float().t()
    top, ref_idx = logits.topk(2, dim=-1)
    ref_gate = torch.softmax(top, dim=-1)
    # A token whose second and third logits are within rounding of each other may legitimately differ.
    margin = (logits.topk(3, dim=-1).values[:, 1] - logits.topk(3, dim=-1).values[:, 2]) > 1e-3
    margin &= (top[:, 0] - top[:, 1]) > 1e-3
    assert margin.float().mean() > 0.95
    assert torch.equal(idx[margin].long(), ref_idx[margin])
    torch.testing.assert_close(gate[margin], ref_gate[margin], atol=2e-3, rtol=2e-3)
    ref_counts = torch.bincount(idx.long().flatten(), minlength=experts)
    assert torch.equal(counts.long(), ref_counts)
    # Slots are a permutation of 0..count-1 inside every expert.
    for e in range(experts):
        s = slot.flatten()[idx.flatten() == e].long().sort().values
        assert torch.equal(s, torch.arange(s.numel(), device="cuda"))


@pytest.mark.parametrize("experts", [2, 8])
def test_router_with_non_finite_rows_stays_inside_its_outputs(experts):
    """NaN / Inf activations give arbitrary but valid routing: two distinct experts in range per
    token, counts that add up, and nothing written outside the output arrays."""
    from pccl_b200.ops import moe
    tokens, hidden = 300, 256
    x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    x[3] = float("nan")
    x[17, 5] = float("inf")
    x[40, :] = float("-inf")
    x[41, 0], x[41, 1] = float("inf"), float("-inf")
    wg = (torch.randn(experts, hidden, device="cuda") * 0.5).to(torch.bfloat16)
    idx, gate, slot, counts = moe.route(x, wg)
    torch.cuda.synchronize()
    assert int(idx.min()) >= 0 and int(idx.max()) < experts
    assert bool((idx[:, 0] != idx[:, 1]).all())
    assert int(counts.sum()) == 2 * tokens
    assert torch.equal(counts.long(), torch.bincount(idx.long().flatten(), minlength=experts))
    finite = torch.isfinite(x.float()).all(dim=-1)
    assert torch.isfinite(gate[finite]).all()
    logits = x[finite].float() @ wg.float().t()
    top, ref_idx = logits.topk(2, dim=-1)
    clear = (top[:, 0] - top[:, 1]) > 1e-3
    assert torch.equal(idx[finite][clear][:, 0].long(), ref_idx[clear][:, 0])


@pytest.mark.parametrize("sms_per_tile", [1, 2])
@pytest.mark.parametrize("tokens,hidden,ffn,experts", [(512, 512, 1024, 8), (200, 256, 400, 4), (1024, 1024, 2048, 8),
                                                       (2048, 512, 768, 2)])
def test_fused_moe_single_gpu(tokens, hidden, ffn, experts, sms_per_tile, monkeypatch):
    """Expert GEMMs on one SM per tile and on SM pairs (two row blocks of one expert per tile; experts
    with an odd number of filled blocks leave half of their last pair empty)."""
    from pccl_b200.ops import moe
    monkeypatch.setenv("PCCL_GEMM_SMS_PER_TILE", str(sms_per_tile))
    native = __import__("pccl_b200.engine", fromlist=["load_native"]).load_native().fused
    native.clear_error()
    wg, w1, w3, w2 = _weights(experts, hidden, ffn)
    layer = moe.FusedMoE(tokens, hidden, ffn, experts, local=True)
    layer.set_weights(wg, w1, w3, w2)
    for call in range(3):
        x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
        out = layer(x)
        torch.cuda.synchronize()
        assert native.read_error() == 0
        ref, ref_idx, _ = moe.moe_reference(x, wg, w1, w3, w2)
        same_route = (layer.topk_idx.long() == ref_idx).all(dim=-1)
        assert same_route.float().mean() > 0.95
        err = (out.float() - ref)[same_route].abs().max().item()
        scale = ref[same_route].abs().max().item()
        assert err <= 2e-2 * scale + 1e-3, f"call {call}: max error {err} against magnitude {scale}"


def test_mixtral_block_single_gpu():
    from pccl_b200.models import MixtralMoEBlock, rms_norm
    from pccl_b200.ops import moe
    tokens, hidden, ffn, experts = 256, 512, 1024, 8
    wg, w1, w3, w2 = _weights(experts, hidden, ffn, seed=3)
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda")).to(torch.bfloat16)
    block = MixtralMoEBlock(tokens, hidden, ffn, experts, gamma, local=True)
    block.load(wg, w1, w3, w2)
    x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    y = block(x)
    torch.cuda.synchronize()
    normed = rms_norm(x, gamma)
    ref, ref_idx, _ = moe.moe_reference(normed, wg, w1, w3, w2)
    same = (block.moe.op.topk_idx.long() == ref_idx).all(dim=-1)
    err = ((y.float() - x.float()) - ref)[same].abs().max().item()
    assert err <= 2e-2 * ref[same].abs().max().item() + 2e-2
