"""The allocation-free router entry point, called through its exported C symbol.

Collected last (file name) so that it also runs after every other GPU test has used the
device; it must pass on its own as well.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from pccl_b200 import engine
    lib = ctypes.CDLL(engine.load_native().__file__)
    fn = lib.pccl_moe_route_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.pccl_moe_route_static_strerror.restype = ctypes.c_char_p
    lib.pccl_moe_route_static_strerror.argtypes = [ctypes.c_int]
    return lib, fn


def _slots_are_permutations(idx, slot, experts):
    for e in range(experts):
        s = slot.flatten()[idx.flatten() == e].long().sort().values
        if not torch.equal(s, torch.arange(s.numel(), device=s.device)):
            return False
    return True


@pytest.mark.parametrize("tokens,hidden,experts", [(777, 512, 8), (4096, 4096, 8)])
def test_static_router_matches_allocating_entry_point(tokens, hidden, experts):
    from pccl_b200.ops import moe
    lib, fn = _entry()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                              # two calls in a row share the scratch array
        x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
        wg = (torch.randn(experts, hidden, device="cuda") * 0.5).to(torch.bfloat16)
        idx = torch.empty(tokens, 2, dtype=torch.int32, device="cuda")
        gate = torch.empty(tokens, 2, dtype=torch.float32, device="cuda")
        slot = torch.empty(tokens, 2, dtype=torch.int32, device="cuda")
        counts = torch.empty(experts, dtype=torch.int32, device="cuda")
        rc = fn(x.data_ptr(), wg.data_ptr(), tokens, hidden, experts, idx.data_ptr(), gate.data_ptr(),
                slot.data_ptr(), counts.data_ptr(), stream)
        assert rc == 0, lib.pccl_moe_route_static_strerror(rc).decode()
        ref_idx, ref_gate, ref_slot, ref_counts = moe.route(x, wg)
        torch.cuda.synchronize()
        assert torch.equal(idx, ref_idx), f"call {call}: expert choices differ"
        torch.testing.assert_close(gate, ref_gate, atol=1e-6, rtol=1e-6)
        assert torch.equal(counts, ref_counts), f"call {call}: per-expert counts differ"
        assert _slots_are_permutations(idx, slot, experts)
        assert _slots_are_permutations(ref_idx, ref_slot, experts)


def test_static_router_with_optional_outputs_left_out_and_non_finite_rows():
    """Every output pointer is optional, and rows holding NaN / Inf must not push the counters
    outside the module's scratch array: the words on either side of the counts stay untouched."""
    lib, fn = _entry()
    tokens, hidden, experts = 333, 256, 8
    x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)
    x[7] = float("nan")
    x[8, 3] = float("-inf")
    wg = (torch.randn(experts, hidden, device="cuda") * 0.5).to(torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(x.data_ptr(), wg.data_ptr(), tokens, hidden, experts, None, None, None, None, stream) == 0
    guarded = torch.full((experts + 8,), -7, dtype=torch.int32, device="cuda")
    counts = guarded[4:4 + experts]
    idx = torch.empty(tokens, 2, dtype=torch.int32, device="cuda")
    assert fn(x.data_ptr(), wg.data_ptr(), tokens, hidden, experts, idx.data_ptr(), None, None,
              counts.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert int(counts.sum()) == 2 * tokens
    assert bool((guarded[:4] == -7).all()) and bool((guarded[4 + experts:] == -7).all())
    assert int(idx.min()) >= 0 and int(idx.max()) < experts and bool((idx[:, 0] != idx[:, 1]).all())
    logits = x.float() @ wg.float().t()
    finite = torch.isfinite(logits).all(dim=-1)
    top, ref_idx = logits[finite].topk(2, dim=-1)
    clear = (top[:, 0] - top[:, 1]) > 1e-3
    assert torch.equal(idx[finite][clear][:, 0].long(), ref_idx[clear][:, 0])


def test_static_router_rejects_oversize_shapes():
    lib, fn = _entry()
    x = torch.zeros(8, 256, dtype=torch.bfloat16, device="cuda")
    wg = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(x.data_ptr(), wg.data_ptr(), 8, 256, 128, None, None, None, None, stream) == 1      # too many experts
    assert fn(x.data_ptr(), wg.data_ptr(), 8, 8192, 64, None, None, None, None, stream) == 1      # router weight too large
    assert fn(None, wg.data_ptr(), 8, 256, 8, None, None, None, None, stream) == 2
    assert b"experts" in lib.pccl_moe_route_static_strerror(1)
