"""tcgen05 GEMM against an fp32 PyTorch reference."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("sms_per_tile", [1, 2])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (384, 768, 1024),
                                   (200, 312, 72), (8192, 4096, 1792), (1024, 1792, 4096),
                                   # tile counts that leave the paired kernel's last round mostly idle: its tiles
                                   # are cut along K (2 tail tiles in 16 slices; 34 in 2; 12 in 6 uneven slices)
                                   (8192, 1792, 4096), (4096, 4096, 4096), (5120, 2048, 2048)])
def test_matmul_nt_matches_fp32_reference(m, n, k, sms_per_tile):
    """Both forms: one SM per 128 x 256 tile, and pairs of SMs on 256 x 256 tiles (cta_group::2)."""
    from pccl_b200.ops import gemm
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    c = gemm.matmul_nt(a, b, sms_per_tile=sms_per_tile)
    torch.cuda.synchronize()
    gemm.check()
    ref = a.float() @ b.float().t()
    # bf16 output rounding: relative 2^-8, plus accumulation-order noise.
    torch.testing.assert_close(c.float(), ref, atol=2e-2 * (k ** 0.5) * 0.05, rtol=2 ** -7)
    # a second call: the split tail's counters must be back at zero
    c2 = gemm.matmul_nt(a, b, sms_per_tile=sms_per_tile)
    torch.cuda.synchronize()
    gemm.check()
    assert torch.equal(c, c2)


@pytest.mark.parametrize("sms_per_tile", [1, 2])
def test_distinct_tiles_land_in_their_own_places(sms_per_tile):
    """A structured input catches swizzle / descriptor mistakes that random data could hide."""
    from pccl_b200.ops import gemm
    m, n, k = 256 + 128 * (sms_per_tile - 1), 512, 128          # an odd number of row blocks for the paired form
    a = torch.zeros(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(n, k, device="cuda", dtype=torch.bfloat16)
    a[:, 0] = torch.arange(m, device="cuda").to(torch.bfloat16) % 64
    a[:, 77] = 1
    b[:, 0] = 1
    b[:, 77] = (torch.arange(n, device="cuda") % 32).to(torch.bfloat16)
    c = gemm.matmul_nt(a, b, sms_per_tile=sms_per_tile)
    torch.cuda.synchronize()
    gemm.check()
    ref = a.float() @ b.float().t()
    assert torch.equal(c.float(), ref)
