"""Self test of the tcgen05 building blocks (shared-memory descriptors, TMEM round trip)
through the C ABI, before anything larger uses them."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b_mn_major", [False, True])
def test_umma_128x128x128(b_mn_major, dtype):
    from flash_moba_b200 import ops
    torch.manual_seed(0)
    a = torch.randn(128, 128, device="cuda").to(dtype)
    b = torch.randn(128, 128, device="cuda").to(dtype)
    d = ops.selftest_umma(a, b, b_mn_major)
    ref = a.float() @ (b.float() if b_mn_major else b.float().t())
    assert torch.allclose(d, ref, atol=1e-2, rtol=1e-3), (d - ref).abs().max().item()
