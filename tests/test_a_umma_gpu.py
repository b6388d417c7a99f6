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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tma_row_gather(dtype):
    from flash_moba_b200 import ops
    torch.manual_seed(1)
    a = torch.randn(1000, 128, device="cuda").to(dtype)
    b = torch.randn(128, 128, device="cuda").to(dtype)
    idx = torch.randint(0, 1000, (128,), device="cuda", dtype=torch.int32)
    idx[5], idx[77], idx[127] = -1, 1000, 999
    d = ops.selftest_gather(a, idx, b)
    g = a[idx.clamp(0, 999).long()].float()
    g[(idx < 0) | (idx >= 1000)] = 0
    ref = g @ b.float().t()
    assert torch.allclose(d, ref, atol=1e-2, rtol=1e-3), (d - ref).abs().max().item()
