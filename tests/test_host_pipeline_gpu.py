"""Host pipeline: results of the head-group pipeline over pinned host tensors equal those of one
call on resident device tensors (heads are independent, so bit for bit)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("heads,heads_k,groups,backward,d", [(8, 8, 4, True, 128), (8, 2, 8, True, 128),
                                                             (6, 6, 4, False, 128), (4, 4, 2, True, 96)])
def test_pipeline_matches_resident_call(heads, heads_k, groups, backward, d):
    import flash_moba_b200 as F
    from flash_moba_b200.host_pipeline import HostPipeline
    lens = [1500, 700, 300]
    T, chunk, topk = sum(lens), 128, 3
    g = torch.Generator().manual_seed(9)
    mk = lambda h: torch.randn(T, h, d, generator=g).bfloat16().pin_memory()
    q_h, k_h, v_h, do_h = mk(heads), mk(heads_k), mk(heads_k), mk(heads)
    cu = torch.tensor([0, 1500, 2200, 2500], dtype=torch.int32, device="cuda")
    out_h = torch.empty_like(q_h).pin_memory()
    dq_h, dk_h, dv_h = (torch.empty_like(t).pin_memory() for t in (q_h, k_h, v_h))
    pipe = HostPipeline(T, heads, heads_k, d, torch.bfloat16, groups=groups, backward=backward)
    for _ in range(2):          # twice: the staging tensors and streams are reused
        if backward:
            pipe.run(q_h, k_h, v_h, do_h, cu, cu, max(lens), max(lens), chunk, topk, out_h, dq_h, dk_h, dv_h)
        else:
            pipe.run(q_h, k_h, v_h, None, cu, cu, max(lens), max(lens), chunk, topk, out_h)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q_h, k_h, v_h))
    out = F.flash_moba_varlen_func(qd, kd, vd, cu, cu, max(lens), max(lens), chunk, topk, causal=True)
    assert torch.equal(out.cpu(), out_h)
    if backward:
        dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), do_h.cuda())
        assert torch.equal(dq.cpu(), dq_h)
        assert torch.equal(dk.cpu(), dk_h)
        assert torch.equal(dv.cpu(), dv_h)


def test_copy_rows_rejects_bad_pitch():
    from flash_moba_b200 import _lib
    x = torch.zeros(16, dtype=torch.uint8).pin_memory()
    y = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = _lib.lib.fmb_copy_rows_async(y.data_ptr(), 4, x.data_ptr(), 4, 8, 2, 0, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"copy_rows" in _lib.lib.fmb_last_error()
