"""This library against the reference's own CUDA kernels on the same GPU.

Runs only where oracle/build_ref.sh has built the reference's extension (oracle/_ref/,
head dims 64 / 128 / 256, bf16, causal).  Same inputs to both: the pattern (pool -> gate -> CSC) is
compared entry by entry, attention forward and backward are compared on one common pattern, and
both are measured against the dense fp32 evaluation of that pattern: the reference's own error is
the yardstick ("no worse than twice the reference's error").
"""
import os
import sys

import pytest
import torch

from conftest import cu_of

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import moba_oracle as O  # noqa: E402
from oracle import ref_cuda  # noqa: E402

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_cuda.available(), reason="reference CUDA extension not built")]
DEV = "cuda"


def _inputs(lens, H, Hk, d, seed):
    torch.manual_seed(seed)
    T = sum(lens)
    q = torch.randn(T, H, d).bfloat16()
    k = torch.randn(T, Hk, d).bfloat16()
    v = torch.randn(T, Hk, d).bfloat16()
    do = torch.randn(T, H, d).bfloat16()
    return q, k, v, do


@pytest.mark.parametrize("lens,H,Hk,d,chunk,topk", [
    ([1024, 2048], 8, 8, 64, 128, 4),          # the reference's CPU-runnable configuration, in bf16
    ([4096], 4, 4, 128, 128, 8),
    ([1500, 700, 333], 4, 2, 128, 64, 3),
    ([2048, 900], 4, 2, 256, 128, 4),          # the wide-head kernels
    ([3000, 1536], 8, 2, 128, 64, 16),         # configuration 4 in miniature: GQA 4:1, chunk 64, lists of 16
])
def test_pattern_and_attention_against_reference_kernels(lens, H, Hk, d, chunk, topk):
    import flash_moba_b200 as F
    from flash_moba_b200 import ops
    from flash_moba_b200.interface import decide_lg_block_m
    q, k, v, do = _inputs(lens, H, Hk, d, 7)
    cs = cu_of(lens).to(DEV)
    S = max(lens)
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))

    # ---- pattern: both from the same pooled centroids
    km, cu_km = ops.mean_pool(kd, cs, S, chunk)
    co_r, cn_r, ind_r = ref_cuda.fused_topk(qd, km, cs, cs, cu_km, S, S, topk, chunk, True)
    co_m, cn_m, ind_m = F.flash_topk_varlen_func(qd, kd, cs, cs, S, S, topk, chunk, causal=True)
    assert torch.equal(co_m.cpu()[..., 0], co_r.cpu()[..., 0])          # same packing of the (sequence, head) regions
    mask_r = O.csc_to_mask(co_r.cpu(), cn_r.cpu(), ind_r.cpu(), cs.cpu(), S)
    mask_m = O.csc_to_mask(co_m.cpu(), cn_m.cpu(), ind_m.cpu(), cs.cpu(), S)
    wrong = (mask_r != mask_m).sum().item() / 2                          # a differing selection flips two entries
    assert wrong <= 0.005 * sum(lens) * H * topk, wrong                  # scores are bf16 products summed in different orders

    # ---- attention on one pattern (the reference's)
    scale = d ** -0.5
    lg_m = decide_lg_block_m(topk, chunk, S, True)
    o_r, lse_r = ref_cuda.attn_fwd(qd, kd, vd, cs, cs, S, S, co_r, cn_r, ind_r, lg_m, chunk, scale)
    dq_r, dk_r, dv_r = ref_cuda.attn_bwd(dod, qd, kd, vd, o_r, lse_r, cs, cs, S, S, co_r, cn_r, ind_r, lg_m, chunk, scale)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (qd, kd, vd))
    o_m, lse_m, _ = F.flash_moba_attn_varlen_func(qg, kg, vg, cs, cs, S, S, co_r, cn_r, ind_r, lg_m, chunk, causal=True,
                                                  return_attn_probs=True)
    dq_m, dk_m, dv_m = torch.autograd.grad(o_m, (qg, kg, vg), dod)
    q32, k32, v32 = (t.clone().requires_grad_(True) for t in (q, k, v))
    o_t, lse_t = O.attention_dense(q32, k32, v32, cs.cpu(), cs.cpu(), mask_r, chunk, True, lowp=False)
    dq_t, dk_t, dv_t = torch.autograd.grad(o_t, (q32, k32, v32), do)
    fin = torch.isfinite(lse_t)
    assert torch.allclose(lse_m.cpu()[fin], lse_r.cpu()[fin], atol=2e-2, rtol=1e-3)
    for name, mine, ref, truth in (("o", o_m, o_r, o_t), ("dq", dq_m, dq_r, dq_t), ("dk", dk_m, dk_r, dk_t),
                                   ("dv", dv_m, dv_r, dv_t)):
        e_mine = (mine.detach().cpu().float() - truth.detach().float()).abs().max().item()
        e_ref = (ref.detach().cpu().float() - truth.detach().float()).abs().max().item()
        assert e_mine <= 2 * e_ref + 1e-4, (name, e_mine, e_ref)


def test_headline_shape_against_reference_kernels():
    """65,536 tokens (4 of the 32 heads), chunk 128, top-k 8: the reference's kernels and this
    library's on the same inputs.  Patterns differ in < 0.5 % of the selections; on one common
    pattern O, LSE and the gradients agree to a few bf16 roundings of the largest value."""
    import flash_moba_b200 as F
    from flash_moba_b200 import ops
    from flash_moba_b200.interface import decide_lg_block_m
    torch.manual_seed(11)
    T, H, d, chunk, topk = 65536, 4, 128, 128, 8
    q, k, v, do = (torch.randn(T, H, d, device=DEV, dtype=torch.bfloat16) for _ in range(4))
    cs = cu_of([T]).to(DEV)
    km, cu_km = ops.mean_pool(k, cs, T, chunk)
    co_r, cn_r, ind_r = ref_cuda.fused_topk(q, km, cs, cs, cu_km, T, T, topk, chunk, True)
    co_m, cn_m, ind_m = F.flash_topk_varlen_func(q, k, cs, cs, T, T, topk, chunk, causal=True)
    assert torch.equal(co_m[..., 0], co_r[..., 0])
    # column lengths differ by the selections that differ: each moves one entry between two columns
    moved = (cn_m.long() - cn_r.long()).abs().sum().item() / 2
    assert moved <= 0.005 * T * H * topk, moved
    scale = d ** -0.5
    lg_m = decide_lg_block_m(topk, chunk, T, True)
    o_r, lse_r = ref_cuda.attn_fwd(q, k, v, cs, cs, T, T, co_r, cn_r, ind_r, lg_m, chunk, scale)
    dq_r, dk_r, dv_r = ref_cuda.attn_bwd(do, q, k, v, o_r, lse_r, cs, cs, T, T, co_r, cn_r, ind_r, lg_m, chunk, scale)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    o_m, lse_m, _ = F.flash_moba_attn_varlen_func(qg, kg, vg, cs, cs, T, T, co_r, cn_r, ind_r, lg_m, chunk, causal=True,
                                                  return_attn_probs=True)
    dq_m, dk_m, dv_m = torch.autograd.grad(o_m, (qg, kg, vg), do)
    assert torch.allclose(lse_m, lse_r, atol=2e-2, rtol=1e-3)
    for name, mine, ref in (("o", o_m, o_r), ("dq", dq_m, dq_r), ("dk", dk_m, dk_r), ("dv", dv_m, dv_r)):
        diff = (mine.detach().float() - ref.float()).abs().max().item()
        assert diff <= 2.0 ** -5 * ref.float().abs().max().item(), (name, diff)
