"""The CPU oracle against golden vectors produced by the reference's own pure-PyTorch code
(tests/golden/make_golden.py).  Runs without a GPU."""
import numpy as np
import pytest
import torch

from conftest import cu_of, from_bits, load_golden
from oracle import moba_oracle as O


def test_pool_matches_reference():
    g = load_golden("pool")
    for i in range(int(g["pool_n"])):
        lens, c = g[f"pool{i}_lens"].tolist(), int(g[f"pool{i}_chunk"])
        k = from_bits(g[f"pool{i}_k"])
        km, cu_km = O.mean_pool(k, cu_of(lens), c)
        ref = from_bits(g[f"pool{i}_km"])
        assert km.shape == ref.shape
        assert torch.equal(km.view(torch.int16), ref.view(torch.int16))
        assert cu_km.tolist() == np.concatenate([[0], np.cumsum([(l + c - 1) // c for l in lens])]).tolist()


def test_gate_topk_and_csc_match_reference():
    g = load_golden("gate")
    for i in range(int(g["gate_n"])):
        B, H, S, d, c, kk, causal = g[f"gate{i}_cfg"].tolist()
        q, k = from_bits(g[f"gate{i}_q"]), from_bits(g[f"gate{i}_k"])
        cs = cu_of([S] * B)
        # the reference gating test pools with .mean() in the input dtype
        # (tests/test_fused_topk.py:11-15); restate that here so the scores are identical
        km = torch.cat([torch.cat([x.mean(dim=0, keepdim=True) for x in k[b * S:(b + 1) * S].split(c, dim=0)])
                        for b in range(B)])
        cu_km, _ = O.chunk_offsets(cs, c)
        idx, val = O.gate_topk(q, km, cs, cs, cu_km, kk, c, bool(causal))
        assert np.array_equal(idx.numpy(), g[f"gate{i}_idx"]), f"case {i}"
        ncol = (S + c - 1) // c
        co, cn, ind = O.build_csc(idx, cs, kk, ncol)
        assert np.array_equal(co.numpy(), g[f"gate{i}_col_offsets"])
        assert np.array_equal(cn.numpy(), g[f"gate{i}_col_nnz"])
        assert np.array_equal(ind.numpy(), g[f"gate{i}_indices"])
        # round trip through the mask form
        mask = O.csc_to_mask(co, cn, ind, cs, S)
        assert int(mask.sum()) == int(cn.sum())


@pytest.mark.parametrize("case", [0, 1, 2, 3])
def test_attention_matches_reference(case):
    g = load_golden("attn")
    i = case
    H, Hk, d, c, kk, causal = g[f"attn{i}_cfg"].tolist()
    lq, lk = g[f"attn{i}_lq"].tolist(), g[f"attn{i}_lk"].tolist()
    B, Sq, Sk = len(lq), max(lq), max(lk)

    def unpad(x, lens):
        return torch.cat([x[b, :lens[b]] for b in range(B)], dim=0)

    q, k, v, do = [from_bits(g[f"attn{i}_{n}"]) for n in ("q", "k", "v", "do")]
    qu, ku, vu, dou = unpad(q, lq), unpad(k, lk), unpad(v, lk), unpad(do, lq)
    mask = torch.from_numpy(g[f"attn{i}_mask"])
    cq, ck = cu_of(lq), cu_of(lk)

    # pattern packing of the reference's mask -> CSC helper
    co, cn, ind = O.mask_to_csc(mask, cq, ck, c)
    assert np.array_equal(cn.numpy(), g[f"attn{i}_col_nnz"])
    assert np.array_equal(ind.numpy(), g[f"attn{i}_indices"])
    nz = cn.numpy() > 0
    assert np.array_equal(co.numpy()[nz], g[f"attn{i}_col_offsets"][nz])
    assert torch.equal(O.csc_to_mask(co, cn, ind, cq, Sq), mask & O.csc_to_mask(co, cn, ind, cq, Sq))

    for tag, lowp, tol in (("fp32", False, 1), ("lowp", True, 4)):
        qq, kk_, vv = [t.clone().requires_grad_(True) for t in (qu, ku, vu)]
        o, lse = O.attention_dense(qq, kk_, vv, cq, ck, mask, c, bool(causal), lowp=lowp)
        dq, dk, dv = torch.autograd.grad(o, (qq, kk_, vv), dou)
        for name, mine, lens in (("o", o, lq), ("dq", dq, lq), ("dk", dk, lk), ("dv", dv, lk)):
            ref = unpad(from_bits(g[f"attn{i}_{tag}_{name}"]), lens).float()
            err = (mine.detach().float() - ref).abs().max().item()
            scale = ref.abs().max().item()
            # both sides round to bf16 at the end: allow `tol` bf16 ulps of the largest value
            assert err <= tol * scale * 2 ** -8, (tag, name, err, scale)


def test_blocked_equals_dense():
    torch.manual_seed(1)
    lens, H, Hk, d, c, kk = [300, 129], 4, 2, 32, 64, 3
    T = sum(lens)
    q, k, v = torch.randn(T, H, d), torch.randn(T, Hk, d), torch.randn(T, Hk, d)
    cs = cu_of(lens)
    idx, co, cn, ind = O.moba_pattern(q, k, cs, cs, max(lens), kk, c, True)
    mask = O.csc_to_mask(co, cn, ind, cs, max(lens))
    qa, ka, va = [t.clone().requires_grad_(True) for t in (q, k, v)]
    qb, kb, vb = [t.clone().requires_grad_(True) for t in (q, k, v)]
    o1, l1 = O.attention_dense(qa, ka, va, cs, cs, mask, c, True)
    o2, l2 = O.attention_blocked(qb, kb, vb, cs, cs, idx, c, True, rows_per_step=50)
    assert torch.allclose(o1, o2, atol=2e-5, rtol=1e-5)
    assert torch.allclose(l1, l2, atol=2e-5, rtol=1e-5)
    do = torch.randn_like(o1)
    g1 = torch.autograd.grad(o1, (qa, ka, va), do)
    g2 = torch.autograd.grad(o2, (qb, kb, vb), do)
    for a, b in zip(g1, g2):
        assert torch.allclose(a, b, atol=1e-4, rtol=1e-4)


def test_c1_end_to_end_matches_reference():
    """The reference's CPU-runnable configuration (2 sequences of 1024 and 2048 tokens, 8 heads, d 64, chunk 128, top-k 4): the oracle's whole path against the reference's
    pure-PyTorch MoBA (fp32, seed 0)."""
    g = load_golden("c1")
    torch.manual_seed(0)
    lens, H, d, c, kk = [1024, 2048], 8, 64, 128, 4
    T = sum(lens)
    q, k, v = torch.randn(T, H, d), torch.randn(T, H, d), torch.randn(T, H, d)
    cs = cu_of(lens)
    out, lse, idx, _ = O.moba_forward(q, k, v, cs, cs, max(lens), max(lens), c, kk, True, blocked=True)
    assert np.array_equal(idx.numpy(), g["c1_idx"].astype(np.int32))
    rows = g["c1_rows"]
    assert np.allclose(out[rows].numpy(), g["c1_o"], atol=2e-5, rtol=1e-5)


def test_tie_rule_higher_index_first():
    gate = np.zeros((1, 4, 6), dtype=np.float32)       # every score equal
    idx, _ = O.select_topk(gate, 3, 1, 4, 6, False)
    assert idx[0, 0].tolist() == [5, 4, 3]
    gate6 = np.zeros((1, 6, 3), dtype=np.float32)
    idx, _ = O.select_topk(gate6, 3, 2, 6, 6, True)
    assert idx[5, 0].tolist() == [2, 1, 0]            # row 5: own chunk 2 first, then 1, 0
    assert idx[0, 0].tolist() == [0, -1, -1]
