"""GPU parity tests: every CUDA stage, called through the C ABI, against the CPU oracle and
the golden vectors of the reference.  Mirrors the reference's own test files
(tests/test_triton_mean_pool.py, test_fused_topk.py, test_fused_topk_epilogue.py,
test_varlen_sort.py, test_moba_attn.py) with their tolerances written out here."""
import math

import numpy as np
import pytest
import torch

from conftest import cu_of, from_bits, load_golden
from oracle import moba_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    from flash_moba_b200 import ops
    return ops


# ----------------------------------------------------------------------------- stage P
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("batch,max_seqlen,heads,d,chunk", [
    (1, 512, 4, 64, 32), (8, 512, 4, 128, 128), (8, 2048, 12, 128, 256), (1, 2048, 4, 256, 512),
    (8, 512, 12, 64, 64), (4, 128, 4, 32, 256), (16, 8, 4, 32, 4), (3, 700, 2, 96, 128),
    (64, 300, 2, 64, 64), (65, 300, 2, 64, 64), (200, 90, 2, 128, 32),   # chunk offsets inside the pool kernel up to 64 sequences, by their own launch above
])
def test_mean_pool_vs_oracle(batch, max_seqlen, heads, d, chunk, dtype):
    # tolerance of the reference test: atol 1e-2, rtol 0 (tests/test_triton_mean_pool.py:63-64)
    g = torch.Generator().manual_seed(42)
    lens = torch.randint(0, max_seqlen, (batch,), generator=g).tolist()
    k = torch.randn(sum(lens), heads, d, generator=g).to(dtype)
    cu = cu_of(lens)
    ref, cu_km_ref = O.mean_pool(k, cu, chunk)
    km, cu_km = _ops().mean_pool(k.to(DEV), cu.to(DEV), max_seqlen, chunk)
    assert cu_km.cpu().tolist() == cu_km_ref.tolist()
    n = int(cu_km_ref[-1])
    assert km.shape[0] >= n
    got = km[:n].cpu().float()
    assert torch.allclose(got, ref.float(), atol=1e-2, rtol=0)
    # in practice the kernel is within one rounding of the fp32 mean
    assert (got - ref.float()).abs().max().item() <= 2 ** -7 * max(ref.float().abs().max().item(), 1e-3)


def test_mean_pool_golden_and_public_form():
    import flash_moba_b200 as F
    g = load_golden("pool")
    for i in range(int(g["pool_n"])):
        lens, c = g[f"pool{i}_lens"].tolist(), int(g[f"pool{i}_chunk"])
        k = from_bits(g[f"pool{i}_k"])
        ref = from_bits(g[f"pool{i}_km"])
        km, cu_km, mx = F.flash_topk_mean_pool(k.to(DEV), cu_of(lens).to(DEV), max(lens), c)
        assert km.shape == ref.shape
        assert mx == (max(lens) + c - 1) // c
        assert torch.allclose(km.cpu().float(), ref.float(), atol=1e-2, rtol=0)


def test_mean_pool_strided_input():
    torch.manual_seed(0)
    kv = torch.randn(300, 2, 4, 64).bfloat16()       # packed (token, 2, head, d): k is a strided view
    k = kv[:, 0]
    cu = cu_of([100, 200])
    ref, _ = O.mean_pool(k.contiguous(), cu, 64)
    km, cu_km = _ops().mean_pool(kv.to(DEV)[:, 0], cu.to(DEV), 200, 64)
    assert torch.allclose(km[: ref.shape[0]].cpu().float(), ref.float(), atol=1e-2, rtol=0)


# ----------------------------------------------------------------------------- stage G
def _gate_case(B, H, Hk, S, d, chunk, topk, causal, dtype=torch.bfloat16, lens_q=None, lens_k=None, seed=0,
               integer=False):
    g = torch.Generator().manual_seed(seed)
    lens_k = lens_k or [S] * B
    lens_q = lens_q or lens_k
    if integer:   # small integers: every fp32 dot product is exact in any summation order
        q = torch.randint(-2, 3, (sum(lens_q), H, d), generator=g).to(dtype)
        k = (torch.randint(-2, 3, (sum(lens_k), Hk, d), generator=g) * 1.0).to(dtype)
    else:
        q = torch.randn(sum(lens_q), H, d, generator=g).to(dtype)
        k = torch.randn(sum(lens_k), Hk, d, generator=g).to(dtype)
    return q, k, cu_of(lens_q), cu_of(lens_k), max(lens_q), max(lens_k)


@pytest.mark.parametrize("topk", [1, 2, 4, 8, 16, 24, 32, 33, 64])
@pytest.mark.parametrize("chunk", [1, 16, 32])
@pytest.mark.parametrize("causal", [True, False])
def test_gate_topk_vs_oracle(topk, chunk, causal):
    # reference bar: index mismatch ratio < 0.5 % (tests/test_fused_topk.py:251-254)
    B, H, S, d = (2, 8, 256, 64) if chunk > 1 else (1, 2, 128, 64)
    q, k, cq, ck, mq, mk = _gate_case(B, H, H, S, d, chunk, topk, causal)
    ops = _ops()
    km, cu_km = ops.mean_pool(k.to(DEV), ck.to(DEV), mk, chunk)
    idx, val = ops.gate_topk(q.to(DEV), km, cq.to(DEV), ck.to(DEV), cu_km, mq, mk, topk, chunk, causal,
                             return_values=True)
    n = int(cu_km[-1])
    ref_idx, ref_val = O.gate_topk(q, km[:n].cpu(), cq, ck, cu_km.cpu(), topk, chunk, causal)
    mism = (idx.cpu() != ref_idx).float().mean().item()
    assert mism < 0.005, mism
    fin = torch.isfinite(ref_val) & (idx.cpu() == ref_idx)
    assert torch.allclose(val.cpu()[fin], ref_val[fin], atol=1e-3, rtol=1e-4)


@pytest.mark.parametrize("cfg", [
    dict(B=2, H=4, Hk=4, S=384, d=64, chunk=32, topk=4, causal=True),
    dict(B=1, H=4, Hk=2, S=1000, d=128, chunk=64, topk=8, causal=True),
    dict(B=2, H=2, Hk=1, S=300, d=128, chunk=16, topk=40, causal=False),
    dict(B=1, H=2, Hk=2, S=512, d=256, chunk=32, topk=3, causal=True),
    dict(B=1, H=4, Hk=2, S=2500, d=256, chunk=8, topk=8, causal=True),      # three score tiles at head dim 256
    dict(B=2, H=2, Hk=2, S=1100, d=256, chunk=4, topk=16, causal=False),    # lists of 16
    dict(B=3, H=2, Hk=2, S=0, d=64, chunk=64, topk=4, causal=True, lens_q=[10, 200, 64], lens_k=[300, 200, 70]),
    dict(B=2, H=2, Hk=2, S=0, d=64, chunk=32, topk=4, causal=True, lens_q=[200, 64], lens_k=[100, 64]),
])
def test_gate_topk_exact_on_identical_scores(cfg):
    """Integer-valued inputs make every fp32 score exact, so scores are identical on both
    sides and ties are frequent: indices must then be bit-exact, tie rule included."""
    q, k, cq, ck, mq, mk = _gate_case(integer=True, **cfg)
    ops = _ops()
    chunk, topk, causal = cfg["chunk"], cfg["topk"], cfg["causal"]
    # power-of-two chunk lengths keep the centroids exact too; ragged tails may round, so
    # the oracle is fed the kernel's own centroids
    km, cu_km = ops.mean_pool(k.to(DEV), ck.to(DEV), mk, chunk)
    idx, val = ops.gate_topk(q.to(DEV), km, cq.to(DEV), ck.to(DEV), cu_km, mq, mk, topk, chunk, causal,
                             return_values=True)
    n = int(cu_km[-1])
    ref_idx, ref_val = O.gate_topk(q, km[:n].cpu(), cq, ck, cu_km.cpu(), topk, chunk, causal)
    assert torch.equal(idx.cpu(), ref_idx)
    assert torch.equal(val.cpu(), ref_val)


def test_gate_and_csc_golden():
    g = load_golden("gate")
    ops = _ops()
    for i in range(int(g["gate_n"])):
        B, H, S, d, c, kk, causal = g[f"gate{i}_cfg"].tolist()
        q, k = from_bits(g[f"gate{i}_q"]), from_bits(g[f"gate{i}_k"])
        cs = cu_of([S] * B).to(DEV)
        km, cu_km = ops.mean_pool(k.to(DEV), cs, S, c)
        idx, _ = ops.gate_topk(q.to(DEV), km, cs, cs, cu_km, S, S, kk, c, bool(causal))
        ref = torch.from_numpy(g[f"gate{i}_idx"])
        mism = (idx.cpu() != ref).float().mean().item()
        assert mism < 0.005, (i, mism)
        # pattern of the REFERENCE's lists must come out bit-exact
        ncol = (S + c - 1) // c
        co, cn, ind = ops.build_csc(ref.to(DEV), cs, S, ncol)
        assert np.array_equal(co.cpu().numpy(), g[f"gate{i}_col_offsets"])
        assert np.array_equal(cn.cpu().numpy(), g[f"gate{i}_col_nnz"])
        assert np.array_equal(ind.cpu().numpy(), g[f"gate{i}_indices"])


# --------------------------------------------------------------------------- stages O/E/S
@pytest.mark.parametrize("lens,H,topk,chunk", [
    ([128], 4, 4, 16), ([256, 256], 8, 8, 32), ([1000, 37, 0, 513], 3, 5, 64), ([5000], 2, 16, 4),
    ([3000, 1500], 2, 64, 16),
])
def test_build_csc_exact(lens, H, topk, chunk):
    # exact equality, as tests/test_fused_topk_epilogue.py:144-145
    g = torch.Generator().manual_seed(3)
    T, ncol = sum(lens), (max(lens) + chunk - 1) // chunk
    idx = torch.full((T, H, topk), -1, dtype=torch.int32)
    r = 0
    for L in lens:
        for t in range(L):
            navail = t // chunk + 1
            for h in range(H):
                kk = min(topk, navail)
                sel = torch.randperm(navail, generator=g)[:kk]
                idx[r, h, :kk] = sel.to(torch.int32)
            r += 1
    cq = cu_of(lens)
    ref = O.build_csc(idx, cq, topk, ncol)
    ops = _ops()
    for layout in ("row_major", "head_major"):
        dev_idx = idx.to(DEV) if layout == "row_major" else idx.to(DEV).permute(1, 0, 2).contiguous().permute(1, 0, 2)
        got = ops.build_csc(dev_idx, cq.to(DEV), max(lens), ncol)
        for a, b in zip(got, ref):
            assert torch.equal(a.cpu(), b), layout


def test_varlen_sort_exact():
    # tests/test_varlen_sort.py:55,83 — exact, including INT32 extremes
    g = torch.Generator().manual_seed(0)
    seg = torch.randint(0, 3000, (37,), generator=g)
    seg[5] = 0
    seg[7] = 70000
    starts = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(seg, 0)[:-1]])
    ends = starts + seg
    n = int(seg.sum())
    src = torch.randint(-2 ** 31, 2 ** 31 - 1, (n,), generator=g, dtype=torch.int64).to(torch.int32)
    src[0], src[1] = -2 ** 31, 2 ** 31 - 1
    ref = torch.zeros_like(src)
    for s, e in zip(starts.tolist(), ends.tolist()):
        ref[s:e] = torch.sort(src[s:e])[0]
    got = _ops().varlen_sort(starts.to(DEV), ends.to(DEV), src.to(DEV))
    assert torch.equal(got.cpu(), ref)


# ----------------------------------------------------------------------------- stages F/B
def _attn_check(q, k, v, do, cq, ck, mask, chunk, causal, engine, pattern=None, check_grad=True):
    """O within 2x, dQ/dK/dV within 3x of the low-precision PyTorch error against the fp32
    truth (tests/test_moba_attn.py:317,326-328), plus a small absolute floor."""
    import flash_moba_b200 as F
    ops = _ops()
    ops.set_engine(engine)
    try:
        lq = (cq[1:] - cq[:-1]).tolist()
        lk = (ck[1:] - ck[:-1]).tolist()
        co, cn, ind = pattern if pattern is not None else O.mask_to_csc(mask, cq, ck, chunk)
        if ind.numel() == 0:
            ind = torch.zeros(1, dtype=torch.int32)
        qd, kd, vd = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
        out, lse, _ = F.flash_moba_attn_varlen_func(
            qd, kd, vd, cq.to(DEV), ck.to(DEV), max(lq), max(lk), co.to(DEV), cn.to(DEV), ind.to(DEV),
            128, chunk, causal=causal, return_attn_probs=True)
        refs = {}
        for tag, lowp in (("fp32", False), ("lowp", True)):
            qq, kk, vv = [t.clone().requires_grad_(True) for t in (q, k, v)]
            o, l = O.attention_dense(qq, kk, vv, cq, ck, mask, chunk, causal, lowp=lowp)
            grads = torch.autograd.grad(o, (qq, kk, vv), do) if check_grad else (None,) * 3
            refs[tag] = (o.detach().float(), l, *[x.float() if x is not None else None for x in grads])
        o_ref, l_ref = refs["fp32"][0], refs["fp32"][1]
        e_pt = (refs["lowp"][0] - o_ref).abs().max().item()
        e = (out.detach().cpu().float() - o_ref).abs().max().item()
        assert e <= 2 * e_pt + 1e-4, ("out", e, e_pt)
        fin = torch.isfinite(l_ref)
        assert torch.equal(torch.isfinite(lse.cpu()), fin)
        assert torch.allclose(lse.cpu()[fin], l_ref[fin], atol=2e-2, rtol=1e-3)
        assert torch.all(lse.cpu()[~fin] == float("inf"))
        if check_grad:
            dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), do.to(DEV))
            for name, mine, j in (("dq", dq, 2), ("dk", dk, 3), ("dv", dv, 4)):
                e_pt = (refs["lowp"][j] - refs["fp32"][j]).abs().max().item()
                e = (mine.cpu().float() - refs["fp32"][j]).abs().max().item()
                assert e <= 3 * e_pt + 1e-4, (name, e, e_pt)
    finally:
        ops.set_engine(1)


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("case", [0, 1, 2, 3])
def test_attention_golden_patterns(case, engine):
    g = load_golden("attn")
    i = case
    H, Hk, d, c, kk, causal = g[f"attn{i}_cfg"].tolist()
    lq, lk = g[f"attn{i}_lq"].tolist(), g[f"attn{i}_lk"].tolist()
    B = len(lq)

    def unpad(x, lens):
        return torch.cat([x[b, :lens[b]] for b in range(B)], dim=0).contiguous()

    q, k, v, do = [from_bits(g[f"attn{i}_{n}"]) for n in ("q", "k", "v", "do")]
    q, k, v, do = unpad(q, lq), unpad(k, lk), unpad(v, lk), unpad(do, lq)
    mask = torch.from_numpy(g[f"attn{i}_mask"])
    pattern = tuple(torch.from_numpy(g[f"attn{i}_{n}"]) for n in ("col_offsets", "col_nnz", "indices"))
    _attn_check(q, k, v, do, cu_of(lq), cu_of(lk), mask, c, bool(causal), engine, pattern=pattern)
    # the reference's golden outputs themselves
    import flash_moba_b200 as F
    co, cn, ind = pattern
    out = F.flash_moba_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu_of(lq).to(DEV), cu_of(lk).to(DEV),
                                        max(lq), max(lk), co.to(DEV), cn.to(DEV), ind.to(DEV), 128, c,
                                        causal=bool(causal))
    ref = unpad(from_bits(g[f"attn{i}_fp32_o"]), lq).float()
    pt = unpad(from_bits(g[f"attn{i}_lowp_o"]), lq).float()
    assert (out.cpu().float() - ref).abs().max().item() <= 2 * (pt - ref).abs().max().item() + 1e-4


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("mha", ["mha", "gqa", "mqa"])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("d,chunk", [(64, 64), (128, 64), (128, 128), (64, 128)])
@pytest.mark.parametrize("lens_q,lens_k", [
    ([113, 203], [113, 203]), ([1, 128], [147, 217]), ([256, 64, 0], [256, 64, 30]), ([1023], [1024]),
])
def test_attention_random_patterns(lens_q, lens_k, d, chunk, causal, mha, engine):
    # the reference's grid in miniature (tests/test_moba_attn.py:36-70, topk 4, random pattern)
    torch.manual_seed(0)
    H = 4
    Hk = {"mha": 4, "gqa": 2, "mqa": 1}[mha]
    Tq, Tk = sum(lens_q), sum(lens_k)
    q = torch.randn(Tq, H, d).bfloat16()
    k = torch.randn(Tk, Hk, d).bfloat16()
    v = torch.randn(Tk, Hk, d).bfloat16()
    do = torch.randn(Tq, H, d).bfloat16()
    cq, ck = cu_of(lens_q), cu_of(lens_k)
    B, Sq, ncol = len(lens_q), max(lens_q), (max(lens_k) + chunk - 1) // chunk
    mask = torch.zeros(B, H, Sq, ncol, dtype=torch.bool)
    g = torch.Generator().manual_seed(1)
    for b in range(B):
        for h in range(H):
            for r in range(lens_q[b]):
                end = lens_k[b] - (lens_q[b] - r - 1) if causal else lens_k[b]
                nb = max(0, math.ceil(end / chunk))
                if nb > 0:
                    sel = torch.randperm(nb - 1, generator=g)[:3] if nb > 1 else torch.zeros(0, dtype=torch.long)
                    mask[b, h, r, sel] = True
                    mask[b, h, r, nb - 1] = True
    _attn_check(q, k, v, do, cq, ck, mask, chunk, causal, engine)


@pytest.mark.parametrize("engine", [0, 1])
def test_attention_rows_with_more_than_32_partials(engine):
    """A dense pattern (every row attends every one of 40 chunks) takes the generic merge path
    next to the fast one (rows with <= 32 partials)."""
    torch.manual_seed(0)
    lens_q, lens_k, H, Hk, d, chunk = [70, 33], [2560, 1000], 2, 1, 64, 64
    q = torch.randn(sum(lens_q), H, d).bfloat16()
    k = torch.randn(sum(lens_k), Hk, d).bfloat16()
    v = torch.randn(sum(lens_k), Hk, d).bfloat16()
    do = torch.randn(sum(lens_q), H, d).bfloat16()
    ncol = (max(lens_k) + chunk - 1) // chunk
    mask = torch.zeros(2, H, max(lens_q), ncol, dtype=torch.bool)
    mask[0, :, :70, :40] = True
    mask[1, :, :33, :16] = True
    _attn_check(q, k, v, do, cu_of(lens_q), cu_of(lens_k), mask, chunk, False, engine)


def _random_mask(lens_q, lens_k, H, chunk, causal, picks, seed=1):
    B, Sq, ncol = len(lens_q), max(lens_q), (max(lens_k) + chunk - 1) // chunk
    mask = torch.zeros(B, H, Sq, ncol, dtype=torch.bool)
    g = torch.Generator().manual_seed(seed)
    for b in range(B):
        for h in range(H):
            for r in range(lens_q[b]):
                end = lens_k[b] - (lens_q[b] - r - 1) if causal else lens_k[b]
                nb = max(0, math.ceil(end / chunk))
                if nb > 0:
                    sel = torch.randperm(nb - 1, generator=g)[:picks] if nb > 1 else torch.zeros(0, dtype=torch.long)
                    mask[b, h, r, sel] = True
                    mask[b, h, r, nb - 1] = True
    return mask


@pytest.mark.parametrize("chunk,d,max_picks", [(64, 64, 31), (64, 128, 31), (128, 128, 20), (256, 128, 15), (256, 64, 15),
                                               (64, 256, 31), (128, 256, 20)])
def test_attention_rows_with_9_to_32_partials(chunk, d, max_picks):
    """Rows with every count of selected chunks from 1 to max_picks + 1 next to each other: the merge
    of a row's partials goes through the 8-lane stage, the warp-per-row stage (9..32 partials; a
    256-key chunk gives two partials per selected chunk) or the generic stage, row by row."""
    torch.manual_seed(0)
    lens, H, Hk = [chunk * (max_picks + 3) + 17], 2, 1
    T = sum(lens)
    q = torch.randn(T, H, d).bfloat16()
    k = torch.randn(T, Hk, d).bfloat16()
    v = torch.randn(T, Hk, d).bfloat16()
    do = torch.randn(T, H, d).bfloat16()
    ncol = (T + chunk - 1) // chunk
    mask = torch.zeros(1, H, T, ncol, dtype=torch.bool)
    g = torch.Generator().manual_seed(5)
    for h in range(H):
        for r in range(T):
            own = r // chunk
            picks = int(torch.randint(0, max_picks + 1, (1,), generator=g))
            if own > 0 and picks > 0:
                mask[0, h, r, torch.randperm(own, generator=g)[:picks]] = True
            mask[0, h, r, own] = True
    _attn_check(q, k, v, do, cu_of(lens), cu_of(lens), mask, chunk, True, 1)


@pytest.mark.parametrize("chunk,d,causal,hk", [(64, 64, True, 4), (128, 128, True, 2), (128, 128, False, 1),
                                               (256, 128, True, 2), (192, 64, True, 4)])
def test_attention_many_work_items_per_cta(chunk, d, causal, hk):
    """Many short, ragged sequences (some empty, some ending inside a key block): the persistent
    CTAs of the main kernels each run through several work items, among them items whose column is
    empty and key blocks that start past a sequence's end, with the next item decoded and its K/V
    staged while the current one is still being worked on."""
    torch.manual_seed(3)
    g = torch.Generator().manual_seed(11)
    lens = [int(x) for x in torch.randint(0, 900, (40,), generator=g)]
    lens[3] = 0
    lens[17] = chunk            # ends exactly on a chunk boundary
    lens[18] = chunk + 1
    H = 4
    T = sum(lens)
    q = torch.randn(T, H, d).bfloat16()
    k = torch.randn(T, hk, d).bfloat16()
    v = torch.randn(T, hk, d).bfloat16()
    do = torch.randn(T, H, d).bfloat16()
    mask = _random_mask(lens, lens, H, chunk, causal, 2, seed=4)
    _attn_check(q, k, v, do, cu_of(lens), cu_of(lens), mask, chunk, causal, 1)


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("chunk,d", [(256, 128), (192, 128), (256, 64), (320, 64)])
def test_attention_chunks_wider_than_a_key_block(chunk, d, engine):
    """Chunks of 192..320 keys are processed as several 64- or 128-key blocks per column
    (the 512K-token benchmark configuration uses chunk 256)."""
    torch.manual_seed(0)
    lens, H, Hk = [700, 301], 4, 2
    T = sum(lens)
    q = torch.randn(T, H, d).bfloat16()
    k = torch.randn(T, Hk, d).bfloat16()
    v = torch.randn(T, Hk, d).bfloat16()
    do = torch.randn(T, H, d).bfloat16()
    mask = _random_mask(lens, lens, H, chunk, True, 2)
    _attn_check(q, k, v, do, cu_of(lens), cu_of(lens), mask, chunk, True, engine)


@pytest.mark.parametrize("d", [128, 256])
def test_attention_in_passes_is_bit_identical(monkeypatch, d):
    """A workspace too small for all heads makes the library walk the heads in passes (whole
    kv-head groups); results must not change by a bit."""
    import flash_moba_b200 as F
    torch.manual_seed(0)
    lens, H, Hk, c, kk = [600, 424], 8, 4, 128, 3
    T = sum(lens)
    q = torch.randn(T, H, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, Hk, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, Hk, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    cs = cu_of(lens).to(DEV)
    res = []
    for gb in ("24", "0.004" if d == 128 else "0.008"):
        monkeypatch.setenv("FMB_WORKSPACE_GB", gb)
        out = F.flash_moba_varlen_func(q, k, v, cs, cs, max(lens), max(lens), c, kk, causal=True)
        grads = torch.autograd.grad(out, (q, k, v), torch.ones_like(out))
        res.append((out.detach().clone(), *[x.clone() for x in grads]))
    for a, b in zip(*res):
        assert torch.equal(a, b)


@pytest.mark.parametrize("engine", [0, 1])
def test_attention_fp16(engine):
    torch.manual_seed(0)
    lens = [200, 130]
    T, H, d, chunk = sum(lens), 2, 64, 64
    q, k, v, do = [torch.randn(T, H, d).half() for _ in range(4)]
    cq = cu_of(lens)
    idx, co, cn, ind = O.moba_pattern(q.float(), k.float(), cq, cq, max(lens), 2, chunk, True)
    mask = O.csc_to_mask(co, cn, ind, cq, max(lens))
    _attn_check(q, k, v, do, cq, cq, mask, chunk, True, engine, pattern=(co, cn, ind))


@pytest.mark.parametrize("d", [32, 40, 96, 100, 128])
def test_attention_head_dims_padded_to_64_or_128(d):
    """Head dimensions below 128 that the kernels are not built for run zero-padded to 64 / 128
    (the reference's grid has 32, 96, ...: tests/test_moba_attn.py); softmax scale from the true d."""
    torch.manual_seed(d)
    lens = [333, 128]
    T, H, chunk = sum(lens), 2, 64
    q, k, v, do = [torch.randn(T, H, d).bfloat16() for _ in range(4)]
    cq = cu_of(lens)
    idx, co, cn, ind = O.moba_pattern(q.float(), k.float(), cq, cq, max(lens), 3, chunk, True)
    mask = O.csc_to_mask(co, cn, ind, cq, max(lens))
    _attn_check(q, k, v, do, cq, cq, mask, chunk, True, 1, pattern=(co, cn, ind))


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d,chunk,causal,hk", [(160, 64, True, 2), (192, 128, True, 4), (224, 128, False, 1),
                                               (256, 64, True, 1), (256, 256, True, 4), (136, 192, True, 2)])
def test_attention_head_dims_above_128(d, chunk, causal, hk, dtype, engine):
    """Head dimensions above 128 (the reference dispatches up to 256 and tests 160,
    tests/test_moba_attn.py:48): run at 192 / 256, zero-padded where they fall between, on both
    engines; ragged sequences, len_q != len_k, GQA / MQA, chunks of 1 to 4 key blocks."""
    torch.manual_seed(d + chunk)
    lens_q, lens_k = [190, 77, 300], [250, 77, 300]
    H = 4
    q = torch.randn(sum(lens_q), H, d).to(dtype)
    k = torch.randn(sum(lens_k), hk, d).to(dtype)
    v = torch.randn(sum(lens_k), hk, d).to(dtype)
    do = torch.randn(sum(lens_q), H, d).to(dtype)
    cq, ck = cu_of(lens_q), cu_of(lens_k)
    mask = _random_mask(lens_q, lens_k, H, chunk, causal, 3, seed=d)
    _attn_check(q, k, v, do, cq, ck, mask, chunk, causal, engine)


# ----------------------------------------------------------------------------- whole path
def test_c1_end_to_end():
    """The reference's CPU-runnable configuration (sequences of 1024 and 2048 tokens, 8 heads, d 64, chunk 128, top-k 4) through the public API: top-k indices against the reference's
    golden lists (mismatch < 0.5 %), forward output against the oracle run on the kernel's
    own pattern (so a flipped near-tie does not pose as numeric error)."""
    import flash_moba_b200 as F
    g = load_golden("c1")
    torch.manual_seed(0)
    lens, H, d, c, kk = [1024, 2048], 8, 64, 128, 4
    T = sum(lens)
    q32, k32, v32 = torch.randn(T, H, d), torch.randn(T, H, d), torch.randn(T, H, d)
    q, k, v = q32.bfloat16(), k32.bfloat16(), v32.bfloat16()
    cs = cu_of(lens)
    csd = cs.to(DEV)
    ops = _ops()
    km, cu_km = ops.mean_pool(k.to(DEV), csd, max(lens), c)
    idx, _ = ops.gate_topk(q.to(DEV), km, csd, csd, cu_km, max(lens), max(lens), kk, c, True)
    ref_idx = torch.from_numpy(g["c1_idx"].astype(np.int32))
    # the golden lists come from fp32 inputs; bf16 inputs move a few near-ties
    mism = (idx.cpu() != ref_idx).float().mean().item()
    assert mism < 0.02, mism
    # against the oracle fed the same bf16 inputs: the reference's 0.5 % bar
    o_idx, _ = O.gate_topk(q, O.mean_pool(k, cs, c)[0], cs, cs, O.chunk_offsets(cs, c)[0], kk, c, True)
    assert (idx.cpu() != o_idx).float().mean().item() < 0.005

    co, cn, ind = F.flash_topk_varlen_func(q.to(DEV), k.to(DEV), csd, csd, max(lens), max(lens), kk, c, causal=True)
    rco, rcn, rind = O.build_csc(idx.cpu(), cs, kk, (max(lens) + c - 1) // c)
    assert torch.equal(co.cpu(), rco) and torch.equal(cn.cpu(), rcn) and torch.equal(ind.cpu(), rind)

    out = F.flash_moba_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), csd, csd, max(lens), max(lens), c, kk, causal=True)
    truth, _ = O.attention_blocked(q.float(), k.float(), v.float(), cs, cs, idx.cpu(), c, True)
    mask = O.csc_to_mask(rco, rcn, rind, cs, max(lens))
    lowp, _ = O.attention_dense(q, k, v, cs, cs, mask, c, True, lowp=True)
    e_pt = (lowp.float() - truth).abs().max().item()
    e = (out.cpu().float() - truth).abs().max().item()
    assert e <= 2 * e_pt + 1e-4, (e, e_pt)
    # and the reference's golden O rows where the pattern of the row is unchanged
    rows = torch.from_numpy(g["c1_rows"])
    same = (idx.cpu()[rows] == ref_idx[rows]).all(dim=-1).all(dim=-1)
    diff = (out.cpu().float()[rows][same] - torch.from_numpy(g["c1_o"])[same]).abs().max().item()
    assert diff <= 0.05, diff


def test_row_lists_handed_from_forward_to_backward(monkeypatch):
    """The backward call takes over the pattern's slot / row lists from the forward call (single-pass
    calls): same gradients bit for bit, fewer launches; a multi-pass workspace falls back to
    building its own."""
    import flash_moba_b200 as F
    from flash_moba_b200 import _lib
    torch.manual_seed(0)
    lens, H, Hk, d, chunk, topk = [700, 333], 4, 2, 128, 128, 3
    T = sum(lens)
    cu = cu_of(lens).to(DEV)
    q, k, v, do = (torch.randn(T, h, d, device=DEV).bfloat16() for h in (H, Hk, Hk, H))

    def run():
        qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
        n0 = _lib.lib.fmb_launch_count()
        out = F.flash_moba_varlen_func(qd, kd, vd, cu, cu, max(lens), max(lens), chunk, topk, causal=True)
        grads = torch.autograd.grad(out, (qd, kd, vd), do)
        torch.cuda.synchronize()
        return (out.detach(),) + grads, _lib.lib.fmb_launch_count() - n0

    monkeypatch.setenv("FMB_SHARE_LISTS", "0")
    ref, n_ref = run()
    monkeypatch.setenv("FMB_SHARE_LISTS", "1")
    got, n_got = run()
    for a, b in zip(ref, got):
        assert torch.equal(a, b)
    assert n_got < n_ref
    monkeypatch.setenv("FMB_WORKSPACE_GB", "0.000001")     # forces one kv-head group per pass
    multi, n_multi = run()
    for a, b in zip(ref, multi):
        assert torch.equal(a, b)


def test_lists_of_a_caller_built_pattern_and_launch_counts(monkeypatch):
    """A pattern that did not come from the library's own builder (here: rebuilt by the oracle from
    the same lists) takes the general path: slot and row lists built by the forward call and handed
    to the backward call.  Same results bit for bit as the library's own pattern, which needs no
    list-building launches at all: a whole step (pool, gating, pattern, forward, backward) is at
    most 12 launches."""
    import flash_moba_b200 as F
    from flash_moba_b200 import _lib
    torch.manual_seed(1)
    lens, H, Hk, d, chunk, topk = [900, 515], 4, 2, 128, 128, 4
    T = sum(lens)
    cu = cu_of(lens).to(DEV)
    q, k, v, do = (torch.randn(T, h, d, device=DEV).bfloat16() for h in (H, Hk, Hk, H))
    mx = max(lens)

    def attn(pattern):
        qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
        n0 = _lib.lib.fmb_launch_count()
        out = F.flash_moba_attn_varlen_func(qd, kd, vd, cu, cu, mx, mx, *pattern, 128, chunk, causal=True)
        grads = torch.autograd.grad(out, (qd, kd, vd), do)
        torch.cuda.synchronize()
        return (out.detach(),) + grads, _lib.lib.fmb_launch_count() - n0

    own = F.flash_topk_varlen_func(q, k, cu, cu, mx, mx, topk, chunk, causal=True)
    got_own, n_own = attn(own)
    copy = tuple(t.clone() for t in own)              # same pattern, unknown to the library
    got_copy, n_copy = attn(copy)
    for a, b in zip(got_own, got_copy):
        assert torch.equal(a, b)
    assert n_own == 5, n_own                          # forward main + combine, dO.O, backward main + combine
    assert n_own < n_copy
    monkeypatch.setenv("FMB_SHARE_LISTS", "0")
    got_off, n_off = attn(copy)
    for a, b in zip(got_own, got_off):
        assert torch.equal(a, b)
    assert n_copy < n_off
    monkeypatch.setenv("FMB_SHARE_LISTS", "1")
    n0 = _lib.lib.fmb_launch_count()
    qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = F.flash_moba_varlen_func(qd, kd, vd, cu, cu, mx, mx, chunk, topk, causal=True)
    torch.autograd.grad(out, (qd, kd, vd), do)
    torch.cuda.synchronize()
    assert _lib.lib.fmb_launch_count() - n0 <= 10


def test_determinism_and_autograd_through_public_api():
    import flash_moba_b200 as F
    torch.manual_seed(0)
    lens = [500, 300]
    T, H, Hk, d, c, kk = sum(lens), 4, 2, 128, 64, 3
    q = torch.randn(T, H, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(T, Hk, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(T, Hk, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    cs = cu_of(lens).to(DEV)
    res = []
    for _ in range(2):
        out = F.flash_moba_varlen_func(q, k, v, cs, cs, max(lens), max(lens), c, kk, causal=True)
        grads = torch.autograd.grad(out, (q, k, v), torch.ones_like(out))
        res.append((out.detach().clone(), *[x.clone() for x in grads]))
    for a, b in zip(*res):
        assert torch.equal(a, b)          # bit-identical run to run (no floating-point atomics)


def test_public_api_at_head_dim_160():
    """The whole path (pool, gating, pattern, attention forward and backward) at a head dimension
    above 128, through the fused public function: the pattern against the oracle on the same
    inputs, O and the gradients against the dense fp32 evaluation of that pattern; two runs
    bit-identical."""
    import flash_moba_b200 as F
    torch.manual_seed(5)
    lens = [700, 333]
    T, H, Hk, d, c, kk = sum(lens), 4, 2, 160, 128, 3
    q, k, v, do = [torch.randn(T, h, d).bfloat16() for h in (H, Hk, Hk, H)]
    cs = cu_of(lens)
    co, cn, ind = F.flash_topk_varlen_func(q.to(DEV), k.to(DEV), cs.to(DEV), cs.to(DEV), max(lens), max(lens), kk, c,
                                           causal=True)
    idx_ref, co_ref, cn_ref, ind_ref = O.moba_pattern(q.float(), k.float(), cs, cs, max(lens), kk, c, True)
    mine = O.csc_to_mask(co.cpu(), cn.cpu(), ind.cpu(), cs, max(lens))
    want = O.csc_to_mask(co_ref, cn_ref, ind_ref, cs, max(lens))
    assert (mine != want).float().mean().item() < 0.005 * kk / mine.shape[-1] * 2   # < 0.5 % of the selections
    res = []
    for _ in range(2):
        qd, kd, vd = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
        out = F.flash_moba_varlen_func(qd, kd, vd, cs.to(DEV), cs.to(DEV), max(lens), max(lens), c, kk, causal=True)
        res.append((out.detach(), *torch.autograd.grad(out, (qd, kd, vd), do.to(DEV))))
    for a, b in zip(*res):
        assert torch.equal(a, b)
    refs = {}
    for tag, lowp in (("fp32", False), ("lowp", True)):
        qq, kk_, vv = [t.clone().requires_grad_(True) for t in (q, k, v)]
        o, _ = O.attention_dense(qq, kk_, vv, cs, cs, mine, c, True, lowp=lowp)
        refs[tag] = (o.detach().float(), *[g.float() for g in torch.autograd.grad(o, (qq, kk_, vv), do)])
    for j, bar in ((0, 2), (1, 3), (2, 3), (3, 3)):
        e_pt = (refs["lowp"][j] - refs["fp32"][j]).abs().max().item()
        e = (res[0][j].cpu().float() - refs["fp32"][j]).abs().max().item()
        assert e <= bar * e_pt + 1e-4, (j, e, e_pt)


def test_reference_argument_checks():
    import flash_moba_b200 as F
    q = torch.randn(64, 2, 64, device=DEV, dtype=torch.float32)
    cs = cu_of([64]).to(DEV)
    with pytest.raises(RuntimeError, match="fp16 and bf16"):
        F.flash_topk_varlen_func(q, q, cs, cs, 64, 64, 2, 32)
    qb = q.bfloat16()
    with pytest.raises(RuntimeError, match="moba_topk"):
        F.flash_topk_varlen_func(qb, qb, cs, cs, 64, 64, 65, 32)
    co, cn, ind = F.flash_topk_varlen_func(qb, qb, cs, cs, 64, 64, 1, 64, causal=True)
    with pytest.raises(RuntimeError, match="lg_block_n"):
        F.flash_moba_attn_varlen_func(qb, qb, qb, cs, cs, 64, 64, co, cn, ind, 128, 32, causal=True)
    with pytest.raises(RuntimeError, match="dropout"):
        F.flash_moba_attn_varlen_func(qb, qb, qb, cs, cs, 64, 64, co, cn, ind, 128, 64, dropout_p=0.1)
    with pytest.raises(RuntimeError, match="int64"):
        F.flash_moba_attn_varlen_func(qb, qb, qb, cs, cs, 64, 64, co.int(), cn, ind, 128, 64)
