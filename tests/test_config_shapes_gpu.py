"""Parity at the shapes of the benchmark configurations 3, 4 and 5 (reduced only in head count).

  c3 : 8 sequences x 8,192 tokens, MHA, d 128, chunk 128, top-k 8
  c4 : 16 ragged sequences (lengths drawn from [2048, 32768], multiples of 64, seeded), GQA 4:1,
       d 128, chunk 64 (64-key blocks: the masked 128-lane backward), top-k 16 (the 16-entry gating list)
  c5 : one sequence of 524,288 tokens, d 128, chunk 256 (two partial planes per chunk), top-k 16,
       2,048 pattern columns, 64-bit offsets, run in several passes over the heads (small workspace cap)

The dense oracle cannot hold these score matrices, so the checks are the size-independent ones of
tests/test_full_size_gpu.py: two runs bit-identical, the device status word read after every call
(conftest sets FMB_CHECK_STATUS), and sampled query rows / key blocks recomputed on the CPU in
fp32 from the inputs: chunk lists (oracle gating rule, mismatch ratio < 0.5 % as in the reference's
tests/test_fused_topk.py:251-254), O, LSE and dQ of the rows, dK and dV of the key blocks (summed
over the q heads of a kv head).  Bars as in tests/test_full_size_gpu.py.
"""
import math
import os
import random
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import moba_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"
D = 128


def _c4_lengths():
    rnd = random.Random(0)
    return [(rnd.randint(2048, 32768) + 63) // 64 * 64 for _ in range(16)]


CONFIGS = {
    # name: (seqlens, q heads, kv heads, chunk, topk, input scale, workspace cap in GiB or None)
    "c3": ([8192] * 8, 8, 8, 128, 8, 1.0, None),
    "c4": (_c4_lengths(), 8, 2, 64, 16, 1.0, None),
    "c5": ([524288], 4, 4, 256, 16, 0.5, 12.0),
}


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def run(request):
    import flash_moba_b200 as F
    lens, H, Hk, chunk, topk, scale_in, cap = CONFIGS[request.param]
    T, mx = sum(lens), max(lens)
    old = os.environ.get("FMB_WORKSPACE_GB")
    if cap is not None:
        os.environ["FMB_WORKSPACE_GB"] = str(cap)
    try:
        g = torch.Generator(device=DEV).manual_seed(77)
        mk = lambda h: (torch.randn(T, h, D, generator=g, device=DEV, dtype=torch.float32) * scale_in).to(torch.bfloat16)
        q, k, v, do = mk(H), mk(Hk), mk(Hk), mk(H)
        cu = torch.tensor([0] + [sum(lens[:i + 1]) for i in range(len(lens))], dtype=torch.int32, device=DEV)
        co, cn, ind = F.flash_topk_varlen_func(q, k, cu, cu, mx, mx, topk, chunk, causal=True)
        outs = []
        for _ in range(2):
            qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
            out, lse, _ = F.flash_moba_attn_varlen_func(qd, kd, vd, cu, cu, mx, mx, co, cn, ind, 128, chunk,
                                                        causal=True, return_attn_probs=True)
            dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), do)
            outs.append(tuple(t.detach().cpu() for t in (out, lse, dq, dk, dv)))
            del qd, kd, vd, out, lse, dq, dk, dv
        torch.cuda.synchronize()
        res = dict(name=request.param, lens=lens, H=H, Hk=Hk, chunk=chunk, topk=topk,
                   q=q.cpu(), k=k.cpu(), v=v.cpu(), do=do.cpu(), cu=cu.cpu(),
                   pattern=(co.cpu(), cn.cpu(), ind.cpu()), runs=outs)
        del q, k, v, do, co, cn, ind
        torch.cuda.empty_cache()
        return res
    finally:
        if cap is not None:
            if old is None:
                os.environ.pop("FMB_WORKSPACE_GB", None)
            else:
                os.environ["FMB_WORKSPACE_GB"] = old


def test_two_runs_bit_identical(run):
    a, b = run["runs"]
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def _sample_rows(run, n, seed):
    """(sequence, local row) samples: random ones plus the chunk edges of the first and last sequence."""
    g = torch.Generator().manual_seed(seed)
    lens, chunk = run["lens"], run["chunk"]
    rows = []
    for _ in range(n):
        b = int(torch.randint(0, len(lens), (1,), generator=g))
        rows.append((b, int(torch.randint(0, lens[b], (1,), generator=g))))
    for b in (0, len(lens) - 1):
        for r in (0, chunk - 1, chunk, chunk + 1, lens[b] - 1):
            if 0 <= r < lens[b]:
                rows.append((b, r))
    return sorted(set(rows))


def _chunks_of_rows(run, h, rows):
    """{(b, r): sorted chunk ids whose CSC column of head h lists the row}, found from the pattern itself."""
    co, cn, ind = run["pattern"]
    res = {br: [] for br in rows}
    for b in sorted({b for b, _ in rows}):
        want = torch.tensor(sorted(r for bb, r in rows if bb == b), dtype=torch.int32)
        nnz = cn[b, h].long()
        total = int(nnz.sum())
        if total == 0:
            continue
        col_id = torch.repeat_interleave(torch.arange(nnz.numel()), nnz)
        first = torch.cumsum(nnz, 0) - nnz
        pos = torch.repeat_interleave(co[b, h], nnz) + (torch.arange(total) - torch.repeat_interleave(first, nnz))
        ent = ind[pos]
        hit = torch.isin(ent, want)
        for c, r in zip(col_id[hit].tolist(), ent[hit].tolist()):
            res[(b, r)].append(c)
    return {br: sorted(cs) for br, cs in res.items()}


def test_pattern_of_sampled_rows(run):
    q, k, cu = run["q"], run["k"], run["cu"]
    H, Hk, chunk, topk = run["H"], run["Hk"], run["chunk"], run["topk"]
    km, cu_km = O.mean_pool(k, cu, chunk)
    rows = _sample_rows(run, 64, 1)
    mism = total = 0
    for h in range(H):
        got_all = _chunks_of_rows(run, h, rows)
        hk = h // (H // Hk)
        for (b, r) in rows:
            own = r // chunk
            kmb = km[int(cu_km[b]):int(cu_km[b + 1]), hk].float()
            sc = (q[int(cu[b]) + r, h].float()[None] * kmb[:own]).sum(-1)      # candidate chunks n < own
            kk = min(topk - 1, own)
            want = {own}
            if kk > 0:   # ties: the higher chunk index first
                want |= set(sorted(range(own), key=lambda n: (-float(sc[n]), -n))[:kk])
            got = set(got_all[(b, r)])
            assert len(got) == len(want), (b, r, h, sorted(got), sorted(want))
            mism += len(want - got)
            total += len(want)
    assert mism / total < 0.005, (mism, total)


def test_sampled_rows_outputs_and_dq(run):
    q, k, v, do, cu = (run[n] for n in ("q", "k", "v", "do", "cu"))
    H, Hk, chunk = run["H"], run["Hk"], run["chunk"]
    out, lse, dq, _, _ = run["runs"][0]
    scale = 1.0 / math.sqrt(D)
    rows = _sample_rows(run, 40, 3)
    worst_o = worst_dq = 0.0
    for h in range(H):
        hk = h // (H // Hk)
        cols = _chunks_of_rows(run, h, rows)
        for (b, r) in rows:
            t0 = int(cu[b])
            keys = torch.cat([torch.arange(c * chunk, min((c + 1) * chunk, r + 1)) for c in cols[(b, r)]]) + t0
            kf, vf = k[keys, hk].float(), v[keys, hk].float()
            s = (kf @ q[t0 + r, h].float()) * scale
            l = torch.logsumexp(s, 0)
            p = torch.exp(s - l)
            o = p @ vf
            assert abs(float(l) - float(lse[h, t0 + r])) < 2e-2
            worst_o = max(worst_o, float((o - out[t0 + r, h].float()).abs().max()))
            dof = do[t0 + r, h].float()
            ds = p * (vf @ dof - float((dof * o).sum()))
            worst_dq = max(worst_dq, float((scale * (ds @ kf) - dq[t0 + r, h].float()).abs().max()))
    # bf16 inputs, P and dS rounded to bf16 inside the kernels: a few bf16 ulps of O(1) values
    assert worst_o < 3e-2, worst_o
    assert worst_dq < 6e-2, worst_dq


def test_sampled_key_blocks_dk_dv(run):
    q, k, v, do, cu = (run[n] for n in ("q", "k", "v", "do", "cu"))
    co, cn, ind = run["pattern"]
    H, Hk, chunk, lens = run["H"], run["Hk"], run["chunk"], run["lens"]
    out, lse, _, dk, dv = run["runs"][0]
    scale = 1.0 / math.sqrt(D)
    group = H // Hk
    g = torch.Generator().manual_seed(5)
    blocks = []
    for b in sorted({0, len(lens) // 2, len(lens) - 1}):
        nchunk = (lens[b] + chunk - 1) // chunk
        for c in sorted({0, 1, nchunk // 2, nchunk - 1, int(torch.randint(0, nchunk, (1,), generator=g))}):
            blocks.append((b, int(torch.randint(0, Hk, (1,), generator=g)), c))
    worst_k = worst_v = scale_ref = 0.0
    for b, hk, c in blocks:
        t0 = int(cu[b])
        keys = torch.arange(c * chunk, min((c + 1) * chunk, lens[b]))
        kf, vf = k[t0 + keys, hk].float(), v[t0 + keys, hk].float()
        dkr, dvr = torch.zeros_like(kf), torch.zeros_like(vf)
        for h in range(hk * group, (hk + 1) * group):
            off, n = int(co[b, h, c]), int(cn[b, h, c])
            rows = ind[off:off + n].long()
            qf, dof, of = q[t0 + rows, h].float(), do[t0 + rows, h].float(), out[t0 + rows, h].float()
            s = (qf @ kf.T) * scale
            vis = keys[None, :] <= rows[:, None]
            p = torch.exp(s - lse[h, t0 + rows][:, None]) * vis
            dvr += p.T @ dof
            ds = p * (dof @ vf.T - (dof * of).sum(-1, keepdim=True))
            dkr += scale * (ds.T @ qf)
        worst_v = max(worst_v, float((dvr - dv[t0 + keys, hk].float()).abs().max()))
        worst_k = max(worst_k, float((dkr - dk[t0 + keys, hk].float()).abs().max()))
        scale_ref = max(scale_ref, float(dvr.abs().max()), float(dkr.abs().max()))
    # sums over up to several thousand rows of bf16-rounded P / dS: relative to the largest entry
    assert worst_v < 0.02 * scale_ref + 2e-2, (worst_v, scale_ref)
    assert worst_k < 0.02 * scale_ref + 2e-2, (worst_k, scale_ref)
