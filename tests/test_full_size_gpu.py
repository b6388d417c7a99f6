"""Parity at the headline sequence length (65,536 tokens, chunk 128, top-k 8, bf16; d 128 with
four heads, and d 256 with two: the wide-head kernels).

The dense oracle cannot hold a 64K x 64K score matrix, so the checks are the size-independent
ones: run-to-run bit identity, and sampled rows / key blocks recomputed on the CPU from the
inputs (fp32) and compared with what the GPU path produced:
  * the chunk lists of sampled query rows (oracle gating of those rows against all centroids),
  * O and LSE of the sampled rows (attention over their selected chunks),
  * dQ of the sampled rows, and dK / dV of sampled key blocks (sum over the rows of the block's
    CSC column), using the GPU's LSE and O only where the definition of the gradient does.
Four heads keep it to about a gigabyte of device memory and a few seconds.
"""
import math
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import moba_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"
S, CHUNK, TOPK = 65536, 128, 8


@pytest.fixture(scope="module", params=[(4, 128), (2, 256)], ids=["d128", "d256"])
def run64k(request):
    import flash_moba_b200 as F
    H, D = request.param
    g = torch.Generator(device=DEV).manual_seed(2024)
    mk = lambda: torch.randn(S, H, D, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, do = mk(), mk(), mk(), mk()
    cu = torch.tensor([0, S], dtype=torch.int32, device=DEV)
    co, cn, ind = F.flash_topk_varlen_func(q, k, cu, cu, S, S, TOPK, CHUNK, causal=True)
    outs = []
    for _ in range(2):
        qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
        out, lse, _ = F.flash_moba_attn_varlen_func(qd, kd, vd, cu, cu, S, S, co, cn, ind, 128, CHUNK, causal=True,
                                                    return_attn_probs=True)
        dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), do)
        outs.append((out.detach(), lse.detach(), dq, dk, dv))
    return dict(q=q, k=k, v=v, do=do, cu=cu, pattern=(co, cn, ind), runs=outs, H=H, D=D)


def test_two_runs_bit_identical(run64k):
    a, b = run64k["runs"]
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def _rows_of_column(pattern, h, c):
    co, cn, ind = pattern
    off, n = int(co[0, h, c]), int(cn[0, h, c])
    return ind[off:off + n].long()


def test_pattern_of_sampled_rows(run64k):
    q, k, H = run64k["q"], run64k["k"], run64k["H"]
    pattern = tuple(t.cpu() for t in run64k["pattern"])
    km, cu_km = O.mean_pool(k.cpu(), run64k["cu"].cpu(), CHUNK)
    g = torch.Generator().manual_seed(1)
    rows = torch.cat([torch.randint(0, S, (96,), generator=g), torch.tensor([0, 1, 127, 128, 129, S - 1])])
    mism = total = 0
    for r in rows.tolist():
        for h in range(H):
            own = r // CHUNK
            sc = (q[r, h].cpu().float()[None] * km[:own, h].float()).sum(-1)      # candidate chunks n < own
            kk = min(TOPK - 1, own)
            want = {own}
            if kk > 0:
                # ties: the higher chunk index first
                order = sorted(range(own), key=lambda n: (-float(sc[n]), -n))[:kk]
                want |= set(order)
            got = set()
            for c in want | set(range(max(0, own - 2), own + 1)):
                if (_rows_of_column(pattern, h, c) == r).any():
                    got.add(c)
            # every wanted chunk lists the row; count the ones that do not (near-tie flips)
            mism += len(want - got)
            total += len(want)
    assert mism / total < 0.005, (mism, total)


def test_sampled_rows_outputs_and_dq(run64k):
    q, k, v, do = (run64k[n] for n in ("q", "k", "v", "do"))
    co, cn, ind = (t.cpu() for t in run64k["pattern"])
    out, lse, dq, _, _ = run64k["runs"][0]
    H, D = run64k["H"], run64k["D"]
    scale = 1.0 / math.sqrt(D)
    # row -> chunks from the CSC itself (the pattern the GPU used): scan the columns of a few heads
    g = torch.Generator().manual_seed(3)
    rows = torch.cat([torch.randint(0, S, (48,), generator=g), torch.tensor([0, 127, 128, 5000, S - 1])]).tolist()
    kf, vf = k.cpu().float(), v.cpu().float()
    worst_o = worst_dq = 0.0
    for h in range(H):
        cols = {r: [] for r in rows}
        nnz = cn[0, h]
        offs = co[0, h]
        for c in range(nnz.numel()):
            n = int(nnz[c])
            if n == 0:
                continue
            seg = ind[int(offs[c]):int(offs[c]) + n]
            for r in rows:
                if c * CHUNK <= r and (seg == r).any():
                    cols[r].append(c)
        for r in rows:
            keys = torch.cat([torch.arange(c * CHUNK, min((c + 1) * CHUNK, r + 1)) for c in cols[r]])
            qs = q[r, h].cpu().float()
            s = (kf[keys, h] @ qs) * scale
            l = torch.logsumexp(s, 0)
            p = torch.exp(s - l)
            o = p @ vf[keys, h]
            assert abs(float(l) - float(lse[h, r])) < 2e-2
            worst_o = max(worst_o, float((o - out[r, h].cpu().float()).abs().max()))
            dof = do[r, h].cpu().float()
            dp = vf[keys, h] @ dof
            dd = float((dof * o).sum())
            ds = p * (dp - dd)
            dqr = scale * (ds @ kf[keys, h])
            worst_dq = max(worst_dq, float((dqr - dq[r, h].cpu().float()).abs().max()))
    # bf16 inputs, P and dS rounded to bf16 inside the kernels: a few bf16 ulps of O(1) values
    assert worst_o < 3e-2, worst_o
    assert worst_dq < 6e-2, worst_dq


def test_sampled_key_blocks_dk_dv(run64k):
    q, k, v, do = (run64k[n] for n in ("q", "k", "v", "do"))
    pattern = tuple(t.cpu() for t in run64k["pattern"])
    out, lse, _, dk, dv = run64k["runs"][0]
    H, D = run64k["H"], run64k["D"]
    scale = 1.0 / math.sqrt(D)
    worst_k = worst_v = 0.0
    scale_ref = 0.0
    for h, c in ((0, 0), (1, 7), (2 % H, 255), (3 % H, 511), (0, 300)):
        rows = _rows_of_column(pattern, h, c)
        keys = torch.arange(c * CHUNK, (c + 1) * CHUNK)
        qf = q[rows, h].cpu().float()
        dof = do[rows, h].cpu().float()
        of = out[rows, h].cpu().float()
        kf, vf = k[keys, h].cpu().float(), v[keys, h].cpu().float()
        s = (qf @ kf.T) * scale
        vis = keys[None, :] <= rows[:, None]
        p = torch.exp(s - lse[h, rows].cpu()[:, None]) * vis
        dvr = p.T @ dof
        dp = dof @ vf.T
        dd = (dof * of).sum(-1, keepdim=True)
        ds = p * (dp - dd)
        dkr = scale * (ds.T @ qf)
        worst_v = max(worst_v, float((dvr - dv[keys, h].cpu().float()).abs().max()))
        worst_k = max(worst_k, float((dkr - dk[keys, h].cpu().float()).abs().max()))
        scale_ref = max(scale_ref, float(dvr.abs().max()), float(dkr.abs().max()))
    # sums over up to several thousand rows of bf16-rounded P / dS: relative to the largest entry
    assert worst_v < 0.02 * scale_ref + 2e-2, (worst_v, scale_ref)
    assert worst_k < 0.02 * scale_ref + 2e-2, (worst_k, scale_ref)
