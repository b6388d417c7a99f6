"""The device-side status path and the longest work items.

  * the bounded wait every kernel uses, run on an mbarrier nobody arrives at: it gives up, the
    status code reaches the host, the time it took is the bound in time, the context stays usable;
  * a pattern whose columns overlap (more entries than `indices` has places): status 7, surfaced
    as a RuntimeError both by the synchronous check and by the deferred one, nothing faults;
  * an "attention sink": every row of a 65,536-token sequence selects chunk 0, so one work item of
    the main kernels is a column of 512 tiles walked by a single CTA (random patterns have 8-40):
    results against a CPU recomputation, status word read.
"""
import math
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_bounded_wait_gives_up_and_reports():
    from flash_moba_b200 import ops
    code, seconds = ops.selftest_wait_expiry()
    assert code == 5
    # far above the longest healthy wait (tens of milliseconds), far below anything that looks like a hang
    assert 0.05 < seconds < 30.0, seconds
    print(f"bounded wait gave up after {seconds:.3f} s")
    a = torch.randn(128, 128, device=DEV).bfloat16()
    d = ops.selftest_umma(a, a, False)            # the context is still usable
    assert torch.allclose(d, a.float() @ a.float().T, atol=0.5, rtol=2e-2)


def _overlapping_pattern(T, H, ncol):
    # two columns that both claim all T places of `indices`
    ind = torch.arange(T, dtype=torch.int32, device=DEV).repeat(H)
    co = torch.zeros((1, H, ncol), dtype=torch.int64, device=DEV)
    cn = torch.zeros((1, H, ncol), dtype=torch.int32, device=DEV)
    for h in range(H):
        co[0, h, :] = h * T
        cn[0, h, 0] = T
        cn[0, h, 1] = T
    return co, cn, ind


def test_overlapping_columns_raise(monkeypatch):
    import flash_moba_b200 as F
    from flash_moba_b200 import ops
    T, H, d, chunk = 256, 2, 128, 128
    q, k, v = (torch.randn(T, H, d, device=DEV).bfloat16() for _ in range(3))
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    pattern = _overlapping_pattern(T, H, T // chunk)
    monkeypatch.setenv("FMB_CHECK_STATUS", "1")
    with pytest.raises(RuntimeError, match="does not fit the slots"):
        F.flash_moba_attn_varlen_func(q, k, v, cu, cu, T, T, *pattern, 128, chunk, causal=False)
    # default mode: the call returns, the status word follows it to the host and raises at the next look
    monkeypatch.setenv("FMB_CHECK_STATUS", "0")
    F.flash_moba_attn_varlen_func(q, k, v, cu, cu, T, T, *pattern, 128, chunk, causal=False)
    with pytest.raises(RuntimeError, match="does not fit the slots"):
        ops.check_pending_status()
    ops.check_pending_status()                     # reported once
    # a well-formed call afterwards is fine
    monkeypatch.setenv("FMB_CHECK_STATUS", "1")
    own = F.flash_topk_varlen_func(q, k, cu, cu, T, T, 2, chunk, causal=True)
    F.flash_moba_attn_varlen_func(q, k, v, cu, cu, T, T, *own, 128, chunk, causal=True)


def test_attention_sink_column():
    import flash_moba_b200 as F
    from flash_moba_b200 import ops
    S, d, chunk = 65536, 128, 128
    g = torch.Generator(device=DEV).manual_seed(5)
    mk = lambda: torch.randn(S, 1, d, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, do = mk(), mk(), mk(), mk()
    cu = torch.tensor([0, S], dtype=torch.int32, device=DEV)
    own = (torch.arange(S, device=DEV) // chunk).to(torch.int32)
    idx = torch.stack([own, torch.where(own > 0, torch.zeros_like(own), torch.full_like(own, -1))], dim=-1)
    idx = idx.view(1, S, 2).permute(1, 0, 2)       # (tokens, heads, topk) view of head-major storage
    co, cn, ind = ops.build_csc(idx, cu, S, S // chunk)
    assert int(cn[0, 0, 0]) == S                   # the sink: every row
    qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
    out, lse, _ = F.flash_moba_attn_varlen_func(qd, kd, vd, cu, cu, S, S, co, cn, ind, 128, chunk, causal=True,
                                                return_attn_probs=True)
    dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), do)
    torch.cuda.synchronize()
    scale = 1.0 / math.sqrt(d)
    qf, kf, vf, dof = (t[:, 0].float() for t in (q, k, v, do))
    outf, lsef = out.detach()[:, 0].float(), lse[0]
    # sampled rows: O, LSE, dQ over {chunk 0} + {own chunk up to the row}
    gg = torch.Generator().manual_seed(6)
    rows = torch.cat([torch.randint(0, S, (64,), generator=gg), torch.tensor([0, 127, 128, 129, S - 1])]).tolist()
    for r in rows:
        c = r // chunk
        keys = torch.arange(0, min(chunk, r + 1), device=DEV) if c == 0 else \
            torch.cat([torch.arange(0, chunk, device=DEV), torch.arange(c * chunk, r + 1, device=DEV)])
        s = (kf[keys] @ qf[r]) * scale
        l = torch.logsumexp(s, 0)
        p = torch.exp(s - l)
        o = p @ vf[keys]
        assert abs(float(l) - float(lsef[r])) < 2e-2
        assert float((o - outf[r]).abs().max()) < 3e-2
        ds = p * (vf[keys] @ dof[r] - float((dof[r] * o).sum()))
        assert float((scale * (ds @ kf[keys]) - dq[r, 0].float()).abs().max()) < 6e-2
    # dK / dV of key block 0: a sum over all 65,536 rows
    keys = torch.arange(0, chunk, device=DEV)
    rr = torch.arange(S, device=DEV)
    s = (qf @ kf[keys].T) * scale
    p = torch.exp(s - lsef[:, None]) * (keys[None, :] <= rr[:, None])
    dvr = p.T @ dof
    ds = p * (dof @ vf[keys].T - (dof * outf).sum(-1, keepdim=True))
    dkr = scale * (ds.T @ qf)
    ref = max(float(dvr.abs().max()), float(dkr.abs().max()))
    assert float((dvr - dv[keys, 0].float()).abs().max()) < 0.02 * ref + 2e-2
    assert float((dkr - dk[keys, 0].float()).abs().max()) < 0.02 * ref + 2e-2
