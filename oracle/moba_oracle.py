"""CPU oracle for the MoBA sparse-attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch/numpy on the CPU, what every stage of the
reference's MoBA path computes.  It is the checker for the CUDA kernels: only the
test-suite, the smoke check and the benchmark's CPU-baseline leg may import it.
The shipped package never imports it and has no CPU fallback.

Pinned against the reference itself: ``tests/golden/make_golden.py`` imports the
reference's pure-PyTorch implementations and stores their outputs;
``tests/test_oracle_golden.py`` checks every function here against those vectors.

Stages and the reference code each one follows (paths inside the reference project):

* ``mean_pool``        tests/test_triton_mean_pool.py:6-26 (fp32 mean -> input dtype),
                       flash_moba/triton_mean_pool.py:112-157 (output layout)
* ``gate_topk``        tests/test_fused_topk.py:11-111 and the kernel's rule for
                       unequal q/k lengths, csrc/flash_topk/src/flash_topk_kernel.h:195-297
* ``build_csc``        tests/test_fused_topk_epilogue.py:19-37,
                       csrc/flash_topk/src/flash_topk_kernel.h:376-402 (offset base),
                       csrc/flash_topk/flash_topk_api.cpp:217 (zero-filled tail)
* ``csc_to_mask`` / ``mask_to_csc``   flash_moba/moba_test_utils.py:142-196
* ``attention_dense``  flash_moba/moba_test_utils.py:653-748 with the key validity rule of
                       csrc/flash_moba/src/mask.h:139-176 and the empty-row rule of
                       csrc/flash_moba/src/flash_fwd_kernel.h:291-333
* ``attention_blocked`` same mathematics, gathering only selected chunks (O(S*topk*C)
                       memory), validated against ``attention_dense`` in the tests
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

NEG_INF = float("-inf")


# --------------------------------------------------------------------------------------
# small helpers
# --------------------------------------------------------------------------------------
def _lens(cu: torch.Tensor) -> list:
    cu = [int(x) for x in cu.tolist()]
    return [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]


def chunk_offsets(cu_seqlens_k: torch.Tensor, chunk: int) -> Tuple[torch.Tensor, int]:
    """cu_seqlens of the centroid table: cumsum(ceil(len/chunk)).

    Follows flash_moba/triton_mean_pool.py:134-138."""
    n = [(l + chunk - 1) // chunk for l in _lens(cu_seqlens_k)]
    cu = np.concatenate([[0], np.cumsum(n)]).astype(np.int32)
    return torch.from_numpy(cu), (max(n) if n else 0)


# --------------------------------------------------------------------------------------
# stage P: per-chunk key mean-pool
# --------------------------------------------------------------------------------------
def mean_pool(k: torch.Tensor, cu_seqlens_k: torch.Tensor, chunk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Centroid of each length-``chunk`` block of every sequence and kv head.

    fp32 mean, divided by the true (possibly short) length of the last chunk, then
    rounded to the dtype of ``k``.  Returns (km (total_chunks, Hk, d), cu_seqlens_km)."""
    cu_km, _ = chunk_offsets(cu_seqlens_k, chunk)
    cu = [int(x) for x in cu_seqlens_k.tolist()]
    out = torch.zeros((int(cu_km[-1]), k.shape[1], k.shape[2]), dtype=k.dtype)
    row = 0
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        for c0 in range(s, e, chunk):
            blk = k[c0:min(c0 + chunk, e)].to(torch.float32)
            out[row] = blk.mean(dim=0).to(k.dtype)
            row += 1
    return out, cu_km


# --------------------------------------------------------------------------------------
# stage G: gating scores + causal chunk rule + top-k
# --------------------------------------------------------------------------------------
def gate_scores(q_seq: torch.Tensor, km_seq: torch.Tensor) -> torch.Tensor:
    """fp32, unscaled gate ``g[h, row, n] = q[row, h] . km[n, h // group]``."""
    H, Hk = q_seq.shape[1], km_seq.shape[1]
    kmf = km_seq.to(torch.float32)
    if Hk != H:
        kmf = kmf.repeat_interleave(H // Hk, dim=1)
    return torch.einsum("shd,nhd->hsn", q_seq.to(torch.float32), kmf)


def select_topk(gate: np.ndarray, topk: int, chunk: int, len_q: int, len_k: int, causal: bool):
    """Top-k selection on a given fp32 score array ``gate`` (H, len_q, nchunks).

    Rule (csrc/flash_topk/src/flash_topk_kernel.h:203-214, 261-285): with
    ``p = row + len_k - len_q``, under ``causal`` the chunk ``p // chunk`` is always taken
    (value +inf, slot 0) and chunk n is a candidate only if ``(n+1)*chunk - 1 < p``;
    rows with p < 0 select nothing.  Among candidates the ``topk`` largest scores are
    kept, sorted by descending score; on exactly equal scores the HIGHER chunk index
    ranks first (tests/test_fused_topk.py:27-37).  Unfilled slots are -1 / -inf.
    Returns (idx int32 (len_q, H, topk), val fp32 (len_q, H, topk))."""
    H, S, N = gate.shape
    g = gate.astype(np.float32).copy()
    if causal:
        p = np.arange(S) + (len_k - len_q)                      # (S,)
        n = np.arange(N)
        cand = ((n[None, :] + 1) * chunk - 1) < p[:, None]      # (S, N)
        own = (p[:, None] // chunk == n[None, :]) & (p[:, None] >= 0)
        g = np.where(cand[None], g, -np.inf)
        g = np.where(own[None], np.inf, g)
    idx = np.full((S, H, topk), -1, dtype=np.int32)
    val = np.full((S, H, topk), -np.inf, dtype=np.float32)
    kk = min(topk, N)
    if kk == 0 or S == 0:
        return idx, val
    # ascending stable order by (score, index): the last kk entries, reversed
    order = np.argsort(g, axis=-1, kind="stable")               # (H, S, N)
    top = order[..., N - kk:][..., ::-1]                        # (H, S, kk)
    tv = np.take_along_axis(g, top, axis=-1)
    ti = np.where(np.isneginf(tv), -1, top).astype(np.int32)
    idx[:, :, :kk] = ti.transpose(1, 0, 2)
    val[:, :, :kk] = tv.transpose(1, 0, 2)
    return idx, val


def gate_topk(q, km, cu_seqlens_q, cu_seqlens_k, cu_seqlens_km, topk: int, chunk: int, causal: bool):
    """Per-row top-k chunk lists for a varlen batch.  Returns (idx (T,H,topk) i32, val fp32)."""
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    ck = [int(x) for x in cu_seqlens_k.tolist()]
    cm = [int(x) for x in cu_seqlens_km.tolist()]
    T, H = q.shape[0], q.shape[1]
    idx = np.full((T, H, topk), -1, dtype=np.int32)
    val = np.full((T, H, topk), -np.inf, dtype=np.float32)
    for b in range(len(cq) - 1):
        lq, lk = cq[b + 1] - cq[b], ck[b + 1] - ck[b]
        if lq == 0 or lk == 0:
            continue
        g = gate_scores(q[cq[b]:cq[b + 1]], km[cm[b]:cm[b + 1]]).numpy()
        i, v = select_topk(g, topk, chunk, lq, lk, causal)
        idx[cq[b]:cq[b + 1]] = i
        val[cq[b]:cq[b + 1]] = v
    return torch.from_numpy(idx), torch.from_numpy(val)


# --------------------------------------------------------------------------------------
# stages O/E/S: per-row top-k lists -> key-block-major CSC pattern
# --------------------------------------------------------------------------------------
def build_csc(topk_idx: torch.Tensor, cu_seqlens_q: torch.Tensor, topk: int, ncol: int):
    """CSC pattern of the top-k lists.

    For (b, h, c): ``indices[col_offsets[b,h,c] : +col_nnz[b,h,c]]`` are the ascending
    sequence-local query rows whose list contains chunk c.  The region of (b, h) starts
    at ``(cu_q[b]*H + len_q[b]*h) * topk``; columns are packed back to back inside it and
    the unused tail of every region stays 0.  ``indices`` has T*H*topk entries."""
    idx = topk_idx.numpy()
    T, H, _ = idx.shape
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    B = len(cq) - 1
    col_offsets = np.zeros((B, H, ncol), dtype=np.int64)
    col_nnz = np.zeros((B, H, ncol), dtype=np.int32)
    indices = np.zeros((T * H * topk,), dtype=np.int32)
    for b in range(B):
        lq = cq[b + 1] - cq[b]
        for h in range(H):
            base = (cq[b] * H + lq * h) * topk
            sel = idx[cq[b]:cq[b + 1], h, :topk]               # (lq, topk)
            rows, slots = np.nonzero(sel >= 0)
            cols = sel[rows, slots]
            order = np.lexsort((rows, cols))                    # by column, then row
            cols_s, rows_s = cols[order], rows[order]
            nnz = np.bincount(cols_s, minlength=ncol)[:ncol].astype(np.int32)
            col_nnz[b, h] = nnz
            col_offsets[b, h] = base + np.concatenate([[0], np.cumsum(nnz)[:-1]])
            indices[base:base + len(rows_s)] = rows_s.astype(np.int32)
    return torch.from_numpy(col_offsets), torch.from_numpy(col_nnz), torch.from_numpy(indices)


def csc_to_mask(col_offsets, col_nnz, indices, cu_seqlens_q, max_seqlen_q: int) -> torch.Tensor:
    """Boolean (B, H, max_seqlen_q, ncol): True where the row attends the chunk."""
    co, cn, ind = col_offsets.numpy(), col_nnz.numpy(), indices.numpy()
    B, H, ncol = co.shape
    mask = np.zeros((B, H, max_seqlen_q, ncol), dtype=bool)
    for b in range(B):
        for h in range(H):
            for c in range(ncol):
                n = int(cn[b, h, c])
                if n:
                    o = int(co[b, h, c])
                    mask[b, h, ind[o:o + n], c] = True
    return torch.from_numpy(mask)


def mask_to_csc(mask: torch.Tensor, cu_seqlens_q, cu_seqlens_k, chunk: int):
    """Pattern triple from a boolean mask, columns packed back to back with one running
    offset over the whole batch (the packing of flash_moba/moba_test_utils.py:172-191,
    which differs from the top-k packing: the attention kernels must honour both)."""
    m = mask.numpy()
    B, H, _, ncol = m.shape
    lq, lk = _lens(cu_seqlens_q), _lens(cu_seqlens_k)
    col_offsets = np.zeros((B, H, ncol), dtype=np.int64)
    col_nnz = np.zeros((B, H, ncol), dtype=np.int32)
    out = []
    off = 0
    for b in range(B):
        nb = (lk[b] + chunk - 1) // chunk
        for h in range(H):
            for c in range(nb):
                rows = np.nonzero(m[b, h, :lq[b], c])[0]
                col_offsets[b, h, c] = off
                col_nnz[b, h, c] = len(rows)
                out.append(rows.astype(np.int32))
                off += len(rows)
    ind = np.concatenate(out) if out else np.zeros((0,), dtype=np.int32)
    return torch.from_numpy(col_offsets), torch.from_numpy(col_nnz), torch.from_numpy(ind.astype(np.int32))


# --------------------------------------------------------------------------------------
# stages F/B: block-sparse attention, forward (+ autograd backward)
# --------------------------------------------------------------------------------------
def _valid_mask(mask_bh: torch.Tensor, lq: int, lk: int, chunk: int, causal: bool) -> torch.Tensor:
    """(H, lq, lk) bool: key col is visible to row iff its chunk is selected, col < lk and,
    under causal, col <= row + lk - lq (bottom-right aligned)."""
    nb = (lk + chunk - 1) // chunk
    keep = mask_bh[:, :lq, :nb].repeat_interleave(chunk, dim=-1)[..., :lk]
    if causal:
        r = torch.arange(lq)[:, None] + (lk - lq)
        c = torch.arange(lk)[None, :]
        keep = keep & (c <= r)[None]
    return keep


def attention_dense(q, k, v, cu_seqlens_q, cu_seqlens_k, mask, chunk: int, causal: bool,
                    softmax_scale: Optional[float] = None, lowp: bool = False):
    """Dense-masked MoBA attention on a varlen batch.

    ``mask`` is (B, H, max_q, ncol) bool.  fp32 mathematics when ``lowp`` is False (the
    truth); when True the computation runs in the input dtype with k pre-scaled, which is
    the reference's low-precision yardstick (flash_moba/moba_test_utils.py:700-703 with
    ``upcast=False, reorder_ops=True``).  Rows without any visible key give O = 0 and
    LSE = +inf.  Differentiable w.r.t. q, k, v.  Returns (out (T,H,d) in q.dtype,
    lse (H,T) fp32)."""
    T, H, d = q.shape
    Hk = k.shape[1]
    g = H // Hk
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    ck = [int(x) for x in cu_seqlens_k.tolist()]
    outs, lses = [], []
    for b in range(len(cq) - 1):
        lq, lk = cq[b + 1] - cq[b], ck[b + 1] - ck[b]
        qb, kb, vb = q[cq[b]:cq[b + 1]], k[ck[b]:ck[b + 1]], v[ck[b]:ck[b + 1]]
        if lq == 0:
            continue
        if lk == 0:
            outs.append(torch.zeros_like(qb))
            lses.append(torch.full((H, lq), float("inf")))
            continue
        if not lowp:
            qb, kb, vb = qb.float(), kb.float(), vb.float()
        kb = kb.repeat_interleave(g, dim=1)
        vb = vb.repeat_interleave(g, dim=1)
        keep = _valid_mask(mask[b], lq, lk, chunk, causal)
        if lowp:
            s = torch.einsum("thd,shd->hts", qb, kb * scale)
        else:
            s = torch.einsum("thd,shd->hts", qb * scale, kb)
        s = s.masked_fill(~keep, NEG_INF)
        empty = ~keep.any(dim=-1, keepdim=True)
        lse = torch.logsumexp(s.float().masked_fill(empty, 0.0), dim=-1)
        lse = lse.masked_fill(empty[..., 0], float("inf"))
        p = torch.softmax(s.masked_fill(empty, 0.0), dim=-1).to(vb.dtype)
        p = p.masked_fill(~keep, 0.0)
        o = torch.einsum("hts,shd->thd", p, vb)
        outs.append(o.to(q.dtype))
        lses.append(lse.detach())
    out = torch.cat(outs, dim=0) if outs else torch.zeros_like(q)
    lse = torch.cat(lses, dim=1) if lses else torch.zeros((H, 0))
    return out, lse


def attention_blocked(q, k, v, cu_seqlens_q, cu_seqlens_k, topk_idx, chunk: int, causal: bool,
                      softmax_scale: Optional[float] = None, rows_per_step: Optional[int] = None):
    """Same result as ``attention_dense`` for a pattern given as per-row chunk lists
    ``topk_idx`` (T, H, K) (-1 = unused), computed by gathering only the selected chunks,
    so memory is O(rows * K * chunk) instead of O(S^2).  fp32.  Differentiable."""
    T, H, d = q.shape
    Hk = k.shape[1]
    g = H // Hk
    K = topk_idx.shape[-1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    if rows_per_step is None:       # keep the gathered K and V tiles near 128 MB each
        rows_per_step = max(1, (32 << 20) // (H * K * chunk * d))
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    ck = [int(x) for x in cu_seqlens_k.tolist()]
    out = []
    lse_all = []
    ar = torch.arange(chunk)
    for b in range(len(cq) - 1):
        lq, lk = cq[b + 1] - cq[b], ck[b + 1] - ck[b]
        if lq == 0:
            continue
        nb = max((lk + chunk - 1) // chunk, 1)
        pad = nb * chunk - lk
        kb = torch.nn.functional.pad(k[ck[b]:ck[b + 1]].float(), (0, 0, 0, 0, 0, pad)).view(nb, chunk, Hk, d)
        vb = torch.nn.functional.pad(v[ck[b]:ck[b + 1]].float(), (0, 0, 0, 0, 0, pad)).view(nb, chunk, Hk, d)
        ob, lb = [], []
        for r0 in range(0, lq, rows_per_step):
            r1 = min(r0 + rows_per_step, lq)
            qs = q[cq[b] + r0:cq[b] + r1].float() * scale                    # (R,H,d)
            sel = topk_idx[cq[b] + r0:cq[b] + r1].long()                     # (R,H,K)
            used = sel >= 0
            selc = sel.clamp(min=0)
            hk = (torch.arange(H) // g)[None, :, None].expand_as(selc)
            kg = kb[selc, :, hk]                                             # (R,H,K,chunk,d)
            vg = vb[selc, :, hk]
            s = torch.einsum("rhd,rhkcd->rhkc", qs, kg)
            col = selc[..., None] * chunk + ar                               # (R,H,K,chunk)
            ok = used[..., None] & (col < lk)
            if causal:
                p = (torch.arange(r0, r1) + (lk - lq))[:, None, None, None]
                ok = ok & (col <= p)
            s = s.masked_fill(~ok, NEG_INF).flatten(2)                       # (R,H,K*chunk)
            empty = ~ok.flatten(2).any(dim=-1, keepdim=True)
            s0 = s.masked_fill(empty, 0.0)
            l = torch.logsumexp(s0, dim=-1).masked_fill(empty[..., 0], float("inf"))
            pr = torch.softmax(s0, dim=-1).masked_fill(~ok.flatten(2), 0.0)
            o = torch.einsum("rhx,rhxd->rhd", pr, vg.flatten(2, 3))
            ob.append(o)
            lb.append(l.detach().transpose(0, 1))
        out.append(torch.cat(ob, dim=0))
        lse_all.append(torch.cat(lb, dim=1))
    o = torch.cat(out, dim=0).to(q.dtype) if out else torch.zeros_like(q)
    lse = torch.cat(lse_all, dim=1) if lse_all else torch.zeros((H, 0))
    return o, lse


# --------------------------------------------------------------------------------------
# whole path
# --------------------------------------------------------------------------------------
def moba_pattern(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_k: int, topk: int, chunk: int, causal: bool):
    """pool -> gate/top-k -> CSC.  Returns (topk_idx, col_offsets, col_nnz, indices)."""
    km, cu_km = mean_pool(k, cu_seqlens_k, chunk)
    idx, _ = gate_topk(q, km, cu_seqlens_q, cu_seqlens_k, cu_km, topk, chunk, causal)
    ncol = (max_seqlen_k + chunk - 1) // chunk
    co, cn, ind = build_csc(idx, cu_seqlens_q, topk, ncol)
    return idx, co, cn, ind


def moba_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int,
                 chunk: int, topk: int, causal: bool = True, blocked: bool = False):
    """The reference's pure-PyTorch MoBA path end to end (pattern + attention)."""
    idx, co, cn, ind = moba_pattern(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_k, topk, chunk, causal)
    if blocked:
        out, lse = attention_blocked(q, k, v, cu_seqlens_q, cu_seqlens_k, idx, chunk, causal)
    else:
        mask = csc_to_mask(co, cn, ind, cu_seqlens_q, max_seqlen_q)
        out, lse = attention_dense(q, k, v, cu_seqlens_q, cu_seqlens_k, mask, chunk, causal)
    return out, lse, idx, (co, cn, ind)
