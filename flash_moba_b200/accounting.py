"""Algorithmic work of the MoBA path: the figures the roofline fractions are computed from.

Selected-block convention: count unmasked (query, key) pairs inside selected chunks only,
the row's own chunk at its causal share.  A causal row in chunk j (0-based) of a sequence with
len_q == len_k selects min(topk, j+1) chunks: that many minus one full past chunks plus its
own.  FLOPs: forward 4*d per pair (QK^T and PV), backward 2.5x, forward+backward 3.5x — the
factors of the reference's benchmark (benchmarks/bench_flash_moba.py:23-26), applied to
selected pairs instead of the dense causal count.
"""
from typing import Sequence


def selected_pairs(seqlens: Sequence[int], chunk: int, topk: int) -> int:
    """Unmasked (q, k) pairs over selected blocks, per query head (causal, len_q == len_k)."""
    total = 0
    for s in seqlens:
        nchunks = (s + chunk - 1) // chunk
        for j in range(nchunks):
            rows = min(chunk, s - j * chunk)
            sel = min(topk, j + 1)
            total += rows * (sel - 1) * chunk + rows * (rows + 1) // 2
    return total


def selected_entries(seqlens: Sequence[int], chunk: int, topk: int) -> int:
    """(query row, key chunk) entries of the pattern, per query head (causal, len_q == len_k)."""
    total = 0
    for s in seqlens:
        for j in range((s + chunk - 1) // chunk):
            total += min(chunk, s - j * chunk) * min(topk, j + 1)
    return total


def attention_flops(seqlens, heads: int, d: int, chunk: int, topk: int):
    """(forward, backward, forward+backward) FLOPs over selected blocks."""
    fwd = 4 * d * selected_pairs(seqlens, chunk, topk) * heads
    return fwd, 2.5 * fwd, 3.5 * fwd


def pool_bytes(seqlens, heads_k: int, d: int, chunk: int, elem: int = 2) -> int:
    """Bytes the mean-pool must move: read every key once, write one centroid per chunk."""
    chunks = sum((s + chunk - 1) // chunk for s in seqlens)
    return (sum(seqlens) + chunks) * heads_k * d * elem


def csc_bytes(seqlens, heads: int, chunk: int, topk: int) -> int:
    """Bytes the pattern build must move: top-k lists read once, indices written once,
    offsets (8 B) and counts (4 B) per column."""
    nnz = heads * sum(min(topk, j + 1) * min(chunk, s - j * chunk)
                      for s in seqlens for j in range((s + chunk - 1) // chunk))
    ncol = max((s + chunk - 1) // chunk for s in seqlens) if seqlens else 0
    return 8 * nnz + 12 * len(seqlens) * heads * ncol


def gating_flops(seqlens, heads: int, d: int, chunk: int) -> int:
    """2*d per (row, candidate centroid) under the causal rule (candidates: chunks entirely
    before the row)."""
    total = 0
    for s in seqlens:
        nchunks = (s + chunk - 1) // chunk
        for j in range(nchunks):
            rows = min(chunk, s - j * chunk)
            total += rows * j
    return 2 * d * total * heads
