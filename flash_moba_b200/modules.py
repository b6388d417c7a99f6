"""Model-level wrappers around the functional API.

The reference stops at the three functions of `flash_moba_interface.py`; an LLM layer that adopts
them needs two more things, both thin host-side glue over the same kernels:

* ``MobaAttention``: an ``nn.Module`` holding the MoBA hyper-parameters.  With a process group of
  more than one rank it runs one long sequence split by query range
  (``sharding.moba_query_range``: centroids, K and V all-gathered, dK/dV reduce-scattered),
  otherwise the single-GPU path (``flash_moba_varlen_func``).
* ``CentroidCache``: the pooled centroids of a growing KV cache for decoding.  Appending keys only
  re-pools the chunks that changed, with the very kernel that pools a whole sequence, so the
  cached table is bit-identical to pooling from scratch; ``pattern()`` then gates new queries
  against the cached table (``flash_moba::_moba_fused_topk``) without touching the old keys.
"""
from typing import List, Optional, Sequence

import torch
from torch import nn

from . import ops
from .interface import decide_lg_block_m, flash_moba_attn_varlen_func, flash_moba_varlen_func


class MobaAttention(nn.Module):
    """MoBA attention over a varlen batch: ``forward(q, k, v, cu_seqlens_q, cu_seqlens_k,
    max_seqlen_q, max_seqlen_k)`` with q (total_q, heads, d), k/v (total_k, heads_k, d).

    process_group: if it has more than one rank, the call is ONE causal sequence whose rows are
    split across the ranks in order (every rank passes its own rows of q, k and v;
    cu_seqlens_* must describe that single local range); see ``sharding.moba_query_range``."""

    def __init__(self, chunk_size: int, topk: int, causal: bool = True, process_group=None):
        super().__init__()
        self.chunk_size, self.topk, self.causal, self.process_group = chunk_size, topk, causal, process_group

    def extra_repr(self) -> str:
        return f"chunk_size={self.chunk_size}, topk={self.topk}, causal={self.causal}"

    def _world(self) -> int:
        import torch.distributed as dist
        if self.process_group is None or not dist.is_available() or not dist.is_initialized():
            return 1
        return dist.get_world_size(self.process_group)

    def forward(self, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int):
        world = self._world()
        if world > 1:
            if not self.causal:
                raise RuntimeError("the query-range split is for causal attention")
            if cu_seqlens_q.numel() != 2 or q.shape[0] != k.shape[0]:
                raise RuntimeError("the query-range split takes one sequence: the rank's rows of q, k and v")
            from .sharding import moba_query_range
            return moba_query_range(q, k, v, q.shape[0] * world, self.chunk_size, self.topk, group=self.process_group)
        return flash_moba_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                      self.chunk_size, self.topk, causal=self.causal)


class CentroidCache:
    """Centroid table of `batch` growing key sequences (decode-time KV cache).

    Sequence b's centroids live in rows [b*capacity_chunks, ...) of ``km`` (capacity layout: rows do
    not move when another sequence grows), ``cu_seqlens_km = arange(batch+1) * capacity_chunks``.
    Under the causal rule a query at position p only competes for chunks n with (n+1)*chunk-1 < p,
    all of which are complete and pooled, so rows past a sequence's last chunk are never read.
    """

    def __init__(self, batch: int, heads_k: int, head_dim: int, chunk_size: int, max_seqlen_k: int,
                 dtype=torch.bfloat16, device="cuda"):
        self.batch, self.chunk = batch, chunk_size
        self.capacity_chunks = (max_seqlen_k + chunk_size - 1) // chunk_size
        self.km = torch.zeros((batch * self.capacity_chunks, heads_k, head_dim), dtype=dtype, device=device)
        self.cu_seqlens_km = (torch.arange(batch + 1, dtype=torch.int32) * self.capacity_chunks).to(device)
        self.lens: List[int] = [0] * batch          # keys pooled so far, per sequence (host side)

    def update(self, k: torch.Tensor, cu_seqlens_k: torch.Tensor, lens: Sequence[int]) -> None:
        """Brings the table up to `lens[b]` keys per sequence.  k (total_k, heads_k, d) is the packed
        key storage, sequence b at rows [cu_seqlens_k[b], cu_seqlens_k[b] + lens[b]) (cu_seqlens_k given
        as a host list or tensor of storage offsets; storage may be larger than what is in use).
        Only chunks that gained keys since the last call are pooled again."""
        starts = [int(x) for x in (cu_seqlens_k.tolist() if torch.is_tensor(cu_seqlens_k) else cu_seqlens_k)]
        pieces, dst_rows = [], []
        for b in range(self.batch):
            new = int(lens[b])
            if new > self.capacity_chunks * self.chunk:
                raise RuntimeError("CentroidCache: sequence longer than max_seqlen_k")
            if new < self.lens[b]:
                raise RuntimeError("CentroidCache: sequences only grow (make a new cache to shrink)")
            if new == self.lens[b]:
                continue
            c0 = self.lens[b] // self.chunk                    # first chunk that changed
            c1 = (new + self.chunk - 1) // self.chunk          # one past the last chunk
            pieces.append((starts[b] + c0 * self.chunk, starts[b] + new))
            dst_rows.append((b * self.capacity_chunks + c0, c1 - c0))
            self.lens[b] = new
        if not pieces:
            return
        # the changed key ranges as one small varlen batch through the pooling kernel
        rows = torch.cat([k[a:e] for a, e in pieces])
        cu = torch.tensor([0] + list(_cumsum(e - a for a, e in pieces)), dtype=torch.int32, device=k.device)
        km_new, _ = ops.mean_pool(rows, cu, max(e - a for a, e in pieces), self.chunk)
        off = 0
        for row0, n in dst_rows:
            self.km[row0:row0 + n] = km_new[off:off + n]
            off += n

    def pattern(self, q, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, topk: int):
        """(col_offsets, col_nnz, indices) for queries q against the cached centroids (causal,
        bottom-right aligned: the queries are the last rows of their sequences).  cu_seqlens_k must give
        the sequences' current lengths (packed, as the attention call will see them)."""
        return torch.ops.flash_moba._moba_fused_topk(q, self.km, cu_seqlens_q, cu_seqlens_k, self.cu_seqlens_km,
                                                     max_seqlen_q, max_seqlen_k, topk, self.chunk, causal=True)

    def attend(self, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, topk: int):
        """Gating against the cache, then block-sparse attention: the decode step."""
        pattern = self.pattern(q, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, topk)
        lg_m = decide_lg_block_m(topk, self.chunk, max_seqlen_k, True)
        return flash_moba_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, *pattern,
                                           lg_m, self.chunk, causal=True)


def _cumsum(xs):
    t = 0
    for x in xs:
        t += x
        yield t
