"""Multi-GPU use of the MoBA path: one process per GPU (torch.distributed), no collective on
the data path unless a single long sequence has to be split.

The reference has no multi-GPU code.  Its path is embarrassingly parallel over
(sequence, kv-head group): nothing flows between them in the forward pass and, in the backward
pass, only inside a kv-head group (dK/dV are summed over the group's query heads).  Two plans:

* ``plan_head_shards`` / ``plan_work_items`` + ``shard_heads``: every rank runs the whole
  single-GPU pipeline on its own heads (or its own (sequence, kv head) items).  No collective.
* ``moba_query_range``: one very long sequence, fewer heads than ranks.  Rank r owns the query
  rows [r*S/R, (r+1)*S/R) and the matching slice of K and V; K and V are all-gathered (NCCL
  over NVLink), the rank's queries attend the gathered keys [0, (r+1)*S/R) with the
  bottom-right aligned causal mask the kernels already implement for len_q < len_k, and in the
  backward pass the partial dK/dV are reduce-scattered back to their owners.
"""
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .accounting import selected_pairs as _pairs


# ------------------------------------------------------------------------------ planning
def plan_head_shards(heads: int, heads_k: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous query-head ranges [h0, h1) per rank, whole kv-head groups, as even as possible."""
    if heads % heads_k != 0:
        raise ValueError("heads must be a multiple of heads_k")
    if world < 1:
        raise ValueError("world must be >= 1")
    group = heads // heads_k
    base, extra = divmod(heads_k, world)
    out, g0 = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((g0 * group, (g0 + n) * group))
        g0 += n
    return out


def selected_pairs(seqlen: int, chunk: int, topk: int) -> int:
    """Unmasked (q, k) pairs over selected chunks of one causal sequence and one query head."""
    return _pairs([seqlen], chunk, topk)


def plan_work_items(seqlens: Sequence[int], heads_k: int, chunk: int, topk: int, world: int):
    """Longest-processing-time assignment of (sequence, kv head) items to ranks by their
    selected-pair count (host arithmetic only).  Returns (items per rank, load per rank)."""
    items = [(selected_pairs(s, chunk, topk), b, hk) for b, s in enumerate(seqlens) for hk in range(heads_k)]
    items.sort(key=lambda x: (-x[0], x[1], x[2]))
    loads = [0] * world
    plan: List[List[Tuple[int, int]]] = [[] for _ in range(world)]
    for cost, b, hk in items:
        r = min(range(world), key=lambda i: (loads[i], i))
        plan[r].append((b, hk))
        loads[r] += cost
    for p in plan:
        p.sort()
    return plan, loads


def shard_heads(q, k, v, heads_range: Tuple[int, int]):
    """Views of q, k, v for the query heads [h0, h1) and their kv heads (no copy: only the last
    dimension has to be contiguous)."""
    h0, h1 = heads_range
    group = q.shape[1] // k.shape[1]
    if h0 % group or h1 % group:
        raise ValueError("head ranges must cover whole kv-head groups")
    return q[:, h0:h1], k[:, h0 // group:h1 // group], v[:, h0 // group:h1 // group]


# ------------------------------------------------------------------------------ collectives
class _AllGatherRows(torch.autograd.Function):
    """all-gather along dim 0 of equally sized shards; backward = reduce-scatter (sum)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        world = dist.get_world_size(ctx.group)
        grad = grad.contiguous()
        out = torch.empty((grad.shape[0] // world,) + tuple(grad.shape[1:]), dtype=grad.dtype, device=grad.device)
        if grad.is_cuda:
            dist.reduce_scatter_tensor(out, grad, op=dist.ReduceOp.SUM, group=ctx.group)
        else:   # gloo has no reduce_scatter_tensor: all-reduce, then keep the own slice
            g = grad.clone()
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
            r = dist.get_rank(ctx.group)
            out.copy_(g[r * out.shape[0]:(r + 1) * out.shape[0]])
        return out, None


def all_gather_rows(x: torch.Tensor, group=None) -> torch.Tensor:
    return _AllGatherRows.apply(x, group)


def moba_query_range(q_local, k_local, v_local, seqlen: int, chunk: int, topk: int, group=None,
                     attention: Optional[Callable] = None):
    """MoBA attention of ONE causal sequence of `seqlen` tokens split by query range.

    Every rank passes its own rows: q_local (S/R, H, d), k_local and v_local (S/R, Hk, d), ranks
    in sequence order, seqlen divisible by the world size.  Returns the rank's output rows
    (S/R, H, d); gradients flow to q_local, k_local and v_local (the key/value gradients through a
    reduce-scatter).  `attention(q, k, v, cu_q, cu_k, max_q, max_k, chunk, topk, causal=True)`
    defaults to this package's `flash_moba_varlen_func`.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if seqlen % world != 0:
        raise ValueError("seqlen must be divisible by the number of ranks")
    share = seqlen // world
    if q_local.shape[0] != share or k_local.shape[0] != share or v_local.shape[0] != share:
        raise ValueError("every rank must hold seqlen / world rows")
    if share % chunk != 0:
        raise ValueError("the per-rank share must be a whole number of chunks")
    if attention is None:
        from .interface import flash_moba_varlen_func as attention
    k_all = all_gather_rows(k_local, group)
    v_all = all_gather_rows(v_local, group)
    len_k = (rank + 1) * share            # causal: keys after the rank's last query are never used
    dev = q_local.device
    cu_q = torch.tensor([0, share], dtype=torch.int32, device=dev)
    cu_k = torch.tensor([0, len_k], dtype=torch.int32, device=dev)
    return attention(q_local, k_all[:len_k], v_all[:len_k], cu_q, cu_k, share, len_k, chunk, topk, causal=True)
