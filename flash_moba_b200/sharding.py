"""Multi-GPU use of the MoBA path: one process per GPU (torch.distributed), no collective on
the data path unless a single long sequence has to be split.

The reference has no multi-GPU code.  Its path is embarrassingly parallel over
(sequence, kv-head group): nothing flows between them in the forward pass and, in the backward
pass, only inside a kv-head group (dK/dV are summed over the group's query heads).  Two plans:

* ``plan_head_shards`` / ``plan_work_items`` + ``shard_heads``: every rank runs the whole
  single-GPU pipeline on its own heads (or its own (sequence, kv head) items).  No collective.
* ``moba_query_range``: one very long sequence, fewer heads than ranks.  Rank r owns the query
  rows [r*S/R, (r+1)*S/R) and the matching slice of K and V.  Each rank pools the centroids of
  its own key range; the centroids, K and V are all-gathered (NCCL over NVLink, issued in that
  order without waiting); gating and the pattern build need only the rank's queries and the
  (small) centroid table, so they run while K and V are still crossing the links; the rank's
  queries then attend the gathered keys [0, (r+1)*S/R) with the bottom-right aligned causal
  mask the kernels already implement for len_q < len_k, and in the backward pass the partial
  dK/dV are reduce-scattered back to their owners.  The kernels only ever read the rank's own
  memory: the collectives land in local buffers first.
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


class _MobaQueryRange(torch.autograd.Function):
    """The query-range split with this package's kernels (see moba_query_range)."""

    @staticmethod
    def forward(ctx, q_local, k_local, v_local, seqlen, chunk, topk, group):
        from . import interface, ops
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        share = seqlen // world
        len_k = (rank + 1) * share        # causal: keys after the rank's last query are never used
        dev = q_local.device
        hk, d = k_local.shape[1], k_local.shape[2]
        cu_q = torch.tensor([0, share], dtype=torch.int32, device=dev)
        cu_k = torch.tensor([0, len_k], dtype=torch.int32, device=dev)
        cu_local = torch.tensor([0, share], dtype=torch.int32, device=dev)
        k_local, v_local = k_local.contiguous(), v_local.contiguous()
        # centroids of the own key range (chunks never straddle ranks: share % chunk == 0), then the
        # three gathers back to back; only the small one is waited for before gating
        km_local, _ = ops.mean_pool(k_local, cu_local, share, chunk)
        nloc = share // chunk
        km_all = torch.empty((world * nloc, hk, d), dtype=k_local.dtype, device=dev)
        k_all = torch.empty((seqlen, hk, d), dtype=k_local.dtype, device=dev)
        v_all = torch.empty((seqlen, hk, d), dtype=v_local.dtype, device=dev)
        w_km = dist.all_gather_into_tensor(km_all, km_local[:nloc].contiguous(), group=group, async_op=True)
        w_k = dist.all_gather_into_tensor(k_all, k_local, group=group, async_op=True)
        w_v = dist.all_gather_into_tensor(v_all, v_local, group=group, async_op=True)
        w_km.wait()
        nk = len_k // chunk
        cu_km = torch.tensor([0, nk], dtype=torch.int32, device=dev)
        pattern = torch.ops.flash_moba._moba_fused_topk(q_local, km_all[:nk], cu_q, cu_k, cu_km, share, len_k, topk,
                                                        chunk, causal=True)
        w_k.wait()
        w_v.wait()
        scale = q_local.shape[-1] ** (-0.5)
        lg_m = interface.decide_lg_block_m(topk, chunk, len_k, True)
        out, lse, _, _ = torch.ops.flash_moba._flash_moba_attn_varlen_forward(
            q_local, k_all[:len_k], v_all[:len_k], cu_q, cu_k, share, len_k, *pattern, lg_m, chunk, 0.0, scale, True)
        ctx.save_for_backward(q_local, k_all, v_all, out, lse, cu_q, cu_k, *pattern)
        ctx.meta = (seqlen, share, len_k, chunk, scale, lg_m, group)
        return out

    @staticmethod
    def backward(ctx, dout):
        q_local, k_all, v_all, out, lse, cu_q, cu_k, co, cn, ind = ctx.saved_tensors
        seqlen, share, len_k, chunk, scale, lg_m, group = ctx.meta
        dq = torch.empty_like(q_local)
        # the whole sequence's dK / dV: rows past this rank's last key get nothing from it
        dk_all, dv_all = torch.zeros_like(k_all), torch.zeros_like(v_all)
        torch.ops.flash_moba._flash_moba_attn_varlen_backward(
            dout.contiguous(), q_local, k_all[:len_k], v_all[:len_k], out, lse, dq, dk_all[:len_k], dv_all[:len_k],
            cu_q, cu_k, share, len_k, co, cn, ind, lg_m, chunk, 0.0, scale, True, 0.0, None, False)
        dk = torch.empty((share,) + tuple(k_all.shape[1:]), dtype=k_all.dtype, device=k_all.device)
        dv = torch.empty_like(dk)
        w_k = dist.reduce_scatter_tensor(dk, dk_all, op=dist.ReduceOp.SUM, group=group, async_op=True)
        w_v = dist.reduce_scatter_tensor(dv, dv_all, op=dist.ReduceOp.SUM, group=group, async_op=True)
        w_k.wait()
        w_v.wait()
        return dq, dk, dv, None, None, None, None


def moba_query_range(q_local, k_local, v_local, seqlen: int, chunk: int, topk: int, group=None,
                     attention: Optional[Callable] = None):
    """MoBA attention of ONE causal sequence of `seqlen` tokens split by query range.

    Every rank passes its own rows: q_local (S/R, H, d), k_local and v_local (S/R, Hk, d), ranks
    in sequence order, seqlen divisible by the world size.  Returns the rank's output rows
    (S/R, H, d); gradients flow to q_local, k_local and v_local (the key/value gradients through a
    reduce-scatter).  By default the package's own kernels run, with the centroids pooled per
    rank and gathered with K and V, and gating overlapped with the K/V gathers.  Passing
    `attention(q, k, v, cu_q, cu_k, max_q, max_k, chunk, topk, causal=True)` (e.g. a CPU
    implementation under gloo) takes the plain route instead: gather K and V, call it.
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
        return _MobaQueryRange.apply(q_local, k_local, v_local, seqlen, chunk, topk, group)
    k_all = all_gather_rows(k_local, group)
    v_all = all_gather_rows(v_local, group)
    len_k = (rank + 1) * share            # causal: keys after the rank's last query are never used
    dev = q_local.device
    cu_q = torch.tensor([0, share], dtype=torch.int32, device=dev)
    cu_k = torch.tensor([0, len_k], dtype=torch.int32, device=dev)
    return attention(q_local, k_all[:len_k], v_all[:len_k], cu_q, cu_k, share, len_k, chunk, topk, causal=True)
