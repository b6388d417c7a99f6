"""Host-side multi-GPU logic on CPU: the planners, and the query-range split run as two gloo
ranks with the CPU oracle standing in for the attention kernels (the collectives, the
bottom-right aligned key ranges and the gradient reduce-scatter are what is under test)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from flash_moba_b200 import sharding  # noqa: E402
from flash_moba_b200.accounting import selected_pairs as acc_pairs  # noqa: E402


def test_head_shards_cover_whole_groups():
    for heads, heads_k, world in [(32, 32, 8), (32, 8, 8), (32, 8, 3), (16, 2, 4), (8, 8, 1)]:
        plan = sharding.plan_head_shards(heads, heads_k, world)
        assert len(plan) == world
        assert plan[0][0] == 0 and plan[-1][1] == heads
        g = heads // heads_k
        for (a0, a1), (b0, _) in zip(plan, plan[1:]):
            assert a1 == b0
        sizes = [(h1 - h0) // g for h0, h1 in plan]
        assert all((h1 - h0) % g == 0 for h0, h1 in plan)
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.plan_head_shards(30, 8, 2)


def test_selected_pairs_matches_accounting():
    for s, c, k in [(4096, 128, 8), (1000, 64, 3), (65536, 128, 8), (100, 128, 8)]:
        mask_pairs = 0          # count from the definition: own chunk + the (topk - 1) earlier chunks at most
        for row in range(s):
            own = row // c
            mask_pairs += (row - own * c + 1) + min(k - 1, own) * c
        assert sharding.selected_pairs(s, c, k) == acc_pairs([s], c, k) == mask_pairs


def test_work_items_balanced_and_complete():
    seqlens = [65536, 8192, 8192, 4096, 1024, 32768, 500, 16384]
    plan, loads = sharding.plan_work_items(seqlens, heads_k=4, chunk=128, topk=8, world=4)
    got = sorted(x for p in plan for x in p)
    assert got == sorted((b, hk) for b in range(len(seqlens)) for hk in range(4))
    assert max(loads) <= 1.05 * (sum(loads) / 4)
    assert sum(loads) == 4 * sum(sharding.selected_pairs(s, 128, 8) for s in seqlens)


def test_shard_heads_views():
    q = torch.randn(10, 8, 4)
    k = torch.randn(10, 2, 4)
    v = torch.randn(10, 2, 4)
    qs, ks, vs = sharding.shard_heads(q, k, v, (4, 8))
    assert qs.shape == (10, 4, 4) and ks.shape == (10, 1, 4)
    assert qs.data_ptr() == q[:, 4:].data_ptr() and torch.equal(ks, k[:, 1:2]) and torch.equal(vs, v[:, 1:2])
    with pytest.raises(ValueError):
        sharding.shard_heads(q, k, v, (2, 8))


# ----------------------------------------------------------------------------- two gloo ranks
def _oracle_attention(q, k, v, cu_q, cu_k, max_q, max_k, chunk, topk, causal=True):
    from oracle import moba_oracle as O
    with torch.no_grad():
        _, co, cn, ind = O.moba_pattern(q.detach(), k.detach(), cu_q, cu_k, max_k, topk, chunk, causal)
        mask = O.csc_to_mask(co, cn, ind, cu_q, max_q)
    out, _ = O.attention_dense(q, k, v, cu_q, cu_k, mask, chunk, causal)
    return out


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, S, H, Hk, d, chunk, topk, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        q = torch.randn(S, H, d, generator=g)
        k = torch.randn(S, Hk, d, generator=g)
        v = torch.randn(S, Hk, d, generator=g)
        do = torch.randn(S, H, d, generator=g)
        share = S // world
        sl = slice(rank * share, (rank + 1) * share)
        ql, kl, vl = (t[sl].clone().requires_grad_(True) for t in (q, k, v))
        out = sharding.moba_query_range(ql, kl, vl, S, chunk, topk, attention=_oracle_attention)
        out.backward(do[sl])
        # the unsplit computation, on every rank
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        cu = torch.tensor([0, S], dtype=torch.int32)
        ref = _oracle_attention(qf, kf, vf, cu, cu, S, S, chunk, topk)
        ref.backward(do)
        errs = [
            (out - ref[sl]).abs().max().item(),
            (ql.grad - qf.grad[sl]).abs().max().item(),
            (kl.grad - kf.grad[sl]).abs().max().item(),
            (vl.grad - vf.grad[sl]).abs().max().item(),
        ]
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_query_range_two_ranks_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, 256, 4, 2, 16, 32, 3, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    for p in procs:
        if p.is_alive():
            p.kill()
        assert p.exitcode == 0
    for r in range(world):
        assert max(ret[r]) < 2e-5, (r, ret[r])


def _ag_main(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = (torch.arange(6, dtype=torch.float32).view(3, 2) + 10 * rank).requires_grad_(True)
        y = sharding.all_gather_rows(x)
        w = torch.arange(y.numel(), dtype=torch.float32).view_as(y) * (rank + 1)
        (y * w).sum().backward()
        ret[rank] = (y.detach().clone(), x.grad.clone())
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_all_gather_rows_backward_is_reduce_scatter():
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_ag_main, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    full = torch.cat([torch.arange(6, dtype=torch.float32).view(3, 2) + 10 * r for r in range(world)])
    wsum = torch.arange(12, dtype=torch.float32).view(6, 2) * 3      # weights of rank 0 + rank 1
    for r in range(world):
        y, gx = ret[r]
        assert torch.equal(y, full)
        assert torch.equal(gx, wsum[r * 3:(r + 1) * 3])
