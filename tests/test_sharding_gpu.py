"""The two multi-GPU plans with the real kernels.

Single GPU: the per-rank calls of the head split and of the query-range split are run one after
the other on one device and compared with the unsplit call (bit-identical outputs are expected:
per (row, head) the same partials are merged in the same order).  Two GPUs (when present): the
query-range split as two NCCL ranks."""
import os
import socket
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu


def _inputs(S, H, Hk, d, seed=3):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h: torch.randn(S, h, d, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    return mk(H), mk(Hk), mk(Hk), mk(H)


def test_head_split_equals_unsplit():
    import flash_moba_b200 as F
    from flash_moba_b200 import sharding
    S, H, Hk, d, chunk, topk = 2048, 8, 4, 128, 128, 4
    q, k, v, do = _inputs(S, H, Hk, d)
    cu = torch.tensor([0, S], dtype=torch.int32, device="cuda")
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = F.flash_moba_varlen_func(qf, kf, vf, cu, cu, S, S, chunk, topk, causal=True)
    dq, dk, dv = torch.autograd.grad(out, (qf, kf, vf), do)
    for world in (2, 3):
        for h0, h1 in sharding.plan_head_shards(H, Hk, world):
            if h0 == h1:
                continue
            qs, ks, vs = (t.clone().requires_grad_(True) for t in sharding.shard_heads(q, k, v, (h0, h1)))
            o = F.flash_moba_varlen_func(qs, ks, vs, cu, cu, S, S, chunk, topk, causal=True)
            gq, gk, gv = torch.autograd.grad(o, (qs, ks, vs), do[:, h0:h1].contiguous())
            g = H // Hk
            assert torch.equal(o, out[:, h0:h1])
            assert torch.equal(gq, dq[:, h0:h1])
            assert torch.equal(gk, dk[:, h0 // g:h1 // g])
            assert torch.equal(gv, dv[:, h0 // g:h1 // g])


def test_query_range_split_single_device():
    """Rank r's call (queries of its range against keys [0, end of range)) reproduces the rows of
    the unsplit call: same pattern, same outputs; dK/dV summed over the ranks match."""
    import flash_moba_b200 as F
    S, H, Hk, d, chunk, topk, world = 4096, 4, 2, 128, 128, 4, 4
    q, k, v, do = _inputs(S, H, Hk, d, seed=5)
    cu = torch.tensor([0, S], dtype=torch.int32, device="cuda")
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = F.flash_moba_varlen_func(qf, kf, vf, cu, cu, S, S, chunk, topk, causal=True)
    dq, dk, dv = torch.autograd.grad(out, (qf, kf, vf), do)
    share = S // world
    dk_sum = torch.zeros_like(dk, dtype=torch.float32)
    dv_sum = torch.zeros_like(dv, dtype=torch.float32)
    for r in range(world):
        sl = slice(r * share, (r + 1) * share)
        lk = (r + 1) * share
        qs = q[sl].clone().requires_grad_(True)
        ks = k[:lk].clone().requires_grad_(True)
        vs = v[:lk].clone().requires_grad_(True)
        cq = torch.tensor([0, share], dtype=torch.int32, device="cuda")
        ck = torch.tensor([0, lk], dtype=torch.int32, device="cuda")
        o = F.flash_moba_varlen_func(qs, ks, vs, cq, ck, share, lk, chunk, topk, causal=True)
        gq, gk, gv = torch.autograd.grad(o, (qs, ks, vs), do[sl])
        assert torch.equal(o, out[sl])
        assert torch.equal(gq, dq[sl])
        dk_sum[:lk] += gk.float()
        dv_sum[:lk] += gv.float()
    # each rank rounds its partial dK/dV to bf16 before the sum: allow a few bf16 ulps
    for got, ref in ((dk_sum, dk.float()), (dv_sum, dv.float())):
        err = (got - ref).abs().max().item()
        assert err <= 0.02 * ref.abs().max().item() + 1e-3, err


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import flash_moba_b200 as F
        from flash_moba_b200 import sharding
        S, H, Hk, d, chunk, topk = 4096, 4, 2, 128, 128, 4
        g = torch.Generator(device="cuda").manual_seed(11)
        mk = lambda h: torch.randn(S, h, d, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        q, k, v, do = mk(H), mk(Hk), mk(Hk), mk(H)
        share = S // world
        sl = slice(rank * share, (rank + 1) * share)
        ql, kl, vl = (t[sl].clone().requires_grad_(True) for t in (q, k, v))
        out = sharding.moba_query_range(ql, kl, vl, S, chunk, topk)
        out.backward(do[sl])
        cu = torch.tensor([0, S], dtype=torch.int32, device="cuda")
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        ref = F.flash_moba_varlen_func(qf, kf, vf, cu, cu, S, S, chunk, topk, causal=True)
        dq, dk, dv = torch.autograd.grad(ref, (qf, kf, vf), do)
        torch.cuda.synchronize()
        ret[rank] = [
            float((out.float() - ref[sl].float()).abs().max()),
            float((ql.grad.float() - dq[sl].float()).abs().max()),
            float((kl.grad.float() - dk[sl].float()).abs().max() / dk.float().abs().max()),
            float((vl.grad.float() - dv[sl].float()).abs().max() / dv.float().abs().max()),
        ]
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", [2, 4])
def test_query_range_ranks_nccl(world):
    """The query-range split as NCCL ranks (centroids pooled per rank and gathered with K and V,
    gating overlapped with the K/V gathers, dK/dV reduce-scattered): O and dQ bit-identical to the
    unsplit call, dK/dV to bf16 rounding of the per-rank partial sums."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(500)
    for p in procs:
        if p.is_alive():
            p.kill()
        assert p.exitcode == 0
    for r in range(world):
        e = ret[r]
        assert e[0] == 0.0 and e[1] == 0.0, e
        assert e[2] < 0.02 and e[3] < 0.02, e
