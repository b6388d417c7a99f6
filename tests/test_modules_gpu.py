"""Model-level wrappers and the forward op's key-span arguments.

  * `leftpad_k` / `seqused_k` of `flash_moba::_flash_moba_attn_varlen_forward` (the reference's
    csrc/flash_moba/src/block_info.h:19-26): keys stored with padding in front and unused rows behind
    give bit for bit what the same keys give when packed;
  * `CentroidCache`: decoding token by token against cached centroids equals gating from scratch,
    and the cached table equals pooling the whole key sequence;
  * `MobaAttention` equals the functional call.
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from conftest import cu_of  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("engine", [0, 1])
def test_leftpad_and_seqused_equal_packed_keys(engine, d):
    import flash_moba_b200 as F
    from flash_moba_b200 import ops
    ops.set_engine(engine)
    try:
        torch.manual_seed(4)
        H, Hk, chunk, topk = 4, 2, 128, 3
        lens_q, lens_k, pad, slack = [200, 77], [520, 333], [64, 8], [40, 0]
        q = torch.randn(sum(lens_q), H, d, device=DEV).bfloat16()
        ks = [torch.randn(n, Hk, d, device=DEV).bfloat16() for n in lens_k]
        vs = [torch.randn(n, Hk, d, device=DEV).bfloat16() for n in lens_k]
        junk = lambda n: torch.full((n, Hk, d), float("nan"), device=DEV).bfloat16()
        k_packed, v_packed = torch.cat(ks), torch.cat(vs)
        k_store = torch.cat([t for i in range(2) for t in (junk(pad[i]), ks[i], junk(slack[i]))])
        v_store = torch.cat([t for i in range(2) for t in (junk(pad[i]), vs[i], junk(slack[i]))])
        cu_q, cu_k = cu_of(lens_q).to(DEV), cu_of(lens_k).to(DEV)
        cu_store = cu_of([pad[i] + lens_k[i] + slack[i] for i in range(2)]).to(DEV)
        leftpad = torch.tensor(pad, dtype=torch.int32, device=DEV)
        seqused = torch.tensor([pad[i] + lens_k[i] for i in range(2)], dtype=torch.int32, device=DEV)
        mq, mk = max(lens_q), max(lens_k)
        pattern = F.flash_topk_varlen_func(q, k_packed, cu_q, cu_k, mq, mk, topk, chunk, causal=True)
        scale = d ** -0.5
        ref = torch.ops.flash_moba._flash_moba_attn_varlen_forward(
            q, k_packed, v_packed, cu_q, cu_k, mq, mk, *pattern, 128, chunk, 0.0, scale, True)
        got = torch.ops.flash_moba._flash_moba_attn_varlen_forward(
            q, k_store, v_store, cu_q, cu_store, mq, mk, *pattern, 128, chunk, 0.0, scale, True,
            leftpad_k=leftpad, seqused_k=seqused)
        assert torch.equal(ref[0], got[0]) and torch.equal(ref[1], got[1])
        assert not torch.isnan(got[0].float()).any()
        with pytest.raises(RuntimeError, match="shape"):
            torch.ops.flash_moba._flash_moba_attn_varlen_forward(
                q, k_store, v_store, cu_q, cu_store, mq, mk, *pattern, 128, chunk, 0.0, scale, True,
                leftpad_k=leftpad[:1].contiguous())
    finally:
        ops.set_engine(1)


def test_centroid_cache_decoding_equals_gating_from_scratch():
    import flash_moba_b200 as F
    from flash_moba_b200 import ops
    from flash_moba_b200.modules import CentroidCache
    torch.manual_seed(9)
    B, H, Hk, d, chunk, topk = 2, 4, 2, 128, 128, 3
    lens = [300, 515]
    ks = [torch.randn(n, Hk, d, device=DEV).bfloat16() for n in lens]
    vs = [torch.randn(n, Hk, d, device=DEV).bfloat16() for n in lens]
    cache = CentroidCache(B, Hk, d, chunk, max_seqlen_k=1024, device=DEV)
    cu_q = cu_of([1] * B).to(DEV)
    for step in range(131):       # crosses a chunk boundary in both sequences
        if step > 0:
            for b in range(B):
                ks[b] = torch.cat([ks[b], torch.randn(1, Hk, d, device=DEV).bfloat16()])
                vs[b] = torch.cat([vs[b], torch.randn(1, Hk, d, device=DEV).bfloat16()])
                lens[b] += 1
        k, v = torch.cat(ks), torch.cat(vs)
        cu_k = cu_of(lens)
        cache.update(k, cu_k, lens)
        if step % 10 and step not in (84, 85, 86, 125, 126):
            continue              # the cache is updated every step; compared at a sample of steps
        q = torch.randn(B, H, d, device=DEV).bfloat16()
        mk = max(lens)
        got = cache.attend(q, k, v, cu_q, cu_k.to(DEV), 1, mk, topk)
        ref = F.flash_moba_varlen_func(q, k, v, cu_q, cu_k.to(DEV), 1, mk, chunk, topk, causal=True)
        assert torch.equal(got, ref), step
    km_full, cu_km = ops.mean_pool(torch.cat(ks), cu_of(lens).to(DEV), max(lens), chunk)
    for b in range(B):
        n = (lens[b] + chunk - 1) // chunk
        a = int(cu_km[b])
        assert torch.equal(cache.km[b * cache.capacity_chunks:b * cache.capacity_chunks + n], km_full[a:a + n])


def test_module_equals_functional():
    import flash_moba_b200 as F
    from flash_moba_b200.modules import MobaAttention
    torch.manual_seed(2)
    lens, H, Hk, d = [640, 130], 4, 4, 64
    q, k, v = (torch.randn(sum(lens), h, d, device=DEV).bfloat16().requires_grad_(True) for h in (H, Hk, Hk))
    cu = cu_of(lens).to(DEV)
    m = MobaAttention(chunk_size=128, topk=2)
    out = m(q, k, v, cu, cu, max(lens), max(lens))
    ref = F.flash_moba_varlen_func(q, k, v, cu, cu, max(lens), max(lens), 128, 2, causal=True)
    assert torch.equal(out, ref)
    g1 = torch.autograd.grad(out, (q, k, v), torch.ones_like(out))
    g2 = torch.autograd.grad(ref, (q, k, v), torch.ones_like(ref))
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)
