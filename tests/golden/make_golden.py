"""Generate the golden vectors under tests/golden/ from the reference's own pure-PyTorch code.

Run once in a container that has the reference checkout (CPU only, no GPU needed):

    python tests/golden/make_golden.py /path/to/reference

It imports, unmodified, the reference's
  * tests/test_triton_mean_pool.py::mean_pool_torch_gappy
  * tests/test_fused_topk.py::moba_fused_topk_ref
  * tests/test_fused_topk_epilogue.py::indices_epilogue_thread_pool
  * flash_moba/moba_test_utils.py::{attention_moba_sparse_ref, prepare_moba_ref_mask,
    generate_moba_params_from_sparse_mask}
(the compiled extension ``flash_moba_cuda`` and ``triton`` kernels are stubbed: none of the
functions above touches them) and stores inputs + reference outputs as compressed .npz.
The files are small on purpose; nothing of the reference's source is copied.
"""
import importlib.util
import math
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load_reference(ref_root):
    sys.modules.setdefault("flash_moba_cuda", types.ModuleType("flash_moba_cuda"))
    sys.path.insert(0, ref_root)

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    utils = load("ref_moba_test_utils", "flash_moba/moba_test_utils.py")
    topk = load("ref_test_fused_topk", "tests/test_fused_topk.py")
    epi = load("ref_test_fused_topk_epilogue", "tests/test_fused_topk_epilogue.py")
    pool = load("ref_test_triton_mean_pool", "tests/test_triton_mean_pool.py")
    return utils, topk, epi, pool


def bits(x):
    """bf16/fp16 tensors are stored as their 16-bit patterns."""
    if x.dtype in (torch.bfloat16, torch.float16):
        return x.view(torch.int16).numpy()
    return x.numpy()


def cu(lens):
    return torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)


def make_pool(pool, out):
    cases = [  # (seqlens, Hk, d, chunk)
        ([100, 0, 257, 64], 2, 64, 64),
        ([37, 5], 3, 32, 128),          # chunk > every sequence
        ([0, 0], 2, 64, 32),            # all empty
        ([512], 2, 128, 128),
    ]
    for i, (lens, hk, d, c) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + i)
        k = torch.randn(sum(lens), hk, d, generator=g).to(torch.bfloat16)
        ref = pool.mean_pool_torch_gappy(k, cu(lens), c)
        out[f"pool{i}_lens"] = np.array(lens)
        out[f"pool{i}_chunk"] = np.array(c)
        out[f"pool{i}_k"] = bits(k)
        out[f"pool{i}_km"] = bits(ref)
    out["pool_n"] = np.array(len(cases))


def make_gate(topk_mod, epi, out):
    cases = [  # (B, H, S, d, chunk, topk, causal)
        (2, 4, 256, 64, 32, 4, True),
        (2, 4, 256, 64, 32, 4, False),
        (1, 2, 128, 128, 16, 16, True),     # topk > chunks available early in the sequence
        (3, 2, 64, 32, 16, 8, False),       # topk > number of chunks
        (1, 2, 96, 64, 1, 3, True),         # chunk size 1
    ]
    for i, (B, H, S, d, c, kk, causal) in enumerate(cases):
        g = torch.Generator().manual_seed(200 + i)
        q = torch.randn(B * S, H, d, generator=g).to(torch.bfloat16)
        k = torch.randn(B * S, H, d, generator=g).to(torch.bfloat16)
        cs = cu([S] * B)
        vals, inds = topk_mod.moba_fused_topk_ref(q, k, cs, cs, kk, c, causal)
        inds = inds[:, :, :kk].contiguous()
        # CSC pattern of those lists, by the reference's row-order scatter
        ncol = (S + c - 1) // c
        nnz = torch.zeros(B, H, ncol, dtype=torch.int64)
        for b in range(B):
            sel = inds[b * S:(b + 1) * S]
            for h in range(H):
                s = sel[:, h].flatten()
                nnz[b, h] = torch.bincount(s[s >= 0].long(), minlength=ncol)
        base = torch.tensor([[(b * S * H + S * h) * kk for h in range(H)] for b in range(B)])
        col_offsets = base[..., None] + torch.cumsum(nnz, -1) - nnz
        flat = torch.zeros(B * S * H * kk, dtype=torch.int32)
        flat_ref, nnz_ref = epi.indices_epilogue_thread_pool(
            col_offsets, nnz.to(torch.int32), flat, inds, cs, kk, max_workers=4)
        out[f"gate{i}_cfg"] = np.array([B, H, S, d, c, kk, int(causal)])
        out[f"gate{i}_q"] = bits(q)
        out[f"gate{i}_k"] = bits(k)
        out[f"gate{i}_idx"] = inds.numpy().astype(np.int32)
        out[f"gate{i}_val"] = vals[:, :, :kk].numpy().astype(np.float32)
        out[f"gate{i}_col_offsets"] = col_offsets.numpy()
        out[f"gate{i}_col_nnz"] = nnz_ref.numpy()
        out[f"gate{i}_indices"] = flat_ref.numpy()
    out["gate_n"] = np.array(len(cases))


def make_attn(utils, out):
    cases = [  # (lens_q, lens_k, H, Hk, d, chunk, topk, causal)
        ([130, 64], [130, 64], 4, 4, 64, 64, 3, True),
        ([200, 77], [200, 77], 4, 2, 32, 64, 2, False),
        ([50, 128], [190, 128], 2, 1, 64, 64, 2, True),    # len_q < len_k, bottom-right causal
        ([140, 64], [140, 64], 2, 1, 160, 64, 2, True),    # a head dim above 128 (tests/test_moba_attn.py:48)
    ]
    for i, (lq, lk, H, Hk, d, c, kk, causal) in enumerate(cases):
        torch.manual_seed(300 + i)
        B, Sq, Sk = len(lq), max(lq), max(lk)
        q = torch.randn(B, Sq, H, d).to(torch.bfloat16)
        k = torch.randn(B, Sk, Hk, d).to(torch.bfloat16)
        v = torch.randn(B, Sk, Hk, d).to(torch.bfloat16)
        do = torch.randn(B, Sq, H, d).to(torch.bfloat16)
        qm = torch.arange(Sq)[None] < torch.tensor(lq)[:, None]
        km = torch.arange(Sk)[None] < torch.tensor(lk)[:, None]
        cq, ck = cu(lq), cu(lk)
        mask = utils.generate_moba_sparse_mask_topk(cq, ck, Sq, Sk, c, H, top_k=kk, causal=causal, device="cpu")
        co, cn, ri = utils.generate_moba_params_from_sparse_mask(mask, cq, ck, c, Sk)
        mref = utils.prepare_moba_ref_mask(mask, c, Sq, Sk, device="cpu")
        res = {}
        for tag, kw in (("fp32", {}), ("lowp", dict(upcast=False, reorder_ops=True))):
            qq, kk_, vv = [t.clone().requires_grad_(True) for t in (q, k, v)]
            o, _ = utils.attention_moba_sparse_ref(qq, kk_, vv, mref, c, qm, km, causal=causal, **kw)
            dq, dk, dv = torch.autograd.grad(o, (qq, kk_, vv), do * qm[..., None, None])
            res[tag] = (o, dq, dk, dv)
        out[f"attn{i}_cfg"] = np.array([H, Hk, d, c, kk, int(causal)])
        out[f"attn{i}_lq"] = np.array(lq)
        out[f"attn{i}_lk"] = np.array(lk)
        for n, t in (("q", q), ("k", k), ("v", v), ("do", do)):
            out[f"attn{i}_{n}"] = bits(t)
        out[f"attn{i}_mask"] = mask.numpy()
        out[f"attn{i}_col_offsets"] = co.numpy()
        out[f"attn{i}_col_nnz"] = cn.numpy()
        out[f"attn{i}_indices"] = ri.numpy()
        for tag, (o, dq, dk, dv) in res.items():
            # fp32-mode outputs are kept before the final rounding to bf16 is visible: the
            # reference rounds to the input dtype, so store exactly what it returns.
            for n, t in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
                out[f"attn{i}_{tag}_{n}"] = bits(t.detach())
    out["attn_n"] = np.array(len(cases))


def make_c1(utils, topk_mod, out):
    """End-to-end CPU-runnable configuration: 2 sequences {1024, 2048}, 8 heads, d 64,
    causal, chunk 128, top-k 4, q/k/v ~ N(0,1) fp32 from seed 0.  Inputs are regenerated
    from the seed by the tests; only outputs are stored (indices in full, O subsampled)."""
    torch.manual_seed(0)
    lens, H, d, c, kk = [1024, 2048], 8, 64, 128, 4
    T = sum(lens)
    q, k, v = torch.randn(T, H, d), torch.randn(T, H, d), torch.randn(T, H, d)
    cs = cu(lens)
    _, inds = topk_mod.moba_fused_topk_ref(q, k, cs, cs, kk, c, True)
    inds = inds[:, :, :kk]
    outs = []
    for b, L in enumerate(lens):
        s, e = int(cs[b]), int(cs[b + 1])
        ncol = math.ceil(L / c)
        mask = torch.zeros(1, H, L, ncol, dtype=torch.bool)
        sel = inds[s:e].long()                                 # (L,H,kk)
        for j in range(kk):
            ok = sel[..., j] >= 0
            r, h = torch.nonzero(ok, as_tuple=True)
            mask[0, h, r, sel[r, h, j]] = True
        mref = utils.prepare_moba_ref_mask(mask, c, L, L, device="cpu")
        o, _ = utils.attention_moba_sparse_ref(q[None, s:e], k[None, s:e], v[None, s:e], mref, c, causal=True)
        outs.append(o[0])
    o = torch.cat(outs, 0)
    out["c1_idx"] = inds.numpy().astype(np.int16)
    out["c1_rows"] = np.arange(0, T, 16)
    out["c1_o"] = o[::16].numpy().astype(np.float32)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of mit-han-lab/flash-moba>")
    ref_root = sys.argv[1]
    utils, topk_mod, epi, pool = _load_reference(ref_root)
    for name, fn, args in (("pool", make_pool, (pool,)), ("gate", make_gate, (topk_mod, epi)),
                           ("attn", make_attn, (utils,)), ("c1", make_c1, (utils, topk_mod))):
        out = {}
        fn(*args, out)
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **out)
        print(name, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
