"""Times the reference's own CUDA kernels (oracle/_ref, built by oracle/build_ref.sh for sm_100)
beside this library's on one GPU, same inputs, CUDA events, L2-exceeding inputs.

    python oracle/time_ref_cuda.py [--tokens 65536] [--heads 32] [--head-dim 128] [--chunk 128] [--topk 8] [--steps 5]

Prints one JSON line.  The reference's mean pool is a Triton kernel of its Python package (not part
of the extension): both sides get the centroids from this library's pool, and the pool is timed
on this library's side only.  Test infrastructure: nothing in the product imports this file.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import ref_cuda  # noqa: E402


def _time(fn, steps, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--chunk", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128, choices=[64, 128, 256])
    ap.add_argument("--steps", type=int, default=5)
    a = ap.parse_args()
    if not ref_cuda.available():
        print(json.dumps({"unavailable": "oracle/_ref/flash_moba_cuda.so not built (bash oracle/build_ref.sh <reference>)"}))
        return
    import flash_moba_b200 as F
    from flash_moba_b200 import ops
    from flash_moba_b200.interface import decide_lg_block_m
    torch.manual_seed(0)
    T, H, d, C, K = a.tokens, a.heads, a.head_dim, a.chunk, a.topk
    q, k, v, do = (torch.randn(T, H, d, device="cuda", dtype=torch.bfloat16) for _ in range(4))
    cs = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    scale = d ** -0.5
    lg_m = decide_lg_block_m(K, C, T, True)
    km, cu_km = ops.mean_pool(k, cs, T, C)
    res = {"tokens": T, "heads": H, "head_dim": d, "chunk": C, "topk": K, "lg_block_m": lg_m, "steps": a.steps}

    # reference kernels
    pat = ref_cuda.fused_topk(q, km, cs, cs, cu_km, T, T, K, C, True)
    out_r, lse_r = ref_cuda.attn_fwd(q, k, v, cs, cs, T, T, *pat, lg_m, C, scale)
    res["reference_ms"] = {
        "topk_and_sort": _time(lambda: ref_cuda.fused_topk(q, km, cs, cs, cu_km, T, T, K, C, True), a.steps),
        "fwd": _time(lambda: ref_cuda.attn_fwd(q, k, v, cs, cs, T, T, *pat, lg_m, C, scale), a.steps),
        "bwd": _time(lambda: ref_cuda.attn_bwd(do, q, k, v, out_r, lse_r, cs, cs, T, T, *pat, lg_m, C, scale), a.steps),
    }
    # this library, same pattern for the attention calls
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))

    def mine_fwd():
        return F.flash_moba_attn_varlen_func(qg, kg, vg, cs, cs, T, T, *pat, lg_m, C, causal=True)

    out_m = mine_fwd()
    res["this_library_ms"] = {
        "pool": _time(lambda: ops.mean_pool(k, cs, T, C), a.steps),
        "topk_and_pattern": _time(lambda: F.flash_topk_varlen_func(q, k, cs, cs, T, T, K, C, causal=True), a.steps),
        "fwd": _time(lambda: mine_fwd(), a.steps),
        "fwd_and_bwd": _time(lambda: torch.autograd.grad(mine_fwd(), (qg, kg, vg), do), a.steps),
    }
    res["max_abs_diff_out"] = (out_m.detach().float() - out_r.float()).abs().max().item()
    r, m = res["reference_ms"], res["this_library_ms"]
    res["reference_fwd_bwd_ms"] = r["fwd"] + r["bwd"]
    res["speedup_fwd_bwd"] = (r["fwd"] + r["bwd"]) / m["fwd_and_bwd"]
    print(json.dumps(res))


if __name__ == "__main__":
    main()
