"""Loader of the reference's own CUDA extension, built by oracle/build_ref.sh (test infrastructure).

The extension (module flash_moba_cuda, oracle/_ref/flash_moba_cuda.so) is the reference's
unmodified C++/CUDA, trimmed to the head-dim 64 / 128 / 256 bf16 causal instantiations; this file only
opens it and calls its four bound functions the way the reference's Python layer does
(flash_moba/flash_moba_interface.py:86-111, 148-160, 200-224, 312-342).  Mean pooling in the
reference is a Triton kernel of its Python package, which is not part of the extension: callers
pass pooled centroids.  Used to compare this library's results with the reference's kernels on
the same GPU and to time those kernels beside this library's; never imported by the product.
"""
import ctypes
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "_ref", "flash_moba_cuda.so")


def available() -> bool:
    return os.path.exists(SO)


_mod = None


def module():
    """The extension module.  Opened with lazy binding: the instantiations left out of the trimmed
    build are undefined symbols that are only missed if a call dispatches to them."""
    global _mod
    if _mod is None:
        import torch  # noqa: F401  (its libraries must be loaded first)
        flags = sys.getdlopenflags()
        sys.setdlopenflags(os.RTLD_LAZY | os.RTLD_GLOBAL)
        try:
            spec = importlib.util.spec_from_file_location("flash_moba_cuda", SO)
            _mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(_mod)
        finally:
            sys.setdlopenflags(flags)
    return _mod


def fused_topk(q, km, cu_q, cu_k, cu_km, max_q, max_k, topk, chunk, causal=True):
    """(col_offsets, col_nnz, indices) with sorted columns, as flash_topk_varlen_func returns them."""
    m = module()
    col_offsets, col_nnz, indices, _, _ = m.moba_fused_topk(q, km, cu_q, cu_k, cu_km, max_q, max_k, topk, chunk, causal)
    ends = col_offsets.view(-1) + col_nnz.view(-1)
    return col_offsets, col_nnz, m.varlen_sort(col_offsets.view(-1), ends, indices)


def attn_fwd(q, k, v, cu_q, cu_k, max_q, max_k, col_offsets, col_nnz, indices, lg_block_m, chunk, scale, causal=True):
    out, lse, _, _ = module().moba_varlen_fwd(q, k, v, None, col_offsets, col_nnz, indices, cu_q, cu_k, None, None,
                                             None, max_q, max_k, 0.0, scale, False, causal, 0.0, False, lg_block_m,
                                             chunk, None)
    return out, lse


def attn_bwd(dout, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, col_offsets, col_nnz, indices, lg_block_m, chunk,
             scale, causal=True):
    import torch
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    module().moba_varlen_bwd(dout, q, k, v, out, lse, dq, dk, dv, col_offsets, col_nnz, indices, cu_q, cu_k, None,
                             max_q, max_k, 0.0, scale, False, causal, 0.0, False, lg_block_m, chunk, None, None)
    return dq, dk, dv
