"""CPU-only checks of the boundary: the library loads, exports every symbol the header
declares, and argument validation fails with the reference's style of RuntimeError."""
import os
import re

import pytest
import torch

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "flash_moba_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fmb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from flash_moba_b200 import _lib
    names = _declared()
    assert len(names) >= 12
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.EXPORTS, f"{n} has no ctypes signature"
    assert _lib.lib.fmb_version() >= 100


def test_workspace_size_queries_need_no_gpu():
    from flash_moba_b200 import _lib
    f = _lib.lib.fmb_attn_fwd_workspace_bytes
    small = f(1024, 4, 4, 64, 1024 * 4 * 4, 1, 1024, 64, 0)
    big = f(2048, 4, 4, 64, 2048 * 4 * 4, 1, 2048, 64, 0)
    assert 0 < small < big
    # passes over half of the heads need about half of the partial storage
    assert f(2048, 4, 4, 64, 2048 * 4 * 4, 1, 2048, 64, 2) < 0.6 * big
    # whole kv-head groups only: asking for 1 head of a group of 2 gives the 2-head size
    assert f(2048, 4, 2, 64, 2048 * 4 * 4, 1, 2048, 64, 1) == f(2048, 4, 2, 64, 2048 * 4 * 4, 1, 2048, 64, 2)
    # a 256-key chunk is two 128-key blocks: twice the partial storage
    assert f(2048, 4, 4, 64, 2048 * 4 * 4, 1, 2048, 256, 0) > 1.8 * f(2048, 4, 4, 64, 2048 * 4 * 4, 1, 2048, 128, 0)
    assert _lib.lib.fmb_build_csc_workspace_bytes(2, 4, 1000, 8) >= 2 * 4 * 2 * 8 * 4
    assert _lib.lib.fmb_attn_bwd_workspace_bytes(1024, 4, 4, 64, 4096, 1, 1024, 64, 0) > 4096 * 64 * 2   # dQ partials in the I/O dtype


def test_bad_arguments_are_rejected_before_any_launch():
    from flash_moba_b200 import _lib
    rc = _lib.lib.fmb_gate_topk(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 4, 4, 64, 16, 16, 65, 16, 1, 0, 0)
    assert rc == 1 and b"moba_topk" in _lib.lib.fmb_last_error()
    rc = _lib.lib.fmb_mean_pool(0, 0, 0, 0, 0, 0, 1, 4, 60, 16, 16, 0, 0)
    assert rc == 1 and b"multiple of 8" in _lib.lib.fmb_last_error()
    rc = _lib.lib.fmb_mean_pool(0, 0, 0, 0, 0, 0, 1, 4, 64, 16, 16, 7, 0)
    assert rc == 1 and b"fp16 and bf16" in _lib.lib.fmb_last_error()
    with pytest.raises(RuntimeError):
        _lib.check(rc)


def test_public_api_surface_matches_reference_names():
    import inspect

    import flash_moba_b200 as F
    sig = inspect.signature(F.flash_moba_varlen_func)
    assert list(sig.parameters) == ["q", "k", "v", "cu_seqlens_q", "cu_seqlens_k", "max_seqlen_q", "max_seqlen_k",
                                    "moba_chunk_size", "moba_topk", "causal"]
    assert sig.parameters["causal"].default is True
    sig = inspect.signature(F.flash_topk_varlen_func)
    assert list(sig.parameters)[6:] == ["moba_topk", "moba_chunk_size", "causal"]
    assert sig.parameters["causal"].default is False
    sig = inspect.signature(F.flash_moba_attn_varlen_func)
    assert list(sig.parameters)[7:] == ["moba_col_offsets", "moba_col_nnz", "moba_row_indices", "lg_block_m",
                                        "lg_block_n", "dropout_p", "softmax_scale", "causal", "softcap",
                                        "alibi_slopes", "deterministic", "return_attn_probs"]
    for op in ("_moba_fused_topk", "_varlen_sort", "_flash_moba_attn_varlen_forward",
               "_flash_moba_attn_varlen_backward"):
        assert hasattr(torch.ops.flash_moba, op)


def test_no_cpu_path():
    import flash_moba_b200 as F
    x = torch.randn(8, 2, 64).bfloat16()
    cu = torch.tensor([0, 8], dtype=torch.int32)
    with pytest.raises(RuntimeError):
        F.flash_moba_varlen_func(x, x, x, cu, cu, 8, 8, 64, 2)


def test_fake_impls_give_reference_shapes():
    q = torch.empty(10, 4, 64, device="meta", dtype=torch.bfloat16)
    cu = torch.empty(3, device="meta", dtype=torch.int32)
    co, cn, ind = torch.ops.flash_moba._moba_fused_topk(q, q, cu, cu, cu, 6, 6, 2, 2, True)
    assert co.shape == (2, 4, 3) and co.dtype == torch.int64
    assert cn.shape == (2, 4, 3) and cn.dtype == torch.int32
    assert ind.shape == (10 * 4 * 2,)


def test_decide_lg_block_m_matches_reference_table():
    import flash_moba_b200 as F
    assert F.decide_lg_block_m(8, 128, 65536, True) == 1024
    assert F.decide_lg_block_m(8, 128, 2048, True) == 128
    assert F.decide_lg_block_m(8, 128, 4096, True) == 256
    assert F.decide_lg_block_m(4, 128, 1024, False) == 128
