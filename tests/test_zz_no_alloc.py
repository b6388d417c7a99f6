"""The allocation-free pattern builder (fmb_build_csc_static), called through the C ABI.

It serves hosts that cannot give the library a workspace because they may not allocate
device memory while running (a runtime that owns all of it, or a pass-through FFI shim).
Its scratch is a fixed device array inside the library, shared by every call and never
cleared, so the test makes two calls in a row with different inputs and requires each to
equal, bit for bit, what the workspace-taking entry point returns.  The file sorts last so
that a `-x` run has already exercised everything else when it gets here; it also passes
when run alone in a fresh process (the first call performs the per-device address lookup).
"""
import pytest
import torch

from conftest import cu_of

pytestmark = pytest.mark.gpu


def _random_lists(lens, heads, topk, chunk, seed):
    g = torch.Generator().manual_seed(seed)
    total = sum(lens)
    idx = torch.full((total, heads, topk), -1, dtype=torch.int32)
    row = 0
    for length in lens:
        for t in range(length):
            avail = t // chunk + 1
            for h in range(heads):
                k = min(topk, avail)
                idx[row, h, :k] = torch.randperm(avail, generator=g)[:k].to(torch.int32)
            row += 1
    return idx


def _call_static(idx, cu, max_q, ncol):
    from flash_moba_b200 import _lib
    total, heads, topk = idx.shape
    batch = cu.numel() - 1
    col_offsets = torch.empty((batch, heads, ncol), dtype=torch.int64, device=idx.device)
    col_nnz = torch.empty((batch, heads, ncol), dtype=torch.int32, device=idx.device)
    indices = torch.empty((total * heads * topk,), dtype=torch.int32, device=idx.device)
    rc = _lib.lib.fmb_build_csc_static(idx.data_ptr(), idx.stride(0), idx.stride(1), cu.data_ptr(),
                                       col_offsets.data_ptr(), col_nnz.data_ptr(), indices.data_ptr(),
                                       batch, heads, topk, max_q, ncol, torch.cuda.current_stream().cuda_stream)
    return rc, (col_offsets, col_nnz, indices)


def test_static_scratch_builder_matches_workspace_builder_twice():
    from flash_moba_b200 import _lib, ops
    assert _lib.lib.fmb_build_csc_static_capacity() == 8 << 20
    cases = [([700, 300], 3, 4, 32, 11), ([1500], 2, 6, 16, 12)]   # second call: other shapes, stale scratch
    for lens, heads, topk, chunk, seed in cases:
        idx = _random_lists(lens, heads, topk, chunk, seed).cuda()
        cu = cu_of(lens).cuda()
        ncol = (max(lens) + chunk - 1) // chunk
        want = ops.build_csc(idx, cu, max(lens), ncol)
        rc, got = _call_static(idx, cu, max(lens), ncol)
        assert rc == 0, _lib.lib.fmb_last_error()
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)


def test_static_scratch_builder_rejects_oversize():
    from flash_moba_b200 import _lib
    idx = torch.zeros((8, 1, 1), dtype=torch.int32, device="cuda")
    cu = cu_of([8]).cuda()
    # 64 heads x 256 tiles x 512 columns of counters = 32 MiB > 8 MiB: refused before any launch
    rc = _lib.lib.fmb_build_csc_static(idx.data_ptr(), 1, 1, cu.data_ptr(), 1, 1, 1, 1, 64, 1, 512 * 256, 512,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 3
    assert b"built-in array" in _lib.lib.fmb_last_error()


def test_static_scratch_builder_at_its_capacity():
    """The largest problem the built-in array holds: exactly 2,097,152 counters (one sequence of
    65,536 rows x 8 heads = 128 tiles, 2,048 columns), the last counter of the array in use.  Same
    pattern as the workspace-taking builder, and no device memory is taken or returned by the call
    (outputs allocated beforehand).  One column more is refused."""
    from flash_moba_b200 import _lib, ops
    rows, heads, topk, ncol = 65536, 8, 2, 2048
    assert heads * (rows // 512) * ncol * 4 == 8 << 20
    g = torch.Generator().manual_seed(21)
    idx = torch.randint(0, ncol, (rows, heads, topk), generator=g, dtype=torch.int32)
    idx[:, :, 1] = torch.where(idx[:, :, 1] == idx[:, :, 0], (idx[:, :, 0] + 1) % ncol, idx[:, :, 1])
    idx = idx.cuda()
    cu = cu_of([rows]).cuda()
    want = ops.build_csc(idx, cu, rows, ncol)
    col_offsets = torch.empty((1, heads, ncol), dtype=torch.int64, device="cuda")
    col_nnz = torch.empty((1, heads, ncol), dtype=torch.int32, device="cuda")
    indices = torch.empty((rows * heads * topk,), dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = _lib.lib.fmb_build_csc_static(idx.data_ptr(), idx.stride(0), idx.stride(1), cu.data_ptr(),
                                       col_offsets.data_ptr(), col_nnz.data_ptr(), indices.data_ptr(),
                                       1, heads, topk, rows, ncol, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.lib.fmb_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    for a, b in zip((col_offsets, col_nnz, indices), want):
        assert torch.equal(a, b)
    rc = _lib.lib.fmb_build_csc_static(idx.data_ptr(), idx.stride(0), idx.stride(1), cu.data_ptr(),
                                       col_offsets.data_ptr(), col_nnz.data_ptr(), indices.data_ptr(),
                                       1, heads, topk, rows, ncol + 1, torch.cuda.current_stream().cuda_stream)
    assert rc == 3
