"""Thin PyTorch wrappers over the C ABI: allocate outputs and workspaces with the torch
caching allocator, pass raw device pointers + the current CUDA stream.  One function per
stage; `flash_moba_b200.interface` composes them into the reference's public API.

The arithmetic lives entirely in libflashmoba_b200.so; nothing here computes on tensors.
"""
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import check, lib


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.FMB_BF16
    if t.dtype == torch.float16:
        return _lib.FMB_FP16
    raise RuntimeError("FlashMoBA only supports fp16 and bf16 data type")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flash_moba_b200: all tensors must be on a CUDA device (there is no CPU path)")


def _i32c(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32:
        raise RuntimeError(f"{name} must have dtype int32")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    return t


def _last_contig(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.stride(-1) != 1:
        raise RuntimeError(f"{name} must have contiguous last dimension")
    return t


def ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


# ---- the pattern's slot / row lists, handed from a forward call to its backward call
# Both attention calls build the same CSR transpose of the pattern in their workspace.  attn_fwd
# keeps a copy of it (a few bytes per pattern entry) that the autograd Function collects with
# take_lists() right after its forward op and offers to the backward op with offer_lists(); the
# custom ops' signatures stay the reference's.  FMB_SHARE_LISTS=0 turns the hand-over off.
import threading as _threading

_tls = _threading.local()


def _share_lists() -> bool:
    import os
    return os.environ.get("FMB_SHARE_LISTS", "1") != "0"


def _lists_key(col_offsets, col_nnz, indices, cu_seqlens_q, total_q, h, hk, d, batch, max_seqlen_k, chunk):
    """What the lists depend on: the pattern tensors and the sequence bounds (storage and version), the geometry."""
    ident = tuple((t.data_ptr(), t._version, t.numel()) for t in (col_offsets, col_nnz, indices, cu_seqlens_q))
    return ident + (int(total_q), h, hk, d, batch, int(max_seqlen_k), int(chunk), str(indices.device))


def take_lists():
    """The lists kept by the last attn_fwd of this thread (None if it kept none); clears the slot."""
    got = getattr(_tls, "kept", None)
    _tls.kept = None
    return got


def offer_lists(lists) -> None:
    """Lists for the next attn_bwd of this thread (used only if they belong to its pattern)."""
    _tls.offered = lists


# ---- the row-major view of a pattern, kept by the pattern builder for the attention calls
# build_csc lets the library write, next to the pattern, where every (row, chunk) pair landed in
# `indices` (fmb_build_csc_rows).  An attention call on exactly that pattern offers those rows to
# the library (fmb_attn_rows_offer) and then launches no list-building kernels of its own.  The
# cache holds the pattern tensors themselves, so a data pointer cannot be reused while its entry
# lives; an in-place write to a pattern tensor changes its version and misses.
import collections as _collections

_rows_cache = _collections.OrderedDict()
_ROWS_CACHE_ENTRIES = 4


def _pattern_key(col_offsets, col_nnz, indices):
    return tuple((t.data_ptr(), t._version, t.numel()) for t in (col_offsets, col_nnz, indices)) + (str(indices.device),)


def _rows_remember(col_offsets, col_nnz, indices, row_slots, topk):
    _rows_cache[_pattern_key(col_offsets, col_nnz, indices)] = (col_offsets, col_nnz, indices, row_slots, topk)
    while len(_rows_cache) > _ROWS_CACHE_ENTRIES:
        _rows_cache.popitem(last=False)


def _rows_offer(col_offsets, col_nnz, indices, total_q, h) -> bool:
    """Offers the builder's rows of this pattern to the next attention call; False if there are none."""
    if not _share_lists():
        return False
    hit = _rows_cache.get(_pattern_key(col_offsets, col_nnz, indices))
    if hit is None:
        return False
    row_slots, topk = hit[3], hit[4]
    if row_slots.numel() != total_q * h * topk or indices.numel() != row_slots.numel():
        return False
    check(lib.fmb_attn_rows_offer(ptr(row_slots), total_q, h, topk))
    return True


def _workspace(query, total_q, h, hk, d, n_indices, batch, max_seqlen_k, chunk, device):
    """Workspace for one attention call: the single-pass size if it fits the cap
    (FMB_WORKSPACE_GB, default 64 GiB of the 180), otherwise the largest pass of whole kv-head groups that
    does; the library then walks the heads in passes of that size."""
    import os
    cap = int(float(os.environ.get("FMB_WORKSPACE_GB", "64")) * (1 << 30))
    group = h // hk
    nh = h
    nbytes = query(total_q, h, hk, d, n_indices, batch, int(max_seqlen_k), int(chunk), nh)
    while nbytes > cap and nh > group:
        nh = max(group, (nh // 2) // group * group)
        nbytes = query(total_q, h, hk, d, n_indices, batch, int(max_seqlen_k), int(chunk), nh)
    return torch.empty((max(nbytes, 1),), dtype=torch.uint8, device=device), nbytes


def _raise_for_status(code: int, what: str) -> None:
    if code == 7:
        raise RuntimeError(f"flash_moba_b200: {what}: the pattern does not fit the slots of a pass "
                           "(overlapping columns, or raise FMB_WORKSPACE_GB)")
    if code != 0:
        raise RuntimeError(f"flash_moba_b200: {what}: a bounded device-side wait expired (code {code})")


# Status words on their way to the host: (event behind the call, ring, slot, which call).  The
# library stores a call's status word straight into mapped pinned memory (fmb_attn_status_mirror),
# so no copy is queued in the stream.
_pending_status = _collections.deque()
_status_rings = {}
_RING = 256
_PENDING = -1


def _drain_status(block: bool) -> None:
    while _pending_status:
        ev, ring, i, what = _pending_status[0]
        if block:
            ev.synchronize()
        elif not ev.query():
            return
        _pending_status.popleft()
        code = int(ring[i])
        _raise_for_status(0 if code == _PENDING else code, what)    # still pending: the call had no rows


def check_pending_status() -> None:
    """Waits for the status words of all attention calls issued so far by this process and raises
    for the first one that reports a failure (see _status_begin)."""
    _drain_status(True)


def _status_begin(dev):
    """Every attention call leaves a device-side status word: 0, or which bounded wait gave up /
    7 = the pattern did not fit the slots.  By default the library mirrors the word into pinned
    host memory at the end of the call, without synchronising, and the attention calls that follow
    (or check_pending_status()) look at it: a failure raises one call late, never silently.  With
    FMB_CHECK_STATUS=1 every call synchronises and raises at once (the tests).  Returns the ticket
    for _status_end."""
    import os
    if os.environ.get("FMB_CHECK_STATUS", "0") == "1":
        return None
    _drain_status(len(_pending_status) >= _RING - 8)
    ring_state = _status_rings.get(dev.index)
    if ring_state is None:
        ring_state = _status_rings[dev.index] = [torch.zeros((_RING,), dtype=torch.int32).pin_memory(), 0]
    ring, i = ring_state
    ring_state[1] = (i + 1) % _RING
    ring[i] = _PENDING
    check(lib.fmb_attn_status_mirror(ring.data_ptr() + 4 * i))
    return ring, i


def _status_end(ticket, ws: torch.Tensor, what: str) -> None:
    if ticket is None:
        _raise_for_status(int(ws[:4].view(torch.int32).item()), what)
        return
    ev = torch.cuda.Event()
    ev.record()
    _pending_status.append((ev, ticket[0], ticket[1], what))


def selftest_umma(a: torch.Tensor, b: torch.Tensor, b_mn_major: bool) -> torch.Tensor:
    """128x128x128 product on the tcgen05 path (see fmb_selftest_umma)."""
    _require_cuda(a, b)
    a, b = a.contiguous(), b.contiguous()
    with torch.cuda.device(a.device):
        d = torch.empty((128, 128), dtype=torch.float32, device=a.device)
        status = torch.zeros((1,), dtype=torch.int32, device=a.device)
        check(lib.fmb_selftest_umma(ptr(a), ptr(b), ptr(d), int(b_mn_major), _dtype_code(a), ptr(status), _stream()))
        if int(status.item()) != 0:
            raise RuntimeError(f"selftest_umma: bounded wait expired (code {int(status.item())})")
    return d


def selftest_wait_expiry(device=None) -> Tuple[int, float]:
    """Runs the library's bounded wait on an mbarrier nobody arrives at (see fmb_selftest_wait_expiry).
    Returns (status code written by the kernel, seconds the wait lasted before it gave up)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        status = torch.full((1,), -1, dtype=torch.int32, device=dev)
        ns = torch.zeros((1,), dtype=torch.int64, device=dev)
        check(lib.fmb_selftest_wait_expiry(ptr(status), ptr(ns), _stream()))
        torch.cuda.synchronize(dev)
    return int(status.item()), int(ns.item()) * 1e-9


def set_engine(engine: int) -> int:
    """0 = CUDA-core validation kernels, 1 = tcgen05 kernels.  Returns the engine in use."""
    return lib.fmb_set_engine(int(engine))


# ------------------------------------------------------------------------------- stage P
def mean_pool(k: torch.Tensor, cu_seqlens_k: torch.Tensor, max_seqlen_k: int, chunk: int
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Centroids of every chunk.  No host sync: km is allocated with an upper bound of
    ceil(total_k/chunk) + batch rows; rows [0, cu_seqlens_km[-1]) are valid."""
    _require_cuda(k, cu_seqlens_k)
    _last_contig(k, "k")
    _i32c(cu_seqlens_k, "cu_seqlens_k")
    total_k, hk, d = k.shape
    batch = cu_seqlens_k.numel() - 1
    rows_ub = (total_k + chunk - 1) // chunk + batch
    with torch.cuda.device(k.device):
        km = torch.empty((rows_ub, hk, d), dtype=k.dtype, device=k.device)
        cu_km = torch.empty((batch + 1,), dtype=torch.int32, device=k.device)
        check(lib.fmb_mean_pool_offsets(ptr(k), k.stride(0), k.stride(1), ptr(cu_seqlens_k), ptr(cu_km), ptr(km),
                                        batch, hk, d, int(max_seqlen_k), chunk, _dtype_code(k), _stream()))
    return km, cu_km


# ------------------------------------------------------------------------------- stage G
def gate_topk(q, km, cu_seqlens_q, cu_seqlens_k, cu_seqlens_km, max_seqlen_q: int, max_seqlen_k: int,
              topk: int, chunk: int, causal: bool, return_values: bool = False):
    """Per-row top-k chunk lists.  Returns idx as a (total_q, heads, topk) VIEW of a
    head-major (heads, total_q, topk) buffer (the layout the pattern builder streams), and
    the scores in the same layout (or None)."""
    _require_cuda(q, km)
    _last_contig(q, "q")
    if not km.is_contiguous():
        raise RuntimeError("km must be contiguous")
    total_q, h, d = q.shape
    hk = km.shape[1]
    batch = cu_seqlens_q.numel() - 1
    with torch.cuda.device(q.device):
        idx = torch.empty((h, total_q, topk), dtype=torch.int32, device=q.device)
        val = torch.empty((h, total_q, topk), dtype=torch.float32, device=q.device) if return_values else None
        check(lib.fmb_gate_topk(ptr(q), q.stride(0), q.stride(1), ptr(km), ptr(_i32c(cu_seqlens_q, "cu_seqlens_q")),
                                ptr(_i32c(cu_seqlens_k, "cu_seqlens_k")), ptr(_i32c(cu_seqlens_km, "cu_seqlens_km")),
                                ptr(idx), ptr(val), topk, total_q * topk, batch, h, hk, d, int(max_seqlen_q),
                                int(max_seqlen_k), int(topk), int(chunk), int(bool(causal)), _dtype_code(q),
                                _stream()))
        import os
        if os.environ.get("FMB_CHECK_STATUS", "0") == "1":
            import ctypes
            code = ctypes.c_int(0)
            check(lib.fmb_gate_status(ctypes.addressof(code)))
            if code.value != 0:
                raise RuntimeError(f"flash_moba_b200: gate_topk: a bounded device-side wait expired (code {code.value})")
    return idx.permute(1, 0, 2), (val.permute(1, 0, 2) if val is not None else None)


# --------------------------------------------------------------------------- stages O/E/S
def build_csc(topk_idx: torch.Tensor, cu_seqlens_q: torch.Tensor, max_seqlen_q: int, ncol: int,
              keep_rows: bool = False):
    """(col_offsets i64 (B,H,ncol), col_nnz i32 (B,H,ncol), indices i32 (T*H*topk)).

    keep_rows: also let the library write the pattern's row-major view and keep it for attention
    calls on the returned tensors (only for lists that name a chunk at most once per row, as the
    lists of gate_topk do)."""
    _require_cuda(topk_idx)
    if topk_idx.dtype != torch.int32 or topk_idx.stride(-1) != 1:
        raise RuntimeError("topk_idx must be int32 with contiguous last dimension")
    total_q, h, topk = topk_idx.shape
    batch = cu_seqlens_q.numel() - 1
    dev = topk_idx.device
    with torch.cuda.device(dev):
        col_offsets = torch.empty((batch, h, ncol), dtype=torch.int64, device=dev)
        col_nnz = torch.empty((batch, h, ncol), dtype=torch.int32, device=dev)
        indices = torch.empty((total_q * h * topk,), dtype=torch.int32, device=dev)
        nbytes = lib.fmb_build_csc_workspace_bytes(batch, h, int(max_seqlen_q), ncol)
        ws = torch.empty((max(nbytes, 1),), dtype=torch.uint8, device=dev)
        if keep_rows and _share_lists() and 0 < indices.numel() < 0xffffffff:
            row_slots = torch.empty((h, total_q, topk), dtype=torch.int32, device=dev)
            check(lib.fmb_build_csc_rows(ptr(topk_idx), topk_idx.stride(0), topk_idx.stride(1),
                                         ptr(_i32c(cu_seqlens_q, "cu_seqlens_q")), ptr(col_offsets), ptr(col_nnz),
                                         ptr(indices), ptr(row_slots), ptr(ws), nbytes, batch, h, topk, total_q,
                                         int(max_seqlen_q), ncol, _stream()))
            _rows_remember(col_offsets, col_nnz, indices, row_slots, topk)
        else:
            check(lib.fmb_build_csc(ptr(topk_idx), topk_idx.stride(0), topk_idx.stride(1),
                                    ptr(_i32c(cu_seqlens_q, "cu_seqlens_q")), ptr(col_offsets), ptr(col_nnz),
                                    ptr(indices), ptr(ws), nbytes, batch, h, topk, int(max_seqlen_q), ncol, _stream()))
    return col_offsets, col_nnz, indices


def varlen_sort(starts: torch.Tensor, ends: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    _require_cuda(starts, ends, src)
    if starts.dtype != torch.int64 or ends.dtype != torch.int64 or src.dtype != torch.int32:
        raise RuntimeError("varlen_sort: offsets must be int64 and keys int32")
    starts, ends, src = starts.contiguous(), ends.contiguous(), src.contiguous()
    with torch.cuda.device(src.device):
        dst = torch.empty_like(src)
        check(lib.fmb_varlen_sort(ptr(starts), ptr(ends), ptr(src), ptr(dst), starts.numel(), src.numel(), _stream()))
    return dst


# ------------------------------------------------------------------------------- stage F
def _check_pattern(col_offsets, col_nnz, indices):
    if col_offsets.dtype != torch.int64:
        raise RuntimeError("moba_col_offsets must have dtype torch.int64")
    if col_nnz.dtype != torch.int32:
        raise RuntimeError("moba_col_nnz must have dtype torch.int32")
    if indices.dtype != torch.int32:
        raise RuntimeError("moba_row_indices must have dtype torch.int32")
    for t, n in ((col_offsets, "moba_col_offsets"), (col_nnz, "moba_col_nnz"), (indices, "moba_row_indices")):
        if not t.is_contiguous():
            raise RuntimeError(f"{n} must be contiguous")
    if col_offsets.shape != col_nnz.shape or col_offsets.dim() != 3:
        raise RuntimeError("moba_col_offsets / moba_col_nnz must both be (batch, heads, ncol)")


def _key_spans(cu_seqlens_k, leftpad_k, seqused_k, batch):
    """(first key row, one past the last key row) per sequence for the reference's leftpad_k /
    seqused_k arguments (csrc/flash_moba/src/block_info.h:19-26): keys start leftpad_k[b] rows into
    the sequence's storage and seqused_k[b] rows of the storage are in use."""
    for t, n in ((leftpad_k, "leftpad_k"), (seqused_k, "seqused_k")):
        if t is not None:
            _require_cuda(t)
            if tuple(_i32c(t, n).shape) != (batch,):
                raise RuntimeError(f"{n} must have shape (batch_size,)")
    begin = cu_seqlens_k[:-1] if leftpad_k is None else cu_seqlens_k[:-1] + leftpad_k
    end = cu_seqlens_k[1:] if seqused_k is None else cu_seqlens_k[:-1] + seqused_k
    return begin.contiguous(), end.contiguous()


def attn_fwd(q, k, v, col_offsets, col_nnz, indices, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int,
             max_seqlen_k: int, chunk: int, softmax_scale: float, causal: bool, out: Optional[torch.Tensor] = None,
             leftpad_k: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None):
    """Block-sparse forward.  Returns (out (T,H,d), lse (H,T) fp32)."""
    _require_cuda(q, k, v, col_offsets, col_nnz, indices)
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _last_contig(t, n)
    if not (q.dtype == k.dtype == v.dtype):
        raise RuntimeError("query, key and value must have the same dtype")
    _check_pattern(col_offsets, col_nnz, indices)
    total_q, h, d = q.shape
    hk = k.shape[1]
    batch = cu_seqlens_q.numel() - 1
    if col_offsets.shape[0] != batch or col_offsets.shape[1] != h:
        raise RuntimeError("pattern shape does not match (batch, heads)")
    ncol_needed = (int(max_seqlen_k) + chunk - 1) // chunk
    if col_offsets.shape[2] != ncol_needed:
        raise RuntimeError(f"pattern has {col_offsets.shape[2]} columns, expected ceil(max_seqlen_k/lg_block_n) = {ncol_needed}")
    dev = q.device
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty_like(q)
        lse = torch.empty((h, total_q), dtype=torch.float32, device=dev)
        ws, nbytes = _workspace(lib.fmb_attn_fwd_workspace_bytes, total_q, h, hk, d, indices.numel(), batch,
                                max_seqlen_k, chunk, dev)
        rows_offered = _rows_offer(col_offsets, col_nnz, indices, total_q, h)
        ticket = _status_begin(dev)
        spans = None
        if leftpad_k is not None or seqused_k is not None:
            spans = _key_spans(_i32c(cu_seqlens_k, "cu_seqlens_k"), leftpad_k, seqused_k, batch)
            check(lib.fmb_attn_key_spans(ptr(spans[0]), ptr(spans[1])))
        check(lib.fmb_attn_fwd(ptr(q), q.stride(0), q.stride(1), ptr(k), k.stride(0), k.stride(1),
                               ptr(v), v.stride(0), v.stride(1), ptr(out), out.stride(0), out.stride(1), ptr(lse),
                               ptr(col_offsets), ptr(col_nnz), ptr(indices), indices.numel(),
                               ptr(_i32c(cu_seqlens_q, "cu_seqlens_q")), ptr(_i32c(cu_seqlens_k, "cu_seqlens_k")),
                               ptr(ws), nbytes, batch, h, hk, d, total_q, int(max_seqlen_q), int(max_seqlen_k),
                               int(chunk), float(softmax_scale), int(bool(causal)), _dtype_code(q), _stream()))
        _status_end(ticket, ws, "attn_fwd")
        _tls.kept = None
        if _share_lists() and indices.numel() > 0 and not rows_offered:
            geo = (total_q, h, hk, d, indices.numel(), batch, int(max_seqlen_k), int(chunk))
            nlist = lib.fmb_attn_lists_bytes(*geo)
            lists = torch.empty((max(nlist, 1),), dtype=torch.uint8, device=dev)
            rc = lib.fmb_attn_lists_save(ptr(ws), nbytes, *geo, ptr(lists), nlist, _stream())
            if rc == 0:
                _tls.kept = (_lists_key(col_offsets, col_nnz, indices, cu_seqlens_q, total_q, h, hk, d, batch,
                                        max_seqlen_k, chunk), lists)
            elif rc != 1:      # 1: the call ran in several passes, nothing to keep
                check(rc)
    return out, lse


# ------------------------------------------------------------------------------- stage B
def attn_bwd(dout, q, k, v, out, lse, dq, dk, dv, col_offsets, col_nnz, indices, cu_seqlens_q, cu_seqlens_k,
             max_seqlen_q: int, max_seqlen_k: int, chunk: int, softmax_scale: float, causal: bool) -> torch.Tensor:
    """Block-sparse backward into caller-allocated dq/dk/dv.  Returns softmax_d (H,T) fp32."""
    _require_cuda(dout, q, k, v, out, lse, dq, dk, dv)
    for t, n in ((dout, "dout"), (q, "q"), (k, "k"), (v, "v"), (out, "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        _last_contig(t, n)
    _check_pattern(col_offsets, col_nnz, indices)
    total_q, h, d = q.shape
    total_k, hk, _ = k.shape
    batch = cu_seqlens_q.numel() - 1
    dev = q.device
    if lse.dtype != torch.float32 or not lse.is_contiguous() or tuple(lse.shape) != (h, total_q):
        raise RuntimeError("softmax_lse must be a contiguous float32 (heads, total_q) tensor")
    with torch.cuda.device(dev):
        softmax_d = torch.empty((h, total_q), dtype=torch.float32, device=dev)
        ws, nbytes = _workspace(lib.fmb_attn_bwd_workspace_bytes, total_q, h, hk, d, indices.numel(), batch,
                                max_seqlen_k, chunk, dev)
        offered = getattr(_tls, "offered", None)
        _tls.offered = None
        if _rows_offer(col_offsets, col_nnz, indices, total_q, h):
            pass        # the pattern builder's rows: no lists to load, none to build
        elif offered is not None and _share_lists() and \
                offered[0] == _lists_key(col_offsets, col_nnz, indices, cu_seqlens_q, total_q, h, hk, d, batch,
                                         max_seqlen_k, chunk):
            rc = lib.fmb_attn_lists_load(ptr(ws), nbytes, total_q, h, hk, d, indices.numel(), batch,
                                         int(max_seqlen_k), int(chunk), ptr(offered[1]), offered[1].numel(), _stream())
            if rc not in (0, 1):
                check(rc)
        ticket = _status_begin(dev)
        check(lib.fmb_attn_bwd(ptr(dout), dout.stride(0), dout.stride(1), ptr(q), q.stride(0), q.stride(1),
                               ptr(k), k.stride(0), k.stride(1), ptr(v), v.stride(0), v.stride(1),
                               ptr(out), out.stride(0), out.stride(1), ptr(lse),
                               ptr(dq), dq.stride(0), dq.stride(1), ptr(dk), dk.stride(0), dk.stride(1),
                               ptr(dv), dv.stride(0), dv.stride(1), ptr(softmax_d),
                               ptr(col_offsets), ptr(col_nnz), ptr(indices), indices.numel(),
                               ptr(_i32c(cu_seqlens_q, "cu_seqlens_q")), ptr(_i32c(cu_seqlens_k, "cu_seqlens_k")),
                               ptr(ws), nbytes, batch, h, hk, d, total_q, total_k, int(max_seqlen_q),
                               int(max_seqlen_k), int(chunk), float(softmax_scale), int(bool(causal)),
                               _dtype_code(q), _stream()))
        _status_end(ticket, ws, "attn_bwd")
    return softmax_d
