"""Public API: a drop-in for the reference's `flash_moba` Python surface
(flash_moba/flash_moba_interface.py:517-727 and flash_moba/triton_mean_pool.py:112-157).

Same function names, positional order, defaults, return values and error behaviour
(RuntimeError on bad dtype/shape); the same four `torch.library.custom_op` names
(`flash_moba::_moba_fused_topk`, `::_varlen_sort`, `::_flash_moba_attn_varlen_forward`,
`::_flash_moba_attn_varlen_backward`) with fake implementations so traced graphs resolve.
Everything below the ops is the sm_100a library behind the C ABI.

Differences that do not change results:
  * the pattern comes out of `_moba_fused_topk` already sorted (the builder is ordered), so
    `flash_topk_varlen_func` does not call `_varlen_sort`; the op still exists and sorts;
  * `lg_block_m` is a partition hint of the reference kernel; it is validated and ignored;
  * dropout, softcap and alibi are rejected if non-default (the reference documents them as
    unsupported for MoBA); `leftpad_k` and `seqused_k` of the forward op are honoured.
"""
from typing import Optional, Tuple

import torch

from . import ops


def round_multiple(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def decide_lg_block_m(top_k: int, chunk_size: int, seqlen: int, causal: bool = False) -> int:
    """The reference's tile-partition hint (flash_moba_interface.py:20-48), kept so callers
    that compute it still work.  These kernels do not need it."""
    budget = top_k * chunk_size
    density = (2 * budget * seqlen - budget ** 2) / seqlen ** 2 if causal else budget / seqlen
    sparsity = 1 - density
    for bound, m in ((0.5, 128), (0.7, 256), (0.8, 512), (0.9, 768)):
        if sparsity <= bound:
            return m
    return 1024


def _fix_last_stride(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def _reject_unsupported(dropout_p, softcap, alibi_slopes):
    if dropout_p != 0.0:
        raise RuntimeError("FlashMoBA does not support dropout (dropout_p must be 0.0)")
    if softcap != 0.0:
        raise RuntimeError("FlashMoBA does not support softcap (softcap must be 0.0)")
    if alibi_slopes is not None:
        raise RuntimeError("FlashMoBA does not support ALiBi (alibi_slopes must be None)")


# ======================================================================================
# custom ops (same names and schemas as the reference)
# ======================================================================================
@torch.library.custom_op("flash_moba::_moba_fused_topk", mutates_args=(), device_types="cuda")
def _moba_fused_topk(
    q: torch.Tensor,
    km: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    cu_seqlens_km: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    moba_topk: int,
    moba_chunk_size: int,
    causal: bool = True,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    q, km = _fix_last_stride(q), km.contiguous()
    idx, _ = ops.gate_topk(q, km, cu_seqlens_q, cu_seqlens_k, cu_seqlens_km, max_seqlen_q, max_seqlen_k,
                           moba_topk, moba_chunk_size, causal)
    ncol = (max_seqlen_k + moba_chunk_size - 1) // moba_chunk_size
    return ops.build_csc(idx, cu_seqlens_q, max_seqlen_q, ncol, keep_rows=True)


@torch.library.register_fake("flash_moba::_moba_fused_topk")
def _moba_fused_topk_fake(q, km, cu_seqlens_q, cu_seqlens_k, cu_seqlens_km, max_seqlen_q, max_seqlen_k,
                          moba_topk, moba_chunk_size, causal=True):
    batch = cu_seqlens_q.numel() - 1
    total_q, heads, _ = q.shape
    ncol = (max_seqlen_k + moba_chunk_size - 1) // moba_chunk_size
    return (torch.empty((batch, heads, ncol), device=q.device, dtype=torch.int64),
            torch.empty((batch, heads, ncol), device=q.device, dtype=torch.int32),
            torch.empty((total_q * heads * moba_topk,), device=q.device, dtype=torch.int32))


@torch.library.custom_op("flash_moba::_varlen_sort", mutates_args=(), device_types="cuda")
def _varlen_sort(col_offsets: torch.Tensor, col_nnz: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    starts = col_offsets.reshape(-1)
    return ops.varlen_sort(starts, starts + col_nnz.reshape(-1), indices)


@torch.library.register_fake("flash_moba::_varlen_sort")
def _varlen_sort_fake(col_offsets, col_nnz, indices):
    return torch.empty_like(indices)


@torch.library.custom_op("flash_moba::_flash_moba_attn_varlen_forward", mutates_args=(), device_types="cuda")
def _flash_moba_attn_varlen_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    moba_col_offsets: torch.Tensor,
    moba_col_nnz: torch.Tensor,
    moba_row_indices: torch.Tensor,
    lg_block_m: int,
    lg_block_n: int,
    dropout_p: float,
    softmax_scale: float,
    causal: bool,
    softcap: float = 0.0,
    alibi_slopes: Optional[torch.Tensor] = None,
    return_softmax: bool = False,
    leftpad_k: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    zero_tensors: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    _reject_unsupported(dropout_p, softcap, alibi_slopes)
    if lg_block_n % 64 != 0:
        raise RuntimeError("lg_block_n must be divisible by 64")
    if lg_block_m % 64 != 0 or not (128 <= lg_block_m <= 1024):
        raise RuntimeError("lg_block_m must be divisible by 64 and within [128, 1024]")
    q, k, v = [_fix_last_stride(x) for x in (q, k, v)]
    out, lse = ops.attn_fwd(q, k, v, moba_col_offsets.contiguous(), moba_col_nnz.contiguous(),
                            moba_row_indices.contiguous(), cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                            max_seqlen_k, lg_block_n, softmax_scale, causal, leftpad_k=leftpad_k, seqused_k=seqused_k)
    p = torch.empty((0,), dtype=q.dtype, device=q.device)
    rng_state = torch.zeros((2,), dtype=torch.int64, device=q.device)
    return out, lse, p, rng_state


@torch.library.register_fake("flash_moba::_flash_moba_attn_varlen_forward")
def _flash_moba_attn_varlen_forward_fake(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                         moba_col_offsets, moba_col_nnz, moba_row_indices, lg_block_m, lg_block_n,
                                         dropout_p, softmax_scale, causal, softcap=0.0, alibi_slopes=None,
                                         return_softmax=False, leftpad_k=None, seqused_k=None, zero_tensors=False):
    total_q, heads, _ = q.shape
    return (torch.empty_like(q), torch.empty((heads, total_q), dtype=torch.float32, device=q.device),
            torch.empty((0,), dtype=q.dtype, device=q.device), torch.empty((2,), dtype=torch.int64, device=q.device))


@torch.library.custom_op("flash_moba::_flash_moba_attn_varlen_backward", mutates_args=("dq", "dk", "dv"),
                         device_types="cuda")
def _flash_moba_attn_varlen_backward(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    dq: Optional[torch.Tensor],
    dk: Optional[torch.Tensor],
    dv: Optional[torch.Tensor],
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    moba_col_offsets: torch.Tensor,
    moba_col_nnz: torch.Tensor,
    moba_row_indices: torch.Tensor,
    lg_block_m: int,
    lg_block_n: int,
    dropout_p: float,
    softmax_scale: float,
    causal: bool,
    softcap: float,
    alibi_slopes: Optional[torch.Tensor],
    deterministic: bool,
    rng_state: Optional[torch.Tensor] = None,
    zero_tensors: bool = False,
) -> torch.Tensor:
    _reject_unsupported(dropout_p, softcap, alibi_slopes)
    if dq is None or dk is None or dv is None:
        raise RuntimeError("dq, dk and dv must be pre-allocated by the caller")
    dout, q, k, v, out = [_fix_last_stride(x) for x in (dout, q, k, v, out)]
    return ops.attn_bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, moba_col_offsets.contiguous(),
                        moba_col_nnz.contiguous(), moba_row_indices.contiguous(), cu_seqlens_q, cu_seqlens_k,
                        max_seqlen_q, max_seqlen_k, lg_block_n, softmax_scale, causal)


@torch.library.register_fake("flash_moba::_flash_moba_attn_varlen_backward")
def _flash_moba_attn_varlen_backward_fake(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k,
                                          max_seqlen_q, max_seqlen_k, moba_col_offsets, moba_col_nnz,
                                          moba_row_indices, lg_block_m, lg_block_n, dropout_p, softmax_scale, causal,
                                          softcap, alibi_slopes, deterministic, rng_state=None, zero_tensors=False):
    total_q, heads, _ = q.shape
    return torch.empty((heads, total_q), device=q.device, dtype=torch.float32)


def _op(name: str):
    """The callable behind one of the four custom ops.  Eager callers run the op's plain Python
    body: the dispatcher's per-call work (schema checks, aliasing checks of every output) costs
    about 0.1 ms per op on the host, a third of the whole step's enqueue time at 4 heads per GPU.
    Under torch.compile the registered op is used, so that traced graphs hold `flash_moba::` nodes
    as they do with the reference."""
    if torch.compiler.is_compiling():
        return getattr(torch.ops.flash_moba, name)
    return globals()[name]._init_fn


def _attention_head_dim(d: int) -> int:
    """Head dimension the attention kernels run at: 64, 128 or 256; anything else is zero-padded up
    to the next of them (the reference pads to a multiple of 8 and dispatches on 32 ... 256,
    flash_moba/flash_moba_interface.py:433-436)."""
    for built in (64, 128, 256):
        if d <= built:
            return built
    return d + (-d) % 8          # above 256: rejected by the library with its message


# ======================================================================================
# autograd
# ======================================================================================
class FlashMobaAttnVarlenFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, moba_col_offsets,
                moba_col_nnz, moba_row_indices, lg_block_m, lg_block_n, dropout_p, softmax_scale, causal, softcap,
                alibi_slopes, deterministic, return_softmax, is_grad_enabled):
        is_grad = is_grad_enabled and any(x.requires_grad for x in (q, k, v))
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        d_og = q.size(2)
        d_pad = _attention_head_dim(d_og)
        if d_pad != d_og:      # zero columns change neither the scores nor the first d_og outputs
            pad = [0, d_pad - d_og]
            q, k, v = (torch.nn.functional.pad(x, pad) for x in (q, k, v))
        out_padded, lse, s_dmask, rng_state = _op("_flash_moba_attn_varlen_forward")(
            q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, moba_col_offsets, moba_col_nnz,
            moba_row_indices, lg_block_m, lg_block_n, dropout_p, softmax_scale, causal=causal, softcap=softcap,
            alibi_slopes=alibi_slopes, return_softmax=return_softmax and dropout_p > 0)
        lists = ops.take_lists()     # the pattern's row lists, kept by the forward call for the backward call
        if is_grad:
            ctx.lists = lists
            ctx.save_for_backward(q, k, v, out_padded, lse, cu_seqlens_q, cu_seqlens_k, rng_state,
                                  moba_col_offsets, moba_col_nnz, moba_row_indices)
            ctx.meta = (dropout_p, max_seqlen_q, max_seqlen_k, softmax_scale, causal, softcap, alibi_slopes,
                        deterministic, lg_block_m, lg_block_n)
        out = out_padded[..., :d_og]
        return out if not return_softmax else (out, lse, s_dmask)

    @staticmethod
    def backward(ctx, dout, *args):
        (q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, rng_state, col_offsets, col_nnz, row_indices) = ctx.saved_tensors
        (dropout_p, max_seqlen_q, max_seqlen_k, softmax_scale, causal, softcap, alibi_slopes, deterministic,
         lg_block_m, lg_block_n) = ctx.meta
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        d_og = dout.size(2)
        dout_padded = dout if q.size(2) == d_og else torch.nn.functional.pad(dout, [0, q.size(2) - d_og])
        ops.offer_lists(getattr(ctx, "lists", None))
        _op("_flash_moba_attn_varlen_backward")(
            dout_padded, q, k, v, out, lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
            col_offsets, col_nnz, row_indices, lg_block_m, lg_block_n, dropout_p, softmax_scale, causal, softcap,
            alibi_slopes, deterministic, rng_state=rng_state)
        return (dq[..., :d_og], dk[..., :d_og], dv[..., :d_og]) + (None,) * 17


# ======================================================================================
# public functions
# ======================================================================================
def flash_topk_mean_pool(input, cu_seqlens_input, max_seqlen_input, pool_block_size):
    """Per-chunk mean pool with the reference's return contract
    (flash_moba/triton_mean_pool.py:112-157): (pooled (total_blocks, H, d),
    cu_seqlens_output int32, max_seqlen_output).  The exact output row count needs the last
    cumulative offset on the host, so this stand-alone form synchronises once, exactly like
    the reference; `flash_topk_varlen_func` uses the sync-free internal form."""
    km, cu_km = ops.mean_pool(_fix_last_stride(input), cu_seqlens_input, max_seqlen_input, pool_block_size)
    total_blocks = int(cu_km[-1].item()) if cu_km.numel() > 1 else 0
    max_out = (max_seqlen_input + pool_block_size - 1) // pool_block_size
    return km[:total_blocks], cu_km, max_out


def flash_topk_varlen_func(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, moba_topk,
                           moba_chunk_size, causal=False):
    """MoBA gating for a varlen batch: mean-pool the keys per chunk, score every query
    against the centroids of its sequence, keep the top-k chunks per (query, head) and return
    the key-block-major pattern `(col_offsets, col_nnz, indices)`.

    q: (total_q, nheads, d); k: (total_k, nheads_k, d); cu_seqlens_*: int32 (batch+1,).
    Note the argument order (top-k, then chunk size), as in the reference."""
    d_og = q.size(2)
    d_pad = _attention_head_dim(d_og)      # zero columns change no score; 64 / 128 / 256 run on tensor cores
    if d_pad != d_og:
        pad = [0, d_pad - d_og]
        q, k = torch.nn.functional.pad(q, pad), torch.nn.functional.pad(k, pad)
    km, cu_seqlens_km = ops.mean_pool(_fix_last_stride(k), cu_seqlens_k, max_seqlen_k, moba_chunk_size)
    return _op("_moba_fused_topk")(q, km, cu_seqlens_q, cu_seqlens_k, cu_seqlens_km, max_seqlen_q,
                                                 max_seqlen_k, moba_topk, moba_chunk_size, causal=causal)


def flash_moba_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                moba_col_offsets, moba_col_nnz, moba_row_indices, lg_block_m=64, lg_block_n=64,
                                dropout_p=0.0, softmax_scale=None, causal=False, softcap=0.0, alibi_slopes=None,
                                deterministic=False, return_attn_probs=False):
    """Block-sparse attention over a given pattern (varlen, MQA/GQA by passing fewer KV
    heads, bottom-right aligned causal mask).  `lg_block_n` is the key chunk size of the
    pattern.  Returns out (total_q, nheads, d), or (out, softmax_lse (nheads, total_q), S_dmask)
    when `return_attn_probs`.  Rows that see no key produce zeros."""
    return FlashMobaAttnVarlenFunc.apply(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                         moba_col_offsets, moba_col_nnz, moba_row_indices, lg_block_m, lg_block_n,
                                         dropout_p, softmax_scale, causal, softcap, alibi_slopes, deterministic,
                                         return_attn_probs, torch.is_grad_enabled())


def flash_moba_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, moba_chunk_size,
                           moba_topk, causal=True):
    """End-to-end MoBA attention: gating pattern, then block-sparse attention with it."""
    col_offsets, col_nnz, indices = flash_topk_varlen_func(q, k, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                                                           max_seqlen_k, moba_topk, moba_chunk_size, causal=causal)
    lg_block_m = decide_lg_block_m(moba_topk, moba_chunk_size, max_seqlen_k, causal)
    return flash_moba_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                       col_offsets, col_nnz, indices, lg_block_m, moba_chunk_size,
                                       dropout_p=0.0, causal=causal)
