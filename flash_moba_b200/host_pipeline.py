"""MoBA forward + backward for operands that live in pinned HOST memory.

The heads of a layer are independent, so the work is cut into head groups and pipelined over three
CUDA streams: while the kernels of group g run, the rows of group g+1 are copied host -> device
and the results of group g-1 device -> host (PCIe is full duplex).  End to end the step then costs
about max(copy in, copy out, compute) plus one group's ramp at each end, instead of their sum.

The copies are strided (a head range of a (tokens, heads, d) tensor) and go through
`fmb_copy_rows_async` of the C ABI (cudaMemcpy2DAsync); the kernels run on the head-range views of
full-size device tensors, which the library accepts as they are (only the last dimension has to be
contiguous).  The reference has no counterpart: its operands are device tensors.
"""
from typing import List, Optional, Tuple

import torch

from . import _lib
from .interface import flash_moba_varlen_func


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(_lib.lib.fmb_last_error().decode("utf-8", "replace") or f"flash_moba_b200 error {rc}")


def _copy_heads(dst: torch.Tensor, src: torch.Tensor, direction: int, stream: torch.cuda.Stream) -> None:
    """dst, src: (tokens, heads, d) views with the same shape, last two dims dense (head stride d)."""
    t, h, d = src.shape
    if dst.shape != src.shape or src.stride(2) != 1 or dst.stride(2) != 1 or src.stride(1) != d or dst.stride(1) != d:
        raise ValueError("head-range copy needs equal shapes and dense (heads, d) rows")
    es = src.element_size()
    _check(_lib.lib.fmb_copy_rows_async(dst.data_ptr(), dst.stride(0) * es, src.data_ptr(), src.stride(0) * es,
                                        h * d * es, t, direction, stream.cuda_stream))


class HostPipeline:
    """Device staging tensors and streams for repeated fwd+bwd steps of one layer shape."""

    def __init__(self, total_tokens: int, heads: int, heads_k: int, head_dim: int, dtype=torch.bfloat16,
                 device=None, groups: int = 8, backward: bool = True):
        if heads % heads_k:
            raise ValueError("heads must be a multiple of heads_k")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.heads, self.heads_k, self.backward = heads, heads_k, backward
        per = heads // heads_k
        ngroups = max(1, min(groups, heads_k))
        base, extra = divmod(heads_k, ngroups)
        self.ranges: List[Tuple[int, int, int, int]] = []      # (q head 0, q head 1, kv head 0, kv head 1)
        g0 = 0
        for i in range(ngroups):
            n = base + (1 if i < extra else 0)
            self.ranges.append((g0 * per, (g0 + n) * per, g0, g0 + n))
            g0 += n
        mk = lambda h: torch.empty((total_tokens, h, head_dim), dtype=dtype, device=self.device)
        self.q, self.k, self.v = mk(heads), mk(heads_k), mk(heads_k)
        self.do = mk(heads) if backward else None
        self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(device=self.device) for _ in range(3))

    def run(self, q_h, k_h, v_h, do_h, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, chunk, topk,
            out_h, dq_h=None, dk_h=None, dv_h=None, causal: bool = True) -> None:
        """All *_h tensors are pinned host tensors (tokens, heads, d); results are written into out_h
        (and dq_h, dk_h, dv_h).  Returns once every copy has been enqueued and the device is idle."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        keep = []
        for (h0, h1, k0, k1) in self.ranges:
            loaded = torch.cuda.Event()
            _copy_heads(self.q[:, h0:h1], q_h[:, h0:h1], 0, self.s_in)
            _copy_heads(self.k[:, k0:k1], k_h[:, k0:k1], 0, self.s_in)
            _copy_heads(self.v[:, k0:k1], v_h[:, k0:k1], 0, self.s_in)
            if self.backward:
                _copy_heads(self.do[:, h0:h1], do_h[:, h0:h1], 0, self.s_in)
            loaded.record(self.s_in)
            self.s_comp.wait_event(loaded)
            done = torch.cuda.Event()
            with torch.cuda.stream(self.s_comp):
                qg = self.q[:, h0:h1]
                kg, vg = self.k[:, k0:k1], self.v[:, k0:k1]
                if self.backward:
                    qg, kg, vg = (t.detach().requires_grad_(True) for t in (qg, kg, vg))
                out = flash_moba_varlen_func(qg, kg, vg, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                             chunk, topk, causal=causal)
                res = [out.detach()]
                if self.backward:
                    res += list(torch.autograd.grad(out, (qg, kg, vg), self.do[:, h0:h1]))
                # results of a zero-padded head dimension (d not 64 or 128) are slices of wider rows:
                # the strided copy wants dense (heads, d) rows
                res = [t if t.stride(1) == t.shape[2] else t.contiguous() for t in res]
                done.record(self.s_comp)
            self.s_out.wait_event(done)
            _copy_heads(out_h[:, h0:h1], res[0], 1, self.s_out)
            if self.backward:
                _copy_heads(dq_h[:, h0:h1], res[1], 1, self.s_out)
                _copy_heads(dk_h[:, k0:k1], res[2], 1, self.s_out)
                _copy_heads(dv_h[:, k0:k1], res[3], 1, self.s_out)
            for t in res:
                t.record_stream(self.s_out)
            keep.append(res)
        for s in (self.s_in, self.s_comp, self.s_out):
            cur.wait_stream(s)
        cur.synchronize()
