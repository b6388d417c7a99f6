"""A process whose FIRST use of the library is on the second GPU.

Kernel attributes (dynamic shared memory above 48 KB) and the per-device scratch of the library
are per device: a process-wide "already done" flag set on device 0 would leave device 1 without
them.  The child process below never touches device 0; it runs the whole path (pool, gating,
pattern by both builders, forward, backward) on cuda:1 and compares with the CPU oracle.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

CHILD = r"""
import sys, torch
sys.path.insert(0, {root!r})
import flash_moba_b200 as F
from flash_moba_b200 import ops, _lib
from oracle import moba_oracle as O
torch.cuda.set_device(1)
dev = "cuda:1"
torch.manual_seed(3)
lens, H, Hk, d, chunk, topk = [700, 300], 4, 2, 128, 64, 3
T = sum(lens)
q, k, v, do = [torch.randn(T, h, d).bfloat16() for h in (H, Hk, Hk, H)]
cs = torch.tensor([0, lens[0], T], dtype=torch.int32)
csd = cs.to(dev)
# pattern builder first (its kernels need more than 48 KB of dynamic shared memory)
km, cu_km = ops.mean_pool(k.to(dev), csd, max(lens), chunk)
idx, _ = ops.gate_topk(q.to(dev), km, csd, csd, cu_km, max(lens), max(lens), topk, chunk, True)
ncol = (max(lens) + chunk - 1) // chunk
want = ops.build_csc(idx, csd, max(lens), ncol)
co = torch.empty_like(want[0]); cn = torch.empty_like(want[1]); ind = torch.empty_like(want[2])
rc = _lib.lib.fmb_build_csc_static(idx.data_ptr(), idx.stride(0), idx.stride(1), csd.data_ptr(), co.data_ptr(),
                                   cn.data_ptr(), ind.data_ptr(), 2, H, topk, max(lens), ncol,
                                   torch.cuda.current_stream().cuda_stream)
assert rc == 0, _lib.lib.fmb_last_error()
torch.cuda.synchronize()
assert all(torch.equal(a, b) for a, b in zip((co, cn, ind), want))
qd, kd, vd = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
out = F.flash_moba_varlen_func(qd, kd, vd, csd, csd, max(lens), max(lens), chunk, topk, causal=True)
dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), do.to(dev))
mask = O.csc_to_mask(want[0].cpu(), want[1].cpu(), want[2].cpu(), cs, max(lens))
qq, kk, vv = [t.float().requires_grad_(True) for t in (q, k, v)]
ref, _ = O.attention_dense(qq, kk, vv, cs, cs, mask, chunk, True)
gq, gk, gv = torch.autograd.grad(ref, (qq, kk, vv), do.float())
for name, a, b in (("out", out, ref), ("dq", dq, gq), ("dk", dk, gk), ("dv", dv, gv)):
    err = (a.detach().cpu().float() - b.detach()).abs().max().item()
    assert err <= 0.02 * max(1.0, b.abs().max().item()), (name, err)
assert torch.cuda.memory_allocated(0) == 0          # nothing ever ran on the first device
print("second device ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_first_use_of_the_library_on_the_second_device():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", CHILD.format(root=root)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True, timeout=600)
    assert r.returncode == 0 and "second device ok" in r.stdout, r.stdout[-3000:]
