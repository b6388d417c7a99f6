#!/usr/bin/env python
"""Benchmark of the MoBA hot path (pattern + block-sparse forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload 64k|c2|c3|c4|c5] [--heads H]

A step = one pass of the hot path over one batch of synthetic input through the public API
(`flash_moba_varlen_func` forward, autograd backward): mean-pool -> gating top-k -> pattern
-> block-sparse forward -> backward (dQ, dK, dV).  Prints ONE JSON line (rank 0).

metric  : selected-block TFLOP/s of fwd+bwd attention (FLOPs counted over selected blocks
          only, see flash_moba_b200/accounting.py); ms_per_step beside it.
value   : device-timed, inputs resident in HBM.   e2e: the same through the public API with
          q/k/v/dO copied from pinned host memory and out/dq/dk/dv copied back each step.
N > 1   : query heads are split across ranks (no collective on the data path); value is the
          whole job's FLOPs / max-over-ranks time ("strong": the 64K problem is fixed).
--impl reference : the reference's pure-PyTorch MoBA restated in oracle/ (the reference has
          no CPU build of its CUDA path), timed on the host cores over a bounded sample; that is the
          line's value.  Where oracle/build_ref.sh has built the reference's own CUDA extension for
          sm_100 (oracle/_ref/), the line also carries "reference_cuda": those kernels on the full
          workload on this GPU (1-GPU runs).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

def _c4_lengths():
    """Configuration 4's 16 sequence lengths: uniform in [2048, 32768], rounded up to multiples of 64, seed 0."""
    import random
    rnd = random.Random(0)
    return [(rnd.randint(2048, 32768) + 63) // 64 * 64 for _ in range(16)]


WORKLOADS = {
    # name: (seqlens, heads, heads_k, d, chunk, topk, backward, input scale): the headline workload and
    # the benchmark configurations 2-5 at their full shapes; --heads runs a stated share of the heads
    # (same ratio of q to kv heads) and --tokens a shorter single sequence, for profiler captures
    "64k": ([65536], 32, 32, 128, 128, 8, True, 1.0),
    "c2": ([32768], 16, 16, 128, 128, 8, False, 0.5),
    "c3": ([8192] * 8, 32, 32, 128, 128, 8, True, 1.0),
    "c4": (_c4_lengths(), 32, 8, 128, 64, 16, True, 1.0),
    "c5": ([524288], 32, 32, 128, 256, 16, True, 0.5),
}


def _load_accounting():
    import importlib.util
    spec = importlib.util.spec_from_file_location("fmb_accounting", os.path.join(ROOT, "flash_moba_b200", "accounting.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


ACC = _load_accounting()
BWD_MAIN_DRAM_BYTES_PER_ENTRY = 575.2


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs.

    Polled in-process through NVML every few milliseconds (the timed region of a multi-GPU run
    lasts only tens of milliseconds, shorter than nvidia-smi's loop interval); nvidia-smi is the
    fallback when the NVML binding is missing.  Reading only: nothing is set."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index, period_s=0.004):
        self.index, self.rows, self.proc, self.period = index, [], None, period_s
        self.stop = threading.Event()
        self.nvml = None
        self.error = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        return pynvml, h

    def _poll(self):
        pynvml, h = self.nvml
        try:
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
        except Exception:
            mx = None
        get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self.stop.is_set():
            try:
                sm = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                bits = int(get_reasons(h)) if get_reasons else 0
                self.rows.append((float(sm), float(mx) if mx else None, bits, time.perf_counter()))
            except Exception as e:      # reported in the summary, never fatal
                self.error = repr(e)
            self.stop.wait(self.period)

    def __enter__(self):
        try:
            self.nvml = self._nvml_handle()
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            r = [x.strip() for x in line.split(",")]
            try:
                bits = sum(b for (name, b), v in zip((("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40),
                                                      ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4)), r[2:6])
                           if v.lower().startswith("active"))
                self.rows.append((float(r[0]), float(r[1]), bits, time.perf_counter()))
            except (ValueError, IndexError):
                continue

    def __exit__(self, *a):
        self.stop.set()
        if self.nvml is not None:
            self.t.join(timeout=1)
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def mark(self, which):
        """Host time stamps of the timed region's start and end (the sampler itself runs from the
        warm-up on, so that a slow first NVML call does not eat the timed region)."""
        setattr(self, "t_" + which, time.perf_counter())

    def summary(self):
        t0, t1 = getattr(self, "t_start", None), getattr(self, "t_end", None)
        rows, window = self.rows, "sampler lifetime"
        if t0 is not None and t1 is not None:
            inside = [r for r in self.rows if t0 <= r[3] <= t1]
            if len(inside) >= 3:
                rows, window = inside, "timed region"
            else:   # a box whose NVML calls take tens of milliseconds: the warm-up steps are the same load
                rows, window = [r for r in self.rows if r[3] <= t1], f"warm-up + timed region ({len(inside)} inside the timed region)"
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "error": self.error}
        sm = [r[0] for r in rows]
        mx = [r[1] for r in rows if r[1]]
        bits = 0
        for r in rows:
            bits |= r[2]
        reasons = sorted(n for n, b in self.REASON_BITS.items() if bits & b)
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm), "window": window, "source": "nvml" if self.nvml is not None else "nvidia-smi"}


def cpu_sample(seqlens, d, chunk, topk, rows=4096, threads=None):
    """The oracle (pure-PyTorch MoBA restated from the reference) on the host cores over a
    bounded sample of the workload: the LAST `rows` query rows of one head against all keys of
    the first sequence (pattern + forward + backward).  Returns (seconds, flops)."""
    from oracle import moba_oracle as O
    threads = threads or os.cpu_count()
    torch.set_num_threads(threads)
    S = seqlens[0]
    rows = min(rows, S)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(rows, 1, d, generator=g).bfloat16().float().requires_grad_(True)
    k = torch.randn(S, 1, d, generator=g).bfloat16().float().requires_grad_(True)
    v = torch.randn(S, 1, d, generator=g).bfloat16().float().requires_grad_(True)
    do = torch.randn(rows, 1, d, generator=g)
    cq = torch.tensor([0, rows], dtype=torch.int32)
    ck = torch.tensor([0, S], dtype=torch.int32)
    t0 = time.perf_counter()
    km, cu_km = O.mean_pool(k.detach(), ck, chunk)
    idx, _ = O.gate_topk(q.detach(), km, cq, ck, cu_km, topk, chunk, True)
    out, _ = O.attention_blocked(q, k, v, cq, ck, idx, chunk, True)
    torch.autograd.grad(out, (q, k, v), do)
    dt = time.perf_counter() - t0
    # pairs of those rows (bottom-right aligned): row r sits at position S-rows+r
    pairs = 0
    for r in range(rows):
        p = S - rows + r
        sel = min(topk, p // chunk + 1)
        pairs += (sel - 1) * chunk + (p % chunk + 1)
    return dt, 3.5 * 4 * d * pairs, rows, threads


def workload_of(args):
    """(seqlens, H, Hk, d, chunk, topk, backward, scale) of the run, after --heads / --tokens."""
    seqlens, H, Hk, d, chunk, topk, backward, scale = WORKLOADS[args.workload]
    if args.heads:
        assert args.heads % (H // Hk) == 0 and args.heads <= H, "--heads must keep whole kv-head groups"
        H, Hk = args.heads, args.heads // (H // Hk)
    if args.tokens:
        assert len(seqlens) == 1, "--tokens is for single-sequence workloads"
        seqlens = [args.tokens]
    return seqlens, H, Hk, d, chunk, topk, backward, scale


def config_of(wl, seqlens, H, Hk, d, chunk, topk, backward):
    """What defines the workload: the same dict in both arms' lines."""
    return {"workload": wl, "seqlens": seqlens, "heads": H, "heads_k": Hk, "head_dim": d, "chunk": chunk,
            "topk": topk, "causal": True, "step": "pattern(pool+gate+csc) + fwd" + (" + bwd" if backward else "")}


def reference_cuda_leg(seqlens, H, Hk, d, chunk, topk, backward, scale, steps):
    """The reference's own CUDA extension (built for sm_100 from its sources by oracle/build_ref.sh,
    present as oracle/_ref/flash_moba_cuda.so) on the full workload on this GPU: gating top-k +
    column sort, forward, backward, each timed with CUDA events.  The reference's mean pool is a
    Triton kernel of its Python package, not part of the extension: the centroids are made with
    plain torch outside the timed region.  None when the extension or a GPU is missing."""
    from oracle import ref_cuda
    if not ref_cuda.available() or not torch.cuda.is_available():
        return None
    try:
        torch.manual_seed(0)
        T, S = sum(seqlens), max(seqlens)
        dev = "cuda"
        q = (torch.randn(T, H, d, device=dev) * scale).bfloat16()
        k = (torch.randn(T, Hk, d, device=dev) * scale).bfloat16()
        v = (torch.randn(T, Hk, d, device=dev) * scale).bfloat16()
        do = torch.randn(T, H, d, device=dev).bfloat16()
        cu = [0]
        for n in seqlens:
            cu.append(cu[-1] + n)
        cs = torch.tensor(cu, dtype=torch.int32, device=dev)
        cm = [0]
        pooled = []
        for b, n in enumerate(seqlens):      # per-chunk means, the last chunk over its true length
            kb = k[cu[b]:cu[b + 1]].float()
            full = n // chunk
            if full:
                pooled.append(kb[:full * chunk].view(full, chunk, Hk, d).mean(1))
            if n % chunk:
                pooled.append(kb[full * chunk:].mean(0, keepdim=True))
            cm.append(cm[-1] + (n + chunk - 1) // chunk)
        km = torch.cat(pooled, 0).bfloat16().contiguous()
        cu_km = torch.tensor(cm, dtype=torch.int32, device=dev)
        from flash_moba_b200.interface import decide_lg_block_m     # the reference's own table of five thresholds
        lg_m = decide_lg_block_m(topk, chunk, S, True)
        sm_scale = d ** -0.5

        def timed(fn):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / steps

        pat = ref_cuda.fused_topk(q, km, cs, cs, cu_km, S, S, topk, chunk, True)
        out, lse = ref_cuda.attn_fwd(q, k, v, cs, cs, S, S, *pat, lg_m, chunk, sm_scale)
        ms = {"topk_and_sort": timed(lambda: ref_cuda.fused_topk(q, km, cs, cs, cu_km, S, S, topk, chunk, True)),
              "fwd": timed(lambda: ref_cuda.attn_fwd(q, k, v, cs, cs, S, S, *pat, lg_m, chunk, sm_scale))}
        if backward:
            ms["bwd"] = timed(lambda: ref_cuda.attn_bwd(do, q, k, v, out, lse, cs, cs, S, S, *pat, lg_m, chunk, sm_scale))
        fwd, bwd, both = ACC.attention_flops(seqlens, H, d, chunk, topk)
        total = sum(ms.values())
        return {"ms_per_step": total, "ms": ms, "value": (both if backward else fwd) / total / 1e9, "unit": "TFLOP/s",
                "lg_block_m": lg_m, "steps": steps,
                "what": "the reference's CUDA extension compiled for sm_100 (its own sources, trimmed to the head-dim 64/128/256 "
                        "bf16 causal instantiations), same workload on this GPU, inputs resident; its Triton mean pool is not timed"}
    except Exception as e:      # reported, never fatal: the line's own numbers do not depend on it
        return {"error": repr(e)[:300]}


def reference_cuda_in_child(args):
    """reference_cuda_leg in a process of its own: the extension is the reference's code, and whatever it
    does (an instantiation left out of the trimmed build, a fault) must not take this arm's line with it."""
    from oracle import ref_cuda
    if not ref_cuda.available() or not torch.cuda.is_available():
        return None
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-cuda-leg", "--workload", args.workload,
           "--steps", str(max(1, min(args.steps, 5)))]
    if args.heads:
        cmd += ["--heads", str(args.heads)]
    if args.tokens:
        cmd += ["--tokens", str(args.tokens)]
    try:
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
        last = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        if r.returncode != 0 or not last:
            return {"error": f"child exited {r.returncode}: {r.stderr[-300:]}"}
        return json.loads(last[-1])
    except Exception as e:
        return {"error": repr(e)[:300]}


def run_reference(args, wl):
    seqlens, H, Hk, d, chunk, topk, backward, scale = workload_of(args)
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 2048
    for _ in range(max(args.warmup, 1)):
        cpu_sample(seqlens, d, chunk, topk, rows=256)
    times, flops, threads = [], 0, 0
    for _ in range(args.steps):
        dt, flops, rows, threads = cpu_sample(seqlens, d, chunk, topk, rows=rows)
        times.append(dt)
    t = sum(times) / len(times)
    val = flops / t / 1e12
    line = {
        "impl": "reference", "metric": "moba_fwd_bwd_selected_block_tflops", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(wl, seqlens, H, Hk, d, chunk, topk, backward),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"pattern+fwd+bwd of the last {rows} query rows of 1 head vs all {seqlens[0]} keys, "
                                   "fp32 PyTorch oracle (oracle/moba_oracle.py), per step"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if args.gpus == 1 and not args.no_reference_cuda:
        line["reference_cuda"] = reference_cuda_in_child(args)
    emit(json.dumps(line))


_RESULT_FD = None


def protect_stdout():
    """The result is ONE JSON line on stdout; libraries print there too (NCCL its version line
    when NCCL_DEBUG asks for it).  From here on everything written to file descriptor 1 goes to
    stderr, and only emit() writes to the real stdout."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(text):
    sys.stdout.flush()
    if _RESULT_FD is None:
        print(text, flush=True)
    else:
        os.write(_RESULT_FD, (text + "\n").encode())


def main():
    protect_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda-leg"])
    ap.add_argument("--workload", default="64k", choices=sorted(WORKLOADS))
    ap.add_argument("--heads", type=int, default=0, help="run this many of the workload's q heads (same q:kv ratio)")
    ap.add_argument("--tokens", type=int, default=0, help="single-sequence workloads: this many tokens instead")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-reference-cuda", action="store_true",
                    help="--impl reference: do not also time the reference's CUDA extension (oracle/_ref) on the GPU")
    ap.add_argument("--e2e-groups", type=int, default=8, help="head groups of the host pipeline")
    ap.add_argument("--engine", type=int, default=1)
    ap.add_argument("--shard", default="heads", choices=["heads", "query-range"],
                    help="N > 1: split the heads (no collective), or split one long sequence by query range "
                         "(all-gather of centroids, K and V; reduce-scatter of dK and dV, inside the step)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl = args.workload
    if args.impl == "reference":
        return run_reference(args, wl)
    if args.impl == "reference-cuda-leg":     # the child of reference_cuda_in_child
        seqlens, H, Hk, d, chunk, topk, backward, scale = workload_of(args)
        return emit(json.dumps(reference_cuda_leg(seqlens, H, Hk, d, chunk, topk, backward, scale, args.steps)))

    seqlens, H, Hk, d, chunk, topk, backward, scale = workload_of(args)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    import flash_moba_b200 as F
    from flash_moba_b200 import _lib, ops
    ops.set_engine(args.engine)

    from flash_moba_b200 import sharding
    by_range = args.shard == "query-range" and world > 1
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    if by_range:
        # one long sequence split by query range: every rank holds S / world rows of all heads
        assert len(seqlens) == 1 and seqlens[0] % (world * chunk) == 0, "query-range split: one sequence, whole chunks per rank"
        h0, h1, h_loc, hk_loc = 0, H, H, Hk
        T = seqlens[0] // world
        args.no_e2e = True
    else:
        # q heads (and their kv heads) split across ranks; no data-path collective
        assert Hk >= world, "fewer kv heads than ranks: split the sequence by query range instead (--shard query-range)"
        h0, h1 = sharding.plan_head_shards(H, Hk, world)[rank]
        h_loc, hk_loc = h1 - h0, (h1 - h0) // (H // Hk)
        T = sum(seqlens)
    mk = lambda h: (torch.randn(T, h, d, generator=g, device=dev, dtype=torch.float32) * scale).to(torch.bfloat16)
    q, k, v, do = mk(h_loc).requires_grad_(True), mk(hk_loc).requires_grad_(True), mk(hk_loc).requires_grad_(True), mk(h_loc)
    cu = torch.tensor([0] + list(__import__("itertools").accumulate(seqlens)), dtype=torch.int32, device=dev)
    mx = max(seqlens)

    def step(qq, kk, vv, dd):
        if by_range:
            out = sharding.moba_query_range(qq, kk, vv, seqlens[0], chunk, topk)
        else:
            out = F.flash_moba_varlen_func(qq, kk, vv, cu, cu, mx, mx, chunk, topk, causal=True)
        if backward:
            return (out,) + torch.autograd.grad(out, (qq, kk, vv), dd)
        return (out,)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        for _ in range(args.warmup):
            step(q, k, v, do)
        barrier()
        launches0 = _lib.lib.fmb_launch_count()
        # inside the timed region only the dominant kernel (the backward main kernel, or the forward
        # one of a forward-only workload: the roofline's subject) is bracketed by events; the other
        # kernels are timed in the loop that follows it
        dom_kind = 1 if backward else 0
        _lib.lib.fmb_profile_enable(1)
        _lib.lib.fmb_profile_kinds(1 << dom_kind)
        # a collection pause of the interpreter in the middle of a short timed region (15 ms at 8 GPUs)
        # would stall one rank's launches, and the slowest rank is the result
        import gc
        gc.collect()
        gc.disable()
        barrier()
        clk.mark("start")
        ev0.record()
        for _ in range(args.steps):
            step(q, k, v, do)
        ev1.record()
        barrier()
        clk.mark("end")
        gc.enable()
    ms = ev0.elapsed_time(ev1) / args.steps
    if os.environ.get("FMB_BENCH_VERBOSE") == "1":
        print(f"[rank {rank}] {ms:.4f} ms per step over {args.steps} steps", file=sys.stderr, flush=True)
    launches = _lib.lib.fmb_launch_count() - launches0
    # device-side status words of every attention call so far, and of the gating launches
    status = 0
    try:
        ops.check_pending_status()
        gate_code = __import__("ctypes").c_int(0)
        _lib.check(_lib.lib.fmb_gate_status(__import__("ctypes").addressof(gate_code)))
    except RuntimeError as e:
        status = str(e)
    import ctypes

    def kernel_ms(kind):
        buf = (ctypes.c_float * 256)()
        n = _lib.lib.fmb_profile_read(kind, ctypes.cast(buf, ctypes.c_void_p), 256)
        return (sum(buf[:n]) / n) if n > 0 else None

    dom_ms = kernel_ms(dom_kind)        # over the timed region
    # host time per step: the same loop without waiting for the device (enqueue cost of a step);
    # every kernel kind is bracketed here
    _lib.lib.fmb_profile_enable(1)
    barrier()
    t_h0 = time.perf_counter()
    for _ in range(args.steps):
        step(q, k, v, do)
    host_ms = (time.perf_counter() - t_h0) * 1e3 / args.steps
    barrier()
    kern_ms = {}
    for kind, name in ((0, "fwd_main"), (1, "bwd_main"), (2, "gate"), (3, "pool"), (4, "fwd_combine"),
                       (5, "bwd_combine"), (6, "pattern_build"), (7, "dot_do_o")):
        kern_ms[name] = kernel_ms(kind)
    if dom_ms is not None:
        kern_ms["bwd_main" if backward else "fwd_main"] = dom_ms
    _lib.lib.fmb_profile_enable(0)
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    fwd_f, bwd_f, both_f = ACC.attention_flops(seqlens, H, d, chunk, topk)
    job_flops = both_f if backward else fwd_f
    value = job_flops / (ms * 1e-3) / 1e12

    # ---- end to end: pinned host inputs in, results out, every step, through the host pipeline
    # (head groups: copies of one group overlap the kernels of another)
    e2e = None
    if not args.no_e2e:
        from flash_moba_b200.host_pipeline import HostPipeline
        host_in = [t.detach().cpu().pin_memory() for t in (q, k, v, do)]
        n_out = 4 if backward else 1
        host_out = [torch.empty((T, h_loc if i < 2 else hk_loc, d), dtype=torch.bfloat16).pin_memory() for i in range(n_out)]
        pipe = HostPipeline(T, h_loc, hk_loc, d, torch.bfloat16, dev, groups=args.e2e_groups, backward=backward)

        def e2e_step():
            pipe.run(host_in[0], host_in[1], host_in[2], host_in[3], cu, cu, mx, mx, chunk, topk, *host_out)

        for _ in range(2):
            e2e_step()
        barrier()
        n_e2e = max(2, min(args.steps, 5))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        e_ms = e0.elapsed_time(e1) / n_e2e
        if dist is not None:
            t = torch.tensor([e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        e2e = {"value": job_flops / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e_ms,
               "pipeline": f"{len(pipe.ranges)} head groups on 3 streams (copy in / kernels / copy out)",
               "h2d_bytes_per_step": sum(t.numel() * 2 for t in host_in) * world,
               "d2h_bytes_per_step": sum(t.numel() * 2 for t in host_out) * world}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    clocks = clk.summary()
    # the burst figure is the denominator as long as the clock stayed at its maximum with no power
    # cap during the timed region (a step is milliseconds long); the sustained figure otherwise
    at_max = bool(clocks.get("sm_mhz")) and clocks.get("sm_max_mhz") and \
        clocks["sm_mhz"] >= 0.98 * clocks["sm_max_mhz"] and "sw_power_cap" not in clocks.get("reasons", [])
    peak_burst, peak_sust = peaks.get("bf16_tflops", 1590.0), peaks.get("bf16_tflops_sustained", 1400.0)
    peak_tf = peak_burst if at_max else peak_sust
    peak_src = ("measured (MEASURED_PEAKS.json " if peaks else "fallback (") + \
        ("bf16_tflops, burst: SM clock at its maximum and no power cap during the timed region)" if at_max else
         "bf16_tflops_sustained: the clock dropped or the power cap was active)")
    dom = "bwd_main" if backward else "fwd_main"
    dom_flops = (bwd_f if backward else fwd_f) * (1.0 / world if by_range else h_loc / H)      # rank 0's launch (about, under the range split)
    roof = None
    # DRAM bytes per (row, chunk) entry of the dominant kernel, from one ncu capture of this build on
    # 32K tokens x 32 heads (profiles/main_kernels_traffic_32k.md: dram__bytes_read.sum +
    # dram__bytes_write.sum = 4,759.1 MB over its 8,273,920 entries; the same head-by-head order of
    # work items as the 64K workload); the traffic is per-entry work (gathered rows in, partial rows
    # out), so it scales with the entries.
    entry_bytes = {"bwd_main": BWD_MAIN_DRAM_BYTES_PER_ENTRY}.get(dom) if (d == 128 and chunk == 128) else None
    entries = ACC.selected_entries(seqlens, chunk, topk) * h_loc / (world if by_range else 1)
    if kern_ms.get(dom):
        ach = dom_flops / (kern_ms[dom] * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": dom, "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s",
                "frac": ach / peak_tf, "frac_of_burst": ach / peak_burst, "frac_of_sustained": ach / peak_sust,
                "traffic": (entry_bytes * entries if entry_bytes else None),
                "traffic_source": "ncu dram bytes of a 32K-token x 32-head case of this build, scaled by (row, chunk) entries" if entry_bytes else None,
                "peak_source": peak_src,
                "launch_ms": kern_ms[dom], "flops_per_launch": dom_flops,
                "other_kernels_ms": {k_: v_ for k_, v_ in kern_ms.items() if k_ != dom}}
    line = {
        "metric": "moba_fwd_bwd_selected_block_tflops" if backward else "moba_fwd_selected_block_tflops",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": config_of(wl, seqlens, H, Hk, d, chunk, topk, backward),
        "run": {"sharding": (f"query rows split in {world} ranges, all heads on every rank" if by_range else
                             f"query heads {h0}..{h1 - 1} of {H} on rank 0, whole kv-head groups per rank, no collective"),
                "collective": ("all_gather(centroids, K, V) + reduce_scatter(dK, dV), NCCL, inside the step" if by_range
                               else "none"),
                "l2": f"inputs q,k,v,dO ({4 * T * h_loc * d * 2 >> 20} MB per rank) plus the per-pair partials exceed the 126 MB L2",
                "engine": {"fwd": ["cuda-core", "tcgen05"][_lib.lib.fmb_attn_engine(chunk, d, 0)],
                           "bwd": ["cuda-core", "tcgen05"][_lib.lib.fmb_attn_engine(chunk, d, 1)]}},
        "gpu_launches": int(launches), "launches_per_step": launches / args.steps, "host_ms_per_step": host_ms,
        "status": status, "clocks": clocks, "e2e": e2e, "roofline": roof,
    }
    if world == 1 and not args.no_cpu_baseline:
        dt, fl, rows, threads = cpu_sample(seqlens, d, chunk, topk, rows=8192)
        line["cpu_baseline"] = {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": f"pattern+fwd+bwd of the last {rows} query rows of 1 head vs all "
                                          f"{seqlens[0]} keys, fp32 PyTorch oracle, {dt:.1f} s"}
    emit(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
