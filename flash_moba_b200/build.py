"""In-tree build of libflashmoba_b200.so with nvcc for sm_100a (no torch headers involved).

    python flash_moba_b200/build.py [--force]

Objects go to flash_moba_b200/_build/, the library next to this file, so that the built
library travels with a snapshot of the source tree.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libflashmoba_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
# --use_fast_math must not touch the CUDA-core validation engine or the combine kernels'
# exp/log: those files are built without it.
PRECISE = {"fmb_attn_simt.cu", "fmb_attn_common.cu", "fmb_gate.cu", "fmb_pool.cu"}


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(nvcc, src, obj, log):
    flags = [f for f in NVCC_FLAGS if not (f == "--use_fast_math" and os.path.basename(src) in PRECISE)]
    flags = flags + os.environ.get("FMB_EXTRA_NVCC_FLAGS", "").split()
    cmd = [nvcc] + flags + ["-I", INCLUDE, "-c", src, "-o", obj]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout[-4000:]}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile what is out of date and link the shared library; returns its path."""
    nvcc = _nvcc()
    os.makedirs(BUILD, exist_ok=True)
    dep_t = _deps_mtime()
    jobs, objs = [], []
    for s in _sources():
        src = os.path.join(CSRC, s)
        obj = os.path.join(BUILD, s[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), dep_t):
            jobs.append((src, obj, os.path.join(BUILD, s[:-3] + ".log")))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for fut in [ex.submit(_compile, nvcc, *j) for j in jobs]:
                o = fut.result()
                if verbose:
                    print("compiled", os.path.basename(o))
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout[-4000:])
        if verbose:
            print("linked", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
