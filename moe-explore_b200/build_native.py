"""Build libmoe_sm100.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Usage: python moe-explore_b200/build_native.py [--force] [-v] [--out other/path.so]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libmoe_sm100.so")
SOURCES = ["api.cu", "routing.cu", "rows.cu", "router.cu", "grouped_gemm.cu", "no_alloc.cu"] + \
          [f"gemm_inst_{t}_{c}{g}.cu" for t in ("bf16", "f16") for c in ("pair", "single") for g in ("", "_gather")]
HEADERS = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "gemm_kernel.cuh"),
           os.path.join(os.path.dirname(HERE), "include", "moe_sm100.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, out: str = OUT) -> str:
    """Compile what is stale and link ``out`` (default: the library next to the package; another path gives a second
    build that ``MOE_SM100_LIBRARY`` can point the package at)."""
    sources = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    objs = []
    procs = []
    for src in sources:
        obj = os.path.splitext(src)[0] + ".o"
        objs.append(obj)
        if force or _stale(obj, [src] + HEADERS):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        log, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{log}")
        if verbose:
            print(log)
    if force or procs or _stale(out, objs):
        # link into a temporary name and rename: a process that loads the library while it is being rebuilt sees the
        # old file or the new one, never a partial one
        tmp = out + ".tmp"
        cmd = [_nvcc(), "-shared", "-o", tmp] + objs
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}")
        os.replace(tmp, out)
    return out


if __name__ == "__main__":
    target = sys.argv[sys.argv.index("--out") + 1] if "--out" in sys.argv else OUT
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, out=target)
    print(path)
