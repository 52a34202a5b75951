"""Build libhyacin.so (sm_100a) in-tree with nvcc.  Cross-compiles without a GPU.

Usage: ``python -m hyacinth_b200._build [--force] [--verbose-ptxas]``
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libhyacin.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]
# potrfp.cu must round like the reference's build of the same arithmetic: that build uses --use_fast_math, which
# for FP32 Gram matrices means flush-to-zero and approximate division / square root (FP64 code is unaffected).
PER_FILE_FLAGS = {"potrfp.cu": ["--use_fast_math"]}
LINK_FLAGS = ["-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xlinker", "-Bsymbolic",
              "-lcublas", "-lcusolver", "-lnccl"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, ptxas_verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    jobs = []
    for src in sources():
        obj = os.path.join(OBJ, src + ".o")
        if force or _stale(obj, [os.path.join(CSRC, src)] + headers):
            cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_verbose else []) + PER_FILE_FLAGS.get(src, []) + ["-c", os.path.join(CSRC, src), "-o", obj]
            jobs.append(cmd)
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, res in zip(jobs, ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs)):
                if res.returncode != 0:
                    sys.stderr.write(res.stdout + res.stderr)
                    raise RuntimeError("nvcc failed: " + " ".join(cmd))
                if ptxas_verbose:
                    sys.stderr.write(res.stderr)
    objs = [os.path.join(OBJ, s + ".o") for s in sources()]
    if force or jobs or _stale(LIB, objs):
        subprocess.check_call(["nvcc"] + LINK_FLAGS + ["-o", LIB] + objs)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, ptxas_verbose="--verbose-ptxas" in sys.argv))
