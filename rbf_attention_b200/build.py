"""Builds librbf_b200.so in-tree with nvcc for sm_100a (no torch headers, no libcuda link dependency).

Usage: ``python -m rbf_attention_b200.build [--force] [--verbose]``.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "librbf_b200.so")
SOURCES = ["capi.cu", "rbf_prep.cu", "rbf_fwd.cu", "rbf_fwd_tf32.cu", "rbf_bwd.cu", "rbf_bwd_fused.cu",
           "rbf_bwd_fused128.cu", "ce_loss.cu", "layer_norm.cu", "col_sums.cu", "gelu.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _deps() -> list[str]:
    root_inc = os.path.join(os.path.dirname(HERE), "include", "rbf_b200.h")
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [root_inc]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every translation unit to an object and links the shared library. Returns its path."""
    deps = _deps()
    objs = []
    jobs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, deps):
            cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {cmd[-3]}")

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        list(pool.map(run, jobs))
    if jobs or force or _stale(LIB, objs):
        run([_nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
