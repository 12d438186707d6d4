"""Builds libnova_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m nova_compiler_b200.build [--force] [--verbose] [--trace]

The library is a plain shared object with `extern "C"` entry points (include/nova_b200.h);
it does not link against torch.  nvcc cross-compiles without a GPU present.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libnova_b200.so")
SOURCES = ["gemm_sm100.cu", "gemm_static_scratch.cu", "runtime.cu", "rowops.cu", "frontend_exec.cu",
           "frontend_parse.cpp", "frontend_plan.cpp"]
HEADERS = ["gemm_kernel.cuh", "gemm_kernel_pair.cuh", "ptx_sm100.cuh", "runtime.h", "frontend.h", os.path.join("..", "..", "include", "nova_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """trace=True compiles the kernels' role timelines in (NOVA_B200_TRACE=<file> then dumps them); such a
    build is a few percent slower and is for diagnosis only."""
    headers = [os.path.join(CSRC, h) for h in HEADERS]
    flags = NVCC_FLAGS + (["-DNOVA_B200_TRACE_BUILD"] if trace else [])
    force = force or trace
    objs = []
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, os.path.splitext(src)[0] + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = ["nvcc", *flags, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            for res in ex.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs):
                if verbose or res.returncode != 0:
                    sys.stderr.write(res.stdout + res.stderr)
                if res.returncode != 0:
                    raise RuntimeError("nvcc failed: " + " ".join(res.args))
    if jobs or force or _stale(OUT, objs):
        link = ["nvcc", "-shared", "-o", OUT, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        subprocess.run(link, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
