"""Builds the CPU oracle (oracle/nova_oracle.c) into oracle/libnova_oracle.so.

Test infrastructure only.  The reference itself (an MLIR/LLVM 21.1.6 out-of-tree
compiler) cannot be compiled with gcc alone, so there is no `oracle/_ref` build:
the oracle is a C restatement of the reference's CPU loop nests.

Flags: -ffp-contract=off -fno-fast-math keep one rounding per multiply and per
add (the reference's linalg bodies carry no `contract` flag);
-march=x86-64-v3 (AVX2) is the widest ISA level assumed on the benchmark host.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "nova_oracle.c")
OUT = os.path.join(HERE, "libnova_oracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = [
        "gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
        "-fPIC", "-shared", "-std=c11", "-Wall", "-Wextra", "-o", OUT, SRC, "-lm",
    ]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
