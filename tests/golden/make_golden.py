"""Generates tests/golden/hotpath_cases.npz: small seeded inputs with the CPU oracle's outputs.

The reference (an MLIR compiler) cannot be built or imported here, so these vectors are NOT
outputs of the reference itself: they are outputs of oracle/nova_oracle.c (fp32-accumulate mode),
which is pinned to the reference's own known-answer cases in tests/test_oracle_pins.py.  They
guard the CUDA kernels and the oracle against silent drift.  The reference's constant-input
known answers (test/wrapper.c:93-99, robust_driver.cpp:71-80,100-108) are stored as well.

    python tests/golden/make_golden.py        # rewrites hotpath_cases.npz

Distributions follow the benchmark configs at reduced sizes: f32 U[-1,1]; f16 N(0,1)/sqrt(K);
bf16 linear X~N(0,1), W,b~N(0,0.02); f16 scores N(0,1); ragged bf16 U[-1,1].
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402


def main():
    rng = np.random.default_rng(1234)
    out = {}

    def put(name, **arrays):
        for k, v in arrays.items():
            out[f"{name}.{k}"] = v

    # C1-like: nova.matmul f32
    a = rng.uniform(-1, 1, (64, 80)).astype(np.float32)
    b = rng.uniform(-1, 1, (80, 48)).astype(np.float32)
    put("c1_f32", a=a, b=b, c=O.gemm(a, b))
    # C2-like: linalg.batch_matmul f16, fp32 accumulate, f16 out
    a = O.to_bits(rng.normal(size=(2, 48, 64)).astype(np.float32) / 8, "f16")
    b = O.to_bits(rng.normal(size=(2, 64, 40)).astype(np.float32) / 8, "f16")
    put("c2_f16_bmm", a=a, b=b, c=O.gemm(a, b, dtype_in="f16"))
    # C3-like: linear bf16 + bias + GELU(tanh)
    x = O.to_bits(rng.normal(size=(72, 136)).astype(np.float32), "bf16")
    w = O.to_bits(rng.normal(size=(136, 88)).astype(np.float32) * 0.02, "bf16")
    bias = O.to_bits(rng.normal(size=88).astype(np.float32) * 0.02, "bf16")
    put("c3_bf16_linear_gelu", a=x, b=w, bias=bias, c=O.gemm(x, w, dtype_in="bf16", bias=bias, act="gelu_tanh"))
    # C4-like: attention scores f16
    q = O.to_bits(rng.normal(size=(2, 96, 128)).astype(np.float32), "f16")
    k = O.to_bits(rng.normal(size=(2, 128, 80)).astype(np.float32), "f16")
    put("c4_f16_scores", a=q, b=k, c=O.gemm(q, k, dtype_in="f16"))
    # C5-like: ragged bf16 (odd pitches)
    a = O.to_bits(rng.uniform(-1, 1, (77, 33)).astype(np.float32), "bf16")
    b = O.to_bits(rng.uniform(-1, 1, (33, 45)).astype(np.float32), "bf16")
    put("c5_bf16_ragged", a=a, b=b, c=O.gemm(a, b, dtype_in="bf16"))
    # ltest/test_cpu.mlir: 8x16 @ 16x10 + [1,10] + relu
    a = rng.uniform(-1, 1, (8, 16)).astype(np.float32)
    b = rng.uniform(-1, 1, (16, 10)).astype(np.float32)
    bias = rng.uniform(-1, 1, 10).astype(np.float32)
    put("test_cpu_mlir", a=a, b=b, bias=bias, c=O.gemm(a, b, bias=bias, act="relu"))
    # row ops + gather
    x = rng.normal(size=(6, 384)).astype(np.float32)
    g = rng.normal(size=384).astype(np.float32)
    be = rng.normal(size=384).astype(np.float32)
    y, ms, rs = O.layer_norm(x, g, be)
    put("layer_norm_f32", x=x, gamma=g, beta=be, y=y, mean_sum=ms, rstd=rs)
    put("softmax_f32", x=x, y=O.softmax(x))
    table = rng.normal(size=(50, 12)).astype(np.float32)
    ids = rng.integers(0, 50, size=(2, 7)).astype(np.int16)
    put("gather_i16", table=table, ids=ids, out=O.gather(table, ids)[0])
    # constant-input known answers held by the reference itself
    put("known_answers", wrapper_c=np.float32(4096.5), robust_matmul=np.float32(48.0), robust_gelu=np.float32(32.0))
    np.savez_compressed(os.path.join(HERE, "hotpath_cases.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
