"""The committed golden vectors (tests/golden/hotpath_cases.npz) replayed through the CPU oracle:
bit-exact, since the oracle generated them.  Guards the oracle against drift; the same file is
replayed through the CUDA kernels in tests/test_gemm_gpu.py."""
import os

import numpy as np

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_cases.npz")


def test_oracle_reproduces_golden_vectors(oracle):
    z = np.load(GOLD)
    assert np.array_equal(oracle.gemm(z["c1_f32.a"], z["c1_f32.b"]), z["c1_f32.c"])
    assert np.array_equal(oracle.gemm(z["c2_f16_bmm.a"], z["c2_f16_bmm.b"], dtype_in="f16"), z["c2_f16_bmm.c"])
    assert np.array_equal(
        oracle.gemm(z["c3_bf16_linear_gelu.a"], z["c3_bf16_linear_gelu.b"], dtype_in="bf16",
                    bias=z["c3_bf16_linear_gelu.bias"], act="gelu_tanh"), z["c3_bf16_linear_gelu.c"])
    assert np.array_equal(oracle.gemm(z["c4_f16_scores.a"], z["c4_f16_scores.b"], dtype_in="f16"), z["c4_f16_scores.c"])
    assert np.array_equal(oracle.gemm(z["c5_bf16_ragged.a"], z["c5_bf16_ragged.b"], dtype_in="bf16"),
                          z["c5_bf16_ragged.c"])
    assert np.array_equal(
        oracle.gemm(z["test_cpu_mlir.a"], z["test_cpu_mlir.b"], bias=z["test_cpu_mlir.bias"], act="relu"),
        z["test_cpu_mlir.c"])
    y, ms, rs = oracle.layer_norm(z["layer_norm_f32.x"], z["layer_norm_f32.gamma"], z["layer_norm_f32.beta"])
    assert np.array_equal(y, z["layer_norm_f32.y"]) and np.array_equal(ms, z["layer_norm_f32.mean_sum"])
    assert np.array_equal(rs, z["layer_norm_f32.rstd"])
    assert np.array_equal(oracle.softmax(z["softmax_f32.x"]), z["softmax_f32.y"])
    assert np.array_equal(oracle.gather(z["gather_i16.table"], z["gather_i16.ids"])[0], z["gather_i16.out"])


def test_known_answers_recorded_from_the_reference(oracle):
    z = np.load(GOLD)
    assert float(z["known_answers.wrapper_c"]) == 4096.5      # test/wrapper.c:93-99
    assert float(z["known_answers.robust_matmul"]) == 48.0    # robust_driver.cpp:71-80
    assert float(z["known_answers.robust_gelu"]) == 32.0      # robust_driver.cpp:100-108
