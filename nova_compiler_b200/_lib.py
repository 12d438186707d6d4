"""ctypes view of libnova_b200.so — the structs, enums and prototypes of include/nova_b200.h.

Loading fails loudly when the shared object is missing: there is no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnova_b200.so")

# nova_b200_status
OK, ERR_INVALID_ARG, ERR_LAYOUT, ERR_UNSUPPORTED, ERR_CUDA, ERR_NO_DEVICE, ERR_DEVICE_TIMEOUT, ERR_TOO_LARGE = range(8)
STATUS_NAMES = ["OK", "ERR_INVALID_ARG", "ERR_LAYOUT", "ERR_UNSUPPORTED", "ERR_CUDA", "ERR_NO_DEVICE",
                "ERR_DEVICE_TIMEOUT", "ERR_TOO_LARGE"]
# nova_b200_dtype
F32, F16, BF16, I16, I32, I64, I1 = range(7)
# nova_b200_act
ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_GELU_TANH_GRAD = range(4)
# nova_b200_acc_init
INIT_ZERO, INIT_BIAS_ROW, INIT_RESIDUAL_FULL, INIT_FROM_C, INIT_BIAS_AND_RESIDUAL, INIT_LN_FOLD = range(6)
# nova_b200_binary_op
BIN_ADD, BIN_SUB, BIN_MUL = range(3)
# nova_b200_f32_mode
TF32X3, TF32X1 = range(2)


class GemmArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("dtype_ab", C.c_int32), ("dtype_c", C.c_int32), ("trans_a", C.c_int32),
        ("trans_b", C.c_int32), ("act", C.c_int32), ("init", C.c_int32), ("f32_mode", C.c_int32),
        ("batch", C.c_int64), ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p), ("bias", C.c_void_p), ("residual", C.c_void_p),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64), ("ldr", C.c_int64),
        ("batch_stride_a", C.c_int64), ("batch_stride_b", C.c_int64), ("batch_stride_c", C.c_int64),
        ("batch_stride_r", C.c_int64),
    ]


class GemmPlanInfo(C.Structure):
    _fields_ = [
        ("loader_a", C.c_int32), ("loader_b", C.c_int32), ("store_c", C.c_int32), ("block_m", C.c_int32),
        ("block_n", C.c_int32), ("block_k", C.c_int32), ("stages", C.c_int32), ("grid", C.c_int32),
        ("tiles", C.c_int64), ("scratch_bytes", C.c_int64),
    ]


def _memref(rank: int):
    class MemRef(C.Structure):
        _fields_ = [("allocated", C.c_void_p), ("aligned", C.c_void_p), ("offset", C.c_int64),
                    ("sizes", C.c_int64 * rank), ("strides", C.c_int64 * rank)]
    MemRef.__name__ = f"MemRef{rank}D"
    return MemRef


MemRef1D, MemRef2D, MemRef3D, MemRef4D = _memref(1), _memref(2), _memref(3), _memref(4)


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("rank", C.c_int32), ("shape", C.c_int64 * 6)]


# every extern "C" symbol include/nova_b200.h declares: name -> (restype, argtypes)
PROTOTYPES = {
    "nova_b200_init": (C.c_int32, [C.c_int32]),
    "nova_b200_shutdown": (C.c_int32, []),
    "nova_b200_last_error_string": (C.c_char_p, []),
    "nova_b200_abi_version": (C.c_int32, []),
    "nova_b200_set_option": (C.c_int32, [C.c_char_p, C.c_int64]),
    "nova_b200_get_option": (C.c_int32, [C.c_char_p, C.POINTER(C.c_int64)]),
    "nova_b200_reserve_scratch": (C.c_int32, [C.c_int64, C.c_void_p]),
    "nova_b200_operand_prepare": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                              C.c_void_p, C.POINTER(C.c_void_p)]),
    "nova_b200_operand_view": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "nova_b200_operand_free": (None, [C.c_void_p]),
    "nova_b200_gemm": (C.c_int32, [C.POINTER(GemmArgs), C.c_void_p]),
    "nova_b200_gemm_flat": (C.c_int32, [C.c_int64] * 17 + [C.c_int32] * 7 + [C.c_int64]),
    "nova_b200_gemm_push": (C.c_int32, [C.POINTER(GemmArgs), C.POINTER(C.c_void_p), C.c_int32, C.c_void_p]),
    "nova_b200_peer_buffer_alloc": (C.c_int32, [C.c_int64, C.POINTER(C.c_void_p), C.c_char_p]),
    "nova_b200_peer_buffer_open": (C.c_int32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "nova_b200_peer_buffer_close": (C.c_int32, [C.c_void_p]),
    "nova_b200_peer_buffer_free": (C.c_int32, [C.c_void_p]),
    "nova_b200_gemm_plan": (C.c_int32, [C.POINTER(GemmArgs), C.POINTER(GemmPlanInfo)]),
    "nova_b200_gemm_host": (C.c_int32, [C.POINTER(GemmArgs)]),
    "nova_b200_gemm_f32_static": (C.c_int32, [C.POINTER(GemmArgs), C.c_void_p, C.POINTER(C.c_uint32)]),
    "nova_b200_activation": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p]),
    "nova_b200_sce": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32,
                                  C.c_int32, C.c_void_p, C.c_void_p]),
    "nova_b200_sce_backward": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32,
                                           C.c_int32, C.c_void_p]),
    "nova_b200_f32_presplit": (C.c_int32, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.POINTER(C.c_void_p)]),
    "nova_b200_f32_presplit_release": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "nova_b200_sce_backward_scaled": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32,
                                                  C.c_int32, C.c_float, C.c_void_p]),
    "nova_b200_scatter_add": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                          C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "nova_b200_layer_norm_backward": (C.c_int32, [C.c_void_p] * 8 + [C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "nova_b200_gelu_backward": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]),
    "nova_b200_add_rowbcast": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32,
                                           C.c_int32, C.c_void_p]),
    "nova_b200_binary": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                     C.POINTER(C.c_int64), C.c_int32, C.c_int32, C.c_void_p]),
    "nova_b200_ln_fold_prepare": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                              C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "nova_b200_row_stats": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "nova_b200_layer_norm": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "nova_b200_column_sum": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "nova_b200_softmax": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "nova_b200_gather": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                     C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "nova_b200_interleave_slabs": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int64, C.c_int64,
                                               C.c_int32, C.c_void_p]),
    "nova_b200_device_status": (C.c_int32, [C.POINTER(C.c_uint32)]),
    "nova_b200_module_parse": (C.c_int32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "nova_b200_module_free": (None, [C.c_void_p]),
    "nova_b200_module_signature": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32, C.c_int32, C.POINTER(Tensor),
                                                C.POINTER(C.c_int32)]),
    "nova_b200_module_plan": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_char_p, C.c_int64]),
    "nova_b200_module_run": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(Tensor), C.c_int32, C.POINTER(Tensor),
                                          C.c_int32, C.c_void_p]),
    "_mlir_ciface_nova_b200_matmul": (C.c_int32, [C.POINTER(MemRef2D), C.POINTER(MemRef2D), C.POINTER(MemRef2D),
                                                  C.c_int32]),
    "_mlir_ciface_nova_b200_batch_matmul": (C.c_int32, [C.POINTER(MemRef3D), C.POINTER(MemRef3D), C.POINTER(MemRef3D),
                                                        C.c_int32, C.c_int32]),
    "_mlir_ciface_nova_b200_batch_matmul_4d": (C.c_int32, [C.POINTER(MemRef4D), C.POINTER(MemRef4D), C.POINTER(MemRef4D),
                                                           C.c_int32, C.c_int32]),
    "nova_b200_module_call_ciface": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    "_mlir_ciface_nova_b200_linear": (C.c_int32, [C.POINTER(MemRef2D), C.POINTER(MemRef2D), C.POINTER(MemRef2D),
                                                  C.POINTER(MemRef1D), C.c_int32, C.c_int32]),
}

_lib = None


class NovaB200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"libnova_b200: {name}: {message}")
        self.status = status


def load() -> C.CDLL:
    """Loads libnova_b200.so and binds every prototype.  Raises if the library was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m nova_compiler_b200.build` "
            "(there is no Python/CPU fallback for the CUDA kernels)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here means the .so is stale against the header
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def set_option(name: str, value: int) -> None:
    check(load().nova_b200_set_option(name.encode(), int(value)))


def get_option(name: str) -> int:
    v = C.c_int64(0)
    check(load().nova_b200_get_option(name.encode(), C.byref(v)))
    return int(v.value)


def check(status: int) -> None:
    if status != OK:
        raise NovaB200Error(status, load().nova_b200_last_error_string().decode("utf-8", "replace"))
