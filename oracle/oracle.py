"""ctypes binding of the CPU oracle (oracle/nova_oracle.c).

TEST INFRASTRUCTURE ONLY — imported by tests/, by __graft_entry__.smoke() and
by bench.py's CPU-baseline legs, never by the product package.

16-bit tensors travel as numpy uint16 arrays holding the raw f16 / bf16 bits;
`to_bits` / `from_bits` convert to and from float32.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

F32, F16, BF16 = 0, 1, 2
DTYPES = {"f32": F32, "f16": F16, "bf16": BF16}
ACC = {"f32": 0, "result": 1, "f64": 2}
ACT = {"none": 0, "relu": 1, "gelu_tanh": 2, "gelu_tanh_grad": 3}
INIT_ZERO, INIT_BIAS_ROW, INIT_RESIDUAL_FULL, INIT_BIAS_AND_RESIDUAL = 0, 1, 2, 4


class _GemmArgs(C.Structure):
    _fields_ = [
        ("dtype_in", C.c_int32), ("dtype_out", C.c_int32), ("acc_mode", C.c_int32), ("act", C.c_int32),
        ("init", C.c_int32), ("trans_a", C.c_int32), ("trans_b", C.c_int32), ("bias_after", C.c_int32),
        ("batch", C.c_int64), ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64), ("ldr", C.c_int64),
        ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_c", C.c_int64), ("stride_r", C.c_int64),
        ("A", C.c_void_p), ("B", C.c_void_p), ("bias", C.c_void_p), ("residual", C.c_void_p), ("C", C.c_void_p),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _build.OUT
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(_build.SRC):
            _build.build()
        _lib = C.CDLL(path)
        _lib.nova_oracle_gemm.argtypes = [C.POINTER(_GemmArgs)]
        _lib.nova_oracle_gemm.restype = C.c_int
        _lib.nova_oracle_gemm_scalar_rows.argtypes = [C.POINTER(_GemmArgs), C.c_int64, C.c_int64]
        _lib.nova_oracle_gemm_scalar_rows.restype = C.c_int
        _lib.nova_oracle_gather.restype = C.c_int64
    return _lib


def np_dtype(dt: str):
    return np.float32 if dt == "f32" else np.uint16


def to_bits(x: np.ndarray, dt: str) -> np.ndarray:
    """float32 array -> storage array of dtype `dt` (RNE), via the oracle's own converters."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dt == "f32":
        return x
    out = np.empty(x.shape, dtype=np.uint16)
    fn = lib().nova_oracle_f32_to_bf16 if dt == "bf16" else lib().nova_oracle_f32_to_f16
    fn(C.c_void_p(x.ctypes.data), C.c_void_p(out.ctypes.data), C.c_int64(x.size))
    return out


def from_bits(x: np.ndarray, dt: str) -> np.ndarray:
    """storage array of dtype `dt` -> float32 array (exact)."""
    if dt == "f32":
        return np.asarray(x, dtype=np.float32)
    x = np.ascontiguousarray(x).view(np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    fn = lib().nova_oracle_bf16_to_f32 if dt == "bf16" else lib().nova_oracle_f16_to_f32
    fn(C.c_void_p(x.ctypes.data), C.c_void_p(out.ctypes.data), C.c_int64(x.size))
    return out


def _ptr(a):
    return C.c_void_p(a.ctypes.data) if a is not None else C.c_void_p(0)


def _gemm_args(A, B, Cout, dtype_in, dtype_out, acc, act, bias, residual, trans_a, trans_b, bias_after):
    A3 = A if A.ndim == 3 else A[None]
    shared_b = B.ndim == 2
    B3 = B[None] if shared_b else B
    batch = A3.shape[0]
    M, K = (A3.shape[2], A3.shape[1]) if trans_a else (A3.shape[1], A3.shape[2])
    N, Kb = (B3.shape[1], B3.shape[2]) if trans_b else (B3.shape[2], B3.shape[1])
    if K != Kb:
        raise ValueError(f"K mismatch: {K} vs {Kb}")  # MatmulOp verify, NovaOps.cpp:1247-1254
    if not shared_b and B3.shape[0] != batch:
        raise ValueError("batch mismatch")
    g = _GemmArgs()
    g.dtype_in, g.dtype_out = DTYPES[dtype_in], DTYPES[dtype_out]
    g.acc_mode, g.act = ACC[acc], ACT[act]
    if bias is not None and residual is not None:
        g.init = INIT_BIAS_AND_RESIDUAL
    else:
        g.init = INIT_BIAS_ROW if bias is not None else (INIT_RESIDUAL_FULL if residual is not None else INIT_ZERO)
    g.trans_a, g.trans_b, g.bias_after = int(trans_a), int(trans_b), int(bias_after)
    g.batch, g.M, g.N, g.K = batch, M, N, K
    g.lda, g.ldb, g.ldc, g.ldr = A3.shape[2], B3.shape[2], N, N
    g.stride_a = A3.shape[1] * A3.shape[2]
    g.stride_b = 0 if shared_b else B3.shape[1] * B3.shape[2]
    g.stride_c = M * N
    g.stride_r = M * N
    g.A, g.B, g.C = A.ctypes.data, B.ctypes.data, Cout.ctypes.data
    g.bias = bias.ctypes.data if bias is not None else None
    g.residual = residual.ctypes.data if residual is not None else None
    return g, (batch, M, N)


def gemm(A, B, *, dtype_in="f32", dtype_out=None, acc="f32", act="none", bias=None, residual=None,
         trans_a=False, trans_b=False, bias_after=False, gelu_grad_of=None):
    """C = act(init + A @ B).  A: [M,K] or [B,M,K]; B: [K,N] (shared across the batch) or [B,K,N].
    bias: [N] of dtype_out; residual: [B,M,N] / [M,N] of dtype_out.  gelu_grad_of=Z ([B,M,N] / [M,N]):
    C = (init + A @ B) * gelu_tanh'(Z), the contraction followed by nova.gelu_backward (excludes residual
    and act).  Returns storage array of dtype_out."""
    dtype_out = dtype_out or dtype_in
    if gelu_grad_of is not None:
        if residual is not None or act != "none":
            raise ValueError("gelu_grad_of excludes residual and act")
        act = "gelu_tanh_grad"
    A = np.ascontiguousarray(A, dtype=np_dtype(dtype_in))
    B = np.ascontiguousarray(B, dtype=np_dtype(dtype_in))
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np_dtype(dtype_out)).reshape(-1)
    if residual is not None:
        residual = np.ascontiguousarray(residual, dtype=np_dtype(dtype_out))
    A3 = A if A.ndim == 3 else A[None]
    M = A3.shape[2] if trans_a else A3.shape[1]
    B3 = B[None] if B.ndim == 2 else B
    N = B3.shape[1] if trans_b else B3.shape[2]
    out = np.zeros((A3.shape[0], M, N), dtype=np_dtype(dtype_out))
    g, _ = _gemm_args(A, B, out, dtype_in, dtype_out, acc, act, bias, residual, trans_a, trans_b, bias_after)
    if gelu_grad_of is not None:
        z = np.ascontiguousarray(gelu_grad_of, dtype=np_dtype(dtype_out))
        if z.size != out.size:
            raise ValueError("gelu_grad_of must have the shape of the result")
        g.residual = z.ctypes.data
    rc = lib().nova_oracle_gemm(C.byref(g))
    if rc != 0:
        raise RuntimeError(f"nova_oracle_gemm failed: {rc}")
    return out if A.ndim == 3 else out[0]


def gemm_scalar_rows(A, B, *, dtype_in="f32", dtype_out=None, act="none", bias=None, row_begin=0, row_end=None):
    """The reference's single-threaded i/j/k nest (C re-loaded every k, k unrolled x8) over a slice of
    the (batch*M) rows; rows outside the slice are left zero.  Used for the timed CPU baseline."""
    dtype_out = dtype_out or dtype_in
    A = np.ascontiguousarray(A, dtype=np_dtype(dtype_in))
    B = np.ascontiguousarray(B, dtype=np_dtype(dtype_in))
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np_dtype(dtype_out)).reshape(-1)
    A3 = A if A.ndim == 3 else A[None]
    B3 = B[None] if B.ndim == 2 else B
    out = np.zeros((A3.shape[0], A3.shape[1], B3.shape[2]), dtype=np_dtype(dtype_out))
    g, (batch, M, _) = _gemm_args(A, B, out, dtype_in, dtype_out, "f32", act, bias, None, False, False, False)
    if row_end is None:
        row_end = batch * M
    rc = lib().nova_oracle_gemm_scalar_rows(C.byref(g), C.c_int64(row_begin), C.c_int64(row_end))
    if rc != 0:
        raise RuntimeError(f"nova_oracle_gemm_scalar_rows failed: {rc}")
    return out if A.ndim == 3 else out[0]


def activation(x, dt="f32", act="gelu_tanh", compute_f32=False):
    x = np.ascontiguousarray(x, dtype=np_dtype(dt))
    y = np.empty_like(x)
    lib().nova_oracle_activation(_ptr(x), _ptr(y), C.c_int64(x.size), C.c_int(DTYPES[dt]), C.c_int(ACT[act]),
                                 C.c_int(int(compute_f32)))
    return y


def gelu_backward(grad_out, x, dt="f32", compute_f32=False):
    """grad_out * gelu_tanh'(x) (nova.gelu_backward)."""
    go = np.ascontiguousarray(grad_out, dtype=np_dtype(dt))
    x = np.ascontiguousarray(x, dtype=np_dtype(dt))
    if go.shape != x.shape:
        raise ValueError("gelu_backward: shapes differ")
    y = np.empty_like(x)
    lib().nova_oracle_gelu_backward(_ptr(go), _ptr(x), _ptr(y), C.c_int64(x.size), C.c_int(DTYPES[dt]),
                                    C.c_int(int(compute_f32)))
    return y


def add_rowbcast(a, b, dt="f32"):
    a = np.ascontiguousarray(a, dtype=np_dtype(dt))
    b = np.ascontiguousarray(b, dtype=np_dtype(dt))
    cols = a.shape[-1]
    rows = a.size // cols
    full = int(b.size == a.size)
    if not full and b.size != cols:
        raise ValueError("operand is neither full-shape nor a row vector")
    out = np.empty_like(a)
    lib().nova_oracle_add_rowbcast(_ptr(a), _ptr(b), _ptr(out), C.c_int64(rows), C.c_int64(cols), C.c_int(full),
                                   C.c_int(DTYPES[dt]))
    return out


def softmax(x, dt="f32", compute_f32=False):
    x = np.ascontiguousarray(x, dtype=np_dtype(dt))
    D = x.shape[-1]
    y = np.empty_like(x)
    lib().nova_oracle_softmax(_ptr(x), _ptr(y), C.c_int64(x.size // D), C.c_int64(D), C.c_int(DTYPES[dt]),
                              C.c_int(int(compute_f32)))
    return y


def layer_norm(x, gamma, beta, dt="f32", compute_f32=False):
    x = np.ascontiguousarray(x, dtype=np_dtype(dt))
    gamma = np.ascontiguousarray(gamma, dtype=np_dtype(dt))
    beta = np.ascontiguousarray(beta, dtype=np_dtype(dt))
    D = x.shape[-1]
    rows = x.size // D
    y = np.empty_like(x)
    mean_sum = np.empty(x.shape[:-1], dtype=x.dtype)
    rstd = np.empty(x.shape[:-1], dtype=x.dtype)
    lib().nova_oracle_layer_norm(_ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), _ptr(mean_sum), _ptr(rstd),
                                 C.c_int64(rows), C.c_int64(D), C.c_int(DTYPES[dt]), C.c_int(int(compute_f32)))
    return y, mean_sum, rstd


def layer_norm_backward(grad_y, x, gamma, mean_sum, rstd, dt="f32", compute_f32=False):
    """(dx, dgamma, dbeta) of nova.layer_norm_backward; mean_sum is the raw row sum the forward returned."""
    gy = np.ascontiguousarray(grad_y, dtype=np_dtype(dt))
    x = np.ascontiguousarray(x, dtype=np_dtype(dt))
    gamma = np.ascontiguousarray(gamma, dtype=np_dtype(dt)).reshape(-1)
    mean_sum = np.ascontiguousarray(mean_sum, dtype=np_dtype(dt)).reshape(-1)
    rstd = np.ascontiguousarray(rstd, dtype=np_dtype(dt)).reshape(-1)
    D = x.shape[-1]
    rows = x.size // D
    if gy.shape != x.shape or gamma.size != D or mean_sum.size != rows or rstd.size != rows:
        raise ValueError("layer_norm_backward: operand shapes do not agree")
    dx = np.empty_like(x)
    dgamma = np.empty(D, dtype=x.dtype)
    dbeta = np.empty(D, dtype=x.dtype)
    lib().nova_oracle_layer_norm_backward(_ptr(gy), _ptr(x), _ptr(gamma), _ptr(mean_sum), _ptr(rstd), _ptr(dx),
                                          _ptr(dgamma), _ptr(dbeta), C.c_int64(rows), C.c_int64(D),
                                          C.c_int(DTYPES[dt]), C.c_int(int(compute_f32)))
    return dx, dgamma, dbeta


def column_sum(x, dt="f32", compute_f32=True):
    x = np.ascontiguousarray(x, dtype=np_dtype(dt))
    cols = x.shape[-1]
    rows = x.size // cols
    out = np.empty(cols, dtype=x.dtype)
    lib().nova_oracle_column_sum(_ptr(x), _ptr(out), C.c_int64(rows), C.c_int64(cols), C.c_int(DTYPES[dt]),
                                 C.c_int(int(compute_f32)))
    return out


def gather(inp, idx, axis=0):
    """nova.gather: out[pre..., idx..., post...] = inp[pre..., idx[...], post...].  Index tensors whose
    leading dims equal inp's leading `axis` dims are treated as batched (NovaOps.cpp:1898-1946)."""
    inp = np.ascontiguousarray(inp)
    idx = np.ascontiguousarray(idx)
    if axis < 0:
        axis += inp.ndim
    batch_dims = 0
    for i in range(min(axis, idx.ndim)):
        if inp.shape[i] != idx.shape[i]:
            break
        batch_dims += 1
    batched = batch_dims == axis and axis > 0
    if axis > 0 and not batched and batch_dims != 0:
        raise NotImplementedError("partially batched gather")
    pre = int(np.prod(inp.shape[:axis], dtype=np.int64))
    post = int(np.prod(inp.shape[axis + 1:], dtype=np.int64))
    idx_shape = idx.shape[batch_dims:] if batched else idx.shape
    n_idx = int(np.prod(idx_shape, dtype=np.int64))
    out_shape = inp.shape[:axis] + tuple(idx_shape) + inp.shape[axis + 1:]
    out = np.empty(out_shape, dtype=inp.dtype)
    bits = idx.dtype.itemsize * 8
    if bits == 16:
        idx = idx.view(np.uint16)
    bad = lib().nova_oracle_gather(_ptr(inp), _ptr(idx), _ptr(out), C.c_int64(pre), C.c_int64(inp.shape[axis]),
                                   C.c_int64(post), C.c_int64(n_idx), C.c_int(bits), C.c_int(int(batched)),
                                   C.c_int(inp.dtype.itemsize))
    return out, int(bad)


def _idx_view(idx):
    idx = np.ascontiguousarray(idx)
    bits = idx.dtype.itemsize * 8
    if bits not in (16, 32, 64):
        raise ValueError("index dtype must be 16, 32 or 64 bits wide")
    return (idx.view(np.uint16) if bits == 16 else idx), bits


def sce(logits, targets, dt="f32", compute_f32=False):
    """nova.sce over the last dim: returns (softmax, loss[1], out-of-range target count)."""
    x = np.ascontiguousarray(logits, dtype=np_dtype(dt))
    t, bits = _idx_view(targets)
    Cn = x.shape[-1]
    rows = x.size // Cn
    if t.size != rows:
        raise ValueError("sce: one target per row")
    sm = np.empty_like(x)
    loss = np.empty(1, dtype=x.dtype)
    lib().nova_oracle_sce.restype = C.c_int64
    bad = lib().nova_oracle_sce(_ptr(x), _ptr(t), _ptr(sm), _ptr(loss), C.c_int64(rows), C.c_int64(Cn),
                                C.c_int(DTYPES[dt]), C.c_int(bits), C.c_int(int(compute_f32)))
    return sm, loss, int(bad)


def sce_backward(softmax, targets, dt="f32", compute_f32=False):
    """nova.sce_backward over the last dim: (softmax - one_hot(targets)) / rows."""
    p = np.ascontiguousarray(softmax, dtype=np_dtype(dt))
    t, bits = _idx_view(targets)
    Cn = p.shape[-1]
    rows = p.size // Cn
    if t.size != rows:
        raise ValueError("sce_backward: one target per row")
    g = np.empty_like(p)
    lib().nova_oracle_sce_backward.restype = C.c_int64
    lib().nova_oracle_sce_backward(_ptr(p), _ptr(t), _ptr(g), C.c_int64(rows), C.c_int64(Cn), C.c_int(DTYPES[dt]),
                                   C.c_int(bits), C.c_int(int(compute_f32)))
    return g


def scatter_add(inp, indices, src, axis=0, dt="f32"):
    """nova.scatter_add: a copy of inp with src added at indices along axis; returns (out, skipped count)."""
    out = np.array(inp, dtype=np_dtype(dt), copy=True, order="C")
    src = np.ascontiguousarray(src, dtype=np_dtype(dt))
    t, bits = _idx_view(indices)
    if axis < 0:
        axis += out.ndim
    pre = int(np.prod(out.shape[:axis], dtype=np.int64))
    post = int(np.prod(out.shape[axis + 1:], dtype=np.int64))
    n_idx = src.shape[axis]
    if t.size != n_idx or src.shape[:axis] != out.shape[:axis] or src.shape[axis + 1:] != out.shape[axis + 1:]:
        raise ValueError("scatter_add: shapes must match except at axis; one index per src slice")
    lib().nova_oracle_scatter_add.restype = C.c_int64
    bad = lib().nova_oracle_scatter_add(_ptr(out), _ptr(t), _ptr(src), C.c_int64(pre), C.c_int64(out.shape[axis]),
                                        C.c_int64(post), C.c_int64(n_idx), C.c_int(bits), C.c_int(DTYPES[dt]))
    return out, int(bad)


def transpose_last2(x):
    x = np.ascontiguousarray(x)
    R, Cc = x.shape[-2], x.shape[-1]
    batch = x.size // (R * Cc)
    out = np.empty(x.shape[:-2] + (Cc, R), dtype=x.dtype)
    lib().nova_oracle_transpose_last2(_ptr(x), _ptr(out), C.c_int64(batch), C.c_int64(R), C.c_int64(Cc),
                                      C.c_int(x.dtype.itemsize))
    return out


def rel_fro(a: np.ndarray, b: np.ndarray) -> float:
    """relative Frobenius error ||a-b|| / ||b|| in float64."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b.ravel())
    return float(np.linalg.norm((a - b).ravel()) / (den if den > 0 else 1.0))
