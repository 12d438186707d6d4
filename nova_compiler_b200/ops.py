"""Host-side mirror of the Nova operator surface for the matmul hot path, on torch CUDA tensors.

Each function corresponds to one nova / linalg op as it reaches code generation in the reference
and forwards to ONE call of the C ABI (include/nova_b200.h).  torch is used only to own device
memory and streams; all arithmetic happens in libnova_b200's CUDA kernels.  There is no fallback:
a missing library raises ImportError, a missing GPU raises NovaB200Error(ERR_NO_DEVICE).

Shape and dtype rules follow the reference's op definitions:
  * matmul        MatmulOp::inferReturnTypes (lib/Dialect/nova/NovaOps.cpp:1116-1285): [...,M,K] x [...,K,N],
                  numpy-style batch broadcast, 1-D operands promoted, K mismatch is an error.
  * linear        LinearOp (NovaOps.cpp:2075-2103): rank-2 or rank-3 input, 2-D weight shared across
                  the batch without a copy (NovaToLinalgGeneric.cpp:1726-1753), result dtype = input dtype.
  * gelu/relu/add/softmax/layer_norm/gather/reshape/transpose: see each docstring.
One deliberate difference: 16-bit inputs accumulate in fp32 and return the INPUT dtype (the
reference infers f16 for every 16-bit matmul, including bf16 x bf16, NovaOps.cpp:1198).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib as L

_DT = {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16}
_IDX = {torch.int16: L.I16, torch.int32: L.I32, torch.int64: L.I64}
_ACT = {None: L.ACT_NONE, "none": L.ACT_NONE, "relu": L.ACT_RELU, "gelu": L.ACT_GELU_TANH, "gelu_tanh": L.ACT_GELU_TANH}


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _on_device(fn):
    """Runs the wrapped op with its tensors' device current, so the library's per-device context, the tensor maps
    and torch's current stream all belong to the device that owns the memory; tensors on different devices are
    refused before anything is launched (the library cannot read another GPU's memory by accident)."""
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        dev = None
        for v in list(args) + list(kwargs.values()):
            if isinstance(v, torch.Tensor) and v.is_cuda:
                if dev is None:
                    dev = v.device
                elif v.device != dev:
                    raise L.NovaB200Error(L.ERR_INVALID_ARG, f"tensors live on different devices ({dev} and {v.device})")
        if dev is None or dev.index == torch.cuda.current_device():
            return fn(*args, **kwargs)
        with torch.cuda.device(dev):
            return fn(*args, **kwargs)

    return wrapper


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, f"dtype {t.dtype} has no kernel (f32, f16, bf16 only)") from None


def _require_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise L.NovaB200Error(L.ERR_NO_DEVICE, "tensor is not on a CUDA device; libnova_b200 has no CPU fallback")


def _inner2(t: torch.Tensor) -> Tuple[int, bool]:
    """(row pitch in elements, stored-transposed?) of the last two dims; copies never happen here."""
    r, c = t.shape[-2], t.shape[-1]
    sr, sc = t.stride(-2), t.stride(-1)
    if sc == 1 or c == 1:
        return (sr if r > 1 else max(sr, c)), False
    if sr == 1 or r == 1:
        return (sc if c > 1 else max(sc, r)), True
    raise L.NovaB200Error(L.ERR_LAYOUT, "neither of the two inner strides is 1")


def _batch_stride(t: torch.Tensor) -> int:
    """Stride of a [B, R, C] tensor's batch dim; 0 when the batch is broadcast (expand) or of size 1."""
    return 0 if t.shape[0] == 1 else t.stride(0)


@_on_device
def gemm(a: torch.Tensor, b: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, act: Optional[str] = None, out: Optional[torch.Tensor] = None,
         out_dtype: Optional[torch.dtype] = None, accumulate_into_out: bool = False,
         f32_mode: int = L.TF32X3, gelu_grad_of: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[b] = act(init + A[b] @ B[b]) on rank-3 views; A: [B,M,K], B: [B or 1,K,N] (any of the two inner
    dims may be the contiguous one: transposed views are passed as trans_a / trans_b, not copied).
    gelu_grad_of=Z: C = (init + A @ B) * gelu_tanh'(Z), the contraction fused with a following
    nova.gelu_backward (excludes residual and act)."""
    _require_cuda(a, b, bias, residual, out, gelu_grad_of)
    if gelu_grad_of is not None:
        if residual is not None or act not in (None, "none"):
            raise L.NovaB200Error(L.ERR_INVALID_ARG, "gelu_grad_of excludes residual and act")
    if a.dim() != 3 or b.dim() != 3:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "gemm expects rank-3 views")
    if a.dtype != b.dtype:
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "A and B must share a dtype")
    B_, M, K = a.shape
    Bb, Kb, N = b.shape
    if K != Kb:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, f"contraction dims differ: {K} vs {Kb}")  # NovaOps.cpp:1247-1254
    if Bb not in (1, B_):
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "batch dims do not broadcast")
    out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is None:
        out = torch.empty((B_, M, N), dtype=out_dtype, device=a.device)
    g = L.GemmArgs()
    g.struct_size = C.sizeof(L.GemmArgs)
    g.dtype_ab, g.dtype_c = _dt(a), _DT[out_dtype]
    g.lda, ta = _inner2(a)
    g.ldb, tb = _inner2(b)
    ldc, tc = _inner2(out)
    if tc:
        raise L.NovaB200Error(L.ERR_LAYOUT, "output must have unit inner stride")
    g.trans_a, g.trans_b, g.ldc = int(ta), int(tb), ldc
    g.act = _ACT[act]
    g.f32_mode = f32_mode
    g.batch, g.M, g.N, g.K = B_, M, N, K
    g.A, g.B, g.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    g.batch_stride_a = _batch_stride(a) if B_ > 1 else 0
    g.batch_stride_b = 0 if Bb == 1 else b.stride(0)
    g.batch_stride_c = out.stride(0) if B_ > 1 else M * ldc
    if a.shape[0] > 1 and a.stride(0) == 0:
        g.batch_stride_a = 0
    g.init = L.INIT_ZERO
    if bias is not None:
        if bias.dtype != out_dtype or bias.numel() != N or not bias.is_contiguous():
            raise L.NovaB200Error(L.ERR_INVALID_ARG, "bias must be a contiguous [N] tensor of the output dtype")
        g.init, g.bias = L.INIT_BIAS_ROW, bias.data_ptr()
    if residual is not None:
        r3 = residual if residual.dim() == 3 else residual.unsqueeze(0)
        if r3.dtype != out_dtype or tuple(r3.shape[-2:]) != (M, N) or r3.stride(-1) != 1:
            raise L.NovaB200Error(L.ERR_INVALID_ARG, "residual must be [B,M,N] of the output dtype, unit inner stride")
        g.init = L.INIT_BIAS_AND_RESIDUAL if bias is not None else L.INIT_RESIDUAL_FULL
        g.residual, g.ldr = r3.data_ptr(), r3.stride(-2)
        g.batch_stride_r = 0 if r3.shape[0] == 1 else r3.stride(0)
    if gelu_grad_of is not None:
        z3 = gelu_grad_of if gelu_grad_of.dim() == 3 else gelu_grad_of.unsqueeze(0)
        if z3.dtype != out_dtype or tuple(z3.shape[-2:]) != (M, N) or z3.stride(-1) != 1:
            raise L.NovaB200Error(L.ERR_INVALID_ARG, "gelu_grad_of must be [B,M,N] of the output dtype, unit inner stride")
        g.act, g.residual, g.ldr = L.ACT_GELU_TANH_GRAD, z3.data_ptr(), z3.stride(-2)
        g.batch_stride_r = 0 if z3.shape[0] == 1 else z3.stride(0)
    if accumulate_into_out:
        if bias is not None or residual is not None:
            raise L.NovaB200Error(L.ERR_INVALID_ARG, "accumulate_into_out excludes bias and residual")
        g.init = L.INIT_FROM_C
    L.check(L.load().nova_b200_gemm(C.byref(g), _stream()))
    return out


def matmul(a: torch.Tensor, b: torch.Tensor, *, act: Optional[str] = None, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, f32_mode: int = L.TF32X3) -> torch.Tensor:
    """nova.matmul (NovaMatmulOpLowering, NovaToLinalg.cpp:874-1050): rank 2 -> linalg.matmul; rank 3 ->
    linalg.batch_matmul with a 2-D / batch-1 operand broadcast (here: batch stride 0, no materialised copy);
    rank > 3 -> batch dims collapsed to one (metadata only) and expanded back."""
    if a.dim() == 1 and b.dim() == 1:  # 1-D . 1-D -> scalar (NovaOps.cpp:1227-1240)
        return matmul(a.unsqueeze(0), b.unsqueeze(1), act=act, out_dtype=out_dtype, f32_mode=f32_mode).reshape(())
    squeeze_m = a.dim() == 1
    squeeze_n = b.dim() == 1
    if squeeze_m:
        a = a.unsqueeze(0)
    if squeeze_n:
        b = b.unsqueeze(1)
    batch_shape = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
    M, N = a.shape[-2], b.shape[-1]

    def as3(t: torch.Tensor) -> torch.Tensor:
        if t.dim() == 2 or all(s == 1 for s in t.shape[:-2]):
            return t.reshape(1, t.shape[-2], t.shape[-1]) if t.dim() != 3 else t
        t = t.expand(*batch_shape, t.shape[-2], t.shape[-1])
        if len(batch_shape) == 1:
            return t
        # collapsing several batch dims must stay a view (tensor.collapse_shape is metadata)
        try:
            return t.view(-1, t.shape[-2], t.shape[-1])
        except RuntimeError:
            return t.reshape(-1, t.shape[-2], t.shape[-1])  # broadcast across an outer batch dim: materialise

    a3, b3 = as3(a), as3(b)
    nb = 1
    for s in batch_shape:
        nb *= s
    if a3.shape[0] == 1 and nb > 1:
        a3 = a3.expand(nb, -1, -1)
    out3 = gemm(a3, b3, act=act, bias=bias, out_dtype=out_dtype, f32_mode=f32_mode)
    out = out3.reshape(*batch_shape, M, N)
    if squeeze_m:
        out = out.squeeze(-2)
    if squeeze_n:
        out = out.squeeze(-1)
    return out


def batch_matmul(a: torch.Tensor, b: torch.Tensor, *, out_dtype: Optional[torch.dtype] = None,
                 out: Optional[torch.Tensor] = None, act: Optional[str] = None) -> torch.Tensor:
    """linalg.batch_matmul ins(A[B,M,K], B[B,K,N]) outs(C[B,M,N]) with fp32 accumulation."""
    return gemm(a, b, out=out, out_dtype=out_dtype, act=act)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, *, act: Optional[str] = None) -> torch.Tensor:
    """nova.linear (+ optional trailing nova.gelu / nova.relu fused as the epilogue): Y = act(X @ W + bias),
    X rank 2 or 3, W [K,N] shared across the batch, bias of N elements (any rank: flattened like
    NovaToLinalgGeneric.cpp:1772-1784)."""
    if x.dim() not in (2, 3):
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "linear: input must be rank 2 or 3")  # NovaOps.cpp:2097-2101
    if w.dim() != 2:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "linear: weight must be rank 2")
    x3 = x.unsqueeze(0) if x.dim() == 2 else x
    # a contiguous [B,M,K] input with a shared weight is one [B*M,K] GEMM
    if x3.dim() == 3 and x3.is_contiguous():
        x3 = x3.reshape(1, -1, x3.shape[-1])
    y = gemm(x3, w.unsqueeze(0), bias=bias.reshape(-1), act=act)
    return y.reshape(*x.shape[:-1], w.shape[-1])


class PreparedOperand:
    """A constant 2-D operand (a weight) whose row pitch no tensor map can describe, copied ONCE to a 16-byte-aligned
    pitch (nova_b200_operand_prepare).  `tensor` is a [rows, cols] strided view of the copy: pass it to gemm / matmul /
    linear in place of the original and the call streams it with TMA without the per-call re-pitch copy."""

    def __init__(self, t: torch.Tensor):
        _require_cuda(t)
        if t.dim() != 2 or t.stride(1) != 1:
            raise L.NovaB200Error(L.ERR_LAYOUT, "a prepared operand is a 2-D tensor with unit inner stride")
        self._lib = L.load()
        self._h = C.c_void_p()
        rows, cols = t.shape
        with torch.cuda.device(t.device):
            L.check(self._lib.nova_b200_operand_prepare(t.data_ptr(), _dt(t), 1, rows, cols, t.stride(0), 0, _stream(),
                                                        C.byref(self._h)))
            data, ld, bs = C.c_void_p(), C.c_int64(), C.c_int64()
            L.check(self._lib.nova_b200_operand_view(self._h, C.byref(data), C.byref(ld), C.byref(bs)))
            es = t.element_size()

            class _Raw:  # integer view of the library-owned copy, reinterpreted as t's dtype below
                __cuda_array_interface__ = {"shape": (rows, ld.value), "typestr": {2: "<i2", 4: "<i4"}[es],
                                            "data": (data.value, False), "version": 2}
            self._raw = _Raw()
            full = torch.as_tensor(self._raw, device=t.device).view(t.dtype)
        self.tensor = full[:, :cols]

    def free(self):
        if self._h:
            self.tensor = None
            self._lib.nova_b200_operand_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class LnFoldedLinear:
    """nova.layer_norm + nova.linear (+ activation) as ONE contraction over the un-normalised input: the weight is
    folded once (W' = diag(gamma) W, c = column sums of W', d = beta^T W + bias; nova_b200_ln_fold_prepare), each call
    takes the row statistics in one read of x (nova_b200_row_stats) and runs the contraction with
    NOVA_B200_INIT_LN_FOLD.  The normalised tensor is never written.  The counterpart of the LN-apply prologue
    the reference fuses into the FFN-up contraction (NovaKernelConfig.cpp:1898-1917)."""

    def __init__(self, w: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, bias: Optional[torch.Tensor] = None):
        _require_cuda(w, gamma, beta, bias)
        if w.dim() != 2 or w.stride(1) != 1:
            raise L.NovaB200Error(L.ERR_LAYOUT, "weight must be [K, N] with unit inner stride")
        K, N = w.shape
        if gamma.numel() != K or beta.numel() != K or (bias is not None and bias.numel() != N):
            raise L.NovaB200Error(L.ERR_INVALID_ARG, "gamma / beta must hold K elements, bias N")
        for t in (gamma, beta, bias):
            if t is not None and t.dtype != w.dtype:
                raise L.NovaB200Error(L.ERR_UNSUPPORTED, "mixed dtypes are out of scope")
        self.K, self.N, self.dtype = K, N, w.dtype
        with torch.cuda.device(w.device):
            self.wprime = torch.empty((K, N), dtype=w.dtype, device=w.device)
            self.cd = torch.empty((2, N), dtype=torch.float32, device=w.device)
            g, b = gamma.contiguous().reshape(-1), beta.contiguous().reshape(-1)
            bb = bias.contiguous().reshape(-1) if bias is not None else None
            L.check(L.load().nova_b200_ln_fold_prepare(w.data_ptr(), g.data_ptr(), b.data_ptr(),
                                                       bb.data_ptr() if bb is not None else None, self.wprime.data_ptr(),
                                                       self.cd.data_ptr(), K, N, w.stride(0), _dt(w), _stream()))

    def __call__(self, x: torch.Tensor, act: Optional[str] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(x)
        if x.dtype != self.dtype or x.shape[-1] != self.K:
            raise L.NovaB200Error(L.ERR_INVALID_ARG, "input must be [..., K] of the weight's dtype")
        xc = x.contiguous()
        rows = xc.numel() // self.K
        with torch.cuda.device(xc.device):
            stats = torch.empty((rows, 2), dtype=torch.float32, device=xc.device)
            L.check(L.load().nova_b200_row_stats(xc.data_ptr(), stats.data_ptr(), rows, self.K, _dt(xc), _stream()))
            if out is None:
                out = torch.empty((rows, self.N), dtype=self.dtype, device=xc.device)
            g = L.GemmArgs()
            g.struct_size = C.sizeof(L.GemmArgs)
            g.dtype_ab = g.dtype_c = _dt(xc)
            g.batch, g.M, g.N, g.K = 1, rows, self.N, self.K
            g.A, g.B, g.C = xc.data_ptr(), self.wprime.data_ptr(), out.data_ptr()
            g.lda, g.ldb, g.ldc = self.K, self.N, out.stride(-2)
            g.batch_stride_a, g.batch_stride_b, g.batch_stride_c = rows * self.K, 0, rows * out.stride(-2)
            g.init, g.act = L.INIT_LN_FOLD, _ACT[act]
            g.bias, g.residual = self.cd.data_ptr(), stats.data_ptr()
            L.check(L.load().nova_b200_gemm(C.byref(g), _stream()))
        return out.reshape(*x.shape[:-1], self.N)


@_on_device
def column_sum(x: torch.Tensor) -> torch.Tensor:
    """Sum over all leading dims of x[..., C] -> [C], fp32 accumulation (grad_bias of nova.linear_backward)."""
    _require_cuda(x)
    xc = x.contiguous()
    cols = xc.shape[-1]
    out = torch.empty(cols, dtype=xc.dtype, device=xc.device)
    L.check(L.load().nova_b200_column_sum(xc.data_ptr(), out.data_ptr(), xc.numel() // max(cols, 1), cols, _dt(xc),
                                          _stream()))
    return out


def matmul_backward(grad_out: torch.Tensor, a: torch.Tensor, b: torch.Tensor):
    """nova.matmul_backward (NovaOps.td:771-787; lowering NovaToLinalgGeneric.cpp:160-234):
    grad_a = grad_out @ b^T (an NT contraction), grad_b = a^T @ grad_out (TN).  The transposes are views
    consumed through trans_b / trans_a, never copies."""
    return matmul(grad_out, b.transpose(-1, -2)), matmul(a.transpose(-1, -2), grad_out)


def linear_backward(grad_out: torch.Tensor, x: torch.Tensor, w: torch.Tensor):
    """nova.linear_backward (NovaOps.td:1059-1066; lowering NovaToLinalgGeneric.cpp:1824-1995):
    grad_input = grad_out @ W^T with W shared across the batch (:1867-1906), grad_weight = flatX^T @ flatGo over
    the flattened batch*M rows (:1913-1963), grad_bias = column sum of flatGo (:1970-1985)."""
    k, n = w.shape
    grad_input = matmul(grad_out, w.transpose(0, 1))
    xf = x.reshape(-1, k)
    gf = grad_out.reshape(-1, n)
    grad_weight = matmul(xf.transpose(0, 1), gf)
    return grad_input, grad_weight, column_sum(gf)


@_on_device
def _unary(x: torch.Tensor, act: int) -> torch.Tensor:
    _require_cuda(x)
    xc = x.contiguous()
    y = torch.empty_like(xc)
    L.check(L.load().nova_b200_activation(xc.data_ptr(), y.data_ptr(), xc.numel(), _dt(xc), act, _stream()))
    return y


def gelu(x: torch.Tensor) -> torch.Tensor:
    """nova.gelu, tanh form (NovaGeluForwardPattern, NovaToLinalgGeneric.cpp:1277-1337)."""
    return _unary(x, L.ACT_GELU_TANH)


@_on_device
def gelu_backward(grad_out: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """nova.gelu_backward: grad_out * d/dx gelu_tanh(x) (NovaGeluBackwardPattern, NovaToLinalgGeneric.cpp:1339-1420)."""
    _require_cuda(grad_out, x)
    if grad_out.shape != x.shape or grad_out.dtype != x.dtype:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "gelu_backward: grad_out and input must share shape and dtype")
    gc, xc = grad_out.contiguous(), x.contiguous()
    y = torch.empty_like(xc)
    L.check(L.load().nova_b200_gelu_backward(gc.data_ptr(), xc.data_ptr(), y.data_ptr(), xc.numel(), _dt(xc), _stream()))
    return y


def relu(x: torch.Tensor) -> torch.Tensor:
    """nova.relu -> max(x, 0) (NovaToLinalg.cpp:1053-1084)."""
    return _unary(x, L.ACT_RELU)


@_on_device
def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """nova.add where b either has a's shape or broadcasts along rows ([N] or [1,N] against [...,N]),
    the forms next to a contraction (ltest/test_cpu.mlir: 8x10 + 1x10).  Other broadcasts are out of scope."""
    _require_cuda(a, b)
    if a.dtype != b.dtype:
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "add: mixed dtypes are out of scope")
    ac, bc = a.contiguous(), b.contiguous()
    cols = ac.shape[-1]
    full = bc.numel() == ac.numel() and bc.shape[-1] == cols
    if not full and not (bc.numel() == cols and bc.shape[-1] == cols):
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "add: only same-shape or row-broadcast operands are supported")
    out = torch.empty_like(ac)
    L.check(L.load().nova_b200_add_rowbcast(ac.data_ptr(), bc.data_ptr(), out.data_ptr(), ac.numel() // cols, cols,
                                            int(full), _dt(ac), _stream()))
    return out


@_on_device
def softmax(x: torch.Tensor, dimension: int = -1) -> torch.Tensor:
    """nova.softmax (NovaSoftmaxForwardPattern, NovaToLinalgGeneric.cpp:1427-1534) along `dimension`
    (default -1, negative wraps, :1439-1443).  Non-last dimensions are moved last and back."""
    _require_cuda(x)
    rank = x.dim()
    dim = dimension
    if dim > rank:
        dim = rank - 1
    if dim < 0:
        dim += rank
    xm = x.movedim(dim, -1).contiguous()
    y = torch.empty_like(xm)
    D = xm.shape[-1]
    L.check(L.load().nova_b200_softmax(xm.data_ptr(), y.data_ptr(), xm.numel() // max(D, 1), D, _dt(xm), _stream()))
    return y.movedim(-1, dim)


@_on_device
def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor):
    """nova.layer_norm over the last dim (NovaLayerNormPattern, NovaToLinalgGeneric.cpp:1997-2126).
    Returns (y, mean_sum, rstd): mean_sum is the RAW row sum, as in the reference (:2121-2123)."""
    _require_cuda(x, gamma, beta)
    xc, g, b = x.contiguous(), gamma.contiguous(), beta.contiguous()
    D = xc.shape[-1]
    if g.numel() != D or b.numel() != D or g.dtype != xc.dtype or b.dtype != xc.dtype:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "layer_norm: gamma/beta must be [D] of x's dtype")
    y = torch.empty_like(xc)
    mean_sum = torch.empty(xc.shape[:-1], dtype=xc.dtype, device=xc.device)
    rstd = torch.empty(xc.shape[:-1], dtype=xc.dtype, device=xc.device)
    L.check(L.load().nova_b200_layer_norm(xc.data_ptr(), g.data_ptr(), b.data_ptr(), y.data_ptr(), mean_sum.data_ptr(),
                                          rstd.data_ptr(), xc.numel() // max(D, 1), D, _dt(xc), _stream()))
    return y, mean_sum, rstd


@_on_device
def layer_norm_backward(grad_y: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor, mean_sum: torch.Tensor,
                        rstd: torch.Tensor):
    """nova.layer_norm_backward (NovaLayerNormBackwardPattern, NovaToLinalgGeneric.cpp:2128-2376): returns
    (dx, dgamma, dbeta) from grad_y, x, gamma and the (mean_sum, rstd) the forward saved."""
    _require_cuda(grad_y, x, gamma, mean_sum, rstd)
    gc, xc, g = grad_y.contiguous(), x.contiguous(), gamma.contiguous()
    ms, rs = mean_sum.contiguous(), rstd.contiguous()
    D = xc.shape[-1]
    rows = xc.numel() // max(D, 1)
    if gc.shape != xc.shape or g.numel() != D or ms.numel() != rows or rs.numel() != rows:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "layer_norm_backward: operand shapes do not agree")
    if any(t.dtype != xc.dtype for t in (gc, g, ms, rs)):
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "layer_norm_backward: mixed dtypes are out of scope")
    dx = torch.empty_like(xc)
    dgamma = torch.empty_like(g)
    dbeta = torch.empty_like(g)
    L.check(L.load().nova_b200_layer_norm_backward(gc.data_ptr(), xc.data_ptr(), g.data_ptr(), ms.data_ptr(), rs.data_ptr(),
                                                   dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), rows, D, _dt(xc),
                                                   _stream()))
    return dx, dgamma, dbeta


@_on_device
def gather(inp: torch.Tensor, indices: torch.Tensor, axis: int = 0, *, return_bad_count: bool = False):
    """nova.gather (NovaGatherOpLowering, NovaToLinalgGeneric.cpp:2372-2472; shapes NovaOps.cpp:1898-1946):
    out[pre..., idx..., post...] = inp[pre..., indices[...], post...].  Leading index dims equal to inp's
    leading dims act as batch dims.  i16 indices are zero-extended.  Bit-exact."""
    _require_cuda(inp, indices)
    if indices.dtype not in _IDX:
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "gather: index dtype must be int16, int32 or int64")
    x = inp.contiguous()
    idx = indices.contiguous()
    if axis < 0:
        axis += x.dim()
    batch_dims = 0
    for i in range(min(axis, idx.dim())):
        if x.shape[i] != idx.shape[i]:
            break
        batch_dims += 1
    batched = axis > 0 and batch_dims == axis
    if axis > 0 and not batched and batch_dims != 0:
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "gather: partially batched indices are out of scope")
    pre = 1
    for s in x.shape[:axis]:
        pre *= s
    post = 1
    for s in x.shape[axis + 1:]:
        post *= s
    idx_shape = tuple(idx.shape[batch_dims:]) if batched else tuple(idx.shape)
    n_idx = 1
    for s in idx_shape:
        n_idx *= s
    out = torch.empty(tuple(x.shape[:axis]) + idx_shape + tuple(x.shape[axis + 1:]), dtype=x.dtype, device=x.device)
    bad = torch.zeros(1, dtype=torch.int64, device=x.device)
    L.check(L.load().nova_b200_gather(x.data_ptr(), idx.data_ptr(), out.data_ptr(), pre, x.shape[axis], post, n_idx,
                                      _IDX[idx.dtype], int(batched), x.element_size(), bad.data_ptr(), _stream()))
    return (out, int(bad.item())) if return_bad_count else out


@_on_device
def sce(logits: torch.Tensor, targets: torch.Tensor, *, return_bad_count: bool = False):
    """nova.sce (NovaSceForwardLowering, NovaToLinalgGeneric.cpp:801-1010): sparse softmax cross-entropy over the
    last dim.  Returns (softmax, loss[1]) as the op does (NovaOps.cpp:1648-1677)."""
    _require_cuda(logits, targets)
    if targets.dtype not in _IDX:
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "sce: target dtype must be int16, int32 or int64")
    x, t = logits.contiguous(), targets.contiguous()
    Cn = x.shape[-1] if x.dim() else 1
    rows = x.numel() // max(Cn, 1)
    if t.numel() != rows:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "sce: one target per row of logits")
    sm = torch.empty_like(x)
    loss = torch.empty(1, dtype=x.dtype, device=x.device)
    bad = torch.zeros(1, dtype=torch.int64, device=x.device)
    L.check(L.load().nova_b200_sce(x.data_ptr(), t.data_ptr(), sm.data_ptr(), loss.data_ptr(), rows, Cn, _dt(x),
                                   _IDX[t.dtype], bad.data_ptr(), _stream()))
    return (sm, loss, int(bad.item())) if return_bad_count else (sm, loss)


@_on_device
def sce_backward(softmax_: torch.Tensor, targets: torch.Tensor, dim: int = -1, scale: float = 1.0) -> torch.Tensor:
    """nova.sce_backward (NovaSceBackwardLowering, NovaToLinalgGeneric.cpp:1012-1137): (softmax - one_hot) / rows;
    `scale` is a following multiplication by one scalar (the loss gradient) done in the same pass."""
    _require_cuda(softmax_, targets)
    if dim not in (-1, softmax_.dim() - 1):
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "sce_backward: the class dimension must be the last one")
    if targets.dtype not in _IDX:
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "sce_backward: target dtype must be int16, int32 or int64")
    p, t = softmax_.contiguous(), targets.contiguous()
    Cn = p.shape[-1]
    rows = p.numel() // max(Cn, 1)
    if t.numel() != rows:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "sce_backward: one target per row")
    g = torch.empty_like(p)
    L.check(L.load().nova_b200_sce_backward_scaled(p.data_ptr(), t.data_ptr(), g.data_ptr(), rows, Cn, _dt(p), _IDX[t.dtype],
                                                   float(scale), _stream()))
    return g


@_on_device
def scatter_add(inp: torch.Tensor, indices: torch.Tensor, src: torch.Tensor, axis: int = 0, *,
                return_bad_count: bool = False):
    """nova.scatter_add (NovaScatterAddOpLowering, NovaToLinalg.cpp:1086-1294; verify NovaOps.cpp:1990-2026): a copy
    of inp with src added at `indices` along `axis`; shapes match except at axis, one index per src slice."""
    _require_cuda(inp, indices, src)
    if indices.dtype not in _IDX:
        raise L.NovaB200Error(L.ERR_UNSUPPORTED, "scatter_add: index dtype must be int16, int32 or int64")
    if inp.dim() != src.dim() or inp.dtype != src.dtype:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "scatter_add: input and src must share rank and dtype")
    if axis < 0:
        axis += inp.dim()
    if not 0 <= axis < inp.dim():
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "scatter_add: axis out of bounds")
    for i in range(inp.dim()):
        if i != axis and inp.shape[i] != src.shape[i]:
            raise L.NovaB200Error(L.ERR_INVALID_ARG, "scatter_add: input and src shapes must match except at axis")
    if indices.numel() != src.shape[axis]:
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "scatter_add: src dimension at axis must match index size")
    out = inp.contiguous().clone()
    s, idx = src.contiguous(), indices.contiguous()
    pre = 1
    for d in out.shape[:axis]:
        pre *= d
    post = 1
    for d in out.shape[axis + 1:]:
        post *= d
    bad = torch.zeros(1, dtype=torch.int64, device=out.device)
    L.check(L.load().nova_b200_scatter_add(out.data_ptr(), idx.data_ptr(), s.data_ptr(), pre, out.shape[axis], post,
                                           s.shape[axis], _IDX[idx.dtype], _dt(out), bad.data_ptr(), _stream()))
    return (out, int(bad.item())) if return_bad_count else out


def reshape(x: torch.Tensor, shape) -> torch.Tensor:
    """nova.reshape -> tensor.reshape (ReshapeOpConverter, NovaToLinalg.cpp:2409-2434): a row-major
    reinterpretation with equal element count (verify: NovaOps.cpp:1885-1895); no data movement."""
    n = 1
    for s in shape:
        n *= s
    if n != x.numel():
        raise L.NovaB200Error(L.ERR_INVALID_ARG, "reshape: element counts differ")
    return x.contiguous().view(*shape)


def transpose(x: torch.Tensor, axes1: int = -1, axes2: int = -2) -> torch.Tensor:
    """nova.transpose (NovaOps.td:832-843): swaps two dims; returned as a VIEW so that a following
    matmul consumes it through trans_a / trans_b (the matmul_transpose_a fusion, NovaToLinalg.cpp:824-872)."""
    return x.transpose(axes1, axes2)


def device_status() -> int:
    """Reads and clears the device status word (0 == every bounded in-kernel wait completed)."""
    code = C.c_uint32(0)
    st = L.load().nova_b200_device_status(C.byref(code))
    if st not in (L.OK, L.ERR_DEVICE_TIMEOUT):
        L.check(st)
    return int(code.value)
