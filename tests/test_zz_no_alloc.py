"""nova_b200_gemm_f32_static — the f32 contraction for callers that cannot call cudaMalloc (a graph running
inside a memory-planned region, a plug-in whose host forbids allocation on its streams, a loop that must
not take the allocator's locks).  It keeps its scratch in a fixed array inside the library image.

Checked here, through the C ABI: two calls in a row (different shapes, so the second one finds the first
one's leftovers in the shared array) give what the regular entry point nova_b200_gemm gives, within the
f32 tolerance of the other GPU tests (relative Frobenius <= 1e-5; the kernels are the same, so the results
are in fact identical); requests beyond the 16 MiB limit or outside f32/3xTF32 are refused with a clear
error.  A fresh process makes this entry point its very first library call, checks the result against the CPU
oracle and checks that the free device memory does not move across a further call.  This file sorts last on
purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _args(L, torch, a, b, c, bias=None, act=0):
    g = L.GemmArgs()
    g.struct_size = C.sizeof(L.GemmArgs)
    g.dtype_ab = g.dtype_c = L.F32
    g.f32_mode = L.TF32X3
    g.batch, g.M, g.K = a.shape
    g.N = b.shape[2]
    g.A, g.B, g.C = a.data_ptr(), b.data_ptr(), c.data_ptr()
    g.lda, g.ldb, g.ldc = a.stride(1), b.stride(1), c.stride(1)
    g.batch_stride_a, g.batch_stride_b, g.batch_stride_c = a.stride(0), b.stride(0), c.stride(0)
    g.act = act
    if bias is not None:
        g.init, g.bias = L.INIT_BIAS_ROW, bias.data_ptr()
    return g


def test_static_scratch_entry_point_matches_regular_entry_point(cuda, oracle, lib):
    torch = cuda
    from nova_compiler_b200 import _lib as L
    gen = torch.Generator(device="cuda")
    gen.manual_seed(99)
    # second call is smaller and ragged: it must not see stale hi/lo values or padding from the first
    cases = [((2, 384, 448), (2, 448, 320), True), ((1, 100, 301), (1, 301, 77), False)]
    for (ashape, bshape, with_bias) in cases:
        a = torch.rand(ashape, device="cuda", generator=gen) * 2 - 1
        b = torch.rand(bshape, device="cuda", generator=gen) * 2 - 1
        bias = torch.randn(bshape[2], device="cuda", generator=gen) if with_bias else None
        want = torch.empty(ashape[0], ashape[1], bshape[2], device="cuda")
        got = torch.full_like(want, float("nan"))
        act = L.ACT_GELU_TANH if with_bias else L.ACT_NONE
        L.check(lib.nova_b200_gemm(C.byref(_args(L, torch, a, b, want, bias, act)), None))
        code = C.c_uint32(123)
        L.check(lib.nova_b200_gemm_f32_static(C.byref(_args(L, torch, a, b, got, bias, act)), None, C.byref(code)))
        torch.cuda.synchronize()
        assert code.value == 0
        err = oracle.rel_fro(got.cpu().numpy(), want.cpu().numpy())
        assert err <= 1e-5, f"static-scratch vs regular entry point: rel-Frobenius {err:.3e}"
        ref = oracle.gemm(a.cpu().numpy(), b.cpu().numpy(), bias=None if bias is None else bias.cpu().numpy(),
                          act="gelu_tanh" if with_bias else "none")
        assert oracle.rel_fro(got.cpu().numpy(), ref) <= 1e-5


def test_static_scratch_entry_point_refuses_what_it_cannot_hold(cuda, lib):
    torch = cuda
    from nova_compiler_b200 import _lib as L
    a = torch.zeros(1, 8, 8, device="cuda")
    g = _args(L, torch, a, a, a)
    g.M = g.N = g.K = 2048  # needs 64 MiB of split buffers; validated before anything is launched
    g.lda = g.ldb = g.ldc = 2048
    assert lib.nova_b200_gemm_f32_static(C.byref(g), None, None) == L.ERR_TOO_LARGE
    assert b"static scratch holds" in lib.nova_b200_last_error_string()
    h = torch.zeros(1, 8, 8, device="cuda", dtype=torch.bfloat16)
    g = _args(L, torch, h, h, h)
    g.dtype_ab = g.dtype_c = L.BF16
    assert lib.nova_b200_gemm_f32_static(C.byref(g), None, None) == L.ERR_UNSUPPORTED
    g = _args(L, torch, a, a, a)
    g.f32_mode = L.TF32X1
    assert lib.nova_b200_gemm_f32_static(C.byref(g), None, None) == L.ERR_UNSUPPORTED


_FIRST_CALL_SCRIPT = r"""
import ctypes as C, sys
import numpy as np
import torch
sys.path.insert(0, {root!r})
from nova_compiler_b200 import _lib as L
from oracle import oracle as O
lib = L.load()
torch.cuda.set_device(0)
rng = np.random.default_rng(5)
ah = rng.uniform(-1, 1, (1, 200, 328)).astype(np.float32)
bh = rng.uniform(-1, 1, (1, 328, 136)).astype(np.float32)
a, b = torch.from_numpy(ah).cuda(), torch.from_numpy(bh).cuda()
c = torch.full((1, 200, 136), float("nan"), device="cuda")
g = L.GemmArgs()
g.struct_size = C.sizeof(L.GemmArgs)
g.dtype_ab = g.dtype_c = L.F32
g.batch, g.M, g.K, g.N = 1, 200, 328, 136
g.A, g.B, g.C = a.data_ptr(), b.data_ptr(), c.data_ptr()
g.lda, g.ldb, g.ldc = 328, 136, 136
g.batch_stride_a, g.batch_stride_b, g.batch_stride_c = 200 * 328, 328 * 136, 200 * 136
# the FIRST call into the library in this process: no nova_b200_init, no nova_b200_gemm before it
code = C.c_uint32(9)
L.check(lib.nova_b200_gemm_f32_static(C.byref(g), None, C.byref(code)))
assert code.value == 0
assert O.rel_fro(c.cpu().numpy(), O.gemm(ah, bh)) <= 1e-5
torch.cuda.synchronize()
free0, _ = torch.cuda.mem_get_info()
for _ in range(3):
    L.check(lib.nova_b200_gemm_f32_static(C.byref(g), None, None))  # enqueue only
torch.cuda.synchronize()
free1, _ = torch.cuda.mem_get_info()
assert free1 == free0, (free0, free1)   # nothing was allocated (or freed) by the calls
# an enqueue-only caller reads the wait code through nova_b200_device_status (this is the library's first
# allocation in this process: the regular per-device context)
st = C.c_uint32(7)
L.check(lib.nova_b200_device_status(C.byref(st)))
assert st.value == 0
assert O.rel_fro(c.cpu().numpy(), O.gemm(ah, bh)) <= 1e-5
print("first-call ok")
"""


def test_static_scratch_entry_point_as_first_call_allocates_nothing(cuda):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", _FIRST_CALL_SCRIPT.format(root=root)], capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "first-call ok" in res.stdout, res.stdout + res.stderr
