"""Host-side checks that need no GPU: the C-ABI library loads, exports every function the header
declares, validates arguments, and selects loaders / tiles as documented.  No compute calls here."""
import ctypes as C
import os
import re

import pytest

from nova_compiler_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "nova_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b((?:_mlir_ciface_)?nova_b200_\w+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported_and_bound(lib):
    declared = _declared_functions()
    assert len(declared) >= 16
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/nova_b200.h but not exported"
        assert name in L.PROTOTYPES, f"{name} has no ctypes prototype"
    assert set(L.PROTOTYPES) == set(declared)
    assert lib.nova_b200_abi_version() == 1


def test_struct_layout_matches_the_header(lib):
    assert C.sizeof(L.GemmArgs) == 168
    assert C.sizeof(L.GemmPlanInfo) == 48
    assert C.sizeof(L.MemRef2D) == 56 and C.sizeof(L.MemRef3D) == 72 and C.sizeof(L.MemRef1D) == 40


def _args(M, N, K, dt=L.BF16, batch=1, lda=None, ldb=None, ldc=None, a=0x1000, b=0x2000, c=0x3000, **kw):
    g = L.GemmArgs()
    g.struct_size = C.sizeof(L.GemmArgs)
    g.dtype_ab = g.dtype_c = dt
    g.batch, g.M, g.N, g.K = batch, M, N, K
    g.A, g.B, g.C = a, b, c
    g.lda = lda if lda is not None else K
    g.ldb = ldb if ldb is not None else N
    g.ldc = ldc if ldc is not None else N
    g.batch_stride_a, g.batch_stride_b, g.batch_stride_c = M * g.lda, K * g.ldb, M * g.ldc
    for k, v in kw.items():
        setattr(g, k, v)
    return g


def _plan(lib, g):
    info = L.GemmPlanInfo()
    st = lib.nova_b200_gemm_plan(C.byref(g), C.byref(info))
    return st, info


def test_plan_aligned_operands_use_tma(lib):
    st, info = _plan(lib, _args(8192, 11008, 4096))
    assert st == L.OK
    assert (info.loader_a, info.loader_b, info.store_c) == (0, 0, 0)
    # a wave of 256 x 256 tiles exists: CTA pairs, three ring stages of two 64-element K boxes each per CTA
    assert (info.block_m, info.block_n, info.block_k, info.stages) == (256, 256, 64, 3)
    assert info.tiles == 32 * 43 and info.grid == 148 and info.scratch_bytes == 0
    # a single 2048^3 problem is one wave of 128 x 256 tiles (128 of them): cheaper than one under-filled wave of
    # pairs or two waves of 128 x 128 tiles
    st, info = _plan(lib, _args(2048, 2048, 2048))
    assert st == L.OK and (info.block_m, info.block_n, info.stages, info.tiles, info.grid) == (128, 256, 4, 128, 128)
    # 1536^3: 144 tiles of 128 x 128 fill one wave
    st, info = _plan(lib, _args(1536, 1536, 1536))
    assert st == L.OK and (info.block_m, info.block_n, info.stages, info.tiles, info.grid) == (128, 128, 6, 144, 144)
    # 1024^3: even 64 tiles of 128 x 128 leave most SMs idle; 128 tiles of 128 x 64 (eight 24 KB stages)
    st, info = _plan(lib, _args(1024, 1024, 1024))
    assert st == L.OK and (info.block_m, info.block_n, info.stages, info.tiles, info.grid) == (128, 64, 8, 128, 128)
    # a short contraction (K <= 256) is epilogue-bound: single-CTA 128 x 256 tiles, three 48 KB stages and a
    # second set of epilogue warps
    st, info = _plan(lib, _args(2048, 2048, 128, dt=L.F16, batch=256))
    assert st == L.OK and (info.block_m, info.block_n, info.stages, info.tiles) == (128, 256, 3, 256 * 16 * 8)


def test_plan_ragged_pitches_select_the_non_tma_loader(lib):
    # 1000 x 1000 x 999 bf16: A pitch 1998 B (not 16-byte aligned): re-pitched into scratch (1000 rows of 1000
    # elements), then TMA; B, C pitch 2000 B -> TMA / vector stores
    st, info = _plan(lib, _args(1000, 1000, 999))
    assert st == L.OK and (info.loader_a, info.loader_b, info.store_c) == (2, 0, 0)
    assert info.scratch_bytes == (1000 * 1000 * 2 + 255) // 256 * 256
    # option "repitch" = 0: read in place by the loader warps, no scratch
    L.set_option("repitch", 0)
    try:
        st, info = _plan(lib, _args(1000, 1000, 999))
    finally:
        L.set_option("repitch", 1)
    assert st == L.OK and (info.loader_a, info.loader_b, info.scratch_bytes) == (1, 0, 0)
    # 4095 x 11007 x 4097: every pitch is odd in bytes/16; both operands re-pitched, C written with element stores
    st, info = _plan(lib, _args(4095, 11007, 4097))
    assert st == L.OK and (info.loader_a, info.loader_b, info.store_c) == (2, 2, 1)
    assert (info.block_m, info.block_n) == (256, 256)
    # an aligned pitch with a misaligned base also needs the loader
    st, info = _plan(lib, _args(256, 256, 256, a=0x1002))
    assert st == L.OK and info.loader_a == 2 and info.loader_b == 0


def test_plan_f32_modes(lib):
    st, info = _plan(lib, _args(512, 512, 512, dt=L.F32))
    # 16 tiles of 128 x 128 would use 16 SMs: 128 x 64 tiles, four stages of hi and lo copies of both operands; even
    # those 32 tiles leave most SMs idle, so K runs as four ranges of 128 (32 x 4 work units) summed by a second kernel
    assert st == L.OK and info.block_n == 64 and info.block_k == 32 and info.stages == 4 and info.tiles == 4 * 32
    st2, big = _plan(lib, _args(4096, 4096, 512, dt=L.F32))
    assert st2 == L.OK and big.block_n == 128 and big.stages == 3 and big.tiles == 32 * 32
    # hi and lo copies of A and B, then four fp32 partial matrices
    assert info.scratch_bytes == 2 * 4 * (512 * 512 + 512 * 512) + 4 * 512 * 512 * 4
    st, info = _plan(lib, _args(512, 512, 512, dt=L.F32, f32_mode=L.TF32X1))
    assert st == L.OK and info.scratch_bytes == 4 * 512 * 512 * 4   # no hi/lo copies; the K ranges' partials only
    # unaligned f32 operands are re-laid out by the split, never read through the loader
    st, info = _plan(lib, _args(100, 200, 301, dt=L.F32))
    assert st == L.OK and (info.loader_a, info.loader_b) == (0, 0)
    assert info.scratch_bytes == 2 * 4 * (100 * 304 + 301 * 200)


def test_plan_small_problems_use_narrow_tiles(lib):
    st, info = _plan(lib, _args(8, 10, 16, dt=L.F16))
    assert st == L.OK and info.block_n == 64 and info.tiles == 1 and info.grid == 1
    st, info = _plan(lib, _args(1024, 1024, 1024, dt=L.F16, batch=32))
    assert st == L.OK and (info.block_m, info.block_n) == (256, 256) and info.tiles == 32 * 4 * 4


def test_argument_errors_are_reported_not_thrown(lib):
    g = _args(16, 16, 16)
    g.struct_size = 12
    assert _plan(lib, g)[0] == L.ERR_INVALID_ARG
    assert b"struct_size" in lib.nova_b200_last_error_string()
    assert _plan(lib, _args(16, 16, 16, dt=L.I32))[0] == L.ERR_UNSUPPORTED
    assert _plan(lib, _args(-1, 16, 16))[0] == L.ERR_INVALID_ARG
    assert _plan(lib, _args(16, 16, 16, lda=8))[0] == L.ERR_LAYOUT
    assert _plan(lib, _args(16, 16, 16, ldc=8))[0] == L.ERR_LAYOUT
    assert _plan(lib, _args(16, 16, 16, act=7))[0] == L.ERR_INVALID_ARG
    assert _plan(lib, _args(16, 16, 16, init=L.INIT_BIAS_ROW))[0] == L.ERR_INVALID_ARG  # bias pointer missing
    assert _plan(lib, _args(16, 16, 16, a=0))[0] == L.ERR_INVALID_ARG
    assert _plan(lib, _args(1 << 31, 16, 16))[0] == L.ERR_TOO_LARGE
    g = _args(16, 16, 16, batch=4)
    g.batch_stride_c = 8
    assert _plan(lib, g)[0] == L.ERR_LAYOUT
    assert lib.nova_b200_gemm_plan(None, None) == L.ERR_INVALID_ARG


def test_empty_problems_are_ok(lib):
    for m, n, k in ((0, 16, 16), (16, 0, 16), (16, 16, 0)):
        assert _plan(lib, _args(m, n, k))[0] == L.OK
    assert _plan(lib, _args(16, 16, 16, batch=0))[0] == L.OK


def test_compute_entry_points_fail_loudly_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    g = _args(16, 16, 16)
    assert lib.nova_b200_gemm(C.byref(g), None) == L.ERR_NO_DEVICE
    assert b"no CPU fallback" in lib.nova_b200_last_error_string()
    assert lib.nova_b200_init(0) == L.ERR_NO_DEVICE
    assert lib.nova_b200_softmax(0x1000, 0x2000, 4, 4, L.F32, None) == L.ERR_NO_DEVICE
    # argument errors still take precedence and are reported on a machine without a GPU
    assert lib.nova_b200_gather(0x1000, 0x2000, 0x3000, 1, 4, 4, 4, L.F32, 0, 4, None, None) == L.ERR_UNSUPPORTED
    with pytest.raises(L.NovaB200Error):
        from nova_compiler_b200 import ops
        ops.gemm(torch.zeros(1, 4, 4), torch.zeros(1, 4, 4))


def test_shutdown_without_init_is_safe(lib):
    assert lib.nova_b200_shutdown() == L.OK
