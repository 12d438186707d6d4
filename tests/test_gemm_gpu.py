"""Parity of the CUDA contraction against the CPU oracle, through the C ABI (ops.gemm -> nova_b200_gemm).

Tolerances (relative Frobenius error against the oracle's fp32-accumulate mode):
    f16 / bf16 inputs, fp32 accumulation : <= 1e-3
    f32 via the 3xTF32 split             : <= 1e-5
    f32 single-pass TF32 (what the reference's own GPU path computes): <= 2e-3, informational
"""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_cases.npz")
TOL = {"f32": 1e-5, "f16": 1e-3, "bf16": 1e-3}


def _tdt(torch, dt):
    return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dt]


def to_dev(torch, arr, dt):
    """numpy storage array (float32, or uint16 bits) -> CUDA tensor of dtype dt."""
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if dt != "f32":
        t = t.view(torch.int16).view(_tdt(torch, dt))
    return t.cuda()


def to_host(torch, t, dt):
    t = t.contiguous().cpu()
    if dt != "f32":
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def rand_bits(oracle, rng, shape, dt, dist="uniform", scale=1.0):
    x = rng.uniform(-1, 1, shape) if dist == "uniform" else rng.normal(size=shape)
    return oracle.to_bits((x * scale).astype(np.float32), dt)


def run_gpu(torch, a, b, dt, out_dt=None, **kw):
    from nova_compiler_b200 import ops
    out_dt = out_dt or dt
    ta = to_dev(torch, a, dt)
    tb = to_dev(torch, b, dt)
    a3 = ta if ta.dim() == 3 else ta[None]
    b3 = tb if tb.dim() == 3 else tb[None]
    if kw.pop("trans_a", False):
        a3 = a3.transpose(1, 2)
    if kw.pop("trans_b", False):
        b3 = b3.transpose(1, 2)
    if "bias" in kw and kw["bias"] is not None:
        kw["bias"] = to_dev(torch, kw["bias"], out_dt)
    if "residual" in kw and kw["residual"] is not None:
        kw["residual"] = to_dev(torch, kw["residual"], out_dt)
    c = ops.gemm(a3, b3, out_dtype=_tdt(torch, out_dt), **kw)
    torch.cuda.synchronize()
    out = to_host(torch, c, out_dt)
    return out if ta.dim() == 3 else out[0]


def check(oracle, got, want, dt, tol=None):
    err = oracle.rel_fro(oracle.from_bits(got, dt), oracle.from_bits(want, dt))
    assert err <= (tol or TOL[dt]), f"rel-Frobenius {err:.3e}"
    return err


# ---------------------------------------------------------------- golden fixtures

def test_golden_vectors(cuda, oracle):
    z = np.load(GOLD)
    check(oracle, run_gpu(cuda, z["c1_f32.a"], z["c1_f32.b"], "f32"), z["c1_f32.c"], "f32")
    check(oracle, run_gpu(cuda, z["c2_f16_bmm.a"], z["c2_f16_bmm.b"], "f16"), z["c2_f16_bmm.c"], "f16")
    check(oracle, run_gpu(cuda, z["c3_bf16_linear_gelu.a"], z["c3_bf16_linear_gelu.b"], "bf16",
                          bias=z["c3_bf16_linear_gelu.bias"], act="gelu"), z["c3_bf16_linear_gelu.c"], "bf16")
    check(oracle, run_gpu(cuda, z["c4_f16_scores.a"], z["c4_f16_scores.b"], "f16"), z["c4_f16_scores.c"], "f16")
    check(oracle, run_gpu(cuda, z["c5_bf16_ragged.a"], z["c5_bf16_ragged.b"], "bf16"), z["c5_bf16_ragged.c"], "bf16")
    check(oracle, run_gpu(cuda, z["test_cpu_mlir.a"], z["test_cpu_mlir.b"], "f32", bias=z["test_cpu_mlir.bias"],
                          act="relu"), z["test_cpu_mlir.c"], "f32")


def test_reference_known_answers(cuda, oracle):
    """test/wrapper.c:93-99 (ones x ones + 0.5, at 1024^3 here and at the reference's 4096^3 in
    test_full_size_wrapper_c) and robust_driver.cpp:71-80,100-108.  All exact in fp32."""
    n = 1024
    ones = np.ones((n, n), np.float32)
    c = run_gpu(cuda, ones, ones, "f32", residual=np.full((1, n, n), 0.5, np.float32))
    assert np.all(c == np.float32(n + 0.5))
    three = np.full((16, 16), 3.0, np.float32)
    one = np.ones((16, 16), np.float32)
    assert np.all(run_gpu(cuda, three, one, "f32") == np.float32(48.0))
    x1 = np.ones((64, 64), np.float32)
    xh = np.full((64, 64), 0.5, np.float32)
    assert np.all(run_gpu(cuda, x1, xh, "f32") == np.float32(32.0))
    g = run_gpu(cuda, x1, xh, "f32", act="gelu")
    assert np.allclose(g, 32.0, rtol=1e-6)


# ---------------------------------------------------------------- shape / dtype / layout sweep

SHAPES_FROM_REFERENCE_TESTS = [
    (1, 8, 32, 16),       # ltest/6otherops.mlir 2-D 8x16 . 16x32
    (4, 8, 32, 16),       # ... batch 4
    (1, 100, 200, 300),   # test/pipeline-tests/01_matmul_non_aligned.mlir
    (1, 256, 512, 128),   # 02 aligned
    (4, 64, 64, 256),     # 03 batch -> gpu.block<z>
    (1, 128, 128, 128),   # exact tile
]


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", SHAPES_FROM_REFERENCE_TESTS)
def test_reference_test_shapes(cuda, oracle, dt, shape):
    B, M, N, K = shape
    rng = np.random.default_rng(hash((dt,) + shape) % (1 << 31))
    a = rand_bits(oracle, rng, (B, M, K), dt)
    b = rand_bits(oracle, rng, (B, K, N), dt)
    check(oracle, run_gpu(cuda, a, b, dt), oracle.gemm(a, b, dtype_in=dt), dt)


EDGES = [1, 7, 63, 64, 65, 127, 128, 129, 255, 256, 257]


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_tile_edge_extents(cuda, oracle, dt):
    rng = np.random.default_rng(42)
    combos = [(m, n, k) for m in (1, 127, 129) for n in (1, 65, 257) for k in (1, 63, 129)]
    combos += [(e, e, e) for e in EDGES] + [(33, 300, 40), (300, 33, 1000)]
    for (m, n, k) in combos:
        a = rand_bits(oracle, rng, (m, k), dt)
        b = rand_bits(oracle, rng, (k, n), dt)
        check(oracle, run_gpu(cuda, a, b, dt), oracle.gemm(a, b, dtype_in=dt), dt)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
def test_operand_majors(cuda, oracle, dt, trans_a, trans_b):
    rng = np.random.default_rng(5)
    B, M, N, K = 2, 200, 328, 264
    a = rand_bits(oracle, rng, (B, K, M) if trans_a else (B, M, K), dt)
    b = rand_bits(oracle, rng, (B, N, K) if trans_b else (B, K, N), dt)
    want = oracle.gemm(a, b, dtype_in=dt, trans_a=trans_a, trans_b=trans_b)
    check(oracle, run_gpu(cuda, a, b, dt, trans_a=trans_a, trans_b=trans_b), want, dt)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("act", [None, "relu", "gelu"])
@pytest.mark.parametrize("init", ["zero", "bias", "residual", "bias+residual"])
def test_epilogues(cuda, oracle, dt, act, init):
    rng = np.random.default_rng(17)
    B, M, N, K = 2, 130, 264, 96
    a = rand_bits(oracle, rng, (B, M, K), dt, "normal")
    b = rand_bits(oracle, rng, (B, K, N), dt, "normal", 0.1)
    bias = rand_bits(oracle, rng, (N,), dt, "normal") if "bias" in init else None
    res = rand_bits(oracle, rng, (B, M, N), dt, "normal") if "residual" in init else None
    want = oracle.gemm(a, b, dtype_in=dt, bias=bias, residual=res, act={"gelu": "gelu_tanh"}.get(act, act or "none"))
    check(oracle, run_gpu(cuda, a, b, dt, bias=bias, residual=res, act=act), want, dt)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gelu_backward_epilogue_and_standalone_op(cuda, oracle, dt, with_bias):
    """C = (bias + A @ B) * gelu_tanh'(Z): the contraction followed by nova.gelu_backward, in one launch; and the
    standalone op.  Z spans the region where the derivative dips below zero and where it saturates."""
    torch = cuda
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(29)
    B, M, N, K = 2, 150, 200, 72
    a = rand_bits(oracle, rng, (B, M, K), dt, "normal")
    b = rand_bits(oracle, rng, (B, K, N), dt, "normal", 0.1)
    z = rand_bits(oracle, rng, (B, M, N), dt, "normal", 2.5)
    bias = rand_bits(oracle, rng, (N,), dt, "normal") if with_bias else None
    want = oracle.gemm(a, b, dtype_in=dt, bias=bias, gelu_grad_of=z)
    got = run_gpu(torch, a, b, dt, bias=bias, gelu_grad_of=to_dev(torch, z, dt))
    check(oracle, got, want, dt)
    if not with_bias:
        go = rand_bits(oracle, rng, (B, M, N), dt, "normal")
        y = ops.gelu_backward(to_dev(torch, go, dt), to_dev(torch, z, dt))
        check(oracle, to_host(torch, y, dt), oracle.gelu_backward(go, z, dt, compute_f32=True), dt, tol=TOL[dt] if dt != "f32" else 1e-6)


def test_accumulate_into_live_output(cuda, oracle):
    """A matmul whose outs is a live tensor (readingExistingAccBuffer): C = C + A @ B."""
    torch = cuda
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(23)
    a = rand_bits(oracle, rng, (1, 70, 50), "bf16")
    b = rand_bits(oracle, rng, (1, 50, 90), "bf16")
    c0 = rand_bits(oracle, rng, (1, 70, 90), "bf16")
    out = to_dev(torch, c0, "bf16")
    ops.gemm(to_dev(torch, a, "bf16"), to_dev(torch, b, "bf16"), out=out, accumulate_into_out=True)
    check(oracle, to_host(torch, out, "bf16"), oracle.gemm(a, b, dtype_in="bf16", residual=c0), "bf16")


def test_shared_weight_and_f32_output(cuda, oracle):
    rng = np.random.default_rng(29)
    a = rand_bits(oracle, rng, (5, 96, 72), "bf16")
    w = rand_bits(oracle, rng, (72, 136), "bf16")  # nova.linear rank 3: W shared, never broadcast-copied
    want = oracle.gemm(a, w, dtype_in="bf16", dtype_out="f32")
    got = run_gpu(cuda, a, w[None], "bf16", out_dt="f32")
    check(oracle, got, want, "f32", tol=1e-5)


def test_empty_contraction_and_empty_outputs(cuda, oracle):
    torch = cuda
    from nova_compiler_b200 import ops
    a = torch.zeros(1, 5, 0, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(1, 0, 7, device="cuda", dtype=torch.bfloat16)
    bias = torch.arange(7, device="cuda").to(torch.bfloat16)
    c = ops.gemm(a, b, bias=bias, act="relu")
    assert torch.equal(c[0], bias.expand(5, 7))
    assert ops.gemm(torch.zeros(1, 0, 4, device="cuda"), torch.zeros(1, 4, 3, device="cuda")).shape == (1, 0, 3)
    assert ops.gemm(torch.zeros(0, 2, 4, device="cuda"), torch.zeros(0, 4, 3, device="cuda")).shape == (0, 2, 3)


def test_single_pass_tf32_matches_tf32_rounding(cuda, oracle):
    """TF32X1 is the arithmetic of the reference's own GPU path (one mma per product, no split)."""
    from nova_compiler_b200 import _lib as L
    rng = np.random.default_rng(31)
    a = rng.uniform(-1, 1, (256, 320)).astype(np.float32)
    b = rng.uniform(-1, 1, (320, 192)).astype(np.float32)
    got = run_gpu(cuda, a, b, "f32", f32_mode=L.TF32X1)
    err = check(oracle, got, oracle.gemm(a, b), "f32", tol=2e-3)
    assert err > 1e-5  # it really is single-pass: the 3xTF32 default is two orders tighter
    check(oracle, run_gpu(cuda, a, b, "f32"), oracle.gemm(a, b), "f32")


# ---------------------------------------------------------------- ragged pitches: no padded copies

def test_unaligned_pitch_loader_matches_tma_bit_for_bit(cuda, oracle):
    """The same values in a 16-byte-aligned buffer (TMA path) and in an odd-pitch buffer (ld.global
    loader, element stores) must give identical bits: both feed the same MMA sequence."""
    torch = cuda
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(37)
    M, N, K = 300, 333, 257
    a = to_dev(torch, rand_bits(oracle, rng, (1, M, K), "bf16"), "bf16")
    b = to_dev(torch, rand_bits(oracle, rng, (1, K, N), "bf16"), "bf16")
    ap = torch.zeros(1, M, 264, device="cuda", dtype=torch.bfloat16); ap[:, :, :K] = a
    bp = torch.zeros(1, K, 336, device="cuda", dtype=torch.bfloat16); bp[:, :, :N] = b
    cp = torch.zeros(1, M, 336, device="cuda", dtype=torch.bfloat16)
    aligned = ops.gemm(ap[:, :, :K], bp[:, :, :N], out=cp[:, :, :N])
    from nova_compiler_b200 import _lib as L
    L.set_option("repitch", 0)  # read in place by the loader warps
    try:
        ragged = ops.gemm(a, b)  # pitches 514 B / 666 B: neither is a multiple of 16
        torch.cuda.synchronize()
    finally:
        L.set_option("repitch", 1)
    assert torch.equal(aligned, ragged)
    check(oracle, to_host(torch, ragged, "bf16"), oracle.gemm(to_host(torch, a, "bf16"), to_host(torch, b, "bf16"),
                                                               dtype_in="bf16"), "bf16")


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
def test_unaligned_pitch_repitch_copy_matches_loader_bit_for_bit(cuda, oracle, dt, trans_a, trans_b):
    """An operand no tensor map can describe is read by the loader warps (small contractions) or re-pitched into
    aligned scratch and streamed with TMA (the default).  The option "repitch" forces either: same bits, batched,
    with a batch-shared B, for both operand majors."""
    torch = cuda
    from nova_compiler_b200 import ops, _lib as L
    rng = np.random.default_rng(41)
    Bn, M, N, K = 3, 203, 141, 275
    a_shape = (Bn, K, M) if trans_a else (Bn, M, K)
    b_shape = (1, N, K) if trans_b else (1, K, N)
    a = rand_bits(oracle, rng, a_shape, dt)
    b = rand_bits(oracle, rng, b_shape, dt)
    ta, tb = to_dev(torch, a, dt), to_dev(torch, b, dt)
    a3 = ta.transpose(1, 2) if trans_a else ta
    b3 = tb.transpose(1, 2) if trans_b else tb
    kw = dict(f32_mode=L.TF32X1) if dt == "f32" else {}
    outs = {}
    for mode in ("0", "1"):
        L.set_option("repitch", int(mode))
        try:
            outs[mode] = ops.gemm(a3, b3, act="relu", **kw)
            torch.cuda.synchronize()
        finally:
            L.set_option("repitch", 1)
    assert torch.equal(outs["0"], outs["1"])
    if dt != "f32":
        want = oracle.gemm(a, b[0], dtype_in=dt, act="relu", trans_a=trans_a, trans_b=trans_b)
        check(oracle, to_host(torch, outs["1"], dt), want, dt)


def test_ragged_equals_zero_padded_problem_bit_for_bit(cuda, oracle):
    """Out-of-bounds fill replaces the reference's PadOperands copy: the ragged result is exactly the
    top-left block of the zero-padded problem."""
    torch = cuda
    from nova_compiler_b200 import ops
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    M, N, K = 1000, 1000, 999
    a = (torch.rand(1, M, K, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    b = (torch.rand(1, K, N, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    ap = torch.zeros(1, 1024, 1024, device="cuda", dtype=torch.bfloat16); ap[:, :M, :K] = a
    bp = torch.zeros(1, 1024, 1024, device="cuda", dtype=torch.bfloat16); bp[:, :K, :N] = b
    ragged = ops.gemm(a, b)
    padded = ops.gemm(ap, bp)
    assert torch.equal(ragged, padded[:, :M, :N])


# ---------------------------------------------------------------- full-size configurations

def _sampled_rows_check(torch, oracle, a_t, b_t, c_t, dt, rows, **okw):
    a_rows = to_host(torch, a_t[rows], dt)
    want = oracle.gemm(a_rows, to_host(torch, b_t, dt), dtype_in=dt, **okw)
    return check(oracle, to_host(torch, c_t[rows], dt), want, dt)


def test_full_size_c1_f32_512(cuda, oracle):
    rng = np.random.default_rng(1234)
    a = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    b = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    check(oracle, run_gpu(cuda, a, b, "f32"), oracle.gemm(a, b), "f32")


def test_full_size_c2_f16_batch32(cuda, oracle):
    rng = np.random.default_rng(1234)
    a = oracle.to_bits((rng.normal(size=(32, 1024, 1024)) / 32).astype(np.float32), "f16")
    b = oracle.to_bits((rng.normal(size=(32, 1024, 1024)) / 32).astype(np.float32), "f16")
    check(oracle, run_gpu(cuda, a, b, "f16"), oracle.gemm(a, b, dtype_in="f16"), "f16")


def test_full_size_c3_linear_gelu_sampled_rows(cuda, oracle):
    torch = cuda
    from nova_compiler_b200 import ops
    g = torch.Generator(device="cuda"); g.manual_seed(1234)
    x = torch.randn(8192, 4096, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(4096, 11008, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(11008, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    y = ops.linear(x, w, bias, act="gelu")
    rows = torch.cat([torch.tensor([0, 127, 128, 4095, 8191]), torch.randint(0, 8192, (59,))]).cuda()
    _sampled_rows_check(torch, oracle, x, w, y, "bf16", rows, bias=to_host(torch, bias, "bf16"), act="gelu_tanh")
    # linearity under exact power-of-two scaling: act(none) path, (2X) W == 2 (X W) bit for bit
    y1 = ops.linear(x[:256], w, torch.zeros_like(bias))
    y2 = ops.linear(x[:256] * 2, w, torch.zeros_like(bias))
    assert torch.equal(y2, y1 * 2)


def test_full_size_c4_scores_two_batches_and_identity(cuda, oracle):
    torch = cuda
    from nova_compiler_b200 import ops
    g = torch.Generator(device="cuda"); g.manual_seed(1234)
    q = torch.randn(256, 2048, 128, device="cuda", generator=g).to(torch.float16)
    k = torch.randn(256, 128, 2048, device="cuda", generator=g).to(torch.float16)
    s = ops.batch_matmul(q, k)
    for bidx in (0, 255):
        want = oracle.gemm(to_host(torch, q[bidx], "f16"), to_host(torch, k[bidx], "f16"), dtype_in="f16")
        check(oracle, to_host(torch, s[bidx], "f16"), want, "f16")
    # identity: Q @ [I | 0] reproduces Q exactly (one non-zero product per output)
    eye = torch.zeros(256, 128, 2048, device="cuda", dtype=torch.float16)
    eye[:, torch.arange(128), torch.arange(128)] = 1
    s2 = ops.batch_matmul(q, eye)
    assert torch.equal(s2[:, :, :128], q) and not s2[:, :, 128:].any()


def test_full_size_c5_ragged_sampled_rows(cuda, oracle):
    torch = cuda
    from nova_compiler_b200 import ops
    g = torch.Generator(device="cuda"); g.manual_seed(1234)
    for (M, N, K) in ((1000, 1000, 999), (4095, 11007, 4097)):
        a = (torch.rand(M, K, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
        b = (torch.rand(K, N, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
        c = ops.matmul(a, b)
        rows = torch.cat([torch.tensor([0, 127, 128, M - 1]), torch.randint(0, M, (28,))]).cuda()
        _sampled_rows_check(torch, oracle, a, b, c, "bf16", rows)


def test_full_size_c5a_square_16384_sampled(cuda, oracle):
    torch = cuda
    from nova_compiler_b200 import ops
    g = torch.Generator(device="cuda"); g.manual_seed(1234)
    n = 16384
    a = (torch.rand(n, n, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    b = (torch.rand(n, n, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    c = ops.matmul(a, b)
    rows = torch.cat([torch.tensor([0, 127, 128, n - 1]), torch.randint(0, n, (12,))]).cuda()
    _sampled_rows_check(torch, oracle, a, b, c, "bf16", rows)
    # N-column slab sharding (what 8 GPUs do): slab s of C equals A @ B[:, slab] bit for bit
    slab = ops.matmul(a, b[:, 2048:4096])
    assert torch.equal(slab, c[:, 2048:4096])


def test_full_size_wrapper_c(cuda, oracle):
    """The reference's one numeric assertion at its own size: 4096^3 ones + 0.5 -> 4096.5 (test/wrapper.c:93-99)."""
    torch = cuda
    from nova_compiler_b200 import ops
    n = 4096
    ones = torch.ones(1, n, n, device="cuda")
    c = ops.gemm(ones, ones, residual=torch.full((1, n, n), 0.5, device="cuda"))
    assert torch.all(c == 4096.5)


# ---------------------------------------------------------------- host-buffer and memref entry points

def test_gemm_host_and_memref_entry_points(cuda, oracle, lib):
    from nova_compiler_b200 import _lib as L
    rng = np.random.default_rng(41)
    M, N, K = 96, 104, 72
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    want = oracle.gemm(a, b, bias=bias, act="relu")

    def memref(arr, cls):
        m = cls()
        m.allocated = m.aligned = arr.ctypes.data
        m.offset = 0
        for i in range(arr.ndim):
            m.sizes[i] = arr.shape[i]
            m.strides[i] = arr.strides[i] // arr.itemsize
        return m

    y = np.zeros((M, N), np.float32)
    st = lib._mlir_ciface_nova_b200_linear(C.byref(memref(y, L.MemRef2D)), C.byref(memref(a, L.MemRef2D)),
                                           C.byref(memref(b, L.MemRef2D)), C.byref(memref(bias, L.MemRef1D)),
                                           L.F32, L.ACT_RELU)
    L.check(st)
    check(oracle, y, want, "f32")
    # matmul with a transposed (column-major) A descriptor: the matmul_transpose_a form
    at = np.ascontiguousarray(a.T)
    c = np.zeros((M, N), np.float32)
    L.check(lib._mlir_ciface_nova_b200_matmul(C.byref(memref(c, L.MemRef2D)), C.byref(memref(at.T, L.MemRef2D)),
                                              C.byref(memref(b, L.MemRef2D)), L.F32))
    check(oracle, c, oracle.gemm(a, b), "f32")
    # batch_matmul f16 in / f16 out on host buffers
    a3 = oracle.to_bits(rng.normal(size=(3, 40, 64)).astype(np.float32) / 8, "f16")
    b3 = oracle.to_bits(rng.normal(size=(3, 64, 48)).astype(np.float32) / 8, "f16")
    c3 = np.zeros((3, 40, 48), np.uint16)
    L.check(lib._mlir_ciface_nova_b200_batch_matmul(C.byref(memref(c3, L.MemRef3D)), C.byref(memref(a3, L.MemRef3D)),
                                                    C.byref(memref(b3, L.MemRef3D)), L.F16, L.F16))
    check(oracle, c3, oracle.gemm(a3, b3, dtype_in="f16"), "f16")
    # a descriptor whose inner strides are both non-unit is a layout error, reported not thrown
    bad = memref(a, L.MemRef2D)
    bad.strides[0], bad.strides[1] = 2 * K, 2
    assert lib._mlir_ciface_nova_b200_matmul(C.byref(memref(c, L.MemRef2D)), C.byref(bad),
                                             C.byref(memref(b, L.MemRef2D)), L.F32) == L.ERR_LAYOUT


@pytest.mark.parametrize("shape", [(6, 70, 90, 48), (1, 1100, 136, 64)])  # chunked by batch / by 256-row blocks
def test_gemm_host_pipeline_carries_epilogue_operands(cuda, oracle, lib, shape):
    """nova_b200_gemm_host cuts the problem into chunks that overlap copies and kernels; the residual (an addend, or
    the pre-activation of a fused gelu_backward) has to be cut the same way."""
    from nova_compiler_b200 import _lib as L
    rng = np.random.default_rng(43)
    Bn, M, N, K = shape
    a = oracle.to_bits(rng.normal(size=(Bn, M, K)).astype(np.float32), "bf16")
    b = oracle.to_bits(rng.normal(size=(Bn, K, N)).astype(np.float32) / 8, "bf16")
    bias = oracle.to_bits(rng.normal(size=N).astype(np.float32), "bf16")
    aux = oracle.to_bits(rng.normal(size=(Bn, M, N)).astype(np.float32) * 2, "bf16")
    for mode in ("bias+residual", "gelu_grad"):
        c = np.zeros((Bn, M, N), np.uint16)
        g = L.GemmArgs()
        g.struct_size = C.sizeof(L.GemmArgs)
        g.dtype_ab = g.dtype_c = L.BF16
        g.batch, g.M, g.N, g.K = Bn, M, N, K
        g.lda, g.ldb, g.ldc, g.ldr = K, N, N, N
        g.batch_stride_a, g.batch_stride_b, g.batch_stride_c, g.batch_stride_r = M * K, K * N, M * N, M * N
        g.A, g.B, g.C = a.ctypes.data, b.ctypes.data, c.ctypes.data
        g.bias, g.residual = bias.ctypes.data, aux.ctypes.data
        if mode == "bias+residual":
            g.init = L.INIT_BIAS_AND_RESIDUAL
            want = oracle.gemm(a, b, dtype_in="bf16", bias=bias, residual=aux)
        else:
            g.init, g.act = L.INIT_BIAS_ROW, L.ACT_GELU_TANH_GRAD
            want = oracle.gemm(a, b, dtype_in="bf16", bias=bias, gelu_grad_of=aux)
        L.check(lib.nova_b200_gemm_host(C.byref(g)))
        check(oracle, c, want, "bf16")


@pytest.mark.parametrize("N", [2504, 2500])
def test_gemm_host_tiled_pipeline_writes_only_its_window(cuda, oracle, lib, N):
    """One large product from host memory is cut into (row block) x (column slab) tiles so that results start
    flowing back before all of B has arrived; the slabs are strided 2-D copies on both sides.  Ragged extents,
    bias + residual, and a host C that is a window of a larger buffer whose other bytes must survive."""
    from nova_compiler_b200 import _lib as L
    rng = np.random.default_rng(47)
    M, K, ldc = 1100, 200, 2600   # N = 2500: B's pitch is not 16-byte aligned, so row blocks only
    a = oracle.to_bits(rng.normal(size=(M, K)).astype(np.float32), "bf16")
    b = oracle.to_bits(rng.normal(size=(K, N)).astype(np.float32) / 8, "bf16")
    bias = oracle.to_bits(rng.normal(size=N).astype(np.float32), "bf16")
    res = oracle.to_bits(rng.normal(size=(M, N)).astype(np.float32), "bf16")
    cbuf = np.full((M + 3, ldc), 0x4321, np.uint16)
    g = L.GemmArgs()
    g.struct_size = C.sizeof(L.GemmArgs)
    g.dtype_ab = g.dtype_c = L.BF16
    g.batch, g.M, g.N, g.K = 1, M, N, K
    g.lda, g.ldb, g.ldc, g.ldr = K, N, ldc, N
    g.A, g.B, g.C = a.ctypes.data, b.ctypes.data, cbuf.ctypes.data
    g.bias, g.residual, g.init, g.act = bias.ctypes.data, res.ctypes.data, L.INIT_BIAS_AND_RESIDUAL, L.ACT_RELU
    L.check(lib.nova_b200_gemm_host(C.byref(g)))
    want = oracle.gemm(a, b, dtype_in="bf16", bias=bias, residual=res, act="relu")
    check(oracle, np.ascontiguousarray(cbuf[:M, :N]), want, "bf16")
    assert np.all(cbuf[:M, N:] == 0x4321) and np.all(cbuf[M:] == 0x4321)


@pytest.mark.parametrize("K", [1024, 1000])   # 1000: the last K range is shorter and ends inside a k-block
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (False, True)])
def test_split_k_matches_the_unsplit_product(cuda, oracle, lib, dt, trans_a, trans_b, K):
    """A product with few output tiles and a long K runs its K ranges as the batches of one launch and sums the fp32
    partials in a second kernel that applies the epilogue once.  Forced ranges (option split_k) on every operand
    major, every init / activation, a ragged N and a C window; against the oracle, and against the unsplit kernel
    (same arithmetic up to the association of the fp32 additions)."""
    torch = cuda
    from nova_compiler_b200 import ops, _lib as L
    rng = np.random.default_rng(71)
    M, N = 200, 150
    a = rand_bits(oracle, rng, (K, M) if trans_a else (M, K), dt)
    b = rand_bits(oracle, rng, (N, K) if trans_b else (K, N), dt)
    bias = rand_bits(oracle, rng, (N,), dt)
    res = rand_bits(oracle, rng, (M, N), dt)
    z = rand_bits(oracle, rng, (M, N), dt)
    cases = [dict(), dict(bias=bias, act="relu"), dict(bias=bias, residual=res, act="gelu"), dict(residual=res),
             dict(bias=bias, gelu_grad_of=z)]
    try:
        for kw in cases:
            okw = {k: v for k, v in kw.items() if k != "act"}
            if "act" in kw:
                okw["act"] = {"gelu": "gelu_tanh"}.get(kw["act"], kw["act"])
            want = oracle.gemm(a, b, dtype_in=dt, trans_a=trans_a, trans_b=trans_b, **okw)
            got = {}
            for ranges in (0, 4, 8):
                L.set_option("split_k", ranges)
                gkw = dict(kw)
                if "residual" in gkw:
                    gkw["residual"] = res[None]
                if "gelu_grad_of" in gkw:
                    gkw["gelu_grad_of"] = to_dev(torch, z, dt)[None]
                got[ranges] = run_gpu(torch, a, b, dt, trans_a=trans_a, trans_b=trans_b, **gkw)
                check(oracle, got[ranges], want, dt)
            for ranges in (4, 8):
                assert oracle.rel_fro(oracle.from_bits(got[ranges], dt), oracle.from_bits(got[0], dt)) <= (2e-5 if dt == "f32" else 4e-3)
            if dt == "f32" and not kw:
                # the tensor core adds into its fp32 accumulator with truncation, so the error of the 3xTF32 product
                # grows with the length of one accumulation chain: shorter ranges are MORE accurate against float64
                af = (a.T if trans_a else a).astype(np.float64)
                bf = (b.T if trans_b else b).astype(np.float64)
                truth = af @ bf
                err = {r: oracle.rel_fro(got[r].astype(np.float64), truth) for r in (0, 4, 8)}
                assert err[8] < err[4] < err[0] and err[8] <= 2e-6
        # accumulate into a live C that is a window of a wider buffer; bytes outside the window survive
        L.set_option("split_k", 4)
        ta, tb = to_dev(torch, a, dt)[None], to_dev(torch, b, dt)[None]
        if trans_a:
            ta = ta.transpose(1, 2)
        if trans_b:
            tb = tb.transpose(1, 2)
        buf = torch.full((1, M + 2, N + 10), 3.0, device="cuda", dtype=_tdt(torch, dt))
        win = buf[:, :M, :N]
        ops.gemm(ta, tb, out=win, accumulate_into_out=True)
        torch.cuda.synchronize()
        want = oracle.gemm(a, b, dtype_in=dt, trans_a=trans_a, trans_b=trans_b,
                           residual=oracle.to_bits(np.full((M, N), 3.0, np.float32), dt))
        check(oracle, to_host(torch, win, dt)[0], want, dt)
        mask = torch.ones_like(buf, dtype=torch.bool)
        mask[:, :M, :N] = False
        assert torch.all(buf[mask] == 3.0)
        assert ops.device_status() == 0
    finally:
        L.set_option("split_k", -1)


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_split_k_of_batched_products(cuda, oracle, dt):
    """K ranges of a BATCHED product: launch batch b * ranges + s; bias, residual and a shared B (batch stride 0)."""
    torch = cuda
    from nova_compiler_b200 import _lib as L
    rng = np.random.default_rng(73)
    B, M, N, K = 3, 130, 200, 1500
    a = rand_bits(oracle, rng, (B, M, K), dt)
    bias = rand_bits(oracle, rng, (N,), dt)
    res = rand_bits(oracle, rng, (B, M, N), dt)
    try:
        for b in (rand_bits(oracle, rng, (B, K, N), dt), rand_bits(oracle, rng, (K, N), dt)):
            want = oracle.gemm(a, b, dtype_in=dt, bias=bias, residual=res, act="relu")
            got = {}
            for ranges in (0, 5, -1):
                L.set_option("split_k", ranges)
                got[ranges] = run_gpu(torch, a, b, dt, bias=bias, residual=res, act="relu")
                # (forced to one chain of 1500, the f32 product is ~1.1e-5 off: what the ranges are for)
                check(oracle, got[ranges], want, dt, tol=3e-5 if (dt == "f32" and ranges == 0) else None)
            assert oracle.rel_fro(oracle.from_bits(got[5], dt), oracle.from_bits(got[0], dt)) <= (2e-5 if dt == "f32" else 2e-3)
    finally:
        L.set_option("split_k", -1)


def test_f32_error_does_not_grow_with_k(cuda):
    """The tensor core adds into its fp32 accumulator with truncation, so one long accumulation chain drifts: the
    unsplit 3xTF32 product is 5.7e-5 off float64 at K = 8192 and 3.5e-4 at K = 50304.  With K in ranges of at most
    1024 the error stays under the 1e-5 the f32 path promises, for ragged and very long K alike."""
    torch = cuda
    from nova_compiler_b200 import ops
    g = torch.Generator(device="cuda")
    g.manual_seed(77)
    for Bn, M, N, K in [(1, 200, 150, 1000), (1, 256, 384, 8191), (1, 128, 128, 50304), (4, 256, 192, 8192)]:
        a = torch.rand(Bn, M, K, device="cuda", generator=g) * 2 - 1
        b = torch.rand(Bn, K, N, device="cuda", generator=g) * 2 - 1
        c = ops.gemm(a, b).double()
        truth = a.double() @ b.double()
        err = float((c - truth).norm() / truth.norm())
        assert err <= 1e-5, (Bn, M, N, K, err)


def test_split_k_is_planned_for_few_tiles_only(cuda, lib):
    """The planner's rule, read from the plan record: the 512-cubed f32 product (32 tiles of 128 x 64) runs four K
    ranges; the headline linear layer and a batched product never split."""
    from nova_compiler_b200 import _lib as L

    def plan(dt, batch, M, N, K):
        g = L.GemmArgs()
        g.struct_size = C.sizeof(L.GemmArgs)
        g.dtype_ab = g.dtype_c = dt
        g.batch, g.M, g.N, g.K = batch, M, N, K
        g.lda, g.ldb, g.ldc = K, N, N
        g.batch_stride_a, g.batch_stride_b, g.batch_stride_c = M * K, K * N, M * N
        g.A = g.B = g.C = 4096  # never dereferenced by the planner
        info = L.GemmPlanInfo()
        L.check(lib.nova_b200_gemm_plan(C.byref(g), C.byref(info)))
        return info
    small = plan(L.F32, 1, 512, 512, 512)
    assert small.tiles == 4 * 32 and small.scratch_bytes >= 4 * 512 * 512 * 4
    assert plan(L.BF16, 1, 8192, 11008, 4096).tiles == 32 * 43
    assert plan(L.F16, 32, 1024, 1024, 1024).tiles == 32 * 16
    # a weight gradient: 384 x 1536 outputs from K = 8192 tokens, bf16: 36 tiles of 128 x 128 -> four ranges
    wg = plan(L.BF16, 1, 384, 1536, 8192)
    assert wg.tiles % 36 == 0 and wg.tiles // 36 >= 2


def test_nova_matmul_rank_rules(cuda, oracle):
    """nova.matmul shape rules (MatmulOp::inferReturnTypes, NovaOps.cpp:1116-1285)."""
    torch = cuda
    from nova_compiler_b200 import ops
    g = torch.Generator(device="cuda"); g.manual_seed(7)
    a4 = torch.randn(2, 4, 24, 40, device="cuda", generator=g)
    b4 = torch.randn(2, 4, 40, 16, device="cuda", generator=g)
    ref = oracle.gemm(a4.reshape(8, 24, 40).cpu().numpy(), b4.reshape(8, 40, 16).cpu().numpy())
    got = ops.matmul(a4, b4)
    assert got.shape == (2, 4, 24, 16)
    check(oracle, got.reshape(8, 24, 16).cpu().numpy(), ref, "f32")
    b2 = torch.randn(40, 16, device="cuda", generator=g)  # 2-D rhs broadcast over the batch
    got = ops.matmul(a4, b2)
    check(oracle, got.reshape(8, 24, 16).cpu().numpy(), oracle.gemm(a4.reshape(8, 24, 40).cpu().numpy(), b2.cpu().numpy()), "f32")
    v = torch.randn(40, device="cuda", generator=g)
    assert ops.matmul(v, v).shape == ()
    with pytest.raises(Exception):
        ops.matmul(torch.zeros(4, 5, device="cuda"), torch.zeros(6, 4, device="cuda"))


def test_no_bounded_wait_gave_up(cuda):
    from nova_compiler_b200 import ops
    assert ops.device_status() == 0


def test_randomised_small_problems(cuda, oracle):
    """Seeded random sweep over small extents, dtypes, operand majors, batch forms and epilogues: every
    combination is one call through the C ABI checked against the oracle."""
    rng = np.random.default_rng(20261125)
    dims = list(range(1, 41)) + [63, 64, 65, 127, 128, 129, 255, 256, 257]
    for trial in range(72):
        dt = ("f32", "f16", "bf16")[trial % 3]
        M, N, K = (int(rng.choice(dims)) for _ in range(3))
        B = int(rng.choice([1, 1, 2, 3]))
        ta, tb = bool(rng.integers(2)), bool(rng.integers(2))
        shared_b = B > 1 and bool(rng.integers(2))
        init = ("zero", "bias", "residual")[int(rng.integers(3))]
        act = (None, "relu", "gelu")[int(rng.integers(3))]
        a = rand_bits(oracle, rng, (B, K, M) if ta else (B, M, K), dt)
        b = rand_bits(oracle, rng, ((N, K) if tb else (K, N)) if shared_b else ((B, N, K) if tb else (B, K, N)), dt)
        bias = rand_bits(oracle, rng, (N,), dt) if init == "bias" else None
        res = rand_bits(oracle, rng, (B, M, N), dt) if init == "residual" else None
        want = oracle.gemm(a, b, dtype_in=dt, trans_a=ta, trans_b=tb, bias=bias, residual=res,
                           act={"gelu": "gelu_tanh"}.get(act, act or "none"))
        got = run_gpu(cuda, a, b if not shared_b else b[None], dt, trans_a=ta, trans_b=tb, bias=bias, residual=res, act=act)
        err = oracle.rel_fro(oracle.from_bits(got, dt), oracle.from_bits(want, dt))
        assert err <= TOL[dt], f"trial {trial}: {dt} B={B} M={M} N={N} K={K} ta={ta} tb={tb} shared_b={shared_b} {init} {act}: {err:.3e}"
