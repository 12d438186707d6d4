"""Runtime behaviour around the contraction, on a GPU through the C ABI: per-stream scratch (two streams at once),
graph capture of scratch users, plan cache / launch-mode / prefetch invariance, bytes around an output survive,
prepared operands, the rank-4 and dynamic-argument entry points, the slab re-interleave kernel."""
import ctypes as C

import numpy as np
import pytest

from test_gemm_gpu import TOL, _tdt, check, rand_bits, to_dev, to_host

pytestmark = pytest.mark.gpu


def _gemm_args(L, a, b, c, **kw):
    g = L.GemmArgs()
    g.struct_size = C.sizeof(L.GemmArgs)
    code = {4: L.F32}
    import torch
    dt = {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16}
    g.dtype_ab, g.dtype_c = dt[a.dtype], dt[c.dtype]
    g.batch, g.M, g.K = a.shape
    g.N = b.shape[2]
    g.A, g.B, g.C = a.data_ptr(), b.data_ptr(), c.data_ptr()
    g.lda, g.ldb, g.ldc = a.stride(1), b.stride(1), c.stride(1)
    g.batch_stride_a, g.batch_stride_b, g.batch_stride_c = a.stride(0), b.stride(0), c.stride(0)
    for k, v in kw.items():
        setattr(g, k, v)
    return g


def test_two_streams_run_scratch_users_concurrently(cuda, oracle):
    """Scratch is per (device, stream): two f32 contractions (hi/lo split in scratch) and two re-pitched bf16
    ones, enqueued alternately on two streams without any synchronisation between them, all match the oracle."""
    torch = cuda
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(7)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    cases = []
    for i, (M, N, K) in enumerate([(384, 512, 640), (512, 384, 768), (300, 333, 257), (203, 141, 275)]):
        dt = "f32" if i < 2 else "bf16"
        a = rand_bits(oracle, rng, (1, M, K), dt)
        b = rand_bits(oracle, rng, (1, K, N), dt)
        cases.append((dt, a, b, to_dev(torch, a, dt), to_dev(torch, b, dt)))
    torch.cuda.synchronize()
    outs = [None] * len(cases)
    for rep in range(3):  # several rounds in flight on both streams
        for i, (dt, a, b, ta, tb) in enumerate(cases):
            with torch.cuda.stream(s1 if i % 2 == 0 else s2):
                outs[i] = ops.gemm(ta, tb)
    torch.cuda.synchronize()
    for (dt, a, b, ta, tb), out in zip(cases, outs):
        check(oracle, to_host(torch, out, dt), oracle.gemm(a, b, dtype_in=dt), dt)
    assert ops.device_status() == 0


def test_scratch_users_capture_into_a_graph_and_survive_growth(cuda, oracle):
    """A captured f32 contraction keeps working after a LARGER scratch request on the same stream: growing never
    frees the buffer the graph holds.  Growth during capture is refused with a clear error instead."""
    torch = cuda
    from nova_compiler_b200 import ops, _lib as L
    rng = np.random.default_rng(8)
    a = rng.uniform(-1, 1, (1, 256, 320)).astype(np.float32)
    b = rng.uniform(-1, 1, (1, 320, 192)).astype(np.float32)
    ta, tb = to_dev(torch, a, "f32"), to_dev(torch, b, "f32")
    out = torch.empty(1, 256, 192, device="cuda")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        ops.gemm(ta, tb, out=out)  # the stream's scratch exists before the capture
    side.synchronize()
    big_a = torch.zeros(1, 1024, 1024, device="cuda")
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            ops.gemm(ta, tb, out=out)
            with pytest.raises(L.NovaB200Error) as ei:  # 16 MiB of split buffers: more than the stream owns
                ops.gemm(big_a, big_a)
            assert "captured" in str(ei.value)
    out.zero_()
    with torch.cuda.stream(side):
        ops.gemm(big_a, big_a)  # grows the stream's scratch: the graph's buffer must stay alive
    side.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    check(oracle, to_host(torch, out, "f32"), oracle.gemm(a, b), "f32")


def test_launch_modes_and_prefetch_do_not_change_the_result(cuda, oracle):
    """Plan cache on/off, programmatic dependent launch on/off and the pair kernel's L2 prefetch cursor are
    scheduling choices: the output bits are the same."""
    torch = cuda
    from nova_compiler_b200 import ops, _lib as L
    rng = np.random.default_rng(9)
    a = to_dev(torch, rand_bits(oracle, rng, (2, 512, 1024), "bf16"), "bf16")
    b = to_dev(torch, rand_bits(oracle, rng, (2, 1024, 768), "bf16"), "bf16")
    base = ops.gemm(a, b, act="gelu")
    torch.cuda.synchronize()
    info = L.GemmPlanInfo()
    for opt, val, restore in [("plan_cache", 0, 1), ("pdl", 0, 1), ("prefetch", 3, -1), ("prefetch", 11, -1), ("pair", 0, -1)]:
        L.set_option(opt, val)
        try:
            got = ops.gemm(a, b, act="gelu")
            got2 = ops.gemm(a, b, act="gelu")  # back to back: the second launch's prologue overlaps the first
            torch.cuda.synchronize()
        finally:
            L.set_option(opt, restore)
        assert torch.equal(got, base) and torch.equal(got2, base), opt
    assert L.get_option("prefetch") == -1 and L.get_option("pdl") == 1
    assert ops.device_status() == 0


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_bytes_around_the_output_survive(cuda, oracle, dt):
    """C is a window of a larger buffer (ldc > N, rows past M, a gap between batches): every byte outside the
    window keeps its sentinel.  Ragged extents and an unaligned pitch take the element-store path, aligned ones
    the TMA-store path."""
    torch = cuda
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(10)
    for (Bn, M, N, K, ldc, rows_alloc) in [(2, 200, 328, 264, 384, 256), (2, 130, 77, 100, 83, 140), (1, 256, 256, 256, 320, 300),
                                            (2, 200, 250, 128, 256, 210)]:   # aligned pitch, rows end inside a 16-byte chunk
        a = rand_bits(oracle, rng, (Bn, M, K), dt)
        b = rand_bits(oracle, rng, (Bn, K, N), dt)
        buf = torch.full((Bn, rows_alloc, ldc), -7.0, device="cuda", dtype=_tdt(torch, dt))
        window = buf[:, :M, :N]
        ops.gemm(to_dev(torch, a, dt), to_dev(torch, b, dt), out=window)
        torch.cuda.synchronize()
        check(oracle, to_host(torch, window, dt), oracle.gemm(a, b, dtype_in=dt), dt)
        mask = torch.ones_like(buf, dtype=torch.bool)
        mask[:, :M, :N] = False
        assert torch.all(buf[mask] == -7.0), f"bytes outside the {M}x{N} window of a {rows_alloc}x{ldc} buffer changed"


def test_prepared_operand_skips_the_per_call_copy(cuda, oracle, lib):
    """A weight with an unaligned pitch, prepared once: the call plans as plain TMA (no scratch) and gives the same
    bits as the default per-call re-pitch."""
    torch = cuda
    from nova_compiler_b200 import ops, _lib as L
    rng = np.random.default_rng(11)
    M, N, K = 320, 527, 448   # B [K, N]: pitch 1054 B, not a multiple of 16
    a = to_dev(torch, rand_bits(oracle, rng, (1, M, K), "bf16"), "bf16")
    bh = rand_bits(oracle, rng, (1, K, N), "bf16")
    b = to_dev(torch, bh, "bf16")
    want = ops.gemm(a, b)
    handle = C.c_void_p()
    L.check(lib.nova_b200_operand_prepare(b.data_ptr(), L.BF16, 1, K, N, N, 0, None, C.byref(handle)))
    data, ld, bs = C.c_void_p(), C.c_int64(), C.c_int64()
    L.check(lib.nova_b200_operand_view(handle, C.byref(data), C.byref(ld), C.byref(bs)))
    assert ld.value == 528 and data.value % 16 == 0
    out = torch.empty(1, M, N, device="cuda", dtype=torch.bfloat16)
    g = _gemm_args(L, a, b, out)
    g.B, g.ldb, g.batch_stride_b = data.value, ld.value, 0
    info = L.GemmPlanInfo()
    L.check(lib.nova_b200_gemm_plan(C.byref(g), C.byref(info)))
    assert (info.loader_b, info.scratch_bytes) == (0, 0)
    L.check(lib.nova_b200_gemm(C.byref(g), None))
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    lib.nova_b200_operand_free(handle)
    # the operator-level wrapper: a strided torch view of the library-owned copy
    prep = ops.PreparedOperand(b[0])
    assert prep.tensor.shape == (K, N) and prep.tensor.stride(0) == 528 and torch.equal(prep.tensor, b[0])
    assert torch.equal(ops.gemm(a, prep.tensor[None]), want)
    torch.cuda.synchronize()
    prep.free()


def test_rank4_descriptor_entry_point(cuda, oracle, lib):
    """nova.matmul on rank-4 operands = collapse the batch dims, batch_matmul, expand (NovaToLinalg.cpp:904-989):
    contiguous operands collapse as metadata; a B that broadcasts along one batch dim walks the outer dim."""
    torch = cuda
    from nova_compiler_b200 import _lib as L
    rng = np.random.default_rng(12)

    def desc(t):
        d = L.MemRef4D()
        d.allocated = d.aligned = t.data_ptr()
        d.offset = 0
        for i in range(4):
            d.sizes[i], d.strides[i] = t.shape[i], t.stride(i)
        return d

    for bshape in [(2, 3), (1, 1), (1, 3), (2, 1)]:
        ah = rand_bits(oracle, rng, (2, 3, 64, 96), "f16")
        bh = rand_bits(oracle, rng, bshape + (96, 80), "f16")
        a, b = to_dev(torch, ah, "f16"), to_dev(torch, bh, "f16")
        c = torch.zeros(2, 3, 64, 80, device="cuda", dtype=torch.float16)
        L.check(lib._mlir_ciface_nova_b200_batch_matmul_4d(C.byref(desc(c)), C.byref(desc(a)), C.byref(desc(b)), L.F16, L.F16))
        torch.cuda.synchronize()
        bb = np.broadcast_to(bh, (2, 3, 96, 80)).reshape(6, 96, 80)
        want = oracle.gemm(ah.reshape(6, 64, 96), np.ascontiguousarray(bb), dtype_in="f16")
        check(oracle, to_host(torch, c, "f16").reshape(6, 64, 80), want, "f16")


def test_dynamic_argument_entry_point_with_host_buffers(cuda, oracle, lib):
    """(result*, void** args) in the style of the reference's _mlir_ciface_main wrapper
    (lib/Transforms/GenerateDynamicWrapper.cpp:34-95), host memrefs in and out as robust_driver.cpp passes them."""
    from nova_compiler_b200 import _lib as L
    text = """
    func.func @main(%a: tensor<16x16xf32>, %b: tensor<16x16xf32>, %c: tensor<16x16xf32>) -> tensor<16x16xf32> {
      %s = nova.add %a, %b : tensor<16x16xf32>, tensor<16x16xf32>
      %r = nova.matmul %s, %c : tensor<16x16xf32>, tensor<16x16xf32>
      return %r : tensor<16x16xf32>
    }
    """
    mod = C.c_void_p()
    L.check(lib.nova_b200_module_parse(text.encode(), C.byref(mod)))
    bufs = [np.full((16, 16), v, np.float32) for v in (1.0, 2.0, 1.0)]  # robust_driver.cpp:71-80: (1+2).1 -> 48
    out = np.zeros((16, 16), np.float32)

    def desc(arr):
        d = L.MemRef2D()
        d.allocated = d.aligned = arr.ctypes.data
        d.offset = 0
        d.sizes[0], d.sizes[1] = arr.shape
        d.strides[0], d.strides[1] = arr.shape[1], 1
        return d

    descs = [desc(x) for x in bufs]
    rd = desc(out)
    argv = (C.c_void_p * 3)(*[C.addressof(d) for d in descs])
    L.check(lib.nova_b200_module_call_ciface(mod, b"main", C.byref(rd), argv))
    assert np.all(out == np.float32(48.0))
    lib.nova_b200_module_free(mod)


@pytest.mark.parametrize("n,dt", [(1000, "bf16"), (11008, "bf16"), (333, "f32"), (135, "bf16")])
def test_slab_interleave_kernel(cuda, lib, n, dt):
    """staging = the ranks' column slabs one after the other (as an all-gather leaves them) -> row-major [M, N]."""
    torch = cuda
    from nova_compiler_b200 import _lib as L
    from nova_compiler_b200.sharding import column_slab
    world, m = 4, 37
    tdt = _tdt(torch, dt)
    full = torch.arange(m * n, device="cuda", dtype=torch.float32).reshape(m, n).remainder(251).to(tdt)
    widths = [column_slab(n, world, r)[1] for r in range(world)]
    wmax = max(widths)
    staging = torch.full((world, m, wmax), -1.0, device="cuda", dtype=tdt)
    for r in range(world):
        s, c = column_slab(n, world, r)
        staging[r, :, :c] = full[:, s:s + c]
    out = torch.empty(m, n, device="cuda", dtype=tdt)
    L.check(lib.nova_b200_interleave_slabs(staging.data_ptr(), out.data_ptr(), m, n, world, wmax, 64, out.element_size(), None))
    torch.cuda.synchronize()
    assert torch.equal(out, full)


def test_f32_presplit_is_shared_by_contractions(cuda, lib):
    """An f32 matrix split into its 3xTF32 halves once (nova_b200_f32_presplit): contractions that read it as A, as B
    or through a transposed view give the same bits as when they split it themselves, and forget it on release."""
    torch = cuda
    from nova_compiler_b200 import ops, _lib as L
    g = torch.Generator(device="cuda")
    g.manual_seed(31)
    M, N, K = 320, 264, 1024
    x = torch.randn(M, K, device="cuda", generator=g)          # read as A [M, K], as B [M(K'), K(N')] and transposed
    w = torch.randn(K, N, device="cuda", generator=g)
    u = torch.randn(96, M, device="cuda", generator=g)
    want_a = ops.gemm(x[None], w[None])
    want_b = ops.gemm(u[None], x[None])
    want_t = ops.gemm(x.t()[None], u.t()[None])                # x^T [K, M] . u^T [M, 96]
    handle = C.c_void_p()
    L.check(lib.nova_b200_f32_presplit(x.data_ptr(), M, K, K, None, C.byref(handle)))
    try:
        assert torch.equal(ops.gemm(x[None], w[None]), want_a)
        assert torch.equal(ops.gemm(u[None], x[None]), want_b)
        assert torch.equal(ops.gemm(x.t()[None], u.t()[None]), want_t)
        # the halves are a snapshot: a contraction reading the registered matrix does not see a later change of x
        x2 = x.clone()
        x.add_(1.0)
        assert torch.equal(ops.gemm(x[None], w[None]), want_a)
    finally:
        L.check(lib.nova_b200_f32_presplit_release(handle, None))
    got = ops.gemm(x[None], w[None])                           # forgotten: the new contents are split and used
    assert torch.equal(got, ops.gemm((x2 + 1.0)[None], w[None])) and not torch.equal(got, want_a)
    torch.cuda.synchronize()


def test_operands_on_another_device_are_refused(cuda, lib):
    torch = cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from nova_compiler_b200 import ops, _lib as L
    a = torch.zeros(1, 128, 128, device="cuda:1", dtype=torch.bfloat16)
    out = torch.empty(1, 128, 128, device="cuda:1", dtype=torch.bfloat16)
    g = _gemm_args(L, a, a, out)
    torch.cuda.set_device(0)
    assert lib.nova_b200_gemm(C.byref(g), None) == L.ERR_INVALID_ARG  # cuda:1 memory with cuda:0 current
    assert b"current device" in lib.nova_b200_last_error_string()
    res = ops.gemm(a, a)  # the operator layer makes the operands' device current instead
    assert res.device.index == 1
    b0 = torch.zeros(1, 128, 128, device="cuda:0", dtype=torch.bfloat16)
    with pytest.raises(L.NovaB200Error):
        ops.gemm(a, b0)
    torch.cuda.synchronize(1)
    # kernels that ask for more than 48 KB of dynamic shared memory are configured per device: the same process, first
    # device 0 then device 1, must get the same rows from both
    gen = torch.Generator(device="cpu")
    gen.manual_seed(5)
    x = torch.randn(300, 4096, generator=gen).to(torch.bfloat16)
    wide = torch.randn(20, 50304, generator=gen)
    gam = torch.randn(4096, generator=gen).to(torch.bfloat16)
    got = []
    for dev in (0, 1):
        d = f"cuda:{dev}"
        y = ops.layer_norm(x.to(d), gam.to(d), gam.to(d))[0]
        sm = ops.softmax(wide.to(d))
        sm2 = ops.softmax(x.to(d))
        got.append((y.cpu(), sm.cpu(), sm2.cpu()))
    for u, v in zip(got[0], got[1]):
        assert torch.equal(u, v)
    torch.cuda.set_device(0)


@pytest.mark.parametrize("dt,tol_pair,tol_truth", [("f16", 1e-3, 1.0e-3), ("bf16", 4e-3, 5e-3), ("f32", 1e-5, 1e-5)])
def test_layer_norm_folded_into_the_contraction(cuda, oracle, dt, tol_pair, tol_truth):
    """LN-apply fused into the FFN-up contraction (isPrologue, NovaKernelConfig.cpp:1898-1917) in its algebraic
    form: rstd_i * (x.W' - mean_i c_j) + d_j.  Against the unfused layer_norm -> linear+GELU pair (which rounds the
    normalised tensor to the operand dtype) the difference is about two operand roundings: <= 1e-3 for f16,
    <= 4e-3 for bf16, <= 1e-5 for f32; against float64 the fused result is as close as the unfused one."""
    torch = cuda
    from nova_compiler_b200 import ops
    g = torch.Generator(device="cuda")
    g.manual_seed(21)
    tdt = _tdt(torch, dt)
    rows, K, N = 333, 512, 328
    x = (torch.randn(rows, K, device="cuda", generator=g) + 0.3).to(tdt)
    w = (torch.randn(K, N, device="cuda", generator=g) * 0.05).to(tdt)
    gamma = (1.0 + 0.2 * torch.randn(K, device="cuda", generator=g)).to(tdt)
    beta = (0.1 * torch.randn(K, device="cuda", generator=g)).to(tdt)
    bias = (0.1 * torch.randn(N, device="cuda", generator=g)).to(tdt)
    y, _, _ = ops.layer_norm(x, gamma, beta)
    unfused = ops.linear(y, w, bias, act="gelu")
    folded = ops.LnFoldedLinear(w, gamma, beta, bias)
    fused = folded(x, act="gelu")
    torch.cuda.synchronize()
    d = torch.float64
    truth = torch.nn.functional.gelu(
        torch.nn.functional.layer_norm(x.to(d), (K,), gamma.to(d), beta.to(d), eps=1e-5) @ w.to(d) + bias.to(d), approximate="tanh")
    rel = lambda a, b: float((a.to(d) - b.to(d)).norm() / b.to(d).norm())
    assert rel(fused, unfused) <= tol_pair, rel(fused, unfused)
    assert rel(fused, truth) <= tol_truth and rel(fused, truth) <= 1.5 * rel(unfused, truth) + 1e-6, (rel(fused, truth), rel(unfused, truth))
    # the statistics entry point on its own
    stats = torch.empty(rows, 2, device="cuda")
    from nova_compiler_b200 import _lib as L
    L.check(L.load().nova_b200_row_stats(x.data_ptr(), stats.data_ptr(), rows, K, {"f16": L.F16, "bf16": L.BF16, "f32": L.F32}[dt], None))
    torch.cuda.synchronize()
    xm = x.to(d).mean(dim=1)
    xv = x.to(d).var(dim=1, unbiased=False)
    assert rel(stats[:, 0], xm) <= 1e-5 and rel(stats[:, 1], (xv + 1e-5).rsqrt()) <= 1e-5
