"""Parity of the row-wise kernels (layer_norm, softmax, gather, activation, add) against the CPU oracle.
f32: rel-Frobenius <= 1e-5.  f16/bf16: the kernels compute in fp32 and round once, compared with the
oracle in the same mode, <= 1e-3.  Gather / reshape / transpose: bit-exact."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from test_gemm_gpu import GOLD, TOL, _tdt, check, rand_bits, to_dev, to_host  # noqa: E402

ROW_SHAPES = [(64, 384), (33, 1000), (16, 4096), (5, 8192), (3, 10000), (7, 37), (1, 1), (300, 2048), (3100, 2048)]


@pytest.mark.parametrize("ring", [1, 0])
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_layer_norm(cuda, oracle, dt, ring):
    """`ring`: rows of a few KB through the shared-memory ring kernel (1, the default) or the register kernels (0)."""
    from nova_compiler_b200 import ops, _lib as L0
    L0.set_option("ring_rows", ring)
    try:
        _layer_norm_cases(cuda, oracle, dt)
    finally:
        L0.set_option("ring_rows", 1)


def _layer_norm_cases(cuda, oracle, dt):
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(1)
    for rows, D in ROW_SHAPES:
        x = rand_bits(oracle, rng, (rows, D), dt, "normal", 2.0)
        g = rand_bits(oracle, rng, (D,), dt, "normal")
        b = rand_bits(oracle, rng, (D,), dt, "normal")
        y, ms, rs = ops.layer_norm(to_dev(cuda, x, dt), to_dev(cuda, g, dt), to_dev(cuda, b, dt))
        wy, wms, wrs = oracle.layer_norm(x, g, b, dt, compute_f32=True)
        check(oracle, to_host(cuda, y, dt), wy, dt)
        check(oracle, to_host(cuda, ms, dt), wms, dt, tol=2e-3 if dt != "f32" else 1e-5)  # raw row sum
        check(oracle, to_host(cuda, rs, dt), wrs, dt)


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_softmax(cuda, oracle, dt):
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(2)
    for rows, D in ROW_SHAPES:
        x = rand_bits(oracle, rng, (rows, D), dt, "normal", 3.0)
        y = ops.softmax(to_dev(cuda, x, dt))
        check(oracle, to_host(cuda, y, dt), oracle.softmax(x, dt, compute_f32=True), dt)
    # rows of 4-32 KB, more of them than resident CTAs: the ring kernel refills its slots while rows are in flight
    for rows, D in [(2100, 4608), (1900, 2560)]:
        x = rand_bits(oracle, rng, (rows, D), dt, "normal", 3.0)
        y = ops.softmax(to_dev(cuda, x, dt))
        check(oracle, to_host(cuda, y, dt), oracle.softmax(x, dt, compute_f32=True), dt)
        assert ops.device_status() == 0
    # rows beyond the register cache: staged in shared memory (up to 220 KB) or read twice (longer).  The oracle adds
    # the exponentials one by one in fp32, which drifts ~4e-5 over such rows; f32 is also checked against float64.
    for rows, D in [(4, 50304), (2, 70000)]:
        x = rand_bits(oracle, rng, (rows, D), dt, "normal", 3.0)
        y = to_host(cuda, ops.softmax(to_dev(cuda, x, dt)), dt)
        check(oracle, y, oracle.softmax(x, dt, compute_f32=True), dt, tol=1e-4 if dt == "f32" else None)
        if dt == "f32":
            e = np.exp(x.astype(np.float64) - x.astype(np.float64).max(-1, keepdims=True))
            assert oracle.rel_fro(y, e / e.sum(-1, keepdims=True)) <= 2e-6
    # more vocabulary rows than SMs: every CTA of the streaming kernel takes several rows, so the chunks of its next
    # row are copied in over the row it is still writing; ragged last chunk (50304 * 4 B = 12 chunks + 4.6 KB).  Checked
    # against float64 on every row, and against the kernel that stages one row at a time.
    from nova_compiler_b200 import _lib as L
    for rows, D in [(470, 50304 if dt == "f32" else 100352), (301, 8200)]:
        x = rand_bits(oracle, rng, (rows, D), dt, "normal", 3.0)
        xd = to_dev(cuda, x, dt)
        y = ops.softmax(xd)
        xf = oracle.from_bits(x, dt).astype(np.float64)
        e = np.exp(xf - xf.max(-1, keepdims=True))
        assert oracle.rel_fro(oracle.from_bits(to_host(cuda, y, dt), dt), e / e.sum(-1, keepdims=True)) <= (2e-6 if dt == "f32" else 3e-3)
        assert ops.device_status() == 0
        L.set_option("ring_rows", 0)
        try:
            y0 = ops.softmax(xd)
        finally:
            L.set_option("ring_rows", 1)
        assert oracle.rel_fro(oracle.from_bits(to_host(cuda, y, dt), dt), oracle.from_bits(to_host(cuda, y0, dt), dt)) <= (1e-6 if dt == "f32" else 3e-3)
    # non-last dimension and the attention-score layout
    x = rand_bits(oracle, rng, (4, 96, 50), "f32", "normal")
    y = ops.softmax(to_dev(cuda, x, "f32"), dimension=1)
    want = np.swapaxes(oracle.softmax(np.ascontiguousarray(np.swapaxes(x, 1, 2))), 1, 2)
    check(oracle, to_host(cuda, y, "f32"), want, "f32")


def test_row_ops_golden_vectors(cuda, oracle):
    from nova_compiler_b200 import ops
    z = np.load(GOLD)
    y, ms, rs = ops.layer_norm(to_dev(cuda, z["layer_norm_f32.x"], "f32"), to_dev(cuda, z["layer_norm_f32.gamma"], "f32"),
                               to_dev(cuda, z["layer_norm_f32.beta"], "f32"))
    check(oracle, to_host(cuda, y, "f32"), z["layer_norm_f32.y"], "f32")
    check(oracle, to_host(cuda, ms, "f32"), z["layer_norm_f32.mean_sum"], "f32")
    check(oracle, to_host(cuda, rs, "f32"), z["layer_norm_f32.rstd"], "f32")
    check(oracle, to_host(cuda, ops.softmax(to_dev(cuda, z["softmax_f32.x"], "f32")), "f32"), z["softmax_f32.y"], "f32")
    out = ops.gather(cuda.from_numpy(z["gather_i16.table"]).cuda(), cuda.from_numpy(z["gather_i16.ids"]).cuda())
    assert np.array_equal(out.cpu().numpy(), z["gather_i16.out"])


def test_gather_bit_exact(cuda, oracle):
    torch = cuda
    from nova_compiler_b200 import ops
    g = torch.Generator(device="cuda"); g.manual_seed(5)
    # embedding lookup of ltest/test.mlir:17: [50304,384] table, [8,1024] i16 ids (zero-extended)
    table = torch.randn(50304, 384, device="cuda", generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 50304, (8, 1024), device="cuda", generator=g)
    out = ops.gather(table, ids.to(torch.int16))
    assert torch.equal(out, table[ids])
    want, bad = oracle.gather(to_host(torch, table, "bf16"), ids.cpu().numpy().astype(np.uint16).view(np.int16))
    assert bad == 0 and np.array_equal(to_host(torch, out, "bf16"), want)
    # odd row widths take the narrower copy units; i32 / i64 indices; axis 1 with batched indices
    for width, dt in ((33, torch.float32), (7, torch.float16), (5, torch.int8), (1, torch.float64)):
        t = torch.randint(-100, 100, (257, width), device="cuda", generator=g).to(dt)
        idx = torch.randint(0, 257, (3, 19), device="cuda", generator=g)
        assert torch.equal(ops.gather(t, idx.to(torch.int32)), t[idx])
        assert torch.equal(ops.gather(t, idx), t[idx])
    x = torch.randn(3, 10, 4, device="cuda", generator=g)
    idx = torch.randint(0, 10, (3, 5), device="cuda", generator=g).to(torch.int32)
    out = ops.gather(x, idx, axis=1)
    assert torch.equal(out, torch.stack([x[i, idx[i].long()] for i in range(3)]))
    # out-of-range indices: zero rows, counted
    out, bad = ops.gather(table[:10], torch.tensor([3, 10, -1], device="cuda"), return_bad_count=True)
    assert bad == 2 and torch.equal(out[0], table[3]) and not out[1:].any()


def test_reshape_and_transpose_are_metadata(cuda, oracle):
    torch = cuda
    from nova_compiler_b200 import ops
    x = torch.arange(8 * 1024 * 384, device="cuda", dtype=torch.float32).reshape(8, 1024, 384)
    r = ops.reshape(x, (8192, 384))  # ltest/test.mlir:26-28
    assert r.data_ptr() == x.data_ptr() and torch.equal(r.reshape(8, 1024, 384), x)
    with pytest.raises(Exception):
        ops.reshape(x, (8192, 385))
    t = ops.transpose(x)
    assert t.data_ptr() == x.data_ptr() and t.shape == (8, 384, 1024)
    # a transposed view feeding a matmul is consumed through trans_a, not copied
    a = torch.randn(64, 48, device="cuda")
    b = torch.randn(64, 40, device="cuda")
    got = ops.matmul(ops.transpose(a), b)
    want = oracle.gemm(np.ascontiguousarray(a.cpu().numpy()), b.cpu().numpy(), trans_a=True)
    check(oracle, got.cpu().numpy(), want, "f32")


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_activation_and_add(cuda, oracle, dt):
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(3)
    for shape in ((1000, 333), (64, 64), (7,)):
        x = rand_bits(oracle, rng, shape, dt, "normal", 2.0)
        check(oracle, to_host(cuda, ops.gelu(to_dev(cuda, x, dt)), dt), oracle.activation(x, dt, "gelu_tanh", True), dt)
        assert np.array_equal(to_host(cuda, ops.relu(to_dev(cuda, x, dt)), dt), oracle.activation(x, dt, "relu"))
    a = rand_bits(oracle, rng, (8, 10), dt)
    b = rand_bits(oracle, rng, (1, 10), dt)  # ltest/test_cpu.mlir: 8x10 + 1x10
    assert np.array_equal(to_host(cuda, ops.add(to_dev(cuda, a, dt), to_dev(cuda, b, dt)), dt),
                          oracle.add_rowbcast(a, b, dt))
    assert np.array_equal(to_host(cuda, ops.add(to_dev(cuda, a, dt), to_dev(cuda, a, dt)), dt),
                          oracle.add_rowbcast(a, a, dt))


def test_test_cpu_mlir_graph_unfused(cuda, oracle):
    """ltest/test_cpu.mlir as three separate ops (matmul, add, relu) equals the fused epilogue form."""
    from nova_compiler_b200 import ops
    z = np.load(GOLD)
    a, b, bias = (to_dev(cuda, z[f"test_cpu_mlir.{k}"], "f32") for k in ("a", "b", "bias"))
    unfused = ops.relu(ops.add(ops.matmul(a, b), bias.reshape(1, 10)))
    check(oracle, to_host(cuda, unfused, "f32"), z["test_cpu_mlir.c"], "f32")


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_column_sum_and_backward_ops(cuda, oracle, dt):
    """grad_bias of nova.linear_backward (column sum over batch*M rows) and the NT / TN contractions of
    nova.matmul_backward / nova.linear_backward, through the operator mirror."""
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(6)
    for rows, cols in ((8192, 1536), (777, 333), (5, 1), (1, 40)):
        x = rand_bits(oracle, rng, (rows, cols), dt, "normal")
        got = to_host(cuda, ops.column_sum(to_dev(cuda, x, dt)), dt)
        check(oracle, got, oracle.column_sum(x, dt), dt, tol=2e-3 if dt != "f32" else 1e-5)
    go = rand_bits(oracle, rng, (3, 40, 72), dt, "normal")
    x = rand_bits(oracle, rng, (3, 40, 56), dt, "normal")
    w = rand_bits(oracle, rng, (56, 72), dt, "normal", 0.1)
    gi, gw, gb = ops.linear_backward(to_dev(cuda, go, dt), to_dev(cuda, x, dt), to_dev(cuda, w, dt))
    check(oracle, to_host(cuda, gi, dt), oracle.gemm(go, np.ascontiguousarray(w.T), dtype_in=dt), dt)
    xf, gf = x.reshape(120, 56), go.reshape(120, 72)
    check(oracle, to_host(cuda, gw, dt), oracle.gemm(np.ascontiguousarray(xf.T), gf, dtype_in=dt), dt)
    check(oracle, to_host(cuda, gb, dt), oracle.column_sum(gf, dt), dt, tol=2e-3 if dt != "f32" else 1e-5)
    ga, gbm = ops.matmul_backward(to_dev(cuda, go[0], dt), to_dev(cuda, x[0], dt), to_dev(cuda, w, dt))
    check(oracle, to_host(cuda, ga, dt), oracle.gemm(go[0], np.ascontiguousarray(w.T), dtype_in=dt), dt)
    check(oracle, to_host(cuda, gbm, dt), oracle.gemm(np.ascontiguousarray(x[0].T), go[0], dtype_in=dt), dt)


@pytest.mark.parametrize("ring", [1, 2, 0])
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_layer_norm_backward(cuda, oracle, dt, ring):
    """dx, dgamma, dbeta from the saved (mean_sum, rstd) of the forward; vectorised and element-wise row shapes,
    one to many rows per CTA; fp32 arithmetic rounded once, as the oracle's compute_f32 mode.  `ring`: the default
    kernels (1), the shared-memory-ring backward kernel as well (2), register kernels only (0)."""
    from nova_compiler_b200 import ops, _lib as L0
    L0.set_option("ring_rows", ring)
    try:
        _layer_norm_backward_cases(cuda, oracle, dt)
    finally:
        L0.set_option("ring_rows", 1)


def _layer_norm_backward_cases(cuda, oracle, dt):
    from nova_compiler_b200 import ops
    rng = np.random.default_rng(6)
    for rows, D in [(64, 384), (8192, 384), (33, 1000), (700, 4096), (5, 8192), (7, 37), (1, 1), (300, 2048), (40, 16384)]:
        if dt == "f32" and D > 8192:
            continue  # beyond 2048 sixteen-byte vectors: refused (checked below)
        x = rand_bits(oracle, rng, (rows, D), dt, "normal", 2.0)
        g = rand_bits(oracle, rng, (D,), dt, "normal")
        b = rand_bits(oracle, rng, (D,), dt, "normal")
        gy = rand_bits(oracle, rng, (rows, D), dt, "normal")
        _, ms, rs = oracle.layer_norm(x, g, b, dt, compute_f32=True)
        dx, dg, db = ops.layer_norm_backward(to_dev(cuda, gy, dt), to_dev(cuda, x, dt), to_dev(cuda, g, dt),
                                             to_dev(cuda, ms, dt), to_dev(cuda, rs, dt))
        wdx, wdg, wdb = oracle.layer_norm_backward(gy, x, g, ms, rs, dt, compute_f32=True)
        check(oracle, to_host(cuda, dx, dt), wdx, dt)
        # column sums over `rows` terms: fp32 on both sides, summation order differs
        check(oracle, to_host(cuda, dg, dt), wdg, dt, tol=2e-3 if dt != "f32" else 2e-5)
        check(oracle, to_host(cuda, db, dt), wdb, dt, tol=2e-3 if dt != "f32" else 2e-5)
    # zero rows: the column sums are zeros, nothing else is touched
    z = cuda.zeros(0, 64, device="cuda")
    dx, dg, db = ops.layer_norm_backward(z, z, cuda.ones(64, device="cuda"), cuda.zeros(0, device="cuda"), cuda.zeros(0, device="cuda"))
    assert dx.shape == (0, 64) and float(dg.abs().sum()) == 0.0 and float(db.abs().sum()) == 0.0
    from nova_compiler_b200 import _lib as L
    big = cuda.zeros(2, 8192 + 4, device="cuda")
    with pytest.raises(L.NovaB200Error) as e:
        ops.layer_norm_backward(big, big, cuda.ones(8196, device="cuda"), cuda.zeros(2, device="cuda"), cuda.ones(2, device="cuda"))
    assert e.value.status == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_sce_forward_and_backward(cuda, oracle, dt):
    """nova.sce / nova.sce_backward over the last dim: softmax, mean loss and gradient against the oracle (fp32
    arithmetic rounded once on both sides); short, vector-friendly and vocabulary-sized rows; i16 targets above
    32767 (zero-extended) and an out-of-range target."""
    from nova_compiler_b200 import ops
    torch = cuda
    rng = np.random.default_rng(8)
    for rows, C, it in [(64, 10, np.int32), (33, 1000, np.int64), (24, 50304, np.uint16), (7, 37, np.int32), (300, 2048, np.int64)]:
        x = rand_bits(oracle, rng, (rows, C), dt, "normal", 3.0)
        t = rng.integers(0, C, size=rows).astype(it)
        t_dev = torch.from_numpy(t.view(np.int16) if it == np.uint16 else t).cuda()
        sm, loss = ops.sce(to_dev(torch, x, dt), t_dev)
        wsm, wloss, bad = oracle.sce(x, t.view(np.int16) if it == np.uint16 else t, dt, compute_f32=True)
        assert bad == 0
        # The oracle adds the C exponentials one after the other in fp32, as the reference's reduction does; over a
        # 50304-term row that running sum is itself ~4e-5 off.  The kernel's tree sum is checked against float64 too.
        long_row = dt == "f32" and C > 16384
        check(oracle, to_host(torch, sm, dt), wsm, dt, tol=1e-4 if long_row else None)
        check(oracle, to_host(torch, loss, dt), wloss, dt, tol=2e-3 if dt != "f32" else 1e-5)
        if dt == "f32":
            x64 = x.astype(np.float64)
            e = np.exp(x64 - x64.max(-1, keepdims=True))
            assert oracle.rel_fro(to_host(torch, sm, dt), e / e.sum(-1, keepdims=True)) <= 2e-6
        g = ops.sce_backward(sm, t_dev)
        wg = oracle.sce_backward(to_host(torch, sm, dt), t.view(np.int16) if it == np.uint16 else t, dt, compute_f32=True)
        check(oracle, to_host(torch, g, dt), wg, dt, tol=TOL[dt] if dt != "f32" else 1e-6)
        # the loss gradient's scalar folded into the same pass: the oracle's gradient times that scalar, rounded once
        gs = ops.sce_backward(sm, t_dev, scale=-2.5)
        pf = oracle.from_bits(to_host(torch, sm, dt), dt).astype(np.float32).reshape(rows, C)
        pf[np.arange(rows), t.astype(np.int64)] -= np.float32(1.0)
        want = oracle.to_bits((pf * (np.float32(1.0 / rows) * np.float32(-2.5))).reshape(sm.shape), dt)
        check(oracle, to_host(torch, gs, dt), want, dt, tol=TOL[dt] if dt != "f32" else 1e-6)
    # an out-of-range target: counted, contributes x[target] = 0
    x = rand_bits(oracle, rng, (5, 16), dt, "normal")
    t = np.array([1, 99, 3, 0, 15], dtype=np.int32)
    sm, loss, bad = ops.sce(to_dev(torch, x, dt), torch.from_numpy(t).cuda(), return_bad_count=True)
    wsm, wloss, wbad = oracle.sce(x, t, dt, compute_f32=True)
    assert bad == wbad == 1
    check(oracle, to_host(torch, loss, dt), wloss, dt, tol=2e-3 if dt != "f32" else 1e-5)


def test_scatter_add(cuda, oracle):
    """out = input; out[.., idx[i], ..] += src[.., i, ..]: unique indices compare bit for bit, repeated indices (atomics,
    unspecified order) within fp32 rounding; out-of-range indices are skipped and counted."""
    from nova_compiler_b200 import ops
    torch = cuda
    rng = np.random.default_rng(12)
    inp = rng.normal(size=(500, 96)).astype(np.float32)
    idx = rng.permutation(500)[:128].astype(np.int32)
    src = rng.normal(size=(128, 96)).astype(np.float32)
    out = ops.scatter_add(torch.from_numpy(inp).cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(src).cuda(), 0)
    want, _ = oracle.scatter_add(inp, idx, src, 0)
    assert np.array_equal(out.cpu().numpy(), want)  # the embedding-gradient form of nova.gather's backward
    # repeated + out-of-range indices, middle axis, i16 indices
    inp = rng.normal(size=(3, 40, 8)).astype(np.float32)
    idx = np.array([5, 5, 5, 39, 0, 200, 7, 5], dtype=np.int16)
    src = rng.normal(size=(3, 8, 8)).astype(np.float32)
    out, bad = ops.scatter_add(torch.from_numpy(inp).cuda(), torch.from_numpy(idx).cuda(), torch.from_numpy(src).cuda(), 1,
                               return_bad_count=True)
    want, wbad = oracle.scatter_add(inp, idx, src, 1)
    assert bad == 3 and wbad == 3  # one bad index, seen once per leading slice
    assert oracle.rel_fro(out.cpu().numpy(), want) <= 1e-6
    # the flat form nova.sce_backward lowers to: -1 at row * C + target
    p = rng.random(size=(6 * 10,)).astype(np.float32)
    flat = (np.arange(6) * 10 + rng.integers(0, 10, size=6)).astype(np.int64)
    out = ops.scatter_add(torch.from_numpy(p).cuda(), torch.from_numpy(flat).cuda(), torch.full((6,), -1.0, device="cuda"), 0)
    want, _ = oracle.scatter_add(p, flat, np.full(6, -1.0, np.float32), 0)
    assert np.array_equal(out.cpu().numpy(), want)
    for dt in ("f16", "bf16"):
        a = rand_bits(oracle, rng, (50, 16), dt)
        s = rand_bits(oracle, rng, (20, 16), dt)
        ix = rng.permutation(50)[:20].astype(np.int32)
        out = ops.scatter_add(to_dev(torch, a, dt), torch.from_numpy(ix).cuda(), to_dev(torch, s, dt), 0)
        want, _ = oracle.scatter_add(a, ix, s, 0, dt)
        assert np.array_equal(to_host(torch, out, dt), want)
