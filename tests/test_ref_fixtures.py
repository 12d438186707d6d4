"""The front-end against the reference's OWN .mlir inputs (tests/golden/ref_fixtures/, copied by
tests/golden/copy_ref_fixtures.py from test/pipeline-tests/, ltest/ and test/ of the reference; ltest/test.mlir with
three statements brought up to today's op definitions, see that script).

CPU: every fixture parses, every function plans, and the plans show the fusions FuseMatmulBias and the epilogue
classification would make.  GPU: the contraction fixtures run and match the CPU oracle (f32 through 3xTF32:
relative Frobenius <= 1e-5); the MLP training step (ltest/testing.mlir) and the whole GPT step (ltest/test.mlir,
full size: 8 x 1024 tokens, vocabulary 50304) match float64 autograd of the same graph within 1e-4 / 2e-4 relative
Frobenius (f32 graphs; the contractions run as 3xTF32).
"""
import glob
import os
import re

import numpy as np
import pytest

from nova_compiler_b200.frontend import Module

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_fixtures")


def _text(name):
    return open(os.path.join(FIX, name)).read()


def _functions(text):
    code = re.sub(r"//[^\n]*", "", text)
    return re.findall(r"func\.func\s+(?:private\s+)?@([\w$.-]+)", code)


def test_every_fixture_parses_and_plans():
    files = sorted(glob.glob(os.path.join(FIX, "*.mlir")))
    assert len(files) == 30
    n_funcs = 0
    for f in files:
        text = open(f).read()
        m = Module(text)  # raises with the line number on a parse or inference error
        for fn in _functions(text):
            plan = m.plan(fn)
            assert plan.startswith(f"func @{fn}(") and "return" in plan
            m.signature(fn)
            n_funcs += 1
    assert n_funcs >= 45


def test_plans_of_the_pipeline_tests_show_the_reference_fusions():
    # linalg.generic bias / ReLU consumers fold into the contraction (FuseMatmulBias.cpp:95-193 + isEpilogue)
    p = Module(_text("test__pipeline-tests__04_matmul_bias_fusion.mlir")).plan("matmul_plus_bias")
    assert p.count("gemm") == 1 and "init=residual(%bias) act=none" in p and "fill" not in p
    p = Module(_text("test__pipeline-tests__05_matmul_bias_relu.mlir")).plan("matmul_bias_relu")
    assert p.count("gemm") == 1 and "init=residual(%bias) act=relu" in p and "[linalg.matmul + nova.add + nova.relu]" in p
    # a live accumulator (outs is an argument), a row-broadcast bias through `#map1 = (d0, d1) -> (d1)`, then ReLU
    p = Module(_text("test__pipeline-tests__13_matmul_bias_relu.mlir")).plan("matmul_bias_relu")
    assert "init=bias_row(%arg2)+residual(%arg3) act=relu" in p and p.count("gemm") == 1
    p = Module(_text("test__pipeline-tests__mlp_2layer.mlir")).plan("mlp_2layer")
    assert p.count("gemm") == 2 and "init=residual(%b1) act=relu" in p and "init=residual(%b2) act=none" in p
    # multi-line `ins(...) outs(...)` with a live C: 01, 02, 03, 06
    for name, fn in [("01_matmul_non_aligned", "matmul_non_aligned"), ("02_matmul_aligned", "matmul_aligned"),
                     ("03_batch_matmul", "batch_matmul"), ("06_matmul_exact_tile", "matmul_exact_tile")]:
        assert "gemm init=residual(%C) act=none" in Module(_text(f"test__pipeline-tests__{name}.mlir")).plan(fn)


def test_plan_of_the_gpt_step():
    p = Module(_text("ltest__test.mlir")).plan("main")
    assert "gemm init=bias_row(%10)+residual(%16) act=none" in p          # FFN-down + bias + residual in one epilogue
    assert "act=gelu_tanh_grad(%18)" in p                                   # grad_input of FFN-down x gelu'(pre-activation)
    kinds = [line.split()[0] for line in p.splitlines()[1:]]
    assert kinds.count("gemm") == 9 and kinds.count("layer_norm_backward") == 2 and kinds.count("scatter_add") == 2
    assert "reduce_sum (%37)" in p and kinds.count("store_to_arg") == 12
    assert "[nova.sce_backward + nova.mul by %27]" in p   # the loss gradient's scalar joins the pass that writes dlogits
    p = Module(_text("ltest__testing.mlir")).plan("main")
    kinds = [line.split()[0] for line in p.splitlines()[1:]]
    assert "gemm init=bias_row(%6) act=none" in p and kinds.count("reduce_sum") == 4 and "compare" in kinds and "mse" in kinds
    p = Module(_text("ltest__6otherops.mlir")).plan("matmul_4d")
    assert "tensor<2x4x8x32xf32>" in p


# ---------------------------------------------------------------------------------------------- GPU

def _rand(torch, g, shape):
    return torch.rand(shape, device="cuda", generator=g) * 2 - 1


def _np(t):
    return t.detach().contiguous().cpu().numpy()


@pytest.mark.gpu
def test_pipeline_test_fixtures_match_the_oracle(cuda, oracle):
    torch = cuda
    g = torch.Generator(device="cuda")
    g.manual_seed(2024)
    relu = lambda x: np.maximum(x, 0)
    # fixture, function, expected(args as numpy) using the CPU oracle
    table = [
        ("01_matmul_non_aligned", "matmul_non_aligned", lambda a, b, c: oracle.gemm(a, b, residual=c)),
        ("02_matmul_aligned", "matmul_aligned", lambda a, b, c: oracle.gemm(a, b, residual=c)),
        ("03_batch_matmul", "batch_matmul", lambda a, b, c: oracle.gemm(a, b, residual=c)),
        ("04_matmul_bias_fusion", "matmul_plus_bias", lambda a, b, bias: oracle.gemm(a, b, residual=bias)),
        ("05_matmul_bias_relu", "matmul_bias_relu", lambda a, b, bias: oracle.gemm(a, b, residual=bias, act="relu")),
        ("06_matmul_exact_tile", "matmul_exact_tile", lambda a, b, c: oracle.gemm(a, b, residual=c)),
        ("07_k_tiling_reduction", "k_tiling_test", lambda a, b, bias: oracle.gemm(a, b, residual=bias)),
        ("13_matmul_bias_relu", "matmul_bias_relu",
         lambda a, b, bias, c: relu(oracle.gemm(a, b, residual=c) + bias[None, :]).astype(np.float32)),
        ("mlp_2layer", "mlp_2layer",
         lambda x, w1, b1, w2, b2: oracle.gemm(oracle.gemm(x, w1, residual=b1, act="relu"), w2, residual=b2)),
    ]
    for name, fn, expect in table:
        m = Module(_text(f"test__pipeline-tests__{name}.mlir"))
        arg_sig, _ = m.signature(fn)
        args = [_rand(torch, g, shape) for _, shape in arg_sig]
        got, = m.run(fn, *args)
        torch.cuda.synchronize()
        want = expect(*[_np(a) for a in args])
        err = oracle.rel_fro(_np(got), want)
        assert err <= 2e-5, f"{name}: rel-Frobenius {err:.3e}"


@pytest.mark.gpu
def test_other_ops_fixture_matches_the_oracle(cuda, oracle):
    torch = cuda
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    m = Module(_text("ltest__6otherops.mlir"))
    a, b = _rand(torch, g, (4, 8)), _rand(torch, g, (8, 16))
    mm, tr = m.run("matrix_operations", a, b)
    assert oracle.rel_fro(_np(mm), oracle.gemm(_np(a), _np(b))) <= 1e-5 and torch.equal(tr, a.t())
    a3, b3 = _rand(torch, g, (4, 8, 16)), _rand(torch, g, (4, 16, 32))
    r3, = m.run("matmul_3d", a3, b3)
    assert oracle.rel_fro(_np(r3), oracle.gemm(_np(a3), _np(b3))) <= 1e-5
    a4, b4 = _rand(torch, g, (2, 4, 8, 16)), _rand(torch, g, (2, 4, 16, 32))
    r4, = m.run("matmul_4d", a4, b4)   # rank > 3: batch dims collapse to one, contraction, expand (NovaToLinalg.cpp:904-989)
    want = oracle.gemm(_np(a4).reshape(8, 8, 16), _np(b4).reshape(8, 16, 32)).reshape(2, 4, 8, 32)
    assert oracle.rel_fro(_np(r4), want) <= 1e-5
    # test/matmul_test.mlir: tensor.collapse_shape + nova.matmul + tensor.expand_shape
    mt = Module(_text("test__matmul_test.mlir"))
    x, w = _rand(torch, g, (8, 128, 768)), _rand(torch, g, (768, 768))
    y, = mt.run("matmul", x, w)
    assert oracle.rel_fro(_np(y).reshape(1024, 768), oracle.gemm(_np(x).reshape(1024, 768), _np(w))) <= 1e-5


@pytest.mark.gpu
def test_mlp_training_step_fixture_matches_float64_autograd(cuda):
    """ltest/testing.mlir: forward of a 2-layer MLP, MSE loss, and hand-derived gradients (transposes, broadcast
    multiplies, compare + cast as the ReLU mask, reduce<sum> over leading dims)."""
    torch = cuda
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    m = Module(_text("ltest__testing.mlir"))
    arg_sig, _ = m.signature("main")
    args = [_rand(torch, g, shape) for _, shape in arg_sig]
    x, tgt, scale, gout, thresh, w1, b1, w2, b2 = args[:9]
    m.run("main", *args)
    torch.cuda.synchronize()
    d = torch.float64
    h = x.to(d) @ w1.to(d) + b1.to(d)                      # %9, %10
    a = torch.relu(h)                                      # %11
    out = a @ w2.to(d) + b2.to(d)                          # %12, %13
    loss = ((out - tgt.to(d)) ** 2).mean()                 # %14
    g17 = (out - tgt.to(d)) * gout.to(d) * scale.to(d)     # %15..%17
    g_b2 = g17.sum(dim=(0, 1))                             # %18
    g_a = g17 @ w2.to(d).t()                               # %19, %20
    g_w2 = (a.transpose(1, 2) @ g17).sum(dim=0)            # %21..%23
    mask = (h > thresh.to(d)).to(d)                        # %24, %25
    g_h = g_a * mask                                       # %26
    g_b1 = g_h.sum(dim=(0, 1))                             # %27
    g_w1 = (x.to(d).transpose(1, 2) @ g_h).sum(dim=0)      # %28..%30

    def rel(got, want):
        return float((got.to(d).reshape(-1) - want.reshape(-1)).norm() / want.norm())

    assert rel(args[9], loss.reshape(1)) <= 1e-5
    assert rel(args[10], g_w1) <= 1e-4 and rel(args[11], g_b1) <= 1e-4
    assert rel(args[12], g_w2) <= 1e-4 and rel(args[13], g_b2) <= 1e-4


@pytest.mark.gpu
def test_gpt_step_fixture_matches_float64_autograd(cuda):
    """ltest/test.mlir at its own size: embedding + position gather, pre-norm FFN block with residual, final layer
    norm, the 8192 x 384 x 50304 vocabulary contraction, sparse cross entropy, and the whole backward down to the
    embedding scatter-adds; every gradient is accumulated in place into its writable argument."""
    torch = cuda
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    m = Module(_text("ltest__test.mlir"))
    arg_sig, _ = m.signature("main")
    V, T, D, H = 50304, 1024, 384, 1536
    args = []
    for i, (dt, shape) in enumerate(arg_sig):
        if i in (0, 1):      # token ids / targets, i16 zero-extended: the whole vocabulary is reachable
            args.append(torch.randint(0, V, shape, device="cuda", generator=g).to(torch.int16))
        elif i in (2, 15):   # positions, i64
            args.append(torch.arange(T, device="cuda", dtype=torch.int64).reshape(shape))
        elif i in (3, 4, 7, 9, 13):   # embedding tables and weights: small, as initialised weights are
            args.append(_rand(torch, g, shape) * 0.05)
        elif i in (5, 11):   # layer-norm gains
            args.append(1.0 + 0.1 * _rand(torch, g, shape))
        elif i < 14:         # biases, layer-norm shifts
            args.append(0.1 * _rand(torch, g, shape))
        else:                # the loss slot and the gradient accumulators (the graph ADDS into them)
            args.append(torch.zeros(shape, device="cuda"))
    m.run("main", *args)
    torch.cuda.synchronize()
    first = {i: args[i].clone() for i in range(16, 27)}
    m.run("main", *args)     # a second step with the same inputs: every accumulator now holds twice the gradient
    torch.cuda.synchronize()

    d = torch.float64
    ids = args[0].to(torch.int64) & 0xFFFF
    tg = (args[1].to(torch.int64) & 0xFFFF).reshape(-1)
    leaf = {i: args[i].to(d).requires_grad_(True) for i in (3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13)}
    x = leaf[3][ids] + leaf[4][args[2].reshape(-1)][None]
    ln = torch.nn.functional.layer_norm
    h = ln(x, (D,), leaf[5], leaf[6], eps=1e-5)
    u = h @ leaf[7] + leaf[8]
    v = torch.nn.functional.gelu(u, approximate="tanh") @ leaf[9] + leaf[10]
    r = x + v
    z = ln(r, (D,), leaf[11], leaf[12], eps=1e-5)
    logits = z.reshape(8 * T, D) @ leaf[13]
    loss = torch.nn.functional.cross_entropy(logits, tg)
    loss.backward()

    def rel(got, want):
        return float((got.to(d).reshape(-1) - want.reshape(-1)).norm() / want.norm())

    assert rel(args[14], loss.detach().reshape(1)) <= 1e-5
    # writable argument += gradient of the matching weight (test.mlir:56-91)
    pairs = {16: 3, 17: 4, 18: 5, 19: 6, 20: 7, 21: 8, 22: 9, 23: 10, 24: 11, 25: 12, 26: 13}
    for out_i, w_i in pairs.items():
        err = rel(first[out_i], leaf[w_i].grad)
        assert err <= 2e-4, f"gradient written to argument {out_i} (of argument {w_i}): rel-Frobenius {err:.3e}"
        err2 = rel(args[out_i], 2 * leaf[w_i].grad)
        assert err2 <= 2e-4, f"argument {out_i} after two steps is not twice the gradient: {err2:.3e}"
