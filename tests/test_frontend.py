"""The textual front-end (nova_b200_module_*): the stand-in for the MLIR lowering pass.

CPU part: parsing, shape inference and fusion planning of modules written in the reference's textual forms
(the op syntax of ltest/*.mlir and test/pipeline-tests/*.mlir; shapes here are this test's own).
GPU part: the planned calls run and match the CPU oracle applied op by op."""
import numpy as np
import pytest

from nova_compiler_b200 import _lib as L
from nova_compiler_b200.frontend import Module

MLP = '''
module {
  func.func @main(%arg0: tensor<24x40xf32, #nova.device<"1">>,
      %arg1: tensor<40x56xf32, #nova.device<"1">>,
      %arg2: tensor<1x56xf32>) -> tensor<24x56xf32> {
    %0 = nova.matmul %arg0, %arg1 : tensor<24x40xf32,#nova.device<"1">>, tensor<40x56xf32,#nova.device<"1">>
    %1 = nova.add %0, %arg2 : tensor<24x56xf32>, tensor<1x56xf32>
    %2 = nova.relu %1 : tensor<24x56xf32>
    return %2 : tensor<24x56xf32>
  }
}
'''

BLOCK = '''
func.func @block(%x: tensor<2x48x64xbf16>, %g: tensor<64xbf16>, %b: tensor<64xbf16>, %w1: tensor<64x136xbf16>,
                 %b1: tensor<136xbf16>, %w2: tensor<136x64xbf16>, %b2: tensor<64xbf16>)
    -> (tensor<2x48x64xbf16>, tensor<2x48x48xbf16>) attributes { llvm.emit_c_interface } {
  %ln, %sum, %rstd = nova.layer_norm %x, %g, %b : tensor<2x48x64xbf16>, tensor<64xbf16>, tensor<64xbf16>
  %h = nova.linear %ln, %w1, %b1 : tensor<2x48x64xbf16>, tensor<64x136xbf16>, tensor<136xbf16>
  %a = nova.gelu %h : tensor<2x48x136xbf16>
  %o = nova.linear %a, %w2, %b2 : tensor<2x48x136xbf16>, tensor<136x64xbf16>, tensor<64xbf16>
  %r = nova.add %o, %x : tensor<2x48x64xbf16>, tensor<2x48x64xbf16>
  %t = nova.transpose %ln axes1 = 2 axes2 = 1 : tensor<2x48x64xbf16>
  %s = nova.matmul %ln, %t : tensor<2x48x64xbf16>, tensor<2x64x48xbf16>
  %p = nova.softmax %s : tensor<2x48x48xbf16>
  return %r, %p : tensor<2x48x64xbf16>, tensor<2x48x48xbf16>
}
'''

LINALG = '''
func.func @la(%A: tensor<100x300xf32>, %B: tensor<300x200xf32>, %bias: tensor<100x200xf32>) -> tensor<100x200xf32> {
  %cst = arith.constant 0.000000e+00 : f32
  %e = tensor.empty() : tensor<100x200xf32>
  %f = linalg.fill ins(%cst : f32) outs(%e : tensor<100x200xf32>) -> tensor<100x200xf32>
  %r = linalg.matmul ins(%A, %B : tensor<100x300xf32>, tensor<300x200xf32>) outs(%f : tensor<100x200xf32>) -> tensor<100x200xf32>
  // the FuseMatmulBias output form: the bias IS the matmul's outs
  %q = linalg.matmul ins(%A, %B : tensor<100x300xf32>, tensor<300x200xf32>) outs(%bias : tensor<100x200xf32>) -> tensor<100x200xf32>
  %s = nova.add %r, %q : tensor<100x200xf32>, tensor<100x200xf32>
  return %s : tensor<100x200xf32>
}
func.func @bmm(%A: tensor<4x64x256xf16>, %B: tensor<4x256x64xf16>, %out: memref<4x64x64xf16, 1>) {
  %cst = arith.constant 0.0 : f16
  %e = tensor.empty() : tensor<4x64x64xf16>
  %f = linalg.fill ins(%cst : f16) outs(%e : tensor<4x64x64xf16>) -> tensor<4x64x64xf16>
  %r = linalg.batch_matmul ins(%A, %B : tensor<4x64x256xf16>, tensor<4x256x64xf16>) outs(%f : tensor<4x64x64xf16>) -> tensor<4x64x64xf16>
  bufferization.materialize_in_destination %r in writable %out : (tensor<4x64x64xf16>, memref<4x64x64xf16, 1>) -> ()
  return
}
'''

EMBED = '''
func.func @embed(%table: tensor<500x96xf32>, %ids: tensor<8x16xi16>) -> tensor<128x96xf32> {
  %0 = nova.gather %table [%ids] axis = 0 : tensor<500x96xf32>, tensor<8x16xi16> -> tensor<8x16x96xf32>
  %1 = nova.reshape %0 : tensor<8x16x96xf32> -> tensor<128x96xf32>
  %2 = nova.to_device %1 : tensor<128x96xf32> -> tensor<128x96xf32, #nova.device<"1">>
  return %2 : tensor<128x96xf32>
}
'''


def test_plan_fuses_bias_and_activation_into_one_call():
    m = Module(MLP)
    plan = m.plan("main")
    assert plan.count("gemm") == 1 and "init=bias_row(%arg2)" in plan and "act=relu" in plan
    assert "[nova.matmul + nova.add + nova.relu]" in plan
    args, res = m.signature("main")
    assert args == [(L.F32, (24, 40)), (L.F32, (40, 56)), (L.F32, (1, 56))] and res == [(L.F32, (24, 56))]


def test_plan_of_a_transformer_style_block():
    m = Module(BLOCK)
    plan = m.plan("block")
    lines = [l.strip() for l in plan.splitlines()]
    assert lines[1].startswith("layer_norm")
    assert "gemm init=bias_row(%b1) act=gelu_tanh" in lines[2] and "nova.linear + nova.gelu" in lines[2]
    # the residual add after the second linear joins its bias in one epilogue ("out + x + b_down")
    assert "gemm init=bias_row(%b2)+residual(%x) act=none" in lines[3] and "nova.linear + nova.add" in lines[3]
    assert lines[4].startswith("transpose") and lines[5].startswith("gemm init=zero") and lines[6].startswith("softmax")
    _, res = m.signature("block")
    assert res == [(L.BF16, (2, 48, 64)), (L.BF16, (2, 48, 48))]


def test_plan_of_linalg_forms():
    m = Module(LINALG)
    plan = m.plan("la")
    assert "fill" not in plan  # the zero fill is folded into the contraction
    assert "gemm init=zero act=none (%A, %B) -> (%r" in plan
    assert "gemm init=residual(%bias) act=none (%A, %B) -> (%q" in plan
    plan = m.plan("bmm")
    assert "gemm init=zero" in plan and "store_to_arg (%r, %out)" in plan
    assert m.signature("bmm")[1] == []


def test_errors_are_reported_with_line_numbers(lib):
    import ctypes as C
    h = C.c_void_p()

    def parse(text):
        st = lib.nova_b200_module_parse(text.encode(), C.byref(h))
        return st, lib.nova_b200_last_error_string().decode()

    st, msg = parse(MLP.replace("tensor<40x56xf32, #nova.device<\"1\">>,", "tensor<41x56xf32>,"))
    assert st == L.ERR_UNSUPPORTED and "contraction dims differ: 40 vs 41" in msg and "line" in msg
    st, msg = parse("func.func @f(%a: tensor<4x4xf32>) -> tensor<4x4xf32> {\n %0 = nova.sin %a : tensor<4x4xf32>\n return %0 : tensor<4x4xf32>\n}")
    assert st == L.ERR_UNSUPPORTED and "nova.sin" in msg and "outside the supported subset" in msg
    st, msg = parse("func.func @f(%a: tensor<?x4xf32>) -> tensor<4x4xf32> {\n return %a : tensor<4x4xf32>\n}")
    assert st == L.ERR_INVALID_ARG and "dynamic shapes" in msg
    st, msg = parse("func.func @f(%a: tensor<4x4xf32>) -> tensor<2x9xf32> {\n %0 = nova.reshape %a : tensor<4x4xf32> -> tensor<2x9xf32>\n return %0 : tensor<2x9xf32>\n}")
    assert st == L.ERR_UNSUPPORTED and "element counts differ" in msg
    st, msg = parse("this is not IR")
    assert st == L.ERR_INVALID_ARG
    assert lib.nova_b200_module_parse(None, C.byref(h)) == L.ERR_INVALID_ARG


# ---------------------------------------------------------------------------------------------- GPU

def _bits(torch, t):
    t = t.contiguous().cpu()
    return t.numpy() if t.dtype == torch.float32 else t.view(torch.int16).numpy().view(np.uint16)


@pytest.mark.gpu
def test_run_mlp_matches_oracle(cuda, oracle):
    torch = cuda
    g = torch.Generator(device="cuda"); g.manual_seed(1)
    a = torch.rand(24, 40, device="cuda", generator=g) * 2 - 1
    b = torch.rand(40, 56, device="cuda", generator=g) * 2 - 1
    bias = torch.rand(1, 56, device="cuda", generator=g) * 2 - 1
    y, = Module(MLP).run("main", a, b, bias)
    want = oracle.gemm(a.cpu().numpy(), b.cpu().numpy(), bias=bias.cpu().numpy().reshape(-1), act="relu")
    assert oracle.rel_fro(y.cpu().numpy(), want) <= 1e-5


@pytest.mark.gpu
def test_run_block_matches_oracle_op_by_op(cuda, oracle):
    torch = cuda
    g = torch.Generator(device="cuda"); g.manual_seed(2)
    bf = torch.bfloat16
    mk = lambda *s, sc=1.0: (torch.randn(*s, device="cuda", generator=g) * sc).to(bf)
    x, gm, bt = mk(2, 48, 64), mk(64), mk(64)
    w1, b1, w2, b2 = mk(64, 136, sc=0.1), mk(136, sc=0.1), mk(136, 64, sc=0.1), mk(64, sc=0.1)
    r, p = Module(BLOCK).run("block", x, gm, bt, w1, b1, w2, b2)
    B = lambda t: _bits(torch, t)
    ln, _, _ = oracle.layer_norm(B(x), B(gm), B(bt), "bf16", compute_f32=True)
    h = oracle.gemm(ln, B(w1), dtype_in="bf16", bias=B(b1), act="gelu_tanh")
    want_r = oracle.gemm(h, B(w2), dtype_in="bf16", bias=B(b2), residual=B(x))
    s = oracle.gemm(ln, np.ascontiguousarray(np.swapaxes(ln, 1, 2)), dtype_in="bf16")
    want_p = oracle.softmax(s, "bf16", compute_f32=True)
    f = lambda bits: oracle.from_bits(bits, "bf16")
    assert oracle.rel_fro(f(B(r)), f(want_r)) <= 4e-3   # three chained bf16 roundings
    assert oracle.rel_fro(f(B(p)), f(want_p)) <= 4e-3


@pytest.mark.gpu
def test_run_linalg_forms_and_output_argument(cuda, oracle):
    torch = cuda
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    A = torch.rand(100, 300, device="cuda", generator=g) * 2 - 1
    Bm = torch.rand(300, 200, device="cuda", generator=g) * 2 - 1
    bias = torch.rand(100, 200, device="cuda", generator=g) * 2 - 1
    m = Module(LINALG)
    s, = m.run("la", A, Bm, bias)
    ab = oracle.gemm(A.cpu().numpy(), Bm.cpu().numpy())
    abq = oracle.gemm(A.cpu().numpy(), Bm.cpu().numpy(), residual=bias.cpu().numpy())
    assert oracle.rel_fro(s.cpu().numpy(), ab + abq) <= 1e-5
    a16 = (torch.randn(4, 64, 256, device="cuda", generator=g) / 16).to(torch.float16)
    b16 = (torch.randn(4, 256, 64, device="cuda", generator=g) / 16).to(torch.float16)
    out = torch.zeros(4, 64, 64, device="cuda", dtype=torch.float16)
    assert m.run("bmm", a16, b16, out) == []
    want = oracle.gemm(_bits(torch, a16), _bits(torch, b16), dtype_in="f16")
    assert oracle.rel_fro(oracle.from_bits(_bits(torch, out), "f16"), oracle.from_bits(want, "f16")) <= 1e-3


@pytest.mark.gpu
def test_run_embedding_is_bit_exact(cuda, oracle):
    torch = cuda
    g = torch.Generator(device="cuda"); g.manual_seed(4)
    table = torch.randn(500, 96, device="cuda", generator=g)
    ids = torch.randint(0, 500, (8, 16), device="cuda", generator=g).to(torch.int16)
    y, = Module(EMBED).run("embed", table, ids)
    assert torch.equal(y, table[ids.long()].reshape(128, 96))


BACKWARD = '''
func.func @bw(%go: tensor<4x24x40xf32>, %x: tensor<4x24x56xf32>, %w: tensor<56x40xf32>,
              %g2: tensor<24x40xf32>, %a: tensor<24x56xf32>, %b: tensor<56x40xf32>)
    -> (tensor<4x24x56xf32>, tensor<56x40xf32>, tensor<40xf32>, tensor<24x56xf32>, tensor<56x40xf32>) {
  %gi, %gw, %gb = nova.linear_backward %go, %x, %w : tensor<4x24x40xf32>, tensor<4x24x56xf32>, tensor<56x40xf32>
  %ga, %gbm = nova.matmul_backward %g2, %a, %b : tensor<24x40xf32>, tensor<24x56xf32>, tensor<56x40xf32>
  return %gi, %gw, %gb, %ga, %gbm : tensor<4x24x56xf32>, tensor<56x40xf32>, tensor<40xf32>, tensor<24x56xf32>, tensor<56x40xf32>
}
'''


def test_plan_of_backward_ops_uses_views_not_copies():
    plan = Module(BACKWARD).plan("bw")
    assert plan.count("gemm") == 4 and plan.count("column_sum") == 1
    assert "grad_input = grad_out x W^T" in plan and "grad_weight = flatX^T x flatGo" in plan
    assert "grad_a = grad_out x b^T" in plan and "grad_b = a^T x grad_out" in plan
    _, res = Module(BACKWARD).signature("bw")
    assert [s for _, s in res] == [(4, 24, 56), (56, 40), (40,), (24, 56), (56, 40)]


@pytest.mark.gpu
def test_run_backward_ops_match_oracle(cuda, oracle):
    torch = cuda
    g = torch.Generator(device="cuda"); g.manual_seed(5)
    r = lambda *s: torch.rand(*s, device="cuda", generator=g) * 2 - 1
    go, x, w, g2, a, b = r(4, 24, 40), r(4, 24, 56), r(56, 40), r(24, 40), r(24, 56), r(56, 40)
    gi, gw, gb, ga, gbm = Module(BACKWARD).run("bw", go, x, w, g2, a, b)
    n = lambda t: t.cpu().numpy()
    want_gi = oracle.gemm(n(go), np.ascontiguousarray(n(w).T))
    xf, gf = n(x).reshape(96, 56), n(go).reshape(96, 40)
    want_gw = oracle.gemm(np.ascontiguousarray(xf.T), gf)
    want_gb = oracle.column_sum(gf)
    assert oracle.rel_fro(n(gi), want_gi) <= 1e-5
    assert oracle.rel_fro(n(gw), want_gw) <= 1e-5
    assert oracle.rel_fro(n(gb), want_gb) <= 1e-5
    assert oracle.rel_fro(n(ga), oracle.gemm(n(g2), np.ascontiguousarray(n(b).T))) <= 1e-5
    assert oracle.rel_fro(n(gbm), oracle.gemm(np.ascontiguousarray(n(a).T), n(g2))) <= 1e-5


# the FFN backward chain of ltest/test.mlir:39-42: linear_backward -> gelu_backward -> linear_backward
FFN_BACKWARD = '''
func.func @ffn_bw(%gy: tensor<2x24x40xbf16>, %h: tensor<2x24x72xbf16>, %w2: tensor<72x40xbf16>,
                  %z: tensor<2x24x72xbf16>, %x: tensor<2x24x40xbf16>, %w1: tensor<40x72xbf16>,
                  %m: tensor<24x72xbf16>, %zz: tensor<24x40xbf16>)
    -> (tensor<2x24x40xbf16>, tensor<40x72xbf16>, tensor<72xbf16>, tensor<24x40xbf16>, tensor<2x24x72xbf16>) {
  %gh, %gw2, %gb2 = nova.linear_backward %gy, %h, %w2 : tensor<2x24x40xbf16>, tensor<2x24x72xbf16>, tensor<72x40xbf16>
  %gz = nova.gelu_backward %gh, %z : tensor<2x24x72xbf16>, tensor<2x24x72xbf16>
  %gx, %gw1, %gb1 = nova.linear_backward %gz, %x, %w1 : tensor<2x24x72xbf16>, tensor<2x24x40xbf16>, tensor<40x72xbf16>
  %p = nova.matmul %m, %w2 : tensor<24x72xbf16>, tensor<72x40xbf16>
  %q = nova.gelu_backward %p, %zz : tensor<24x40xbf16>, tensor<24x40xbf16>
  %s = nova.gelu_backward %z, %h : tensor<2x24x72xbf16>, tensor<2x24x72xbf16>
  return %gx, %gw1, %gb1, %q, %s : tensor<2x24x40xbf16>, tensor<40x72xbf16>, tensor<72xbf16>, tensor<24x40xbf16>, tensor<2x24x72xbf16>
}
'''


def test_plan_fuses_gelu_backward_into_the_producing_contraction():
    plan = Module(FFN_BACKWARD).plan("ffn_bw")
    lines = [l.strip() for l in plan.splitlines()]
    # grad_input of the second layer is multiplied by gelu'(%z) in the contraction's epilogue ...
    fused = [l for l in lines if "grad_input = grad_out x W^T + nova.gelu_backward" in l]
    assert len(fused) == 1 and "act=gelu_tanh_grad(%z)" in fused[0] and "-> (%gz" in fused[0]
    # ... its other two contractions still read the unfused %gy, and %gz feeds the first layer's backward
    assert sum("gemm" in l for l in lines) == 5
    assert any(l.startswith("gemm") and "nova.matmul + nova.gelu_backward" in l and "act=gelu_tanh_grad(%zz)" in l for l in lines)
    # a gelu_backward whose grad_out is not a contraction result stays a step of its own
    assert sum(l.startswith("gelu_backward") for l in lines) == 1


@pytest.mark.gpu
def test_run_ffn_backward_chain_matches_oracle(cuda, oracle):
    torch = cuda
    g = torch.Generator(device="cuda"); g.manual_seed(9)
    bf = torch.bfloat16
    r = lambda *s, sc=1.0: ((torch.rand(*s, device="cuda", generator=g) * 2 - 1) * sc).to(bf)
    gy, h, w2, z = r(2, 24, 40), r(2, 24, 72), r(72, 40, sc=0.3), r(2, 24, 72, sc=2.0)
    x, w1, m, zz = r(2, 24, 40), r(40, 72, sc=0.3), r(24, 72), r(24, 40, sc=2.0)
    gx, gw1, gb1, q, s = Module(FFN_BACKWARD).run("ffn_bw", gy, h, w2, z, x, w1, m, zz)
    B = lambda t: _bits(torch, t)
    f = lambda bits: oracle.from_bits(bits, "bf16")
    T = lambda bits: np.ascontiguousarray(np.swapaxes(bits, -1, -2))
    gz = oracle.gemm(B(gy), T(B(w2)), dtype_in="bf16", gelu_grad_of=B(z))       # fused epilogue form
    want_gx = oracle.gemm(gz, T(B(w1)), dtype_in="bf16")
    want_gw1 = oracle.gemm(T(B(x).reshape(48, 40)), gz.reshape(48, 72), dtype_in="bf16")
    want_gb1 = oracle.column_sum(gz.reshape(48, 72), "bf16")
    want_q = oracle.gemm(B(m), B(w2), dtype_in="bf16", gelu_grad_of=B(zz))
    want_s = oracle.gelu_backward(B(z), B(h), "bf16", compute_f32=True)
    assert oracle.rel_fro(f(B(gx)), f(want_gx)) <= 4e-3    # two chained bf16 roundings
    assert oracle.rel_fro(f(B(gw1)), f(want_gw1)) <= 4e-3
    assert oracle.rel_fro(f(B(gb1)), f(want_gb1)) <= 4e-3
    assert oracle.rel_fro(f(B(q)), f(want_q)) <= 1e-3
    assert oracle.rel_fro(f(B(s)), f(want_s)) <= 1e-3


# forward + backward of one pre-norm FFN block, the op chain of ltest/test.mlir:20-43 at small sizes
BLOCK_TRAIN = '''
func.func @train(%x: tensor<2x16x40xf32>, %g: tensor<40xf32>, %b: tensor<40xf32>, %w1: tensor<40x72xf32>,
                 %b1: tensor<72xf32>, %w2: tensor<72x40xf32>, %b2: tensor<40xf32>, %gy: tensor<2x16x40xf32>)
    -> (tensor<2x16x40xf32>, tensor<2x16x40xf32>, tensor<40xf32>, tensor<40xf32>, tensor<40x72xf32>, tensor<72x40xf32>) {
  %ln, %sum, %rstd = nova.layer_norm %x, %g, %b : tensor<2x16x40xf32>, tensor<40xf32>, tensor<40xf32>
  %z = nova.linear %ln, %w1, %b1 : tensor<2x16x40xf32>, tensor<40x72xf32>, tensor<72xf32>
  %h = nova.gelu %z : tensor<2x16x72xf32>
  %o = nova.linear %h, %w2, %b2 : tensor<2x16x72xf32>, tensor<72x40xf32>, tensor<40xf32>
  %y = nova.add %o, %x : tensor<2x16x40xf32>, tensor<2x16x40xf32>
  %gh, %gw2, %gb2 = nova.linear_backward %gy, %h, %w2 : tensor<2x16x40xf32>, tensor<2x16x72xf32>, tensor<72x40xf32>
  %gz = nova.gelu_backward %gh, %z : tensor<2x16x72xf32>, tensor<2x16x72xf32>
  %gln, %gw1, %gb1 = nova.linear_backward %gz, %ln, %w1 : tensor<2x16x72xf32>, tensor<2x16x40xf32>, tensor<40x72xf32>
  %gx0, %gg, %gbeta = nova.layer_norm_backward %gln, %x, %g, %sum, %rstd : tensor<2x16x40xf32>, tensor<2x16x40xf32>, tensor<40xf32>, tensor<2x16xf32>, tensor<2x16xf32>
  %gx = nova.add %gx0, %gy : tensor<2x16x40xf32>, tensor<2x16x40xf32>
  return %y, %gx, %gg, %gbeta, %gw1, %gw2 : tensor<2x16x40xf32>, tensor<2x16x40xf32>, tensor<40xf32>, tensor<40xf32>, tensor<40x72xf32>, tensor<72x40xf32>
}
'''


def test_plan_of_a_training_step_keeps_the_pre_activation_for_the_backward():
    plan = Module(BLOCK_TRAIN).plan("train")
    lines = [l.strip() for l in plan.splitlines()]
    # %z is needed by gelu_backward, so the forward GELU is NOT folded into the first linear's epilogue
    assert any(l.startswith("gemm init=bias_row(%b1) act=none") for l in lines)
    assert any(l.startswith("activation") for l in lines)
    assert any("act=gelu_tanh_grad(%z)" in l for l in lines)
    assert sum(l.startswith("layer_norm_backward") for l in lines) == 1


@pytest.mark.gpu
def test_run_training_step_matches_autograd(cuda):
    """The whole block, forward and backward, against torch autograd in float64 (an independent check of the chain
    rule; the per-op parity against the oracle is in the other tests)."""
    torch = cuda
    g = torch.Generator(device="cuda"); g.manual_seed(11)
    r = lambda *s, sc=1.0: (torch.rand(*s, device="cuda", generator=g) * 2 - 1) * sc
    x, gm, bt = r(2, 16, 40), r(40) + 1.5, r(40)
    w1, b1, w2, b2, gy = r(40, 72, sc=0.3), r(72, sc=0.3), r(72, 40, sc=0.3), r(40, sc=0.3), r(2, 16, 40)
    y, gx, gg, gbeta, gw1, gw2 = Module(BLOCK_TRAIN).run("train", x, gm, bt, w1, b1, w2, b2, gy)
    d = lambda t: t.detach().double().requires_grad_(True)
    X, G, Bt, W1, B1, W2, B2 = map(d, (x, gm, bt, w1, b1, w2, b2))
    ln = torch.nn.functional.layer_norm(X, (40,), G, Bt, eps=1e-5)
    Y = torch.nn.functional.gelu(ln @ W1 + B1, approximate="tanh") @ W2 + B2 + X
    Y.backward(gy.double())
    rel = lambda a, b: float((a.double() - b).norm() / b.norm())
    assert rel(y, Y.detach()) <= 1e-5
    assert rel(gx, X.grad) <= 2e-5 and rel(gg, G.grad) <= 2e-5 and rel(gbeta, Bt.grad) <= 2e-5
    assert rel(gw1, W1.grad) <= 2e-5 and rel(gw2, W2.grad) <= 2e-5


# the loss end of ltest/test.mlir:24-30,33-34: vocabulary matmul -> sce -> sce_backward -> the two backward matmuls
LOSS = '''
func.func @loss(%h: tensor<2x12x40xf32>, %wv: tensor<40x96xf32>, %tgt: tensor<2x12xi16>, %emb: tensor<96x40xf32>)
    -> (tensor<1xf32>, tensor<24x40xf32>, tensor<40x96xf32>, tensor<96x40xf32>) {
  %0 = nova.reshape %h : tensor<2x12x40xf32> -> tensor<24x40xf32>
  %1 = nova.matmul %0, %wv : tensor<24x40xf32>, tensor<40x96xf32>
  %2 = nova.reshape %1 : tensor<24x96xf32> -> tensor<2x12x96xf32>
  %sm, %l = nova.sce %2, %tgt : tensor<2x12x96xf32>, tensor<2x12xi16>
  %g = nova.sce_backward %sm, %tgt {dim = -1 : i64} : tensor<2x12x96xf32>, tensor<2x12xi16>
  %3 = nova.reshape %g : tensor<2x12x96xf32> -> tensor<24x96xf32>
  %4 = nova.transpose %0 : tensor<24x40xf32>
  %5 = nova.transpose %wv : tensor<40x96xf32>
  %gh = nova.matmul %3, %5 : tensor<24x96xf32>, tensor<96x40xf32>
  %gw = nova.matmul %4, %3 : tensor<40x24xf32>, tensor<24x96xf32>
  %ids = nova.reshape %tgt : tensor<2x12xi16> -> tensor<24xi16>
  %ge = nova.scatter_add %emb, %ids, %gh axis = 0 : tensor<96x40xf32>, tensor<24xi16>, tensor<24x40xf32> -> tensor<96x40xf32>
  return %l, %gh, %gw, %ge : tensor<1xf32>, tensor<24x40xf32>, tensor<40x96xf32>, tensor<96x40xf32>
}
'''


def test_plan_of_the_loss_end():
    plan = Module(LOSS).plan("loss")
    lines = [l.strip() for l in plan.splitlines()]
    assert sum(l.startswith("sce ") for l in lines) == 1 and sum(l.startswith("sce_backward") for l in lines) == 1
    assert sum(l.startswith("scatter_add") for l in lines) == 1 and sum(l.startswith("gemm") for l in lines) == 3
    _, res = Module(LOSS).signature("loss")
    assert res == [(L.F32, (1,)), (L.F32, (24, 40)), (L.F32, (40, 96)), (L.F32, (96, 40))]
    bad = LOSS.replace("{dim = -1 : i64}", "{dim = 0 : i64}")
    with pytest.raises(Exception) as e:
        Module(bad).plan("loss")
    assert "last dimension" in str(e.value)


@pytest.mark.gpu
def test_run_loss_end_matches_autograd(cuda):
    torch = cuda
    g = torch.Generator(device="cuda"); g.manual_seed(21)
    r = lambda *s, sc=1.0: (torch.rand(*s, device="cuda", generator=g) * 2 - 1) * sc
    h, wv, emb = r(2, 12, 40), r(40, 96, sc=0.5), r(96, 40)
    tgt = torch.randint(0, 96, (2, 12), device="cuda", generator=g).to(torch.int16)
    l, gh, gw, ge = Module(LOSS).run("loss", h, wv, tgt, emb)
    H, W = h.double().reshape(24, 40).requires_grad_(True), wv.double().requires_grad_(True)
    loss = torch.nn.functional.cross_entropy(H @ W, tgt.long().reshape(-1))
    loss.backward()
    rel = lambda a, b: float((a.double() - b).norm() / b.norm())
    assert abs(float(l[0]) - float(loss.detach())) <= 1e-5 * abs(float(loss.detach()))
    assert rel(gh, H.grad) <= 2e-5 and rel(gw, W.grad) <= 2e-5
    want_ge = emb.double().index_add(0, tgt.long().reshape(-1), H.grad)
    assert rel(ge, want_ge) <= 1e-6
