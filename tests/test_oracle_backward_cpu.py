"""The oracle's restatements of the backward and loss ops (nova.gelu_backward, nova.layer_norm_backward, nova.sce,
nova.sce_backward, nova.scatter_add and the fused epilogue forms) against float64 autograd on the CPU: an
independent statement of the same mathematics.  The reference has no numeric fixtures for these ops
(ltest/_gelu.mlir, ltest/_layernorm.mlir carry shapes only)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def O():
    from oracle import build
    build.build()
    from oracle import oracle
    return oracle


def test_gelu_backward_matches_autograd(O):
    rng = np.random.default_rng(3)
    x = (rng.normal(size=(5, 33)) * 2.5).astype(np.float32)
    go = rng.normal(size=(5, 33)).astype(np.float32)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    torch.nn.functional.gelu(xt, approximate="tanh").backward(torch.tensor(go, dtype=torch.float64))
    assert O.rel_fro(O.gelu_backward(go, x), xt.grad.numpy()) <= 1e-6
    # 16-bit: every step rounded through the element type (the reference's generic) stays within a few ulp
    xb, gb = O.to_bits(x, "bf16"), O.to_bits(go, "bf16")
    got = O.from_bits(O.gelu_backward(gb, xb, "bf16"), "bf16")
    xr = torch.tensor(O.from_bits(xb, "bf16"), dtype=torch.float64, requires_grad=True)
    torch.nn.functional.gelu(xr, approximate="tanh").backward(torch.tensor(O.from_bits(gb, "bf16"), dtype=torch.float64))
    assert O.rel_fro(got, xr.grad.numpy()) <= 3e-2


def test_fused_epilogues_equal_their_unfused_chains(O):
    rng = np.random.default_rng(4)
    a = rng.normal(size=(2, 9, 12)).astype(np.float32)
    b = rng.normal(size=(2, 12, 7)).astype(np.float32)
    bias = rng.normal(size=7).astype(np.float32)
    res = rng.normal(size=(2, 9, 7)).astype(np.float32)
    z = (rng.normal(size=(2, 9, 7)) * 2).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64) + bias + res
    assert O.rel_fro(O.gemm(a, b, bias=bias, residual=res), want) <= 1e-6
    fused = O.gemm(a, b, bias=bias, gelu_grad_of=z)
    assert np.array_equal(fused, O.gelu_backward(O.gemm(a, b, bias=bias), z))
    with pytest.raises(ValueError):
        O.gemm(a, b, residual=res, gelu_grad_of=z)


def test_layer_norm_backward_matches_autograd(O):
    rng = np.random.default_rng(5)
    x = rng.normal(size=(4, 6, 48)).astype(np.float32)
    g = (rng.normal(size=48) + 1.5).astype(np.float32)
    b = rng.normal(size=48).astype(np.float32)
    gy = rng.normal(size=(4, 6, 48)).astype(np.float32)
    _, ms, rstd = O.layer_norm(x, g, b)
    dx, dg, db = O.layer_norm_backward(gy, x, g, ms, rstd)
    xt, gt, bt = (torch.tensor(v, dtype=torch.float64, requires_grad=True) for v in (x, g, b))
    torch.nn.functional.layer_norm(xt, (48,), gt, bt, eps=1e-5).backward(torch.tensor(gy, dtype=torch.float64))
    assert O.rel_fro(dx, xt.grad.numpy()) <= 1e-5
    assert O.rel_fro(dg, gt.grad.numpy()) <= 1e-5 and O.rel_fro(db, bt.grad.numpy()) <= 1e-5


@pytest.mark.parametrize("idx_dtype", [np.int16, np.int32, np.int64])
def test_sce_and_its_backward_match_autograd(O, idx_dtype):
    rng = np.random.default_rng(6)
    x = (rng.normal(size=(3, 5, 70)) * 3).astype(np.float32)
    t = rng.integers(0, 70, size=(3, 5)).astype(idx_dtype)
    sm, loss, bad = O.sce(x, t)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    l = torch.nn.functional.cross_entropy(xt.reshape(-1, 70), torch.tensor(t.astype(np.int64)).reshape(-1))
    l.backward()
    assert bad == 0 and abs(float(loss[0]) - float(l.detach())) <= 1e-6 * float(l.detach())
    assert O.rel_fro(sm, torch.softmax(xt.detach(), -1).numpy()) <= 1e-6
    assert O.rel_fro(O.sce_backward(sm, t), xt.grad.numpy()) <= 1e-6


def test_sce_zero_extends_narrow_targets_and_counts_bad_ones(O):
    x = np.zeros((2, 40000), dtype=np.float32)
    x[0, 39999] = 5.0
    t = np.array([39999, 7], dtype=np.uint16).view(np.int16)  # 39999 is negative as a signed i16
    _, loss, bad = O.sce(x, t)
    want = 0.5 * ((np.log(39999 + np.exp(5.0)) - 5.0) + np.log(40000.0))
    # (the oracle adds the 40000 exponentials one by one in fp32, as the reference's reduction does: ~3e-5 of drift)
    assert bad == 0 and abs(float(loss[0]) - want) <= 1e-4 * want
    _, _, bad = O.sce(np.zeros((1, 8), np.float32), np.array([8], np.int32))
    assert bad == 1


def test_scatter_add_is_index_add(O):
    rng = np.random.default_rng(7)
    inp = rng.normal(size=(3, 11, 4)).astype(np.float32)
    idx = np.array([0, 10, 3, 3, 25, 3], dtype=np.int32)
    src = rng.normal(size=(3, 6, 4)).astype(np.float32)
    out, bad = O.scatter_add(inp, idx, src, axis=1)
    keep = idx < 11
    want = torch.tensor(inp).index_add(1, torch.tensor(idx[keep].astype(np.int64)), torch.tensor(src[:, keep])).numpy()
    assert bad == 3 and np.allclose(out, want, atol=1e-6)
    with pytest.raises(ValueError):
        O.scatter_add(inp, idx[:5], src, axis=1)
