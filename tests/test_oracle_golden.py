"""Pins the CPU oracle (oracle/sage_ref.py + oracle/sage_oracle.c) to the
reference's own known-answer vectors.  Each case restates one reference unit
test; the literals come from tests/golden/reference_vectors.json, produced by
tests/golden/extract_reference_vectors.py from the reference's Rust sources.
Tolerances are the reference's own (absolute, Tensor::all_close, src/tensor.rs:320-328).
"""
import json
import os

import numpy as np
import pytest

from oracle import sage_ref as R

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_vectors.json")) as f:
    GOLD = json.load(f)


def vec(test, name, nth=0, dtype=np.float32):
    hits = [v["value"] for v in GOLD[test]["vectors"] if v["name"] == name]
    return np.array(hits[nth], dtype=dtype)


def close(t, gt, eps):
    a = t.numpy() if isinstance(t, R.Tensor) else t
    assert a.shape == gt.shape, (a.shape, gt.shape)
    assert np.all(np.abs(a.astype(np.float64) - gt) < eps), np.abs(a - gt).max()


def V(a, dtype=None):
    return R.Var.new(R.Tensor.new(a, dtype))


def test_nullary_map():  # src/ops/map.rs:1383
    close(R.scalar(3.0, [3, 3]).eval(), vec("map.test_nullary_map", "y_gt"), 1e-3)


def test_unary_map():  # src/ops/map.rs:1394
    x, y = vec("map.test_unary_map", "x"), vec("map.test_unary_map", "y_gt")
    close(R.sin(V(x)).eval(), y, 1e-3)
    close(R.sin(R.transpose(V(x), 0, 1)).eval(), y.transpose(1, 0, 2), 1e-3)


def test_binary_map():  # src/ops/map.rs:1518
    x1, x2, y = (vec("map.test_binary_map", n) for n in ("x1", "x2", "y_gt"))
    close(R.sub(V(x1), V(x2)).eval(), y, 1e-3)
    close(R.sub(R.tr(V(x1)), R.tr(V(x2))).eval(), np.swapaxes(y, 0, 1), 1e-3)


def test_ternary_map():  # src/ops/map.rs:1621
    x1, x2, y = (vec("map.test_ternary_map", n) for n in ("x1", "x2", "y_gt"))
    close(R.cond(R.gt(V(x1), 0.0), V(x1), V(x2)).eval(), y, 1e-3)


def test_variadic_map():  # src/ops/map.rs:1644
    x1, x2, x3, y = (vec("map.test_variadic_map", n) for n in ("x1", "x2", "x3", "y_gt"))
    a, b, c = V(x1), V(x2), V(x3)
    close((((a + b * 3.0) - c / 2.0) / b).eval(), y, 1e-2)


def test_reshape():  # src/ops/core.rs:946
    a = vec("core.test_reshape", "a")
    b_gt, c_gt = vec("core.test_reshape", "b_gt"), vec("core.test_reshape", "c_gt")
    b = R.reshape(V(a), R.Shape([4, 2, 3]))
    close(b.eval(), b_gt, 1e-3)
    # a transposed view is not default-strided, so reshape() goes through organize()
    c = R.reshape(R.transpose(b, 0, 1), R.Shape([4, 2, 3]))
    close(c.eval(), c_gt, 1e-3)


def test_expand():  # src/ops/core.rs:994
    close(R.expand(V(vec("core.test_expand", "x")), [3, 4]).eval(), vec("core.test_expand", "y_gt"), 1e-3)


def test_permute():  # src/ops/core.rs:1010
    close(R.permute(V(vec("core.test_permute", "x")), [2, 3, 4, 1, 0]).eval(), vec("core.test_permute", "y_gt"), 1e-3)


def test_slice():  # src/ops/core.rs:1076
    close(R.slice_(V(vec("core.test_slice", "x")), 1, 1, 2).eval(), vec("core.test_slice", "y_gt"), 1e-3)


def test_unslice():  # src/ops/core.rs:1108
    close(R.unslice(V(vec("core.test_unslice", "x")), 1, 1, 3).eval(), vec("core.test_unslice", "y_gt"), 1e-3)


def test_gather():  # src/ops/core.rs:1141
    x = vec("core.test_gather", "x")
    t = vec("core.test_gather", "t", dtype=np.uint32)
    close(R.gather(V(x), V(t, R.UINT), 2).eval(), vec("core.test_gather", "y_gt"), 1e-3)


def test_concat():  # src/ops/core.rs:1196 (the reference prints instead of asserting)
    x1, x2, x3, y = (vec("core.test_concat", n) for n in ("x1", "x2", "x3", "y_gt"))
    close(R.concat([V(x1), V(x2), V(x3)], 1).eval(), y, 1e-3)


def test_reduce_mean():  # src/ops/reduce.rs:446
    close(R.mean(V(vec("reduce.test_reduce", "x")), [0, 2, 3], False).eval(), vec("reduce.test_reduce", "y_gt"), 1e-3)


def test_reduce_arg():  # src/ops/reduce.rs:501
    y = R.argmax(V(vec("reduce.test_reduce_arg", "x")), 1, False).eval().numpy()
    gt = vec("reduce.test_reduce_arg", "y_gt", dtype=np.uint32)
    assert y.dtype == np.uint32 and np.array_equal(y, gt)


def test_gemm():  # src/ops/gemm.rs:432
    a, b, c = vec("gemm.test_gemm", "a", 0), vec("gemm.test_gemm", "b", 0), vec("gemm.test_gemm", "c_gt")
    close(R.gemm(V(a), V(b), False, False).eval(), c, 1e-3)
    a, b = vec("gemm.test_gemm", "a", 1), vec("gemm.test_gemm", "b", 1)
    for name, ta, tb in (("cff_gt", False, False), ("ctf_gt", True, False), ("cft_gt", False, True), ("ctt_gt", True, True)):
        for fma in (0, 1):
            R.USE_FMA = fma
            close(R.gemm(V(a), V(b), ta, tb).eval(), vec("gemm.test_gemm", name), 1e-3)
    R.USE_FMA = 1


def test_im2col():  # src/ops/conv.rs:509
    close(R.im2col(V(vec("conv.test_im2col", "x")), [3, 2], [1, 1], [0, 0], [1, 1]).eval(), vec("conv.test_im2col", "y_gt"), 1e-3)


def test_col2im():  # src/ops/conv.rs:699
    close(R.col2im(V(vec("conv.test_col2im", "x")), [4, 5], [3, 2], [1, 1], [0, 0], [1, 1]).eval(), vec("conv.test_col2im", "y_gt"), 1e-3)


def test_conv2d():  # src/ops/conv.rs:995
    x, f, y = (vec("conv.test_conv2d", n) for n in ("x", "filter", "y_gt"))
    close(R.conv_2d(V(x), V(f), [1, 1], [1, 1], [1, 1]).eval(), y, 1e-3)


def test_relu():  # src/ops/nn.rs:111
    close(R.relu(V(vec("nn.test_relu", "x"))).eval(), vec("nn.test_relu", "y_gt"), 1e-3)


def test_softmax():  # src/ops/nn.rs:133
    close(R.softmax(V(vec("nn.test_softmax", "x")), 1).eval(), vec("nn.test_softmax", "y_gt"), 1e-3)


def test_softmax_cross_entropy():  # src/ops/nn.rs:157 (gx_gt is declared there but never asserted)
    x = vec("nn.test_softmax_cross_entropy", "x")
    label = vec("nn.test_softmax_cross_entropy", "label", dtype=np.uint32)
    xv = V(x)
    loss = R.softmax_cross_entropy(xv, V(label, R.UINT))
    close(loss.eval(), vec("nn.test_softmax_cross_entropy", "loss_gt"), 1e-3)
    # gx_gt was generated with a mean-reduced loss (PyTorch default), hence the 1/5
    gx = xv.grad(loss).eval().numpy() / np.float32(x.shape[0])
    close(gx, vec("nn.test_softmax_cross_entropy", "gx_gt"), 1e-3)


def test_max_pool_2d():  # src/ops/nn.rs:224
    close(R.max_pool_2d(V(vec("nn.test_max_pool_2d", "x")), 3, 1, 0, 1).eval(), vec("nn.test_max_pool_2d", "y_gt"), 1e-2)


@pytest.mark.parametrize("name,fn,tol", [
    ("abs", R.abs_, 0.01), ("neg", R.neg, 0.01), ("exp", R.exp, 0.01), ("square", R.square, 0.01),
    ("sin", R.sin, 0.01), ("cos", R.cos, 0.01), ("tanh", R.tanh, 0.01), ("erf", R.erf, 0.01)])
def test_grad_check_unary(name, fn, tol):
    """Pattern B of the reference's tests (src/var.rs:107-148): symbolic grad vs
    central differences, eps 1e-4 in the reference; float64 differences here."""
    x = vec("map.test_unary_map", "x")
    xv = V(x)
    g = xv.grad(fn(xv)).eval().numpy()
    f64 = {"abs": np.sign, "neg": lambda v: -np.ones_like(v), "exp": np.exp, "square": lambda v: 2 * v,
           "sin": np.cos, "cos": lambda v: -np.sin(v), "tanh": lambda v: 1 / np.cosh(v) ** 2,
           "erf": lambda v: 2 / np.sqrt(np.pi) * np.exp(-v * v)}[name](x.astype(np.float64))
    assert np.abs(g - f64).max() < tol
