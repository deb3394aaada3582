"""GPU parity: the CUDA path (through the C ABI of libsagecuda.so) against the CPU oracle on the
same seeded inputs, and against the reference's golden vectors.

Tolerances (from the task's north star): gather / scatter(unique) / argmax / integer casts are
bit-exact; f32 results have max relative error <= 1e-4 measured as
|a - b| / max(|b|, 1e-6 * max|b|)  for elementwise work, and for contractions (whose outputs can
cancel to ~0, where any two fp32 summation orders differ by more than 1e-4 of the value)
|a - b| / max(|b|, 1e-3 * max|b|);  full model logits <= 1e-3.
"""
import json
import os

import numpy as np
import pytest

import sage_b200 as S
from oracle import sage_ref as R
from parity_metrics import check_envelope

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_vectors.json")) as f:
    GOLD = json.load(f)


def vec(test, name, nth=0, dtype=np.float32):
    hits = [v["value"] for v in GOLD[test]["vectors"] if v["name"] == name]
    return np.array(hits[nth], dtype=dtype)


def rel_err(a, b, floor=1e-6):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.size == 0:
        return 0.0
    scale = np.maximum(np.abs(b), floor * max(np.abs(b).max(), 1e-30))
    return float((np.abs(a - b) / scale).max())


@pytest.fixture(scope="module")
def ctx():
    c = S.Context(0)
    yield c
    c.close()


def RV(a, dtype=None):
    return R.Var.new(R.Tensor.new(a, dtype))


# ------------------------------------------------------------------------------ golden vectors on the GPU
def test_golden_maps(ctx):  # src/ops/map.rs:1383-1676
    close = lambda y, gt, eps: np.testing.assert_allclose(y, gt, atol=eps, rtol=0)
    close(S.scalar(3.0, [3, 3]).eval(ctx), vec("map.test_nullary_map", "y_gt"), 1e-3)
    x, y = vec("map.test_unary_map", "x"), vec("map.test_unary_map", "y_gt")
    xv = ctx.var(x)
    close(S.sin(xv).eval(ctx), y, 1e-3)
    close(S.sin(xv.transpose(0, 1)).eval(ctx), y.transpose(1, 0, 2), 1e-3)
    x1, x2, y = (vec("map.test_binary_map", n) for n in ("x1", "x2", "y_gt"))
    a, b = ctx.var(x1), ctx.var(x2)
    close(S.sub(a, b).eval(ctx), y, 1e-3)
    close(S.sub(a.tr(), b.tr()).eval(ctx), np.swapaxes(y, 0, 1), 1e-3)
    x1, x2, y = (vec("map.test_ternary_map", n) for n in ("x1", "x2", "y_gt"))
    a, b = ctx.var(x1), ctx.var(x2)
    close(S.cond(S.gt(a, 0.0), a, b).eval(ctx), y, 1e-3)
    x1, x2, x3, y = (vec("map.test_variadic_map", n) for n in ("x1", "x2", "x3", "y_gt"))
    a, b, c = ctx.var(x1), ctx.var(x2), ctx.var(x3)
    close((((a + b * 3.0) - c / 2.0) / b).eval(ctx), y, 1e-2)


def test_golden_core(ctx):  # src/ops/core.rs:946-1233
    close = lambda y, gt: np.testing.assert_allclose(y, gt, atol=1e-3, rtol=0)
    a = ctx.var(vec("core.test_reshape", "a"))
    b = a.view([4, 2, 3])
    close(b.eval(ctx), vec("core.test_reshape", "b_gt"))
    close(b.transpose(0, 1).view([4, 2, 3]).eval(ctx), vec("core.test_reshape", "c_gt"))
    close(S.expand(ctx.var(vec("core.test_expand", "x")), [3, 4]).organize().eval(ctx), vec("core.test_expand", "y_gt"))
    close(S.permute(ctx.var(vec("core.test_permute", "x")), [2, 3, 4, 1, 0]).organize().eval(ctx), vec("core.test_permute", "y_gt"))
    close(S.slice_(ctx.var(vec("core.test_slice", "x")), 1, 1, 2).organize().eval(ctx), vec("core.test_slice", "y_gt"))
    close(S.unslice(ctx.var(vec("core.test_unslice", "x")), 1, 1, 3).eval(ctx), vec("core.test_unslice", "y_gt"))
    t = ctx.var(vec("core.test_gather", "t", dtype=np.uint32))
    close(S.gather(ctx.var(vec("core.test_gather", "x")), t, 2).eval(ctx), vec("core.test_gather", "y_gt"))
    xs = [ctx.var(vec("core.test_concat", n)) for n in ("x1", "x2", "x3")]
    close(S.concat(xs, 1).eval(ctx), vec("core.test_concat", "y_gt"))


def test_golden_reduce_gemm_conv_nn(ctx):
    close = lambda y, gt, eps=1e-3: np.testing.assert_allclose(y, gt, atol=eps, rtol=0)
    close(S.mean(ctx.var(vec("reduce.test_reduce", "x")), [0, 2, 3], False).eval(ctx), vec("reduce.test_reduce", "y_gt"))
    y = S.argmax(ctx.var(vec("reduce.test_reduce_arg", "x")), 1, False).eval(ctx)
    assert y.dtype == np.uint32 and np.array_equal(y, vec("reduce.test_reduce_arg", "y_gt", dtype=np.uint32))
    a, b = ctx.var(vec("gemm.test_gemm", "a", 0)), ctx.var(vec("gemm.test_gemm", "b", 0))
    close(S.gemm(a, b).eval(ctx), vec("gemm.test_gemm", "c_gt"))
    a, b = ctx.var(vec("gemm.test_gemm", "a", 1)), ctx.var(vec("gemm.test_gemm", "b", 1))
    for name, ta, tb in (("cff_gt", 0, 0), ("ctf_gt", 1, 0), ("cft_gt", 0, 1), ("ctt_gt", 1, 1)):
        close(S.gemm(a, b, ta, tb).eval(ctx), vec("gemm.test_gemm", name))
    close(S.im2col(ctx.var(vec("conv.test_im2col", "x")), [3, 2], [1, 1], [0, 0], [1, 1]).eval(ctx), vec("conv.test_im2col", "y_gt"))
    close(S.col2im(ctx.var(vec("conv.test_col2im", "x")), [4, 5], [3, 2], [1, 1], [0, 0], [1, 1]).eval(ctx), vec("conv.test_col2im", "y_gt"))
    x, f = ctx.var(vec("conv.test_conv2d", "x")), ctx.var(vec("conv.test_conv2d", "filter"))
    close(S.conv_2d(x, f, [1, 1], [1, 1], [1, 1]).eval(ctx), vec("conv.test_conv2d", "y_gt"))
    close(S.relu(ctx.var(vec("nn.test_relu", "x"))).eval(ctx), vec("nn.test_relu", "y_gt"))
    close(S.softmax(ctx.var(vec("nn.test_softmax", "x")), 1).eval(ctx), vec("nn.test_softmax", "y_gt"))
    x = ctx.var(vec("nn.test_softmax_cross_entropy", "x"))
    lab = ctx.var(vec("nn.test_softmax_cross_entropy", "label", dtype=np.uint32))
    loss = S.softmax_cross_entropy(x, lab)
    close(loss.eval(ctx), vec("nn.test_softmax_cross_entropy", "loss_gt"))
    close(x.grad(loss).eval(ctx) / np.float32(5), vec("nn.test_softmax_cross_entropy", "gx_gt"))
    close(S.max_pool_2d(ctx.var(vec("nn.test_max_pool_2d", "x")), 3, 1, 0, 1).eval(ctx), vec("nn.test_max_pool_2d", "y_gt"), 1e-2)


# ------------------------------------------------------------------------------ maps vs oracle
UNARY = ["abs", "neg", "recip", "log", "exp", "sqrt", "square", "erf", "sign", "ceil", "floor", "round", "sin", "sinh", "cos",
         "cosh", "tan", "tanh", "asin", "asinh", "acos", "acosh", "atan", "atanh"]


@pytest.mark.parametrize("name", UNARY)
def test_unary_vs_oracle(ctx, name):
    rng = np.random.default_rng(7)
    x = rng.uniform(-3, 3, (37, 129)).astype(np.float32)
    if name in ("log", "sqrt"):
        x = np.abs(x) + np.float32(0.01)
    if name in ("asin", "acos", "atanh"):
        x = (x / 3.5).astype(np.float32)
    if name == "acosh":
        x = np.abs(x) + np.float32(1.01)
    if name in ("ceil", "floor", "round", "sign"):
        x[0, :5] = [0.5, -0.5, 1.5, -2.5, 0.0]
    ref = getattr(R, name + "_" if name in ("abs", "round") else name)(RV(x)).eval().numpy()
    got = getattr(ctx.var(x), name)().eval(ctx)
    if name in ("ceil", "floor", "round", "sign", "abs", "neg"):
        assert np.array_equal(got, ref)
    else:
        assert rel_err(got, ref) <= 1e-4


def test_binary_logic_casts_exact(ctx):
    rng = np.random.default_rng(8)
    a = rng.integers(-5, 5, (33, 65)).astype(np.float32)
    b = rng.integers(-5, 5, (33, 65)).astype(np.float32)
    va, vb = ctx.var(a), ctx.var(b)
    for name in ("eq", "ne", "gt", "ge", "lt", "le", "minimum", "maximum", "add", "sub", "mul"):
        got = getattr(S, name)(va, vb).eval(ctx)
        ref = getattr(R, name)(RV(a), RV(b)).eval().numpy()
        assert got.dtype == ref.dtype and np.array_equal(got, ref), name
    x = rng.uniform(-100, 100, (1000,)).astype(np.float32)
    gi = ctx.var(x).int().eval(ctx)
    assert gi.dtype == np.int32 and np.array_equal(gi, np.trunc(x).astype(np.int32))  # (int)x truncates toward zero
    u = rng.integers(0, 2, (1000,)).astype(np.uint32)
    gf = ctx.var(u).float().eval(ctx)
    assert gf.dtype == np.float32 and np.array_equal(gf, u.astype(np.float32))


def test_div_mod_pow_and_logic_vs_oracle(ctx):
    """The binary / unary maps of src/ops/map.rs:224-302 that have no other value test: `/`, `mod`, `pow`,
    `&&`, `||`, `!`.  Logic results are uint and bit-exact, also on float operands (C truthiness: non-zero is
    true, so -0.0 is false and NaN is true); div is one correctly rounded division: bit-exact; fmod is exact by
    definition; pow goes through the device's powf: rel <= 1e-4."""
    rng = np.random.default_rng(81)
    a = rng.uniform(-4, 4, (37, 129)).astype(np.float32)
    b = rng.uniform(0.25, 4, (37, 129)).astype(np.float32) * np.where(rng.random((37, 129)) < 0.5, -1, 1).astype(np.float32)
    va, vb = ctx.var(a), ctx.var(b)
    got = S.div(va, vb).eval(ctx)
    assert got.dtype == np.float32 and np.array_equal(got, R.div(RV(a), RV(b)).eval().numpy())
    got = S.modular(va, vb).eval(ctx)
    assert np.array_equal(got, R.modular(RV(a), RV(b)).eval().numpy())
    base = np.abs(a) + np.float32(0.05)
    got = S.pow_(ctx.var(base), vb).eval(ctx)
    assert rel_err(got, R.pow_(RV(base), RV(b)).eval().numpy()) <= 1e-4
    # broadcast + scalar operand forms (into_var of a literal, map.rs:412-429)
    row = rng.uniform(0.5, 2, (129,)).astype(np.float32)
    assert np.array_equal((va / ctx.var(row)).eval(ctx), (RV(a) / RV(row)).eval().numpy())
    assert np.array_equal((va / 3.0).eval(ctx), (RV(a) / 3.0).eval().numpy())
    # logic on uint operands (the results of compares) and on floats with the awkward values
    x = rng.integers(-2, 3, (33, 65)).astype(np.float32)
    y = rng.integers(-2, 3, (33, 65)).astype(np.float32)
    x[0, :4] = [0.0, -0.0, np.nan, 1e-30]
    y[0, :4] = [1.0, 1.0, 0.0, -0.0]
    vx, vy = ctx.var(x), ctx.var(y)
    for name in ("and_", "or_"):
        got = getattr(S, name)(vx, vy).eval(ctx)
        ref = getattr(R, name)(RV(x), RV(y)).eval().numpy()
        assert got.dtype == np.uint32 == ref.dtype and np.array_equal(got, ref), name
        got = getattr(S, name)(S.gt(vx, 0.0), S.lt(vy, 1.0)).eval(ctx)
        ref = getattr(R, name)(R.gt(RV(x), 0.0), R.lt(RV(y), 1.0)).eval().numpy()
        assert got.dtype == np.uint32 and np.array_equal(got, ref), name
    got = S.not_(vx).eval(ctx)
    ref = R.not_(RV(x)).eval().numpy()
    assert got.dtype == np.uint32 == ref.dtype and np.array_equal(got, ref)
    assert np.array_equal(S.not_(S.ge(vx, vy)).eval(ctx), R.not_(R.ge(RV(x), RV(y))).eval().numpy())
    # gradients of div and pow (map.rs:1014-1042) through the same kernels
    vbase = ctx.var(base)
    out = S.sum_(S.pow_(vbase, vb) / vb, [0, 1])
    rbase, rb = RV(base), RV(b)
    rout = R.sum_(R.pow_(rbase, rb) / rb, [0, 1])
    g1, g2 = vbase.grad(out).eval(ctx), vb.grad(out).eval(ctx)
    r1, r2 = [t.numpy() for t in R.evaluate([rbase.grad(rout), rb.grad(rout)])]
    assert rel_err(g1, r1, floor=1e-5) <= 1e-4 and rel_err(g2, r2, floor=1e-5) <= 1e-4


@pytest.mark.parametrize("shape", [(3, 9, 11, 16), (2, 5, 7, 3), (4, 8, 8, 64)])
def test_batch_norm_2d_vs_oracle(ctx, shape):
    """batch_norm_2d (src/ops/conv.rs:167-185): gamma * (x - mean) / sqrt(var + eps) + beta with per-channel running
    statistics and [1] gamma / beta, as BatchNorm2d::pass builds it (src/layers.rs:535-545)."""
    rng = np.random.default_rng(82)
    c = shape[3]
    x = rng.standard_normal(shape).astype(np.float32)
    mean_ = rng.standard_normal((c,)).astype(np.float32)
    var_ = rng.uniform(0.3, 2.0, (c,)).astype(np.float32)
    for gamma, beta in ((np.float32([1.0]), np.float32([0.0])), (np.float32([0.7]), np.float32([-0.3])),
                        (rng.uniform(0.5, 1.5, (c,)).astype(np.float32), rng.standard_normal((c,)).astype(np.float32))):
        got = S.batch_norm_2d(ctx.var(x), ctx.var(gamma), ctx.var(beta), ctx.var(mean_), ctx.var(var_), 1e-5).eval(ctx)
        ref = R.batch_norm_2d(RV(x), RV(gamma), RV(beta), RV(mean_), RV(var_), 1e-5).eval().numpy()
        assert got.shape == ref.shape and rel_err(got, ref, floor=1e-4) <= 1e-4
    xv = ctx.var(x)
    g, b = ctx.var(np.float32([0.7])), ctx.var(np.float32([-0.3]))
    out = S.sum_(S.square(S.batch_norm_2d(xv, g, b, ctx.var(mean_), ctx.var(var_), 1e-5)), [0, 1, 2, 3])
    rx, rg, rb = RV(x), RV(np.float32([0.7])), RV(np.float32([-0.3]))
    rout = R.sum_(R.square(R.batch_norm_2d(rx, rg, rb, RV(mean_), RV(var_), 1e-5)), [0, 1, 2, 3])
    gx, gg = xv.grad(out).eval(ctx), g.grad(out).eval(ctx)
    rgx, rgg = [t.numpy() for t in R.evaluate([rx.grad(rout), rg.grad(rout)])]
    assert rel_err(gx, rgx, floor=1e-4) <= 1e-4 and rel_err(gg, rgg, floor=1e-4) <= 1e-4


def test_broadcast_and_strided_views(ctx):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((6, 5, 8)).astype(np.float32)
    bias = rng.standard_normal((8,)).astype(np.float32)
    col = rng.standard_normal((6, 1, 1)).astype(np.float32)
    got = ((ctx.var(x) + ctx.var(bias)) * ctx.var(col)).eval(ctx)
    ref = ((RV(x) + RV(bias)) * RV(col)).eval().numpy()
    assert rel_err(got, ref) <= 1e-4
    # transposed + sliced inputs: generic strided index path
    xv = ctx.var(x)
    got = (xv.transpose(0, 2).slice(1, 1, 4) * 2.0).eval(ctx)
    ref = (R.slice_(R.transpose(RV(x), 0, 2), 1, 1, 4) * 2.0).eval().numpy()
    assert np.array_equal(got, ref)
    # ragged (not a multiple of 4) and tiny sizes
    for n in (1, 3, 5, 1023):
        v = rng.standard_normal((n,)).astype(np.float32)
        assert np.array_equal((ctx.var(v) * 2.0 + 1.0).eval(ctx), (RV(v) * 2.0 + 1.0).eval().numpy()) or \
            rel_err((ctx.var(v) * 2.0 + 1.0).eval(ctx), (RV(v) * 2.0 + 1.0).eval().numpy()) <= 1e-6


# ------------------------------------------------------------------------------ reductions
@pytest.mark.parametrize("shape,axes,preserve", [
    ((64, 1000), [1], True), ((64, 1000), [0], False), ((7, 9, 11, 5), [0, 2], False), ((7, 9, 11, 5), [3, 1], True),
    ((3, 20000), [1], False), ((5000, 3), [0], False), ((2, 3, 4), [0, 1, 2], False), ((1, 1), [1], True),
    ((128, 7, 7, 64), [0, 1, 2], False), ((6272, 100), [0], True), ((40000, 33), [0], False), ((70, 512), [0], False),
    ((2048, 1536), [0, 1], False), ((2, 300000), [1], True), ((3, 512, 256), [1, 2], False),  # long runs, few outputs: two stages
    ((4096, 768), [0], False), ((1000, 260), [0], True),      # column sums cut into row chunks, 16-byte loads
    ((2, 8192), [0], False), ((8, 16384), [0], True), ((11, 4100), [0], False), ((63, 4096), [0], False),  # few slices of a long run
    ((20000, 128), [1], False), ((16384, 68), [1], True), ((10000, 512), [1], False)])  # many short rows: eight lanes per row
@pytest.mark.parametrize("kind", ["sum", "max", "min", "prod"])
def test_reduce_vs_oracle(ctx, shape, axes, preserve, kind):
    rng = np.random.default_rng(10)
    x = rng.uniform(-1.5, 1.5, shape).astype(np.float32)
    if kind == "prod":
        x = rng.uniform(0.9, 1.1, shape).astype(np.float32)
    got = getattr(ctx.var(x), kind)(axes, preserve).eval(ctx)
    ref = R.reduce(RV(x), axes, preserve, kind).eval().numpy()
    if kind in ("max", "min", "prod"):  # prod is identically 0 in the reference (accumulator starts at 0)
        assert np.array_equal(got, ref)
    else:
        n_red = int(np.prod([shape[a] for a in axes]))
        # a sum of n terms in a different order: bounded by n * eps * sum|x|; compare against that scale
        scale = np.abs(x).sum(axis=tuple(axes), keepdims=preserve).reshape(ref.shape)
        assert np.all(np.abs(got.astype(np.float64) - ref) <= 1e-6 * np.maximum(scale, 1e-30) * max(1, np.log2(n_red)))


def test_column_sums_repeat_bit_for_bit(ctx):
    # The block that draws the last ticket of a column tile combines the chunks' partial rows; the tickets must be
    # back at zero for the next launch, and the order of combination must not depend on which block came last.
    rng = np.random.default_rng(110)
    for shape in ((4096, 768), (6272, 100), (5000, 2304)):
        x = rng.standard_normal(shape).astype(np.float32)
        first = ctx.var(x).sum([0], False).eval(ctx)
        for _ in range(5):
            assert np.array_equal(ctx.var(x).sum([0], False).eval(ctx), first)
        assert np.all(np.abs(first - x.astype(np.float64).sum(0)) <= 1e-5 * np.abs(x).sum(0))
    xi = rng.integers(-1000, 1000, (3000, 520)).astype(np.int32)
    assert np.array_equal(ctx.var(xi).sum([0], False).eval(ctx), xi.sum(axis=0, dtype=np.int32))
    assert np.array_equal(ctx.var(xi).max([0], False).eval(ctx), np.maximum(xi.max(axis=0), 0))  # the accumulator starts at 0


def test_reduce_int_exact_and_true_identities():
    c = S.Context(0, ref_compat=0)
    try:
        x = np.random.default_rng(11).integers(-50, 50, (17, 33)).astype(np.int32)
        assert np.array_equal(c.var(x).sum([1]).eval(c), x.sum(axis=1, dtype=np.int32))
        assert np.array_equal(c.var(x).max([0]).eval(c), x.max(axis=0))
        f = -np.abs(np.random.default_rng(12).standard_normal((5, 9))).astype(np.float32)
        assert np.array_equal(c.var(f).max([1]).eval(c), f.max(axis=1))  # with true identities max of negatives is negative
    finally:
        c.close()


def test_argmax_argmin_exact(ctx):
    rng = np.random.default_rng(13)
    for shape, axis in (((40, 300), 1), ((300, 40), 0), ((6, 7, 8), 1), ((3, 5000), 1)):
        x = rng.integers(-3, 3, shape).astype(np.float32)  # many ties: first extremum must win
        x.flat[::17] = np.nan
        for fn, rfn in ((S.argmax, R.argmax), (S.argmin, R.argmin)):
            got = fn(ctx.var(x), axis, False).eval(ctx)
            ref = rfn(RV(x), axis, False).eval().numpy()
            assert got.dtype == np.uint32 and np.array_equal(got, ref)


# ------------------------------------------------------------------------------ gather / scatter
def test_gather_scatter_exact(ctx):
    rng = np.random.default_rng(14)
    x = rng.standard_normal((50, 64)).astype(np.float32)
    idx = rng.integers(0, 64, (50, 1)).astype(np.uint32)
    got = S.gather(ctx.var(x), ctx.var(idx), 1).eval(ctx)
    assert np.array_equal(got, R.gather(RV(x), RV(idx, R.UINT), 1).eval().numpy())
    # embedding-style: stride-0 expanded index along the last axis (src/layers.rs:438-446)
    w = rng.standard_normal((100, 24)).astype(np.float32)
    ids = rng.integers(0, 100, (33,)).astype(np.uint32)
    iv = S.expand(ctx.var(ids).view([33, 1]), [33, 24])
    got = S.gather(ctx.var(w), iv, 0).eval(ctx)
    assert np.array_equal(got, w[ids])
    # rows that are not a whole number of 16-byte chunks take the per-element kernel; a batched table takes the row kernel
    w2 = rng.standard_normal((100, 26)).astype(np.float32)
    assert np.array_equal(S.gather(ctx.var(w2), S.expand(ctx.var(ids).view([33, 1]), [33, 26]), 0).eval(ctx), w2[ids])
    w3 = rng.standard_normal((5, 100, 32)).astype(np.float32)
    ids3 = rng.integers(0, 100, (5, 33, 1)).astype(np.uint32)
    got = S.gather(ctx.var(w3), S.expand(ctx.var(ids3), [5, 33, 32]), 1).eval(ctx)
    assert np.array_equal(got, np.take_along_axis(w3, np.broadcast_to(ids3, (5, 33, 32)).astype(np.int64), axis=1))
    big = rng.standard_normal((3000, 768)).astype(np.float32)
    idb = rng.integers(0, 3000, (4096,)).astype(np.uint32)
    assert np.array_equal(S.gather(ctx.var(big), S.expand(ctx.var(idb).view([4096, 1]), [4096, 768]), 0).eval(ctx), big[idb])
    # scatter with unique indices is bit-exact with the reference's read-modify-write
    g = rng.standard_normal((50, 1)).astype(np.float32)
    got = S.scatter(ctx.var(g), ctx.var(idx), 1, [50, 64]).eval(ctx)
    ref = R.scatter(RV(g), RV(idx, R.UINT), 1, [50, 64]).eval().numpy()
    assert np.array_equal(got, ref)


# ------------------------------------------------------------------------------ composites
@pytest.mark.parametrize("shape", [(64, 128), (33, 768), (5, 1000), (7, 130), (3, 5000), (2, 3, 16, 16)])
def test_softmax_lse_layernorm_vs_oracle(ctx, shape):
    rng = np.random.default_rng(15)
    x = (rng.standard_normal(shape) * 3).astype(np.float32)
    ax = len(shape) - 1
    assert rel_err(S.softmax(ctx.var(x), [ax]).eval(ctx), R.softmax(RV(x), [ax]).eval().numpy()) <= 1e-4
    assert rel_err(S.log_sum_exp(ctx.var(x), [ax]).eval(ctx), R.log_sum_exp(RV(x), [ax]).eval().numpy()) <= 1e-4
    g, b = np.float32([1.3]), np.float32([-0.2])
    got = S.layer_norm(ctx.var(x), [ax], ctx.var(g), ctx.var(b), 1e-5).eval(ctx)
    ref = R.layer_norm(RV(x), [ax], RV(g), RV(b), 1e-5).eval().numpy()
    # normalised outputs cross zero: an fp32 rounding of ~1 ulp of an O(1) value is a large fraction
    # of an output that happens to be ~0, so the floor is 1e-2 of the largest output
    assert rel_err(got, ref, floor=1e-2) <= 1e-4


def test_fused_and_unfused_composites_agree():
    rng = np.random.default_rng(16)
    x = rng.standard_normal((40, 96)).astype(np.float32)
    outs = []
    for fusion in (1, 0):
        c = S.Context(0, pattern_fusion=fusion)
        try:
            v = c.var(x)
            g, b = c.var(np.float32([1.0])), c.var(np.float32([0.5]))
            outs.append((S.softmax(v, [1]).eval(c), S.layer_norm(v, [1], g, b, 1e-5).eval(c), S.log_sum_exp(v, [1]).eval(c)))
        finally:
            c.close()
    for a, b in zip(*outs):
        assert rel_err(a, b, floor=1e-2) <= 1e-4


# ------------------------------------------------------------------------------ config 1 (BASELINE): fused map + reduce graph
def config1(n, c, seed=1001):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, c), dtype=np.float32)
    y = rng.standard_normal((n, c), dtype=np.float32)
    labels = rng.integers(0, c, (n, 1)).astype(np.uint32)
    return x, y, labels


def test_config1_forward_and_grad(ctx):
    x, y, labels = config1(1024, 1024)
    xv, yv, lv = ctx.var(x), ctx.var(y), ctx.var(labels)
    loss = S.softmax_cross_entropy(xv * yv + xv * 3.14, lv)
    gx = xv.grad(loss)
    ctx.eval(loss, gx)
    rx, ry, rl = RV(x), RV(y), RV(labels, R.UINT)
    rloss = R.softmax_cross_entropy(rx * ry + rx * 3.14, rl)
    rgx = rx.grad(rloss)
    ref_loss, ref_gx = [t.numpy() for t in R.evaluate([rloss, rgx])]
    assert rel_err(ctx.read(loss), ref_loss) <= 1e-4
    assert rel_err(ctx.read(gx), ref_gx, floor=1e-5) <= 1e-4


def row_graph(M, x, y, idx, pick):
    """A graph that stays inside one [R, C] row space: maps, all four reductions over axis 1 (both
    `preserve` forms), a gather and a scatter along the row, integer and uint values, a broadcast scalar."""
    n = x.extent(0)
    z = x * y + M.abs_(x) * 0.5
    hi, lo = M.max_(z, [1], True), M.min_(z, [1], False)
    e = M.exp(z - hi)
    soft = e / M.sum_(e, [1], True)
    picked = M.gather(z, idx, 1)                                      # [R, 1]
    onehot = M.scatter(picked * 2.0, pick, 1, [n, x.extent(1)])
    count = M.sum_(M.float_(M.gt(z, M.scalar(0.0, [1]))), [1], True)  # uint -> float
    small = M.prod(y * 0.01 + 1.0, [1], True)
    full = soft * count + onehot - M.view(lo, [n, 1]) * M.float_(M.int_(z)) + small
    row = M.sum_(full, [1], False) + M.view(picked, [n])
    return full, row, hi


@pytest.mark.parametrize("rows,cols", [(1024, 1024), (37, 301), (5, 130), (9, 4100), (3, 8192), (4, 10000), (2, 16384)])
def test_row_program_vs_oracle_and_kernel_by_kernel(rows, cols):
    rng = np.random.default_rng(1100 + cols)
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    y = rng.standard_normal((rows, cols), dtype=np.float32)
    idx = rng.integers(0, cols, (rows, 1)).astype(np.uint32)
    pick = rng.integers(0, cols, (rows, 1)).astype(np.int32)
    outs = []
    for fusion in (1, 5):  # 1: whole-row program; 5: the same graph kernel by kernel
        c = S.Context(0, pattern_fusion=fusion)
        try:
            targets = row_graph(S, c.var(x), c.var(y), c.var(idx), c.var(pick))
            c.trace_begin()
            c.eval(*targets)
            assert (c.trace() == ["sage_row_program"]) == (fusion == 1)
            outs.append([c.read(t) for t in targets])
            assert c.status_word() == 0
        finally:
            c.close()
    ref = [t.numpy() for t in R.evaluate(list(row_graph(R, RV(x), RV(y), RV(idx, R.UINT), RV(pick, R.INT))))]
    for a, b, r in zip(outs[0], outs[1], ref):
        assert a.shape == b.shape == r.shape
        assert rel_err(a, b, floor=1e-4) <= 1e-4      # f32 rel <= 1e-4 between the two partitions into kernels
        assert rel_err(a, r, floor=1e-4) <= 1e-4      # and against the oracle
    assert np.array_equal(outs[0][2], outs[1][2])      # the row maxima are exact either way


def test_row_program_reads_evaluated_states(ctx):
    """Leaves of a row program may be values the session already holds."""
    rng = np.random.default_rng(1200)
    x = rng.standard_normal((64, 512), dtype=np.float32)
    xv = ctx.var(x)
    z = (xv * 2.0).exp()
    ctx.eval(z)                                   # now a state of the session
    out = (z / z.sum([1], True) + xv).max([1], False)
    ctx.trace_begin()
    got = out.eval(ctx)
    assert ctx.trace() == ["sage_row_program"] and "(2 inputs -> 1 outputs)" in ctx.describe()
    e = np.exp(2.0 * x.astype(np.float64))
    ref = (e / e.sum(1, keepdims=True) + x).max(1)
    assert rel_err(got, ref.astype(np.float32), floor=1e-4) <= 1e-4
    ctx.clear()


# ------------------------------------------------------------------------------ config 2: contractions
def gemm_err(got, ref):
    """Contractions: |a - b| / max(|b|, rms(b)).  An output that cancels to ~0 carries the rounding of
    K products of ordinary size, so it is measured against the typical output, not against itself."""
    a, b = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert a.shape == b.shape
    rms = max(float(np.sqrt((b ** 2).mean())), 1e-30)
    return float((np.abs(a - b) / np.maximum(np.abs(b), rms)).max())


@pytest.mark.parametrize("m,n,k", [(1024, 1024, 1024), (1, 1, 1), (7, 13, 5), (129, 257, 63), (128, 768, 3072), (300, 2, 768),
                                   (576, 64, 6272), (128, 512, 4608), (64, 128, 2052)])  # the last three: split over K
def test_matmul_vs_oracle(ctx, m, n, k):
    rng = np.random.default_rng(2001)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    got = S.matmul(ctx.var(a), ctx.var(b)).eval(ctx)
    ref = R.matmul(RV(a), RV(b)).eval().numpy()
    assert gemm_err(got, ref) <= 1e-4
    f64 = a.astype(np.float64) @ b.astype(np.float64)
    assert np.linalg.norm(got - f64) / max(np.linalg.norm(f64), 1e-30) <= 2e-6
    # the strict elementwise metric against the envelope of the oracle's FMA / non-FMA sums
    check_envelope("matmul %dx%dx%d" % (m, n, k), got, lambda: R.matmul(RV(a), RV(b)).eval().numpy(), f64)


def test_matmul_operand_split_at_the_edges_of_the_format(ctx):
    """The tf32 hi / lo split of the operands: values whose rounding to tf32 would overflow are truncated instead,
    a subnormal stays harmless, a NaN poisons exactly its row, ties round away from zero."""
    rng = np.random.default_rng(2011)
    m, n, k = 256, 128, 64
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(0.25, 1, (k, n)).astype(np.float32)
    a[3, :] = 0.0
    a[3, 5] = np.float32(3.4028234e38)          # the largest finite value: rounds to infinity in tf32, must not
    b[5, :] = 0.5
    a[7, :] = 0.0
    a[7, 9] = np.float32(1e-41)                 # subnormal
    a[11, 2] = np.nan
    a[13, :] = 0.0
    a[13, 1] = np.frombuffer(np.uint32(0x3f801000).tobytes(), np.float32)[0]   # exactly half way between two tf32 values
    a[13, 2] = -a[13, 1]
    b[1, :] = 1.0
    b[2, :] = 0.5
    got = S.matmul(ctx.var(a), ctx.var(b)).eval(ctx)
    f64 = a.astype(np.float64) @ b.astype(np.float64)
    assert np.all(np.isfinite(got[3])) and np.allclose(got[3], f64[3], rtol=1e-6)
    assert np.all(np.isfinite(got[7])) and np.all(np.abs(got[7]) <= 2e-41)   # (the tensor core may flush a subnormal operand)
    assert np.all(np.isnan(got[11]))
    finite_rows = [r for r in range(m) if r != 11]
    assert np.all(np.isfinite(got[finite_rows]))
    assert np.allclose(got[13], f64[13], rtol=1e-6)   # hi + lo carry the value exactly whichever way the tie went
    rest = [r for r in range(m) if r not in (3, 7, 11, 13)]
    assert gemm_err(got[rest], f64[rest]) <= 1e-5
    assert ctx.status_word() == 0


@pytest.mark.parametrize("m,n,k", [(200, 136, 72), (320, 72, 4480)])  # the second: few tiles, long K, split over K
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_transposes_vs_oracle(ctx, ta, tb, m, n, k):
    rng = np.random.default_rng(2002)
    a = rng.uniform(-1, 1, (k, m) if ta else (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, k) if tb else (k, n)).astype(np.float32)
    got = S.gemm(ctx.var(a), ctx.var(b), ta, tb).eval(ctx)
    ref = R.gemm(RV(a), RV(b), bool(ta), bool(tb)).eval().numpy()
    assert gemm_err(got, ref) <= 1e-4
    f64 = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    check_envelope("gemm t%d%d %dx%dx%d" % (ta, tb, m, n, k), got, lambda: R.gemm(RV(a), RV(b), bool(ta), bool(tb)).eval().numpy(), f64)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_skinny_gemm_vs_oracle(ctx, ta, tb):
    """Few outputs, long K (the classifier head's shape): the warp-per-output kernel."""
    rng = np.random.default_rng(2004)
    m, n, k = 32, 3, 771
    a = rng.uniform(-1, 1, (k, m) if ta else (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, k) if tb else (k, n)).astype(np.float32)
    ctx.trace_begin()
    got = S.gemm(ctx.var(a), ctx.var(b), ta, tb).eval(ctx)
    assert "gemm_simt" in ctx.trace()
    ref = R.gemm(RV(a), RV(b), bool(ta), bool(tb)).eval().numpy()
    assert gemm_err(got, ref) <= 1e-4
    f64 = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    check_envelope("skinny gemm t%d%d" % (ta, tb), got, lambda: R.gemm(RV(a), RV(b), bool(ta), bool(tb)).eval().numpy(), f64)
    a3 = rng.uniform(-1, 1, (5, 8, 300)).astype(np.float32)
    b3 = rng.uniform(-1, 1, (5, 300, 2)).astype(np.float32)
    got = S.matmul_batched(ctx.var(a3), ctx.var(b3)).eval(ctx)
    assert gemm_err(got, a3.astype(np.float64) @ b3.astype(np.float64)) <= 1e-4


@pytest.mark.parametrize("sa,sb", [((16, 512, 64), (16, 64, 512)), ((16, 512, 512), (16, 512, 64)), ((3, 5, 7), (3, 7, 2))])
def test_batch_matmul_vs_oracle(ctx, sa, sb):
    rng = np.random.default_rng(2003)
    a = rng.uniform(-1, 1, sa).astype(np.float32)
    b = rng.uniform(-1, 1, sb).astype(np.float32)
    got = S.matmul_batched(ctx.var(a), ctx.var(b)).eval(ctx)
    ref = R.matmul_batched(RV(a), RV(b)).eval().numpy()
    assert gemm_err(got, ref) <= 1e-4
    check_envelope("matmul_batched %s x %s" % (sa, sb), got, lambda: R.matmul_batched(RV(a), RV(b)).eval().numpy(),
                   a.astype(np.float64) @ b.astype(np.float64))


@pytest.mark.parametrize("n", [4096, 8192])
def test_matmul_large_properties(ctx, n):
    """At the full BASELINE sizes the oracle is too slow; use size-independent properties:
    sampled rows against float64, and linearity A(B1 + B2) = A B1 + A B2."""
    rng = np.random.default_rng(2004 + n)
    a = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    va, vb = ctx.var(a), ctx.var(b)
    got = S.matmul(va, vb).eval(ctx)
    rows = rng.integers(0, n, 16)
    f64 = a[rows].astype(np.float64) @ b.astype(np.float64)
    # With K >= 4096 any fp32 accumulation (the reference's sequential one included) is ~1e-4
    # absolute away from the exact value, which exceeds 1e-4 of outputs that cancel to ~0.  So the
    # error is measured against max(|c|, rms(c)), and must not exceed what the oracle's own
    # sequential-k fp32 sum shows on the same rows (with a factor 2 of slack).
    rms = float(np.sqrt((f64 ** 2).mean()))
    err = lambda c: float((np.abs(c - f64) / np.maximum(np.abs(f64), rms)).max())
    oracle_rows = R.matmul(RV(a[rows]), RV(b)).eval().numpy()
    assert err(got[rows]) <= max(1e-4, 2 * err(oracle_rows))
    assert err(got[rows]) <= 1e-4
    b2 = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    vb2 = ctx.var(b2)
    lhs = S.matmul(va, vb + vb2).eval(ctx)
    rhs = got + S.matmul(va, vb2).eval(ctx)
    assert np.linalg.norm(lhs - rhs) / np.linalg.norm(rhs) <= 1e-5


# ------------------------------------------------------------------------------ conv / pooling
def test_conv_pool_vs_oracle(ctx):
    rng = np.random.default_rng(5001)
    x = rng.standard_normal((3, 17, 19, 5)).astype(np.float32)
    f = (rng.standard_normal((3, 3, 5, 8)) * 0.2).astype(np.float32)
    for stride, pad in ((1, 1), (2, 1), (2, 0)):
        got = S.conv_2d(ctx.var(x), ctx.var(f), stride, pad, 1).eval(ctx)
        ref = R.conv_2d(RV(x), RV(f), stride, pad, 1).eval().numpy()
        assert gemm_err(got, ref) <= 1e-4
        cols = R.im2col(RV(x), [3, 3], stride, pad, 1).eval().numpy().astype(np.float64)
        f64 = cols.reshape(-1, 45) @ f.astype(np.float64).reshape(45, 8)
        check_envelope("conv_2d stride %d pad %d" % (stride, pad), got.reshape(-1, 8),
                       lambda: R.conv_2d(RV(x), RV(f), stride, pad, 1).eval().numpy().reshape(-1, 8), f64)
    got = S.max_pool_2d(ctx.var(x), 3, 2, 1, 1).eval(ctx)
    assert np.array_equal(got, R.max_pool_2d(RV(x), 3, 2, 1, 1).eval().numpy())
    got = S.avg_pool_2d(ctx.var(x), [19, 17], [19, 17], 0, 1).eval(ctx)
    assert rel_err(got, R.avg_pool_2d(RV(x), [19, 17], [19, 17], 0, 1).eval().numpy(), floor=1e-3) <= 1e-4


@pytest.mark.parametrize("shape,filt,stride,pad", [((3, 17, 19, 5), (3, 3, 5, 8), 2, 1), ((2, 40, 40, 64), (3, 3, 64, 96), 1, 1)])
def test_conv2d_entry_point_on_caller_buffers(ctx, shape, filt, stride, pad):
    """sage_conv2d_nhwc: conv_2d (src/ops/conv.rs:61-96) over buffers the caller owns; the second case has
    C % 32 == 0 and an image above 128 KiB, so it runs as an implicit GEMM on the tensor cores."""
    rng = np.random.default_rng(5002)
    x = rng.standard_normal(shape).astype(np.float32)
    f = (rng.standard_normal(filt) * 0.1).astype(np.float32)
    ref = R.conv_2d(RV(x), RV(f), stride, pad, 1).eval().numpy()
    xt, ft, yt = ctx.tensor(x), ctx.tensor(f), ctx.empty(ref.shape)
    cx, cf, cy = xt.c(), ft.c(), yt.c()
    win = S.window(1, stride, pad, 1)
    import ctypes
    ctx._ck(S.lib.sage_conv2d_nhwc(ctx.h, ctypes.byref(cx), ctypes.byref(cf), ctypes.byref(win), ctypes.byref(cy)))
    assert gemm_err(yt.numpy(), ref) <= 1e-4
    bad = ctx.empty((1, 2, 3, 4)).c()
    assert S.lib.sage_conv2d_nhwc(ctx.h, ctypes.byref(cx), ctypes.byref(cf), ctypes.byref(win), ctypes.byref(bad)) == 1
    assert ctx.status_word() == 0
    for t in (xt, ft, yt):
        t.release()


# ------------------------------------------------------------------------------ models
def init_params(rng, shapes, std=0.02):
    return [(rng.standard_normal(s) * std).astype(np.float32) for s in shapes]


def run_bert(ctx, cfg, batch, seq, seed, pad=False, **ref_kw):
    rng = np.random.default_rng(seed)
    model = S.Bert(**cfg)
    params = model.params()
    values = init_params(rng, [p.extents for p in params])
    for p, v in zip(params, values):
        ctx.set(p, v)
    ids = rng.integers(0, cfg.get("num_vocabs", 30522), (batch, seq)).astype(np.uint32)
    mask = np.ones((batch, seq), np.float32)
    if pad:
        for i, p in enumerate(rng.integers(0, seq // 4 + 1, batch)):
            mask[i, seq - p:] = 0
    logits = model.pass_(ctx.var(ids), ctx.var(mask)).eval(ctx)
    rc = R.BertConfig(embed_dim=cfg.get("embed_dim", 768), num_vocabs=cfg.get("num_vocabs", 30522),
                      max_num_tokens=cfg.get("max_num_tokens", 512), hidden_dim=cfg.get("hidden_dim", 3072),
                      num_layers=cfg.get("num_layers", 12), num_heads=cfg.get("num_heads", 12),
                      num_classes=cfg.get("num_classes", 2), **ref_kw)
    rm = R.Bert(rc)
    rp = rm.params()
    assert [tuple(p.extents) for p in rp] == [tuple(p.extents) for p in params]  # same traversal order
    for p, v in zip(rp, values):
        p.set(v)
    ref = rm(RV(ids, R.UINT), RV(mask)).eval().numpy()
    return logits, ref


def test_bert_small_vs_oracle(ctx):
    cfg = dict(embed_dim=64, num_vocabs=150, max_num_tokens=64, hidden_dim=128, num_layers=2, num_heads=2, num_classes=10)
    got, ref = run_bert(ctx, cfg, batch=3, seq=20, seed=3001, pad=True)
    assert got.shape == (3, 10) and rel_err(got, ref, floor=1e-3) <= 1e-3


def test_bert_gelu_variant_vs_oracle(ctx):
    cfg = dict(embed_dim=64, num_vocabs=150, max_num_tokens=64, hidden_dim=128, num_layers=2, num_heads=2, num_classes=4,
               gelu=1, layer_norm_eps=1e-12)
    got, ref = run_bert(ctx, cfg, batch=2, seq=16, seed=3002, gelu=True, ln_eps=1e-12)
    assert rel_err(got, ref, floor=1e-3) <= 1e-3


def test_bert_base_vs_oracle(ctx):
    """BASELINE config 3 at reduced batch (the oracle's sequential-k CPU GEMM sets the time):
    the reference's BertConfig::base(), seq 128, batch 2."""
    got, ref = run_bert(ctx, {}, batch=2, seq=128, seed=3001)
    assert got.shape == (2, 2) and rel_err(got, ref, floor=1e-3) <= 1e-3


def test_bert_base_gelu_eps_variant_vs_oracle(ctx):
    """The extra variant of BASELINE config 3: erf-GELU feed-forward and LayerNorm eps 1e-12 at base width
    (12 layers, 768, 12 heads, FFN 3072), seq 128, batch 2, the same seeded weights as the ReLU test."""
    cfg = dict(gelu=1, layer_norm_eps=1e-12)
    got, ref = run_bert(ctx, cfg, batch=2, seq=128, seed=3001, gelu=True, ln_eps=1e-12)
    assert got.shape == (2, 2) and rel_err(got, ref, floor=1e-3) <= 1e-3
    ctx.clear()


@pytest.mark.parametrize("batch_norm", [False, True])
def test_resnet18_vs_oracle(ctx, batch_norm):
    """batch_norm=True: the extra variant of BASELINE config 5 — inference BatchNorm after every convolution where
    the reference has it commented out (src/models/resnet.rs:80,167,170), running mean 0 / variance 1, gamma 1,
    beta 0, eps 1e-5; a second pass uses non-trivial statistics so that the normalisation really acts."""
    rng = np.random.default_rng(5002)
    model = S.ResNet18(3, 10, batch_norm=batch_norm)
    params = model.params()
    values = []
    for p in params:
        if len(p.extents) == 4:
            fan_in = p.extents[0] * p.extents[1] * p.extents[2]
            values.append((rng.standard_normal(p.extents) * np.sqrt(2.0 / fan_in)).astype(np.float32))
        elif len(p.extents) == 2:
            values.append((rng.standard_normal(p.extents) * 0.02).astype(np.float32))
        else:
            values.append((rng.standard_normal(p.extents) * 0.01).astype(np.float32))
    if batch_norm:  # gamma / beta are the only [1] parameters; set them by name order: gamma first
        flip = 0
        for i, p in enumerate(params):
            if tuple(p.extents) == (1,):
                values[i] = np.float32([1.0 if flip == 0 else 0.0])
                flip ^= 1
    for p, v in zip(params, values):
        ctx.set(p, v)
    x = rng.standard_normal((2, 64, 64, 3)).astype(np.float32)
    rm = R.resnet18(3, 10, batch_norm)
    rp = rm.params()
    assert [tuple(p.extents) for p in rp] == [tuple(p.extents) for p in params]
    for p, v in zip(rp, values):
        p.set(v)
    bufs, rbufs = model.buffers(), rm.buffers()
    assert len(bufs) == len(rbufs) == (34 if batch_norm else 0)
    for trial in range(2 if batch_norm else 1):
        for i, (b, rb) in enumerate(zip(bufs, rbufs)):
            if trial == 0:
                v = np.zeros(b.extents, np.float32) if i % 2 == 0 else np.ones(b.extents, np.float32)
            else:
                v = (rng.standard_normal(b.extents) * 0.1 if i % 2 == 0 else rng.uniform(0.5, 1.5, b.extents)).astype(np.float32)
            ctx.set(b, v)
            rb.set(v)
        ctx.clear()
        got = model.pass_(ctx.var(x)).eval(ctx)
        ref = rm(RV(x)).eval().numpy()
        assert got.shape == (2, 10) and rel_err(got, ref, floor=1e-3) <= 1e-3
    assert ctx.status_word() == 0


# ------------------------------------------------------------------------------ runtime behaviour
@pytest.mark.parametrize("name,shape", [("densenet121", (8, 32, 32, 3)), ("densenet169", (2, 16, 16, 1)), ("mobilenet_v2", (4, 64, 64, 3))])
def test_densenet_and_mobilenet_vs_oracle(ctx, name, shape):
    """The reference's other two image models (src/models/densenet.rs, src/models/mobilenet.rs) as it builds them:
    DenseNet without BatchNorm or dropout, channel concatenation after every bottleneck; MobileNetV2 with full
    3 x 3 convolutions of padding 0 and dilation 0.  Logits rel <= 1e-3 against the oracle evaluating the same graph."""
    rng = np.random.default_rng(5100)
    if name == "densenet121":
        model, rmodel = S.DenseNet(shape[3], 10), R.densenet(shape[3], 10)
    elif name == "densenet169":
        model, rmodel = S.DenseNet(shape[3], 7, 169, 24), R.densenet(shape[3], 7, 169, 24)
    else:
        model, rmodel = S.MobileNetV2(shape[3], 10), R.mobilenet_v2(shape[3], 10)
    params, rparams = model.params(), rmodel.params()
    assert [tuple(p.extents) for p in params] == [tuple(r.extents) for r in rparams]
    for p, r in zip(params, rparams):
        e = p.extents
        v = (rng.standard_normal(e) * (np.sqrt(1.0 / (e[0] * e[1] * e[2])) if len(e) == 4 else 0.05)).astype(np.float32)
        ctx.set(p, v)
        r.set(v.copy())
    x = rng.standard_normal(shape).astype(np.float32)
    got = model.pass_(ctx.var(x)).eval(ctx)
    ref = rmodel(RV(x)).eval().numpy()
    assert got.shape == ref.shape and np.isfinite(ref).all() and float(np.abs(ref).max()) > 0
    assert gemm_err(got, ref) <= 1e-3
    assert ctx.status_word() == 0
    ctx.clear()


def test_random_tensors_with_explicit_seeds(ctx):
    """ops::rand::uniform / normal (src/ops/rand.rs): the reference's one-round xorshift mix of (seed + index), with
    the seeds as arguments.  uniform is integer arithmetic and one correctly rounded product: equal bits;
    normal goes through log / sqrt / cos / sin: |a - b| <= 1e-5 (values of order 1)."""
    for extents, sx, sy in (([3, 1001], 12345, 678), ([4096], 0xFFFFFFF0, 0xDEADBEEF), ([1], 1, 2), ([5, 7, 3], 42, 43)):
        got = S.uniform(extents, sx, sy).eval(ctx)
        ref = R.uniform(extents, sx, sy).eval().numpy()
        assert got.shape == ref.shape and np.array_equal(got, ref)
        assert (got >= 0).all() and (got <= 1).all()
        gz = S.normal(extents, sx, sy).eval(ctx)
        rz = R.normal(extents, sx, sy).eval().numpy()
        ok = np.isfinite(rz)
        assert gz.shape == rz.shape and np.array_equal(np.isfinite(gz), ok)
        assert np.abs(gz[ok] - rz[ok]).max(initial=0.0) <= 1e-5 * max(1.0, float(np.abs(rz[ok]).max(initial=0.0)))
    a, b = S.uniform([64], 5, 6), S.uniform([64], 5, 6)
    assert np.array_equal(a.eval(ctx), b.eval(ctx))      # same seeds, same tensor
    ctx.clear()


def test_bounded_wait_runs_out_and_reports():
    """Every device-side wait has a limit.  The self-test kernel waits on a barrier nothing arrives on:
    after about a second the wait gives up, the kernel returns, the status word says so, and the
    context goes on working (no trap, no hang, no fault)."""
    import time
    c = S.Context(0)
    try:
        assert c.status_word() == 0
        t0 = time.perf_counter()
        c._ck(S.lib.sage_selftest_bounded_wait(c.h))
        assert c.status_word() == 0x140              # reading synchronises and clears the word
        assert 0.2 < time.perf_counter() - t0 < 10.0
        a = np.random.default_rng(1).uniform(-1, 1, (256, 256)).astype(np.float32)
        got = S.matmul(c.var(a), c.var(a)).eval(c)   # the context is still good
        assert gemm_err(got, a.astype(np.float64) @ a.astype(np.float64)) <= 1e-4
        assert c.status_word() == 0
    finally:
        c.close()



def test_program_cache_and_allocator_reuse(ctx):
    x = ctx.var(np.ones((256, 256), np.float32))
    y = S.softmax(x * 2.0 + 1.0, [1])
    before = ctx.programs_compiled()
    allocs0 = ctx.mem_stats()["num_device_allocs"]
    outs = []
    for i in range(5):
        ctx.set(x, np.full((256, 256), float(i), np.float32))
        ctx.clear()
        outs.append(y.eval(ctx))
    assert ctx.programs_compiled() == before + 1          # compiled once, replayed 4 times
    assert ctx.mem_stats()["num_device_allocs"] - allocs0 <= 2  # blocks are recycled, not re-allocated
    assert all(np.allclose(o, 1.0 / 256) for o in outs)
    assert ctx.status_word() == 0


@pytest.mark.parametrize("m,n,k,batch", [(4096, 3072, 768, 1), (4096, 3072, 96, 1), (2048, 1500, 160, 1), (1024, 1216, 64, 6), (3000, 1100, 100, 1)])
def test_gemm_with_ragged_column_tiles(ctx, monkeypatch, m, n, k, batch):
    """A launch of 256-wide tiles whose last wave would be badly filled ends each row block with 192-wide tiles instead
    (4096 x 3072: nine 256-wide and four 192-wide column tiles).  A narrow tile runs the same code with a smaller N in its
    MMAs, so every element is computed exactly as with uniform tiles: equal bits with SAGE_GEMM_RAGGED=0; also against
    float64, and with the bias + relu epilogue and transposed operands."""
    rng = np.random.default_rng(77 + n + k)
    a = rng.uniform(-1, 1, (batch, m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (batch, k, n)).astype(np.float32)
    bias = rng.standard_normal((n,)).astype(np.float32)
    f64 = a.astype(np.float64) @ b.astype(np.float64)
    va, vb, vbias = ctx.var(a), ctx.var(b), ctx.var(bias)
    vbt = ctx.var(np.ascontiguousarray(b.transpose(0, 2, 1)))  # the same B stored [n, k]
    outs = {}
    for ragged in ("1", "0"):
        monkeypatch.setenv("SAGE_GEMM_RAGGED", ragged)  # read at every launch
        ctx.clear()
        y = S.matmul_batched(va, vb) if batch > 1 else S.matmul(va.view([m, k]), vb.view([k, n]))
        plain = y.eval(ctx).reshape(batch, m, n)
        fused = None
        if batch == 1:
            fused = S.relu(S.matmul(va.view([m, k]), vb.view([k, n])) + vbias).eval(ctx)
            tb = S.gemm(va.view([m, k]), vbt.view([n, k]), False, True).eval(ctx)
            assert np.array_equal(tb, plain[0])
        outs[ragged] = (plain, fused)
    assert np.array_equal(outs["1"][0], outs["0"][0])
    assert gemm_err(outs["1"][0], f64) <= 1e-4
    assert np.linalg.norm(outs["1"][0] - f64) / np.linalg.norm(f64) <= 2e-6
    if batch == 1:
        assert np.array_equal(outs["1"][1], outs["0"][1])
        assert gemm_err(outs["1"][1], np.maximum(f64[0] + bias, 0)) <= 1e-4
    assert ctx.status_word() == 0
    ctx.clear()


@pytest.mark.parametrize("m,n,k,batch", [(4096, 768, 768, 1), (4096, 3072, 768, 1), (4096, 768, 3072, 1), (128, 25600, 512, 1), (512, 640, 1024, 5),
                                         (300, 1000, 2100, 1), (4096, 768, 200, 1)])
def test_gemm_shapes_whose_tiles_are_shared_between_ctas(ctx, monkeypatch, m, n, k, batch):
    """Shapes whose whole tiles would fill the 148 SMs badly (64 pair tiles on 74 SM pairs, 2.6 waves, 100 tiles on 148
    CTAs ...): with SAGE_GEMM_STREAMK=1 the CTAs share the (tile, K-block) space evenly and a tile cut between two or
    three CTAs is summed through scratch (stream-K; off by default because it measured slower).  Checked against
    float64 and the oracle, with the bias + residual epilogue of the model on the first shapes, run twice (the
    hand-over flags change value per launch) with equal bits."""
    monkeypatch.setenv("SAGE_GEMM_STREAMK", "1")  # read at every launch
    rng = np.random.default_rng(2100 + n)
    a = rng.uniform(-1, 1, (batch, m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (batch, k, n)).astype(np.float32)
    f64 = a.astype(np.float64) @ b.astype(np.float64)
    va, vb = ctx.var(a), ctx.var(b)
    outs = []
    for _ in range(2):
        ctx.clear()
        y = S.matmul_batched(va, vb) if batch > 1 else S.matmul(va.view([m, k]), vb.view([k, n]))
        outs.append(y.eval(ctx).reshape(batch, m, n))
    assert np.array_equal(outs[0], outs[1])
    assert gemm_err(outs[0], f64) <= 1e-4
    assert np.linalg.norm(outs[0] - f64) / np.linalg.norm(f64) <= 2e-6
    if batch == 1 and m * n * k <= 4096 * 768 * 3072:
        ref = R.matmul(RV(a[0]), RV(b[0])).eval().numpy()
        assert gemm_err(outs[0][0], ref) <= 1e-4
    if batch == 1 and n <= 3072:  # x W + bias + residual, as the output projection and the feed-forward products run
        bias = rng.standard_normal((n,)).astype(np.float32)
        res = rng.standard_normal((m, n)).astype(np.float32)
        got = (S.matmul(va.view([m, k]), vb.view([k, n])) + ctx.var(bias) + ctx.var(res)).eval(ctx)
        assert "gemm{" in ctx.describe()
        assert gemm_err(got, f64[0] + bias + res) <= 1e-4
    assert ctx.status_word() == 0
    ctx.clear()
