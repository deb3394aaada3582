"""The op-level entry points of include/sage_cuda.h, called the way a Rust `backend::cuda` would call them:
through the C ABI, with `sage_tensor` descriptors over buffers the caller owns (strided and broadcast
operands, non-zero offsets), no graph and no session.  Every result is compared with the CPU oracle
evaluating the same operator on the same seeded arrays (call sites mirrored: src/ops/reduce.rs:258-325,
src/ops/core.rs:571-934, src/ops/map.rs:898-1175, src/ops/nn.rs:42-100, src/ops/conv.rs:289-498,
src/ops/gemm.rs:176-421, src/session/device.rs:149-164, 215-318).

Tolerances: index work (gather, scatter with unique indices, unslice, concat, argmax, im2col, max pooling,
memset) is bit-exact; f32 maps, reductions, softmax / log_sum_exp / layer_norm, average pooling and col2im are
within 1e-4 by |a - b| / max(|b|, floor * max|b|); contractions by |a - b| / max(|b|, rms(b)) <= 1e-4.
"""
import ctypes

import numpy as np
import pytest

import sage_b200 as S
from oracle import sage_ref as R

pytestmark = pytest.mark.gpu
L = ctypes.c_int64
REF = ctypes.byref


def RV(a, dtype=None):
    return R.Var.new(R.Tensor.new(a, dtype))


def rel_err(a, b, floor=1e-6):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    scale = np.maximum(np.abs(b), floor * max(float(np.abs(b).max(initial=0.0)), 1e-30))
    return float((np.abs(a - b) / scale).max(initial=0.0))


def gemm_err(got, ref):
    a, b = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    rms = max(float(np.sqrt((b ** 2).mean())), 1e-30)
    return float((np.abs(a - b) / np.maximum(np.abs(b), rms)).max())


@pytest.fixture(scope="module")
def ctx():
    c = S.Context(0)
    yield c
    assert c.status_word() == 0
    c.close()


class Held:
    """Device tensors of one test, released together."""

    def __init__(self, ctx):
        self.ctx, self.items = ctx, []

    def put(self, array):
        t = self.ctx.tensor(array)
        self.items.append(t)
        return t

    def empty(self, shape, dtype=S.F32):
        t = self.ctx.empty(shape, dtype)
        self.items.append(t)
        return t

    def embedded(self, array, lead=5, tail=3):
        """The array stored `lead` elements into a larger buffer: a tensor with a non-zero offset."""
        a = np.ascontiguousarray(array)
        flat = np.concatenate([np.full(lead, 77, a.dtype), a.ravel(), np.full(tail, 99, a.dtype)])
        t = self.put(flat)
        return t.view(a.shape, [s // 4 for s in a.strides], lead)

    def close(self):
        for t in self.items:
            t.release()


@pytest.fixture()
def held(ctx):
    h = Held(ctx)
    yield h
    h.close()


def ctensors(ts):
    arr = (S.CTensor * len(ts))()
    for i, t in enumerate(ts):
        arr[i] = t.c()
    return arr


# ------------------------------------------------------------------------------ sage_map
def test_map_entry_point_strided_broadcast_and_offset(ctx, held):
    rng = np.random.default_rng(901)
    a = rng.standard_normal((6, 5, 8)).astype(np.float32)
    b = rng.standard_normal((8,)).astype(np.float32)
    c = rng.standard_normal((8, 5, 6)).astype(np.float32)
    ta = held.embedded(a)                                  # offset 5
    tb = held.put(b).view((6, 5, 8), (0, 0, 1))            # broadcast over two axes (stride 0)
    tc = held.put(c).view((6, 5, 8), (1, 6, 30))           # a transposed view: axes (2, 1, 0) of c
    y = held.empty((6, 5, 8))
    xs = ctensors([ta, tb, tc])
    cy = y.c()
    ctx._ck(S.lib.sage_map(ctx.h, b"((x0 * x1) + (x2 * 3.14f))", xs, 3, REF(cy)))
    ref = (RV(a) * RV(b) + R.transpose(RV(c), 0, 2) * 3.14).eval().numpy()
    assert np.array_equal(y.numpy(), ref) or rel_err(y.numpy(), ref) <= 1e-6
    # a compare writes uint; a cast writes int; a nullary map has no operand at all
    yu = held.empty((6, 5, 8), S.U32)
    cu = yu.c()
    ctx._ck(S.lib.sage_map(ctx.h, b"(x0 > x1)", xs, 2, REF(cu)))
    assert np.array_equal(yu.numpy(), R.gt(RV(a), RV(b)).eval().numpy())
    yi = held.empty((6, 5, 8), S.I32)
    ci = yi.c()
    ctx._ck(S.lib.sage_map(ctx.h, b"((int)(x0 * 10.0f))", xs, 1, REF(ci)))
    assert np.array_equal(yi.numpy(), np.trunc(a * np.float32(10)).astype(np.int32))
    ctx._ck(S.lib.sage_map(ctx.h, b"(2.5f)", None, 0, REF(cy)))
    assert np.array_equal(y.numpy(), np.full((6, 5, 8), 2.5, np.float32))
    # errors, not crashes: rank mismatch, strided output
    bad = held.put(b).c()
    assert S.lib.sage_map(ctx.h, b"(x0)", REF(bad), 1, REF(cy)) == 1
    ys = y.view((6, 5, 4), (40, 8, 2)).c()
    assert S.lib.sage_map(ctx.h, b"(x0)", xs, 1, REF(ys)) == 1


# ------------------------------------------------------------------------------ sage_reduce / sage_reduce_arg
@pytest.mark.parametrize("kind,name", [(0, "sum"), (1, "prod"), (2, "max"), (3, "min")])
def test_reduce_entry_point(ctx, held, kind, name):
    rng = np.random.default_rng(902)
    x = rng.uniform(-1.5, 1.5, (7, 9, 11, 5)).astype(np.float32)
    if name == "prod":
        x = rng.uniform(0.9, 1.1, x.shape).astype(np.float32)
    tx = held.embedded(x)
    for axes in ([1], [0, 2], [3, 1], [0, 1, 2, 3]):
        ref = R.reduce(RV(x), axes, False, name).eval().numpy()
        y = held.empty(ref.shape)
        cx, cy = tx.c(), y.c()
        ax = (ctypes.c_int32 * len(axes))(*axes)
        ctx._ck(S.lib.sage_reduce(ctx.h, kind, REF(cx), ax, len(axes), REF(cy)))
        got = y.numpy()
        if name == "sum":
            scale = np.abs(x).sum(axis=tuple(axes)).reshape(ref.shape)
            assert np.all(np.abs(got.astype(np.float64) - ref) <= 1e-5 * np.maximum(scale, 1e-30))
        else:  # max / min are exact; prod is identically 0 (the reference's accumulator starts at 0)
            assert np.array_equal(got, ref)
    # a permuted (strided) input: reduce over what is axis 0 of the view
    xt = tx.view((11, 9, 7, 5), (5, 55, 495, 1), tx.offset)
    ref = R.reduce(R.transpose(RV(x), 0, 2), [0], False, name).eval().numpy()
    y = held.empty(ref.shape)
    cx, cy = xt.c(), y.c()
    ax = (ctypes.c_int32 * 1)(0)
    ctx._ck(S.lib.sage_reduce(ctx.h, kind, REF(cx), ax, 1, REF(cy)))
    assert rel_err(y.numpy(), ref, floor=1e-5) <= 1e-4
    wrong = held.empty((3,)).c()
    assert S.lib.sage_reduce(ctx.h, kind, REF(cx), ax, 1, REF(wrong)) == 1
    # integer input keeps its type
    xi = rng.integers(-50, 50, (17, 33)).astype(np.int32)
    ti, yi = held.put(xi), held.empty((17,), S.I32)
    ci, cyi = ti.c(), yi.c()
    ax = (ctypes.c_int32 * 1)(1)
    ctx._ck(S.lib.sage_reduce(ctx.h, kind, REF(ci), ax, 1, REF(cyi)))
    assert np.array_equal(yi.numpy(), R.reduce(RV(xi, R.INT), [1], False, name).eval().numpy())


def test_reduce_arg_entry_point(ctx, held):
    rng = np.random.default_rng(903)
    x = rng.integers(-3, 3, (6, 70, 8)).astype(np.float32)   # many ties: the first extremum wins
    x.flat[::17] = np.nan
    tx = held.embedded(x)
    for axis in (0, 1, 2):
        for is_max, rfn in ((1, R.argmax), (0, R.argmin)):
            ref = rfn(RV(x), axis, False).eval().numpy()
            y = held.empty(ref.shape, S.U32)
            cx, cy = tx.c(), y.c()
            ctx._ck(S.lib.sage_reduce_arg(ctx.h, is_max, REF(cx), axis, REF(cy)))
            assert np.array_equal(y.numpy(), ref)
    ci = held.put(np.zeros((4, 4), np.int32)).c()
    cy = held.empty((4,), S.U32).c()
    assert S.lib.sage_reduce_arg(ctx.h, 1, REF(ci), 1, REF(cy)) == 7   # only float input, like the reference's kernel


# ------------------------------------------------------------------------------ softmax / log_sum_exp / layer_norm
@pytest.mark.parametrize("rows,inner", [(33, 768), (5, 1000), (7, 130), (3, 5000), (64, 64)])
def test_row_composites_entry_points(ctx, held, rows, inner):
    rng = np.random.default_rng(904)
    x = (rng.standard_normal((rows, inner)) * 3).astype(np.float32)
    tx = held.embedded(x, lead=8)        # offset 8 keeps the rows 16-byte aligned or not, depending on `inner`
    y = held.empty((rows, inner))
    cx, cy = tx.c(), y.c()
    ctx._ck(S.lib.sage_softmax(ctx.h, REF(cx), L(rows), L(inner), REF(cy)))
    assert rel_err(y.numpy(), R.softmax(RV(x), [1]).eval().numpy()) <= 1e-4
    yl = held.empty((rows,))
    cl = yl.c()
    ctx._ck(S.lib.sage_log_sum_exp(ctx.h, REF(cx), L(rows), L(inner), REF(cl)))
    assert rel_err(yl.numpy(), R.log_sum_exp(RV(x), [1]).eval().numpy().reshape(rows)) <= 1e-4
    for g, b in ((np.float32([1.3]), np.float32([-0.2])),
                 (rng.uniform(0.5, 1.5, (inner,)).astype(np.float32), rng.standard_normal((inner,)).astype(np.float32))):
        cg, cb = held.put(g).c(), held.put(b).c()
        ctx._ck(S.lib.sage_layer_norm(ctx.h, REF(cx), L(rows), L(inner), REF(cg), REF(cb), ctypes.c_float(1e-5), REF(cy)))
        ref = R.layer_norm(RV(x), [1], RV(g), RV(b), 1e-5).eval().numpy()
        assert rel_err(y.numpy(), ref, floor=1e-2) <= 1e-4
    assert S.lib.sage_softmax(ctx.h, REF(cx), L(rows + 1), L(inner), REF(cy)) == 1
    cg3 = held.put(np.ones(3, np.float32)).c()
    assert S.lib.sage_layer_norm(ctx.h, REF(cx), L(rows), L(inner), REF(cg3), REF(cg3), ctypes.c_float(1e-5), REF(cy)) == 1


# ------------------------------------------------------------------------------ gather / scatter / unslice / concat
def test_gather_scatter_entry_points(ctx, held):
    rng = np.random.default_rng(905)
    x = rng.standard_normal((50, 64)).astype(np.float32)
    idx = rng.integers(0, 64, (50, 1)).astype(np.uint32)
    tx, ti = held.embedded(x), held.embedded(idx)
    y = held.empty((50, 1))
    cx, ci, cy = tx.c(), ti.c(), y.c()
    ctx._ck(S.lib.sage_gather(ctx.h, REF(cx), REF(ci), 1, REF(cy)))
    assert np.array_equal(y.numpy(), R.gather(RV(x), RV(idx, R.UINT), 1).eval().numpy())
    # the embedding lookup of src/layers.rs:438-446: a [n] index read as an expanded [n, dim] view (stride 0)
    w = rng.standard_normal((100, 24)).astype(np.float32)
    ids = rng.integers(0, 100, (33,)).astype(np.uint32)
    tw, tids = held.put(w), held.embedded(ids)
    ye = held.empty((33, 24))
    cw, cids, cye = tw.c(), tids.view((33, 24), (1, 0), tids.offset).c(), ye.c()
    ctx._ck(S.lib.sage_gather(ctx.h, REF(cw), REF(cids), 0, REF(cye)))
    assert np.array_equal(ye.numpy(), w[ids])
    # gather from a transposed source
    cwt = tw.view((24, 100), (1, 24)).c()
    idt = rng.integers(0, 100, (24, 3)).astype(np.uint32)
    cidt, yt = held.put(idt).c(), held.empty((24, 3))
    cyt = yt.c()
    ctx._ck(S.lib.sage_gather(ctx.h, REF(cwt), REF(cidt), 1, REF(cyt)))
    assert np.array_equal(yt.numpy(), R.gather(R.tr(RV(w)), RV(idt, R.UINT), 1).eval().numpy())
    # scatter (unique indices per row: same bits as the reference's read-modify-write); the entry point clears y first
    g = rng.standard_normal((50, 1)).astype(np.float32)
    tg = held.embedded(g)
    ys = held.put(np.full((50, 64), 5.0, np.float32))      # stale contents must not survive
    cg, cys = tg.c(), ys.c()
    for _ in range(2):
        ctx._ck(S.lib.sage_scatter(ctx.h, REF(cg), REF(ci), 1, REF(cys)))
        assert np.array_equal(ys.numpy(), R.scatter(RV(g), RV(idx, R.UINT), 1, [50, 64]).eval().numpy())
    assert S.lib.sage_gather(ctx.h, REF(cx), REF(cids), 1, REF(cy)) == 1   # output size does not match the index


def test_unslice_concat_entry_points(ctx, held):
    rng = np.random.default_rng(906)
    x = rng.standard_normal((7, 40, 9)).astype(np.float32)
    tx = held.embedded(x)
    for axis, start, total in ((1, 13, 70), (0, 2, 11), (2, 0, 9), (2, 5, 14)):
        shape = list(x.shape)
        shape[axis] = total
        y = held.put(np.full(shape, 3.0, np.float32))
        cx, cy = tx.c(), y.c()
        ctx._ck(S.lib.sage_unslice(ctx.h, REF(cx), axis, L(start), REF(cy)))
        ref = R.unslice(RV(x), axis, start, total).eval().numpy()   # (axis, start, end): `end` is the padded extent
        assert ref.shape == tuple(shape) and np.array_equal(y.numpy(), ref)
    # a strided source (a slice along the last axis of a wider tensor)
    wide = rng.standard_normal((7, 40, 12)).astype(np.float32)
    tw = held.put(wide)
    src = tw.view((7, 40, 9), (480, 12, 1), 2)
    y = held.empty((7, 50, 9))
    cs, cy = src.c(), y.c()
    ctx._ck(S.lib.sage_unslice(ctx.h, REF(cs), 1, L(10), REF(cy)))
    ref = np.zeros((7, 50, 9), np.float32)
    ref[:, 10:50] = wide[:, :, 2:11]
    assert np.array_equal(y.numpy(), ref)
    # concat of three operands, one of them a transposed view, along every axis
    for axis in (0, 1, 2):
        shapes = [list(x.shape) for _ in range(3)]
        shapes[0][axis], shapes[1][axis], shapes[2][axis] = 3, 1, 6
        arrs = [rng.standard_normal(s).astype(np.float32) for s in shapes]
        ts = [held.embedded(arrs[0]), held.put(arrs[1]), None]
        tr = np.ascontiguousarray(arrs[2].transpose(0, 2, 1))            # stored transposed, read back through strides
        tt = held.put(tr)
        ts[2] = tt.view(arrs[2].shape, (tr.shape[1] * tr.shape[2], 1, tr.shape[2]))
        ref = R.concat([RV(a) for a in arrs], axis).eval().numpy()
        y = held.empty(ref.shape)
        cy = y.c()
        ctx._ck(S.lib.sage_concat(ctx.h, ctensors(ts), 3, axis, REF(cy)))
        assert np.array_equal(y.numpy(), ref)


# ------------------------------------------------------------------------------ GEMM entry points
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("batch,m,n,k", [(16, 128, 96, 64), (3, 5, 7, 2), (70000, 2, 3, 4)])
def test_gemm_strided_batched_entry_point(ctx, held, ta, tb, batch, m, n, k):
    """GemmBatched::compute_direct (src/ops/gemm.rs:338-421) with padded leading dimensions, batch strides
    larger than a matrix and an offset into every buffer.  The last case has more batches than a grid's y / z
    extent allows."""
    if batch > 1000 and (ta or tb):
        pytest.skip("the many-batches case runs once")
    rng = np.random.default_rng(907)
    ar, ac = (k, m) if ta else (m, k)
    br, bc = (n, k) if tb else (k, n)
    lda, ldb, ldc = ac + 4, bc + 8, n + 4
    sa, sb, sc = ar * lda + 16, br * ldb + 4, m * ldc + 8
    A = rng.uniform(-1, 1, (batch, sa)).astype(np.float32)
    B = rng.uniform(-1, 1, (batch, sb)).astype(np.float32)
    a = np.stack([A[i, :ar * lda].reshape(ar, lda)[:, :ac] for i in range(batch)])
    b = np.stack([B[i, :br * ldb].reshape(br, ldb)[:, :bc] for i in range(batch)])
    ta_, tb_, tc_ = held.embedded(A, lead=4), held.embedded(B, lead=8), held.put(np.full((batch * sc + 12,), -7.0, np.float32))
    ctx._ck(S.lib.sage_gemm_strided_batched(ctx.h, ta, tb, L(m), L(n), L(k), ta_.buf, L(4), L(lda), L(sa), tb_.buf, L(8), L(ldb), L(sb),
                                            tc_.buf, L(12), L(ldc), L(sc), L(batch)))
    raw = tc_.numpy()
    got = np.stack([raw[12 + i * sc: 12 + i * sc + m * ldc].reshape(m, ldc)[:, :n] for i in range(batch)])
    if batch <= 1000:
        ref = R.gemm_batched(RV(a), RV(b), bool(ta), bool(tb)).eval().numpy()
    else:
        ref = np.einsum("bmk,bkn->bmn", a.astype(np.float64), b.astype(np.float64))
    assert gemm_err(got, ref) <= 1e-4
    # nothing outside the [m, n] windows was written
    pad = np.stack([raw[12 + i * sc: 12 + i * sc + m * ldc].reshape(m, ldc)[:, n:] for i in range(batch)])
    assert np.all(pad == -7.0) and np.all(raw[:12] == -7.0)


# ------------------------------------------------------------------------------ im2col / col2im / pool2d
WINDOWS = [((3, 2), (1, 1), (0, 0), (1, 1)), ((3, 3), (2, 2), (1, 1), (1, 1)), ((3, 3), (1, 2), (2, 1), (2, 1)), ((1, 1), (2, 2), (0, 0), (1, 1)),
           ((7, 7), (2, 2), (3, 3), (1, 1))]


@pytest.mark.parametrize("ker,stride,pad,dil", WINDOWS)
def test_im2col_col2im_pool_entry_points(ctx, held, ker, stride, pad, dil):
    rng = np.random.default_rng(908)
    x = rng.standard_normal((3, 17, 19, 5)).astype(np.float32)
    win = S.window(ker, stride, pad, dil)
    ref = R.im2col(RV(x), list(ker), list(stride), list(pad), list(dil)).eval().numpy()
    tx, y = held.embedded(x), held.empty(ref.shape)
    cx, cy = tx.c(), y.c()
    ctx._ck(S.lib.sage_im2col(ctx.h, REF(cx), REF(win), REF(cy)))
    assert np.array_equal(y.numpy(), ref)
    # col2im of a random column tensor (the gradient path), with the reference's dilation quirk reproduced by the oracle
    col = rng.standard_normal(ref.shape).astype(np.float32)
    rimg = R.col2im(RV(col), [19, 17], list(ker), list(stride), list(pad), list(dil)).eval().numpy()
    tcol, img = held.embedded(col), held.put(np.full(rimg.shape, 9.0, np.float32))
    cc, ci = tcol.c(), img.c()
    ctx._ck(S.lib.sage_col2im(ctx.h, REF(cc), REF(win), REF(ci)))
    assert rel_err(img.numpy(), rimg, floor=1e-4) <= 1e-4
    for is_max, rfn in ((1, R.max_pool_2d), (0, R.avg_pool_2d)):
        rp = rfn(RV(x), list(ker), list(stride), list(pad), list(dil)).eval().numpy()
        yp = held.empty(rp.shape)
        cp = yp.c()
        ctx._ck(S.lib.sage_pool2d(ctx.h, is_max, REF(cx), REF(win), REF(cp)))
        if is_max:
            assert np.array_equal(yp.numpy(), rp)
        else:
            assert rel_err(yp.numpy(), rp, floor=1e-4) <= 1e-4
    flat = held.empty((3, 17 * 19 * 5)).c()
    assert S.lib.sage_im2col(ctx.h, REF(flat), REF(win), REF(cy)) == 1


# ------------------------------------------------------------------------------ sage_module_get + sage_launch + sage_memset
KERNEL = rb"""
struct Affine { float scale; float shift; int n; };
extern "C" __global__ void affine(const float *x, float *y, Affine p, float extra, int stride, long long limit, unsigned flip) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < p.n && (long long)i < limit) y[i] = x[i * stride] * p.scale + p.shift + extra + (flip ? 1.0f : 0.0f);
}
"""


class Affine(ctypes.Structure):
    _fields_ = [("scale", ctypes.c_float), ("shift", ctypes.c_float), ("n", ctypes.c_int32)]


class SageArg(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("buf", ctypes.c_void_p), ("i", ctypes.c_int64), ("f", ctypes.c_float),
                ("bytes", ctypes.c_void_p), ("nbytes", ctypes.c_size_t)]


def test_launch_and_memset_entry_points(ctx, held):
    """KernelProgram::kernel + Kernel::arg_tensor / arg / launch (src/session/device.rs:215-318) and Buffer::fill
    (:149-164): every argument kind of sage_arg reaches the kernel with the right width."""
    rng = np.random.default_rng(909)
    n = 1000
    x = rng.standard_normal((2 * n,)).astype(np.float32)
    tx, ty = held.put(x), held.put(np.full((n + 24,), 4.0, np.float32))
    ctx._ck(S.lib.sage_memset(ctx.h, ty.buf, ctypes.c_size_t(0), 0, ctypes.c_size_t(n * 4)))       # Tensor::fill_zero
    got = ty.numpy()
    assert np.all(got[:n] == 0) and np.all(got[n:] == 4.0)
    ctx._ck(S.lib.sage_memset(ctx.h, ty.buf, ctypes.c_size_t(16), 0xFF, ctypes.c_size_t(8)))
    assert np.array_equal(ty.numpy().view(np.uint32)[4:6], np.uint32([0xFFFFFFFF] * 2))
    mod = ctypes.c_void_p()
    ctx._ck(S.lib.sage_module_get(ctx.h, KERNEL, REF(mod)))
    mod2 = ctypes.c_void_p()
    before = ctx.launch_count()
    ctx._ck(S.lib.sage_module_get(ctx.h, KERNEL, REF(mod2)))                                    # cached by source text
    par = Affine(2.0, -1.0, n)
    args = (SageArg * 7)()
    args[0].kind, args[0].buf = 0, tx.buf
    args[1].kind, args[1].buf = 0, ty.buf
    args[2].kind, args[2].bytes, args[2].nbytes = 5, ctypes.cast(ctypes.pointer(par), ctypes.c_void_p), ctypes.sizeof(par)
    args[3].kind, args[3].f = 3, 0.5
    args[4].kind, args[4].i = 1, 2
    args[5].kind, args[5].i = 4, 900
    args[6].kind, args[6].i = 2, 1
    grid, block = (ctypes.c_uint32 * 3)(8, 1, 1), (ctypes.c_uint32 * 3)(128, 1, 1)
    ctx._ck(S.lib.sage_launch(ctx.h, mod, b"affine", grid, block, 0, args, 7))
    got = ty.numpy()
    assert np.array_equal(got[:900], x[0:1800:2] * np.float32(2.0) + np.float32(-1.0) + np.float32(0.5) + np.float32(1.0))
    assert ctx.launch_count()[0] == before[0] + 1
    assert S.lib.sage_launch(ctx.h, mod, b"no_such_kernel", grid, block, 0, args, 7) != 0
    bad = ctypes.c_void_p()
    assert S.lib.sage_module_get(ctx.h, b"extern \"C\" __global__ void broken( { }", REF(bad)) == 4  # SAGE_ERR_COMPILE
    assert b"error" in S.lib.sage_last_error(ctx.h).lower()
