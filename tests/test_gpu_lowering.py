"""The evaluator's GEMM lowering on the GPU: operand views instead of organize() copies, epilogue
fusion, store patterns, grouped launches and producer-written tf32 planes must not change results.
Every case is evaluated three ways — lowered (default), with pattern_fusion = 0 (the reference's
decomposition, every operator its own kernel) and in float64 NumPy — and the lowered program is
checked to really contain the folds it is meant to exercise.

Tolerance: contractions are compared as |a - b| / max(|b|, rms(b)) <= 1e-4 against float64 (the
bound stated for f32 results); lowered vs decomposed differ only by the order of a few fp32
roundings in the epilogue (x*W + b evaluated in one kernel instead of two), so they agree to 1e-5.
"""
import numpy as np
import pytest

import sage_b200 as S

pytestmark = pytest.mark.gpu


def gemm_err(got, ref):
    a, b = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    rms = max(float(np.sqrt((b ** 2).mean())), 1e-30)
    return float((np.abs(a - b) / np.maximum(np.abs(b), rms)).max())


def softmax64(x):
    e = np.exp(x - x.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def attention_block(ctx, a, heads):
    """One post-LN transformer block written with the public ops, as src/models/bert.rs does."""
    n, l, e = a["x"].shape
    d = e // heads
    x = ctx.var(a["x"])
    v = {k: ctx.var(a[k]) for k in a if k != "x"}

    def split(t):
        return S.view(t, (n, l, heads, d)).permute((0, 2, 1, 3))
    q, k, val = (split(x.matmul(v["w" + s]) + v["b" + s]) for s in "qkv")
    scores = q.matmul_batched(k.transpose(-1, -2)) / float(np.sqrt(d)) + v["mask"]
    p = S.softmax(scores, [-1])
    merged = S.view(p.matmul_batched(val).permute((0, 2, 1, 3)), (n, l, e))
    o = merged.matmul(v["wo"]) + v["bo"] + x
    h = S.relu(o.matmul(v["w1"]) + v["b1"])
    out = h.matmul(v["w2"]) + v["b2"] + o
    return dict(scores=scores, p=p, merged=merged, o=o, out=out), v


def attention_block64(a, heads):
    f = {k: np.asarray(t, np.float64) for k, t in a.items()}
    n, l, e = f["x"].shape
    d = e // heads

    def split(t):
        return t.reshape(n, l, heads, d).transpose(0, 2, 1, 3)
    q, k, v = (split(f["x"] @ f["w" + s] + f["b" + s]) for s in "qkv")
    scores = q @ k.transpose(0, 1, 3, 2) / np.float64(np.float32(np.sqrt(d))) + f["mask"]
    p = softmax64(scores)
    merged = (p @ v).transpose(0, 2, 1, 3).reshape(n, l, e)
    o = merged @ f["wo"] + f["bo"] + f["x"]
    h = np.maximum(o @ f["w1"] + f["b1"], 0)
    out = h @ f["w2"] + f["b2"] + o
    return dict(scores=scores, p=p, merged=merged, o=o, out=out)


def block_inputs(rng, n, l, e, f):
    a = {"x": rng.standard_normal((n, l, e)).astype(np.float32)}
    for s in "qkvo":
        a["w" + s] = (rng.standard_normal((e, e)) / np.sqrt(e)).astype(np.float32)
        a["b" + s] = (rng.standard_normal(e) * 0.1).astype(np.float32)
    a["w1"] = (rng.standard_normal((e, f)) / np.sqrt(e)).astype(np.float32)
    a["b1"] = (rng.standard_normal(f) * 0.1).astype(np.float32)
    a["w2"] = (rng.standard_normal((f, e)) / np.sqrt(f)).astype(np.float32)
    a["b2"] = (rng.standard_normal(e) * 0.1).astype(np.float32)
    mask = np.zeros((n, 1, 1, l), np.float32)
    for i in range(n):  # ragged padding, as config 4 has it
        mask[i, 0, 0, l - int(rng.integers(0, l // 4 + 1)):] = -100000.0
    a["mask"] = mask
    return a


@pytest.mark.parametrize("n,l,e,heads,f", [(4, 96, 256, 4, 512), (2, 128, 768, 12, 3072), (3, 200, 128, 2, 320)])
def test_transformer_block_lowered_vs_decomposed_vs_float64(n, l, e, heads, f):
    a = block_inputs(np.random.default_rng(100 + l), n, l, e, f)
    ref = attention_block64(a, heads)
    lowered, plain = S.Context(0), S.Context(0, pattern_fusion=0)
    try:
        t1, _ = attention_block(lowered, a, heads)
        t0, _ = attention_block(plain, a, heads)
        names = list(t1)
        lowered.eval(*[t1[k] for k in names])
        plain.eval(*[t0[k] for k in names])
        d = lowered.describe()
        # the folds this test is about are really in the program
        assert "gemm_grouped" in d and "slab(" in d            # q, k, v projections: one launch
        assert "[store]" in d                                   # head merge
        assert "gemm_batched{((x0 / sg_lit(" in d               # scale + mask in the scores epilogue
        assert "planes" in d                                    # producers write the tf32 planes of what GEMMs read
        dp = plain.describe()
        assert "gemm{" not in dp and "[store]" not in dp and "gemm_grouped" not in dp and "planes" not in dp
        for k in names:
            got, dec = lowered.read(t1[k]), plain.read(t0[k])
            assert gemm_err(got, ref[k]) <= 1e-4, k
            assert gemm_err(dec, ref[k]) <= 1e-4, k
            assert gemm_err(got, dec) <= 1e-5, k
        assert lowered.status_word() == 0 and plain.status_word() == 0
    finally:
        lowered.close()
        plain.close()


def test_rewriting_a_weight_invalidates_cached_planes_and_grouped_copies():
    """Weights are split once and (for grouped launches) copied once; Var::set must make both stale."""
    rng = np.random.default_rng(7)
    a = block_inputs(rng, 2, 128, 256, 512)
    ctx = S.Context(0)
    try:
        t, v = attention_block(ctx, a, 4)
        ctx.eval(t["out"])
        first = ctx.read(t["out"])
        assert gemm_err(first, attention_block64(a, 4)["out"]) <= 1e-4
        for name in ("wk", "bq", "w2"):
            a[name] = (a[name] * np.float32(-0.5) + np.float32(0.01)).astype(np.float32)
            ctx.set(v[name], a[name])
        ctx.clear()
        ctx.eval(t["out"])
        second = ctx.read(t["out"])
        assert gemm_err(second, attention_block64(a, 4)["out"]) <= 1e-4
        assert gemm_err(second, first) > 1e-2  # and it did change
    finally:
        ctx.close()


@pytest.mark.parametrize("m,n,k", [(130, 70, 147), (257, 36, 64), (64, 33, 32), (300, 513, 100)])
def test_epilogue_on_ragged_shapes(m, n, k):
    """N not a multiple of 4 (element-wise epilogue path), K with a row pitch TMA cannot address (operand
    gathered into compact planes), tiles that hang over M and N."""
    rng = np.random.default_rng(m * 1000 + n)
    x = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n,)).astype(np.float32)
    r = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    col = rng.uniform(-1, 1, (m, 1)).astype(np.float32)
    ctx = S.Context(0)
    try:
        X, W, B, Rr, C = (ctx.var(t) for t in (x, w, b, r, col))
        y1 = S.relu(X.matmul(W) + B)
        y2 = (X.matmul(W) + B) * C + Rr       # three epilogue operands: row vector, column vector, full tensor
        y3 = (X.matmul(W) * 0.5).exp()
        ctx.eval(y1, y2, y3)
        d = ctx.describe()
        assert d.count("gemm{") == 3
        p = x.astype(np.float64) @ w.astype(np.float64)
        assert gemm_err(ctx.read(y1), np.maximum(p + b, 0)) <= 1e-4
        assert gemm_err(ctx.read(y2), (p + b) * col + r) <= 1e-4
        assert gemm_err(ctx.read(y3), np.exp(p * 0.5)) <= 1e-4
        assert ctx.status_word() == 0
    finally:
        ctx.close()


def test_transposed_and_strided_operand_views():
    """gemm(a^T), gemm over a sliced batch, and a product consumed by another product through a permute."""
    rng = np.random.default_rng(11)
    a = rng.uniform(-1, 1, (6, 96, 160)).astype(np.float32)
    b = rng.uniform(-1, 1, (6, 96, 72)).astype(np.float32)
    ctx = S.Context(0)
    try:
        A, B = ctx.var(a), ctx.var(b)
        y = A.transpose(-1, -2).matmul_batched(B)                       # [6,160,96] x [6,96,72]: A read transposed
        z = A.slice(0, 1, 5).transpose(-1, -2).matmul_batched(B.slice(0, 1, 5))
        ctx.eval(y, z)
        assert "map{(x0)}" not in ctx.describe()                        # no organize() copy survived
        ref = np.einsum("bki,bkj->bij", a.astype(np.float64), b.astype(np.float64))
        assert gemm_err(ctx.read(y), ref) <= 1e-4
        assert gemm_err(ctx.read(z), ref[1:5]) <= 1e-4
        assert ctx.status_word() == 0
    finally:
        ctx.close()


def test_planes_only_intermediates():
    """When a product (or a softmax) is read by one GEMM and nothing else, only its tf32 planes are
    written.  Evaluating just the block's output makes q/k/v, the merged context and the FFN activation
    such intermediates (and the probabilities, when the attention is kept decomposed: pattern_fusion bit 3);
    evaluating them as targets as well must give the same output."""
    a = block_inputs(np.random.default_rng(321), 2, 128, 256, 512)
    ref = attention_block64(a, 4)
    ctx, ctx2, ctx3 = S.Context(0, pattern_fusion=9), S.Context(0, pattern_fusion=9), S.Context(0)
    try:
        t, _ = attention_block(ctx, a, 4)
        ctx.eval(t["out"])
        d = ctx.describe()
        assert d.count("=planes") >= 4 and "softmax=planes" in d    # the probabilities exist only as tf32 planes
        got = ctx.read(t["out"])
        assert gemm_err(got, ref["out"]) <= 1e-4
        t2, _ = attention_block(ctx2, a, 4)
        ctx2.eval(*t2.values())                      # every intermediate materialised in fp32 too
        assert "softmax=planes" not in ctx2.describe()
        assert np.array_equal(got, ctx2.read(t2["out"]))  # the same kernels computed the same planes
        assert ctx.status_word() == 0
        # with the fused attention kernel the probabilities do not exist at all; q / k / v and its output are planes only
        t3, _ = attention_block(ctx3, a, 4)
        ctx3.eval(t3["out"])
        d3 = ctx3.describe()
        assert "softmax" not in d3 and "[store]=planes" in d3 and d3.count("=planes") >= 4 and "attention{" in d3
        assert gemm_err(ctx3.read(t3["out"]), ref["out"]) <= 1e-4 and gemm_err(ctx3.read(t3["out"]), got) <= 1e-5
        assert ctx3.status_word() == 0
    finally:
        ctx.close()
        ctx2.close()
        ctx3.close()


def conv64(x, f, stride, pad, dil):
    """float64 NHWC convolution with [KH, KW, C, OC] filters ([w, h] ordered pairs like the reference)."""
    (sw, sh), (pw, ph), (dw, dh) = stride, pad, dil
    n, h, w, c = x.shape
    kh, kw, _, oc = f.shape
    oh = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    ow = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    xp = np.zeros((n, h + 2 * ph, w + 2 * pw, c), np.float64)
    xp[:, ph:ph + h, pw:pw + w] = x
    out = np.zeros((n, oh, ow, oc), np.float64)
    for ky in range(kh):
        for kx in range(kw):
            patch = xp[:, ky * dh:ky * dh + (oh - 1) * sh + 1:sh, kx * dw:kx * dw + (ow - 1) * sw + 1:sw]
            out += patch @ f[ky, kx].astype(np.float64)
    return out


@pytest.mark.parametrize("shape,filt,stride,pad,dil", [
    ((6, 30, 34, 64), (3, 3, 64, 64), (1, 1), (1, 1), (1, 1)),      # ResNet basic block
    ((5, 31, 29, 64), (3, 3, 64, 128), (2, 2), (1, 1), (1, 1)),     # strided, odd extents, tiles span rows and images
    ((4, 28, 28, 128), (1, 1, 128, 96), (2, 2), (0, 0), (1, 1)),    # 1x1 downsample
    ((3, 20, 24, 32), (3, 5, 32, 40), (1, 2), (2, 0), (2, 1)),      # unequal window, stride, padding and dilation
    ((2, 40, 40, 96), (7, 7, 96, 32), (2, 2), (3, 3), (1, 1)),      # large window
])
@pytest.mark.parametrize("raw", [0, 1])
def test_implicit_gemm_convolution(monkeypatch, raw, shape, filt, stride, pad, dil):
    """conv_2d with C % 32 == 0 runs as an implicit GEMM: im2col-mode TMA loads from the image's tf32
    planes.  Checked against float64 and against the explicit im2col + GEMM decomposition."""
    # raw = 1: the opt-in variant that reads the image as plain fp32 and splits each tile inside the SM (measured slower)
    monkeypatch.setenv("SAGE_CONV_RAW", str(raw))
    rng = np.random.default_rng(sum(shape) + sum(filt))
    x = rng.standard_normal(shape).astype(np.float32)
    f = (rng.standard_normal(filt) / np.sqrt(filt[0] * filt[1] * filt[2])).astype(np.float32)
    b = rng.standard_normal(filt[3]).astype(np.float32)
    ref = np.maximum(conv64(x, f, stride, pad, dil) + b, 0)
    lowered, plain = S.Context(0), S.Context(0, pattern_fusion=0)
    try:
        outs = []
        for ctx in (lowered, plain):
            ctx.trace_begin()
            y = S.relu(S.conv_2d(ctx.var(x), ctx.var(f), list(stride), list(pad), list(dil)) + ctx.var(b))
            outs.append(y.eval(ctx))
        assert "<implicit conv>" in lowered.describe() and "im2col" not in lowered.trace()
        assert "im2col" in plain.trace()
        assert outs[0].shape == ref.shape
        assert gemm_err(outs[0], ref) <= 1e-4 and gemm_err(outs[1], ref) <= 1e-4
        assert gemm_err(outs[0], outs[1]) <= 1e-5
        assert lowered.status_word() == 0
    finally:
        lowered.close()
        plain.close()


@pytest.mark.parametrize("shape,filt,pad", [
    ((3, 56, 56, 64), (3, 3, 64, 64), (1, 1)),      # ResNet-18 layer 1: two output rows of 58 positions per CTA
    ((5, 28, 28, 128), (3, 3, 128, 128), (1, 1)),   # layer 2: four rows per CTA, 7 CTA tiles per image (pairs span images)
    ((2, 13, 50, 32), (3, 3, 32, 64), (1, 1)),      # odd height: the last tile of an image is partly outside it
    ((3, 9, 30, 64), (3, 3, 64, 96), (0, 0)),       # no padding; output channels short of the tile width
    ((2, 20, 36, 32), (2, 4, 32, 32), (1, 2)),      # even window, unequal padding
    ((1, 24, 60, 32), (3, 3, 32, 64), (1, 1)),      # the widest rows that fit: a window of 248 pixel rows
    ((9, 3, 40, 32), (3, 3, 32, 32), (1, 1)),       # an image is lower than a CTA tile: one tile per image, pairs span images
    ((3, 16, 40, 64), (1, 3, 64, 64), (0, 1)),      # a single filter row: the window has no extra rows
])
@pytest.mark.parametrize("halo", [1, 0])
def test_convolution_with_tap_reuse(monkeypatch, halo, shape, filt, pad):
    """A stride-1 convolution with few output channels loads each CTA's input window once per 32 channels and
    reads all taps out of it (SAGE_CONV_HALO=0: one im2col load per tap).  With a bias, a residual and relu in
    the epilogue, against float64 and the explicit decomposition."""
    monkeypatch.setenv("SAGE_CONV_HALO", str(halo))
    rng = np.random.default_rng(sum(shape) + sum(filt) + 7)
    x = rng.standard_normal(shape).astype(np.float32)
    f = (rng.standard_normal(filt) / np.sqrt(filt[0] * filt[1] * filt[2])).astype(np.float32)
    b = rng.standard_normal(filt[3]).astype(np.float32)
    conv = conv64(x, f, (1, 1), pad, (1, 1))
    r = rng.standard_normal(conv.shape).astype(np.float32)
    ref = np.maximum(conv + b + r, 0)
    lowered, plain = S.Context(0), S.Context(0, pattern_fusion=0)
    try:
        outs = []
        for ctx in (lowered, plain):
            y = S.relu(S.conv_2d(ctx.var(x), ctx.var(f), [1, 1], list(pad), [1, 1]) + ctx.var(b) + ctx.var(r))
            outs.append(y.eval(ctx))
        assert "<implicit conv>" in lowered.describe()
        assert outs[0].shape == ref.shape
        assert gemm_err(outs[0], ref) <= 1e-4 and gemm_err(outs[1], ref) <= 1e-4
        assert gemm_err(outs[0], outs[1]) <= 1e-5
        assert lowered.status_word() == 0
    finally:
        lowered.close()
        plain.close()


@pytest.mark.parametrize("b,lq,lk,d", [(6, 128, 128, 64), (5, 70, 96, 32), (3, 300, 200, 64), (4, 64, 256, 32), (2, 130, 33, 64)])
def test_row_softmax_in_the_gemm_epilogue(b, lq, lk, d):
    """softmax(q k^T * scale + mask) with the keys of a row inside one tile (L_k <= 256) can be computed by
    the scores GEMM's epilogue warps (pattern_fusion bit 1; off by default because it measured slower on
    the BERT step).  Ragged extents exercise partial tiles in both directions; the mask has
    padded keys (-1e5) like the attention of config 4."""
    rng = np.random.default_rng(b * 100 + lk)
    q = rng.standard_normal((b, lq, d)).astype(np.float32)
    k = rng.standard_normal((b, lk, d)).astype(np.float32)
    v = rng.standard_normal((b, lk, d)).astype(np.float32)
    mask = np.zeros((b, 1, lk), np.float32)
    for i in range(b):
        mask[i, 0, lk - int(rng.integers(0, lk // 3 + 1)):] = -100000.0
    scale = np.float32(1.0 / np.sqrt(d))
    s64 = q.astype(np.float64) @ k.astype(np.float64).transpose(0, 2, 1) * np.float64(scale) + mask
    p64 = softmax64(s64)
    o64 = p64 @ v.astype(np.float64)
    lowered, plain = S.Context(0, pattern_fusion=3), S.Context(0, pattern_fusion=0)
    try:
        res = []
        for ctx in (lowered, plain):
            Q, K, V, M = (ctx.var(t) for t in (q, k, v, mask))
            P = S.softmax(Q.matmul_batched(K.transpose(-1, -2)) * float(scale) + M, [-1])
            O = P.matmul_batched(V)
            ctx.trace_begin()
            ctx.eval(P, O) if ctx is plain else ctx.eval(O)
            res.append((ctx.read(O), ctx.trace()))
        assert "|softmax" in lowered.describe() and "softmax_rows" not in res[0][1]
        if lk % 4 == 0:  # the probabilities feed P.V as planes; an unaligned row pitch goes through the gather path
            assert "|softmax=planes" in lowered.describe()
        assert gemm_err(res[0][0], o64) <= 1e-4 and gemm_err(res[1][0], o64) <= 1e-4
        assert gemm_err(res[0][0], res[1][0]) <= 1e-5
        # the probabilities themselves, as a target
        ctx = lowered
        Q, K, M = (ctx.var(t) for t in (q, k, mask))
        P = S.softmax(Q.matmul_batched(K.transpose(-1, -2)) * float(scale) + M, [-1])
        got = P.eval(ctx)
        assert "|softmax" in ctx.describe()
        assert np.abs(got - p64).max() <= 1e-6 and np.abs(got.sum(-1) - 1).max() <= 1e-5
        assert lowered.status_word() == 0
    finally:
        lowered.close()
        plain.close()


@pytest.mark.parametrize("n,l,e", [(4, 32, 256), (2, 7, 96), (3, 16, 1024)])
def test_row_groups_inside_a_larger_program(n, l, e):
    """LayerNorm's backward pass sits between GEMMs: its states (maps and row reductions over [n*l, e])
    run as ONE generated kernel inside the larger program.  Gradients with the groups on (pattern_fusion
    1) and off (5: kernel by kernel) agree to fp32 rounding, and both match float64."""
    rng = np.random.default_rng(900 + e)
    x = rng.standard_normal((n, l, e)).astype(np.float32)
    w1 = (rng.standard_normal((e, e)) / np.sqrt(e)).astype(np.float32)
    w2 = (rng.standard_normal((e, 8)) / np.sqrt(e)).astype(np.float32)
    gamma, beta = np.float32([1.3]), np.float32([0.2])
    outs = []
    for fusion in (1, 5):
        c = S.Context(0, pattern_fusion=fusion)
        try:
            xv, w1v, w2v, gv, bv = (c.var(a) for a in (x, w1, w2, gamma, beta))
            h = S.layer_norm(S.matmul(xv, w1v) + xv, [2], gv, bv, 1e-5)
            y = S.matmul(S.relu(h), w2v)
            loss = (y * y).sum([0, 1, 2], False)
            grads = S.grad(loss, [xv, w1v, w2v, gv, bv])
            c.trace_begin()
            c.eval(loss, *grads)
            assert ("sage_row_program" in c.trace()) == (fusion == 1)
            if fusion == 1:
                assert "row_program[%dx%d" % (n * l, e) in c.describe()
            outs.append([c.read(loss)] + [c.read(g) for g in grads])
            assert c.status_word() == 0
        finally:
            c.close()
    for a, b in zip(*outs):
        assert gemm_err(a, b) <= 1e-4
    # float64 reference of the same graph
    X, W1, W2 = (a.astype(np.float64) for a in (x, w1, w2))
    t = X @ W1 + X
    mu, var = t.mean(-1, keepdims=True), (t * t).mean(-1, keepdims=True) - t.mean(-1, keepdims=True) ** 2
    xh = (t - mu) / np.sqrt(var + 1e-5)
    h = xh * 1.3 + 0.2
    r = np.maximum(h, 0)
    y = r @ W2
    gy = 2 * y
    gw2 = np.einsum("nle,nlo->eo", r, gy)
    gh = (gy @ W2.T) * (h > 0)
    ggamma, gbeta = (gh * xh).sum(), gh.sum()
    gxh = gh * 1.3
    gt = (gxh - gxh.mean(-1, keepdims=True) - xh * (gxh * xh).mean(-1, keepdims=True)) / np.sqrt(var + 1e-5)
    gw1 = np.einsum("nle,nlo->eo", X, gt)
    gx = gt @ W1.T + gt
    for got, ref in zip(outs[0], [(y * y).sum().reshape(1), gx, gw1, gw2, np.array([ggamma]), np.array([gbeta])]):
        assert gemm_err(got, ref.astype(np.float32)) <= 2e-4


def test_out_of_memory_evicts_recomputes_and_gives_the_same_values():
    """Program::exec's out-of-memory path (src/session.rs:259-331) on the device: with a tight capacity the
    evaluator drops the intermediates that are cheapest to recompute per element (device time from events)
    and rebuilds them on demand; the result equals, bit for bit, the one computed with room to spare."""
    n = 1 << 20  # 4 MiB tensors
    x = np.random.default_rng(77).standard_normal(n).astype(np.float32) * 1e-3
    outs, launches = [], []
    for cap in (0, 44 << 20):
        c = S.Context(0, **({"mem_capacity_bytes": cap} if cap else {}))
        try:
            xv = c.var(x)
            a = [xv * float(i + 2) + 1.0 for i in range(12)]
            s = [v.sum([0], True) for v in a]
            z = s[0]
            for v in s[1:]:
                z = z + v
            t = [(v * z.expand([n])).sum([0], True) for v in a]
            out = s[0] * 0.0
            for v, w in zip(t, s):
                out = out + v + v * 2.0 + w
            c.trace_begin()
            for _ in range(2):   # the second pass uses the device times measured in the first
                c.clear()
                c.eval(out)
            outs.append(c.read(out))
            launches.append(len(c.trace()))
            if cap:
                assert c.mem_stats()["mem_peak"] <= cap
            assert c.status_word() == 0
        finally:
            c.close()
    assert np.array_equal(outs[0], outs[1]) and np.isfinite(outs[0]).all()
    assert launches[1] > launches[0]   # states were evicted and computed again


def test_row_groups_do_not_swallow_a_state_that_lies_between_them():
    """a (row space) feeds a GEMM g and, together with g, a second row-space state b.  Merging a and b into
    one kernel would need g both after and before it; they stay two generated kernels around the GEMM, and
    the values match the kernel-by-kernel evaluation and float64."""
    rng = np.random.default_rng(950)
    x = rng.standard_normal((192, 256)).astype(np.float32)
    w = (rng.standard_normal((256, 256)) / 16).astype(np.float32)
    outs = []
    for fusion in (1, 5):
        c = S.Context(0, pattern_fusion=fusion)
        try:
            xv, wv = c.var(x), c.var(w)
            a = (xv - xv.max([1], True)).exp()
            g = S.matmul(a, wv)
            b = ((a + g) * a).sum([1], False) + a.sum([1], False)
            c.trace_begin()
            c.eval(b, g)
            t = c.trace()
            if fusion == 1:
                assert t.count("sage_row_program") == 2 and t.index("sage_row_program") < t.index("gemm_tc_3xtf32") < len(t) - 1 - t[::-1].index("sage_row_program")
            outs.append((c.read(b), c.read(g)))
        finally:
            c.close()
    for p, q in zip(*outs):
        assert gemm_err(p, q) <= 1e-4
    A = np.exp(np.maximum(x.astype(np.float64) - np.maximum(x.max(1, keepdims=True), 0), -1e30))  # the reference's max starts from 0
    G = A @ w.astype(np.float64)
    B = ((A + G) * A).sum(1) + A.sum(1)
    assert gemm_err(outs[0][0], B.astype(np.float32)) <= 1e-4 and gemm_err(outs[0][1], G.astype(np.float32)) <= 1e-4


# ------------------------------------------------------------------------------ fused attention
def attention_graph(M, q, k, v, mask, n, heads, l, d):
    """The attention block of src/models/bert.rs:250-280 with the public ops: separate heads, scores / sqrt(d) +
    extended mask, softmax over the keys, probabilities x values, merge heads."""
    def split(t):
        return M.transpose(M.view(t, [n, l, heads, d]), 2, 1)
    scores = M.matmul_batched(split(q), M.transpose(split(k), -1, -2)) / float(np.sqrt(np.float32(d)))
    ext = (-(M.view(mask, [n, 1, 1, l])) + 1.0) * -1e5
    p = M.softmax(scores + ext, [3])
    av = M.transpose(M.matmul_batched(p, split(v)), 2, 1)
    return M.view(av, [n, l, heads * d])


@pytest.mark.parametrize("n,heads,l,d", [(2, 2, 128, 64), (3, 4, 512, 64), (2, 2, 70, 32), (2, 3, 200, 64), (1, 1, 64, 64), (2, 2, 129, 48),
                                         (32, 12, 128, 64)])
def test_fused_attention_vs_oracle_and_decomposed(n, heads, l, d):
    """scores -> scale + mask -> softmax -> probabilities x values as ONE kernel (tcgen05, P kept in tensor memory)
    against the oracle evaluating the reference's four-step composition, against the same graph evaluated kernel by
    kernel (pattern_fusion bit 3 keeps the attention decomposed) and against float64.  Ragged padding masks; key
    counts that are not multiples of the 64-key block (70, 129, 200); head widths 32 / 48 / 64; more than one key
    block, where the running maximum rescales the partial sums: |a - b| / max(|b|, rms(b)) <= 1e-4 in every case."""
    rng = np.random.default_rng(7000 + l + d)
    e = heads * d
    q, k, v = (rng.standard_normal((n, l, e)).astype(np.float32) * np.float32(s) for s in (1.5, 1.5, 1.0))
    mask = np.ones((n, l), np.float32)
    for i in range(n):
        mask[i, l - int(rng.integers(0, l // 4 + 1)):] = 0
    outs = []
    for fusion in (1, 9):
        c = S.Context(0, pattern_fusion=fusion)
        try:
            # the operands are results of kernels, as in the model: their producers write the tf32 planes
            qv, kv, vv = (c.var(t) * 1.0 for t in (q, k, v))
            y = attention_graph(S, qv, kv, vv, c.var(mask), n, heads, l, d)
            c.trace_begin()
            got = y.eval(c)
            tr, desc = c.trace(), c.describe()
            if fusion == 1:
                assert "attention{" in desc and "attention_tc_3xtf32" in tr and "softmax_rows" not in tr, desc
                assert sum(1 for t in tr if t.startswith("gemm")) == 0
            else:
                assert "attention" not in desc and "softmax_rows" in tr
            assert c.status_word() == 0
            outs.append(got)
        finally:
            c.close()
    fused, plain = outs
    q64, k64, v64 = (t.astype(np.float64).reshape(n, l, heads, d).transpose(0, 2, 1, 3) for t in (q, k, v))
    s64 = q64 @ k64.transpose(0, 1, 3, 2) / np.float64(np.sqrt(np.float32(d))) + ((1.0 - mask.astype(np.float64)) * -1e5)[:, None, None, :]
    ref64 = (softmax64(s64) @ v64).transpose(0, 2, 1, 3).reshape(n, l, e)
    assert fused.shape == ref64.shape
    assert gemm_err(fused, ref64) <= 1e-4 and gemm_err(plain, ref64) <= 1e-4
    assert gemm_err(fused, plain) <= 1e-4
    if n * heads * l * l <= 3 * 4 * 512 * 512:  # the oracle's scalar loops
        from oracle import sage_ref as R
        RV = lambda a: R.Var.new(R.Tensor.new(a))
        ref = attention_graph(R, RV(q) * 1.0, RV(k) * 1.0, RV(v) * 1.0, RV(mask), n, heads, l, d).eval().numpy()
        assert gemm_err(fused, ref) <= 1e-4


def test_fused_attention_without_ref_compat_and_with_large_scores():
    """With true identities (ref_compat = 0) the row maximum starts at -inf instead of 0, and scores far from 0 make the
    running maximum move between key blocks: the rescaling path."""
    rng = np.random.default_rng(7100)
    n, heads, l, d = 2, 2, 256, 64
    e = heads * d
    q, k, v = (rng.standard_normal((n, l, e)).astype(np.float32) * np.float32(s) for s in (3.0, 3.0, 1.0))
    q += np.float32(0.5)  # rows whose scores are all far below zero exist as well
    mask = np.ones((n, l), np.float32)
    mask[1, 200:] = 0
    q64, k64, v64 = (t.astype(np.float64).reshape(n, l, heads, d).transpose(0, 2, 1, 3) for t in (q, k, v))
    s64 = q64 @ k64.transpose(0, 1, 3, 2) / 8.0 + ((1.0 - mask.astype(np.float64)) * -1e5)[:, None, None, :]
    ref64 = (softmax64(s64) @ v64).transpose(0, 2, 1, 3).reshape(n, l, e)
    for compat in (0, 1):
        c = S.Context(0, ref_compat=compat)
        try:
            y = attention_graph(S, c.var(q) * 1.0, c.var(k) * 1.0, c.var(v) * 1.0, c.var(mask), n, heads, l, d)
            got = y.eval(c)
            assert "attention{" in c.describe()
            if compat == 0:
                assert gemm_err(got, ref64) <= 1e-4
            else:
                # rows whose scores are all negative keep exp(x - 0): smaller terms, same quotient up to rounding
                assert gemm_err(got, ref64) <= 1e-3
            assert c.status_word() == 0
        finally:
            c.close()


@pytest.mark.parametrize("shape,filt,stride,pad,dil", [
    ((4, 64, 64, 3), (7, 7, 3, 64), (2, 2), (3, 3), (1, 1)),        # the first convolution of ResNet (112-wide rows at full size)
    ((3, 40, 44, 1), (3, 3, 1, 32), (1, 1), (1, 1), (1, 1)),        # one channel (the training example's 28 x 28 x 1 images)
    ((2, 45, 51, 3), (3, 5, 3, 40), (3, 2), (2, 0), (1, 2)),        # unequal window / stride / padding, dilated rows
    ((5, 32, 32, 3), (3, 3, 3, 32), (1, 1), (1, 1), (1, 1)),        # MobileNet's first layer (K = 27)
    ((2, 50, 50, 4), (2, 8, 4, 32), (2, 1), (0, 1), (1, 1)),        # four channels, the widest window (8 taps x 4 floats = one 128-byte row)
    ((2, 40, 40, 3), (3, 3, 3, 32), (1, 1), (1, 1), (2, 1)),        # dilated COLUMNS: not this path, the column planes are built
])
def test_convolution_with_few_input_channels(shape, filt, stride, pad, dil):
    """conv_2d with C <= 4 (src/ops/conv.rs:61-96 at the first layer of the reference's image models).  A 12-byte channel
    run cannot be a TMA box, so the image is re-laid with 4-float pixels (zero-padded in space as well) and the GEMM
    reads overlapping 32-float windows of it: no column matrix is written.  Against float64, against the same graph
    evaluated operator by operator, and — for the small cases — against the oracle."""
    rng = np.random.default_rng(sum(shape) + sum(filt))
    x = rng.standard_normal(shape).astype(np.float32)
    f = (rng.standard_normal(filt) / np.sqrt(filt[0] * filt[1] * filt[2])).astype(np.float32)
    b = rng.standard_normal(filt[3]).astype(np.float32)
    ref = np.maximum(conv64(x, f, stride, pad, dil) + b, 0)
    lowered, plain = S.Context(0), S.Context(0, pattern_fusion=0)
    try:
        outs = []
        for ctx in (lowered, plain):
            ctx.trace_begin()
            y = S.relu(S.conv_2d(ctx.var(x), ctx.var(f), list(stride), list(pad), list(dil)) + ctx.var(b))
            outs.append(y.eval(ctx))
            outs.append(y.eval(ctx) if ctx is plain else None)
        padded = dil[0] == 1
        if padded:
            assert "channels padded to 4" in lowered.describe() and "im2col" not in lowered.trace() and "pack_small_c" in lowered.trace()
        else:
            assert "channels padded" not in lowered.describe()
        assert outs[0].shape == ref.shape
        assert gemm_err(outs[0], ref) <= 1e-4 and gemm_err(outs[2], ref) <= 1e-4
        assert gemm_err(outs[0], outs[2]) <= 1e-5
        # a second evaluation reuses the re-laid filter; rewriting the filter must invalidate it
        fv = lowered.var(f)
        y2 = S.conv_2d(lowered.var(x), fv, list(stride), list(pad), list(dil))
        first = y2.eval(lowered)
        lowered.set(fv, (f * np.float32(-2)).astype(np.float32))
        lowered.clear()
        second = y2.eval(lowered)
        assert gemm_err(second, -2 * conv64(x, f, stride, pad, dil)) <= 1e-4 and gemm_err(first, conv64(x, f, stride, pad, dil)) <= 1e-4
        from oracle import sage_ref as R
        RV = lambda a: R.Var.new(R.Tensor.new(a))
        oref = R.conv_2d(RV(x), RV(f), list(stride), list(pad), list(dil)).eval().numpy()
        assert gemm_err(first, oref) <= 1e-4
        assert lowered.status_word() == 0
    finally:
        lowered.close()
        plain.close()
