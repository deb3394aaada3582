"""The training path on the GPU against the CPU oracle: gradients of whole models (src/var.rs:56-103 over
the operators' grad rules), ops::metric::accuracy, and the optimizers of src/optim.rs driven the way
examples/train.rs drives them (evaluate loss + gradients, Optimizer::update, Context::data.clear()).

Tolerances: gradients are sums of products like contractions, so they are measured against the rms of
the reference tensor (|a - b| / max(|b|, rms) <= 1e-3, the bound used for full-model outputs);
parameters after Adam steps of whole models: see adam_close (Adam divides by sqrt(v): an element's step is
~lr whatever the gradient's size, so rounding differences of small gradients show as a fraction of lr).  Given
the SAME gradients, the update itself is bit-exact (test_optimizer_update_given_gradients_matches_to_the_last_bits).
"""
import numpy as np
import pytest

import sage_b200 as S
from oracle import sage_ref as R

pytestmark = pytest.mark.gpu


def RV(a, dtype=None):
    return R.Var.new(R.Tensor.new(a, dtype))


def rms_err(got, ref, floor=0.0):
    """max |a - b| / max(|b|, rms(b), floor).  `floor` (an absolute value) is for gradients that cancel to
    ~0: sums of terms of ordinary size whose fp32 rounding noise any evaluation order shows."""
    a, b = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    rms = max(float(np.sqrt((b ** 2).mean())), floor, 1e-30)
    return float((np.abs(a - b) / np.maximum(np.abs(b), rms)).max())


def adam_close(a, b, lr, steps):
    """|a - b| <= 1e-4 |b| + 0.02 lr per step, for all but one element in a thousand; those may differ by up
    to a full step each time.  An element's Adam step is lr * m / (sqrt(v) + 1e-8): once its gradient lies
    within fp32 rounding noise of zero (a few in every large tensor do), sign and size of the step are
    decided by that noise in any implementation, bounded by lr."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    d = np.abs(a - b)
    bad = d > 1e-4 * np.abs(b) + 0.02 * lr * steps
    return bool(bad.mean() <= 1e-3 and d.max() <= 2.0 * lr * steps)


def rel_err(a, b, floor):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    scale = np.maximum(np.abs(b), floor * max(np.abs(b).max(), 1e-30))
    return float((np.abs(a - b) / scale).max())


class Params:
    def __init__(self, ps):
        self.ps = ps

    def params(self):
        return self.ps


@pytest.fixture(scope="module")
def ctx():
    c = S.Context(0)
    yield c
    c.close()


def mlp(M, x, lab, w1, b1, w2):
    h = M.relu(M.matmul(x, w1) + b1)
    logits = M.matmul(h, w2)
    return logits, M.mean(M.softmax_cross_entropy(logits, lab), [0], False)


@pytest.mark.parametrize("opt_name,lr,wd", [("Adam", 1e-2, 0.0), ("Adam", 1e-2, 0.1), ("Sgd", 0.1, 0.0), ("Sgd", 0.1, 0.05)])
def test_optimizer_steps_vs_oracle(ctx, opt_name, lr, wd):
    rng = np.random.default_rng(4200)
    n, din, dh, dout = 64, 300, 129, 10   # 300 x 129 and 129 x 10: slots that are not multiples of 4 or of a chunk
    x = rng.standard_normal((n, din)).astype(np.float32)
    lab = rng.integers(0, dout, (n, 1)).astype(np.uint32)
    init = [(rng.standard_normal(s) * 0.1).astype(np.float32) for s in ((din, dh), (dh,), (dh, dout))]
    gp = [ctx.var(v) for v in init]
    rp = [RV(v) for v in init]
    logits, loss = mlp(S, ctx.var(x), ctx.var(lab), *gp)
    acc = S.accuracy(logits, ctx.var(lab))
    rlogits, rloss = mlp(R, RV(x), RV(lab, R.UINT), *rp)
    racc = R.accuracy(rlogits, RV(lab, R.UINT))
    grads, rgrads = S.grad_param(loss, Params(gp)), R.grad_param(rloss, Params(rp))
    opt, ropt = getattr(S, opt_name)(lr), getattr(R, opt_name)(lr)
    opt.set_weight_decay(wd)
    ropt.weight_decay = wd
    opt.init(ctx)
    ropt.init()
    for step in range(5):
        ctx.eval(*grads.values(), loss, acc)          # Program::exec in examples/train.rs:52
        got_loss, got_acc = ctx.read(loss), ctx.read(acc)
        opt.update(grads, ctx)
        ctx.clear()
        ref_loss, ref_acc = [t.numpy() for t in R.evaluate([rloss, racc])]
        ropt.update(rgrads)
        assert rel_err(got_loss, ref_loss, 1e-6) <= 1e-4, step
        assert np.array_equal(got_acc, ref_acc), step   # a count of matches divided by n: exact
        for g, r in zip(gp, rp):
            assert rel_err(ctx.read(g), r.data.numpy(), 1e-2) <= 1e-3, step
    assert ctx.status_word() == 0


@pytest.mark.parametrize("opt_name,wd", [("Adam", 0.0), ("Adam", 0.01), ("Sgd", 0.0), ("Sgd", 0.01)])
def test_optimizer_update_given_gradients_matches_to_the_last_bits(ctx, opt_name, wd):
    """With gradients supplied as data, the fused update and the oracle's expression-by-expression update
    (optim.rs:134-177) perform the same correctly rounded fp32 operations.  Sgd: equal bits after every
    step.  Adam: the bias corrections 1 - beta^t come from two powf implementations (the host's libm here,
    the oracle's map kernel there) that may differ in the last bit, so a step of size ~lr may differ by one
    unit in its last places: |a - b| <= 2^-20 * max(|b|, lr).  40 parameters (two launches of 32 slots), sizes
    around the vector width and the chunk."""
    rng = np.random.default_rng(4250)
    sizes = [1, 2, 3, 4, 5, 7, 8, 31, 33, 127, 128, 129, 1000, 4095, 4096, 4097, 8191, 8193, 12289, 20000] * 2
    ps = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    gp, rp = [ctx.var(v) for v in ps], [RV(v) for v in ps]
    gg = [ctx.var(np.zeros(n, np.float32)) for n in sizes]
    rg = [RV(np.zeros(n, np.float32)) for n in sizes]
    opt, ropt = getattr(S, opt_name)(1e-2), getattr(R, opt_name)(1e-2)
    opt.set_weight_decay(wd)
    ropt.weight_decay = wd
    opt.init(ctx)
    grads, rgrads = dict(zip(gp, gg)), dict(zip(rp, rg))
    for step in range(4):
        for g, r, n in zip(gg, rg, sizes):
            v = (rng.standard_normal(n) * 10.0 ** rng.integers(-6, 2)).astype(np.float32)
            ctx.set(g, v)
            r.set(v.copy())
        opt.update(grads, ctx)
        ropt.update(rgrads)
        for i, (g, r) in enumerate(zip(gp, rp)):
            a, b = ctx.read(g), r.data.numpy()
            if opt_name == "Sgd":
                assert np.array_equal(a, b), (step, i, sizes[i])
            else:
                assert (np.abs(a - b) <= 2.0 ** -20 * np.maximum(np.abs(b), 1e-2)).all(), (step, i, sizes[i])


def test_update_refreshes_the_tf32_planes_of_gemm_weights(ctx):
    """A weight that a tensor-core GEMM has read keeps hi / lo planes beside it; the update rewrites them,
    so the next GEMM multiplies by the new values."""
    rng = np.random.default_rng(4260)
    x = rng.uniform(-1, 1, (256, 384)).astype(np.float32)
    w = rng.uniform(-1, 1, (384, 128)).astype(np.float32)
    g = rng.uniform(-1, 1, (384, 128)).astype(np.float32)
    xv, wv, gv = ctx.var(x), ctx.var(w), ctx.var(g)
    y = S.matmul(xv, wv)
    before = y.eval(ctx)
    ctx.clear()
    opt = S.Sgd(0.5)
    opt.update({wv: gv}, ctx)
    after = y.eval(ctx)
    ctx.clear()
    w_new = w - g * np.float32(0.5)
    assert np.array_equal(ctx.read(wv), w_new)
    f64 = x.astype(np.float64) @ w_new.astype(np.float64)
    assert np.linalg.norm(after - f64) / np.linalg.norm(f64) <= 2e-6
    assert np.linalg.norm(before - f64) / np.linalg.norm(f64) > 1e-2


def test_update_refuses_a_parameter_that_is_not_data(ctx):
    """"param is not data tensor" (optim.rs:52-54): the reference panics, the library returns an error."""
    w = ctx.var(np.ones((4, 4), np.float32))
    y = (w * w).sum([0, 1], False)
    opt = S.Adam(0.1)
    with pytest.raises(S.SageError):
        opt.update({w * 2.0: w.grad(y)}, ctx)


def test_resnet18_training_step_vs_oracle(ctx):
    """examples/train.rs at a small batch: ResNet d18(1, 10) on 28 x 28 x 1 images, mean softmax cross
    entropy, gradients of all 42 parameters, Adam."""
    rng = np.random.default_rng(4300)
    batch = 4
    model, rmodel = S.ResNet18(1, 10), R.resnet18(1, 10)
    params, rparams = model.params(), rmodel.params()
    for p, r in zip(params, rparams):
        e = p.extents
        v = (rng.standard_normal(e) * (np.sqrt(2.0 / (e[0] * e[1] * e[2])) if len(e) == 4 else 0.05)).astype(np.float32)
        ctx.set(p, v)
        r.set(v.copy())
    x = rng.standard_normal((batch, 28, 28, 1)).astype(np.float32)
    lab = rng.integers(0, 10, (batch, 1)).astype(np.uint32)
    xin, lin = S.Var.empty([batch, 28, 28, 1]), S.Var.empty([batch, 1], S.U32)
    logits = model.pass_(xin)
    loss = S.softmax_cross_entropy(logits, lin).mean([0], False)
    rlogits = rmodel(RV(x))
    rloss = R.mean(R.softmax_cross_entropy(rlogits, RV(lab, R.UINT)), [0], False)
    grads, rgrads = S.grad_param(loss, model), R.grad_param(rloss, rmodel)
    params = list(grads)  # the same variables as above, under the handles grad_param made
    opt, ropt = S.Adam(1e-3), R.Adam(1e-3)
    opt.init(ctx)
    for step in range(3):
        ctx.set(xin, x)
        ctx.set(lin, lab)
        ctx.eval(*grads.values(), loss)
        ref = R.evaluate([rgrads[p] for p in rparams] + [rloss])
        assert rel_err(ctx.read(loss), ref[-1].numpy(), 1e-6) <= 1e-3, step
        if step == 0:
            gmax = max(float(np.abs(r.numpy()).max()) for r in ref[:-1])
            for i, (p, r) in enumerate(zip(params, ref[:-1])):
                assert rms_err(ctx.read(grads[p]), r.numpy(), 1e-5 * gmax) <= 1e-3, (i, p.extents)
        opt.update(grads, ctx)
        ropt.update(rgrads)
        ctx.clear()
        for i, (p, r) in enumerate(zip(params, rparams)):
            assert adam_close(ctx.read(p), r.data.numpy(), 1e-3, step + 1), (step, i)
    assert ctx.status_word() == 0


def test_bert_training_step_vs_oracle(ctx):
    """A small Bert (2 layers, width 64, 4 heads, FFN 128, 16 tokens): gradients through embeddings
    (scatter-add with repeated token ids), LayerNorm, masked softmax, batched and transposed
    contractions; then Adam steps, after which the forward pass must see the new weights (the tf32
    planes of every GEMM weight are rewritten by the update itself)."""
    rng = np.random.default_rng(4400)
    cfg = dict(embed_dim=64, num_vocabs=50, max_num_tokens=16, hidden_dim=128, num_layers=2, num_heads=4, num_classes=3)
    batch, seq = 8, 16
    model = S.Bert(**cfg)
    rmodel = R.Bert(R.BertConfig(**cfg))
    params, rparams = model.params(), rmodel.params()
    for p, r in zip(params, rparams):
        v = (rng.standard_normal(p.extents) * 0.1).astype(np.float32)
        if p.extents == (1,):  # LayerNorm's scalar gamma / beta
            v = np.float32([rng.uniform(0.5, 1.5)])
        ctx.set(p, v)
        r.set(v.copy())
    ids = rng.integers(0, 50, (batch, seq)).astype(np.uint32)
    mask = np.ones((batch, seq), np.float32)
    mask[1, 10:] = 0
    lab = rng.integers(0, 3, (batch, 1)).astype(np.uint32)
    logits = model.pass_(ctx.var(ids), ctx.var(mask))
    loss = S.softmax_cross_entropy(logits, ctx.var(lab)).mean([0], False)
    rlogits = rmodel(RV(ids, R.UINT), RV(mask))
    rloss = R.mean(R.softmax_cross_entropy(rlogits, RV(lab, R.UINT)), [0], False)
    grads, rgrads = S.grad_param(loss, model), R.grad_param(rloss, rmodel)
    params = list(grads)  # the same variables as above, under the handles grad_param made
    opt, ropt = S.Adam(1e-3), R.Adam(1e-3)
    opt.init(ctx)
    noise = set()
    for step in range(3):
        ctx.eval(*grads.values(), loss)
        ref = R.evaluate([rgrads[p] for p in rparams] + [rloss])
        assert rel_err(ctx.read(loss), ref[-1].numpy(), 1e-6) <= 1e-3, step
        if step == 0:
            gmax = max(float(np.abs(r.numpy()).max()) for r in ref[:-1])
            for i, (p, r) in enumerate(zip(params, ref[:-1])):
                assert rms_err(ctx.read(grads[p]), r.numpy(), 1e-5 * gmax) <= 1e-3, (i, p.extents)
                # The key projection's bias shifts every score of a query by the same amount, which softmax
                # ignores: its gradient is exactly 0, what is computed is rounding noise, and Adam turns
                # noise into a step of arbitrary sign.  Such parameters are left out of the final comparison.
                if float(np.abs(r.numpy()).max()) < 1e-5 * gmax:
                    noise.add(i)
        opt.update(grads, ctx)
        ropt.update(rgrads)
        ctx.clear()
    assert len(noise) == cfg["num_layers"]
    for i, (p, r) in enumerate(zip(params, rparams)):
        if i not in noise:
            assert adam_close(ctx.read(p), r.data.numpy(), 1e-3, 3), i
    assert ctx.status_word() == 0
