"""CPU-only checks of the host side: the C-ABI library loads and exports every declared symbol,
graph construction / shape inference / grad / fusion / state selection behave like the reference,
generated map kernels compile (real NVRTC, no device needed), and the allocator follows its
policy.  A planning context (device = -1) records launches and computes nothing."""
import ctypes
import os
import re

import numpy as np
import pytest

import sage_b200 as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in ("sage_cuda.h", "sage_graph.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(sage_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    syms = declared_symbols()
    assert len(syms) > 80
    missing = [s for s in syms if not hasattr(S.lib, s)]
    assert not missing, missing


def test_no_device_means_errors_not_fallbacks():
    if S.device_count() > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(S.SageError) as e:
        S.Context(0)
    assert e.value.code == 5  # SAGE_ERR_NO_DEVICE
    ctx = S.Context(-1)
    x = ctx.var(np.ones((4, 4), np.float32))
    y = x * 2.0
    ctx.eval(y)  # planning: compiles + records
    with pytest.raises(S.SageError) as e:
        ctx.read(y)  # but there is nothing to read
    assert e.value.code == 5


@pytest.fixture()
def ctx():
    c = S.Context(-1)
    yield c
    c.close()


def test_shapes_broadcast_views(ctx):
    x = ctx.var(np.zeros((2, 3, 4), np.float32))
    assert x.transpose(0, 2).extents == (4, 3, 2) and x.transpose(0, 2).strides == (1, 4, 12)
    assert x.view([6, -1]).extents == (6, 4)
    assert S.expand(ctx.var(np.zeros((3, 1), np.float32)), [2, 3, 5]).strides == (0, 1, 0)
    assert x.unsqueeze(1).strides == (12, 0, 4, 1)  # a fresh unit axis has stride 0 (src/shape.rs:190-195)
    assert x.slice(1, 1, 3).offset == 4 and x.slice(1, 1, 3).extents == (2, 2, 4)
    assert (x + ctx.var(np.zeros((4,), np.float32))).extents == (2, 3, 4)
    assert x.sum([0, 2], False).extents == (3,) and x.sum([0, 2], True).extents == (1, 3, 1)
    assert x.sum(None, False).extents == (1,)
    assert x.argmax(1).dtype == S.U32 and S.gt(x, 0.0).dtype == S.U32 and x.int().dtype == S.I32
    for bad in (lambda: x.view([5, -1]), lambda: x + ctx.var(np.zeros((5,), np.float32)), lambda: x.squeeze(0),
                lambda: S.matmul(x, x), lambda: x.transpose(0, 7)):
        with pytest.raises(S.SageError) as e:
            bad()
        assert e.value.code == 1


def test_matmul_shapes(ctx):
    a = ctx.var(np.zeros((2, 5, 7), np.float32))
    assert S.matmul(a, ctx.var(np.zeros((7, 3), np.float32))).extents == (2, 5, 3)
    q = ctx.var(np.zeros((2, 4, 6, 8), np.float32))
    assert S.matmul_batched(q, q.transpose(-1, -2)).extents == (2, 4, 6, 6)
    assert S.conv_2d(ctx.var(np.zeros((1, 5, 5, 4), np.float32)), ctx.var(np.zeros((3, 3, 4, 8), np.float32)), 1, 1, 1).extents == (1, 5, 5, 8)
    assert S.max_pool_2d(ctx.var(np.zeros((2, 112, 112, 64), np.float32)), 3, 2, 1, 1).extents == (2, 56, 56, 64)


def test_config1_program_matches_reference_fusion():
    """src/session.rs + src/ops.rs::fuse: z = x*y + x*3.14 is ONE variadic kernel with x bound twice and
    the literal folded in; z is materialised (it has several consumers).  pattern_fusion bit 2 keeps the
    whole-row program off, so the reference's own partition into kernels shows."""
    ctx = S.Context(-1, pattern_fusion=5)
    x = ctx.var(np.zeros((1024, 1024), np.float32))
    y = ctx.var(np.zeros((1024, 1024), np.float32))
    lab = ctx.var(np.zeros((1024, 1), np.uint32))
    z = x * y + x * 3.14
    loss = S.softmax_cross_entropy(z, lab)
    ctx.trace_begin()
    ctx.eval(loss)
    d = ctx.describe().strip().split("\n")
    assert d[0] == "variadic{((x0 * x1) + (x2 * sg_lit(0x4048f5c3u)))}(data,data,data)"
    assert "log_sum_exp(state)" in d[-1] and "gather" in d[-1]
    assert ctx.trace() == ["sage_map", "lse_rows", "sage_map", "gather", "reduce_g1", "sage_map"]
    ctx.close()
    # without pattern fusion the reference's own kernel sequence appears (max, exp, sum, log...)
    c2 = S.Context(-1, pattern_fusion=0)
    x2 = c2.var(np.zeros((64, 64), np.float32))
    c2.trace_begin()
    c2.eval(S.log_sum_exp(x2, [1]))
    assert [k.split("_g")[0] for k in c2.trace()] == ["reduce", "sage_map", "reduce", "sage_map"]
    c2.close()


def test_config1_runs_as_one_row_program(ctx):
    """The whole forward + gradient graph of config 1 (maps, row reductions, gather, scatter over one
    [R, C] space) becomes ONE generated kernel; graphs that leave the row space are compiled the ordinary way."""
    x = ctx.var(np.zeros((1024, 1024), np.float32))
    y = ctx.var(np.zeros((1024, 1024), np.float32))
    lab = ctx.var(np.zeros((1024, 1), np.uint32))
    loss = S.softmax_cross_entropy(x * y + x * 3.14, lab)
    gx = x.grad(loss)
    ctx.trace_begin()
    ctx.eval(loss, gx)
    assert ctx.trace() == ["sage_row_program"]
    d = ctx.describe()
    assert d.startswith("row_program[1024x1024; 128 threads x 8]") and "(3 inputs -> 2 outputs)" in d
    n = ctx.programs_compiled()
    ctx.clear()
    ctx.eval(loss, gx)
    assert ctx.programs_compiled() == n
    # a reduction across rows is not row-local: ordinary program
    ctx.clear()
    ctx.trace_begin()
    ctx.eval(loss.mean(0))
    assert "sage_row_program" not in ctx.trace()
    # rows that do not fill the block exactly, scalar accesses (C % 4 != 0), int data
    w = ctx.var(np.zeros((7, 301), np.float32))
    ctx.trace_begin()
    ctx.eval(S.softmax(w, [1]).int().float().sum([1], True) * w)
    assert ctx.trace() == ["sage_row_program"] and "[7x301; 96 threads x 4]" in ctx.describe()


def test_grad_graph_and_program_cache(ctx):
    x = ctx.var(np.zeros((8, 8), np.float32))
    y = (x.exp() * x).sum([0, 1], False)
    gx = x.grad(y)
    assert gx.extents == (8, 8)
    ctx.eval(gx)
    n = ctx.programs_compiled()
    ctx.clear()
    ctx.eval(gx)
    assert ctx.programs_compiled() == n  # same targets, same inputs: compiled program is reused
    with pytest.raises(S.SageError):
        S.grad(y, [ctx.var(np.zeros((2,), np.float32))])  # unrelated variable


def test_map_kernels_compile_for_every_op(ctx):
    """Every op of the reference's map tables (src/ops/map.rs:224-302) goes through the CUDA emitter and NVRTC."""
    f = ctx.var(np.zeros((5, 8), np.float32))
    for name in S._UN:
        if name in ("not_",):
            continue
        ctx.eval(getattr(f, name)())
    u = S.gt(f, 0.0)
    ctx.eval(u.not_(), S.and_(u, u), S.or_(u, u), S.cond(u, f, 1.0))
    for name in S._BIN:
        if name in ("and_", "or_"):
            continue
        ctx.eval(getattr(S, name + "_" if name == "pow" else name)(f, f.transpose(0, 1).organize().view([5, 8])))
    i = f.int()
    ctx.eval(i + i, i * i, S.minimum(i, i), i.float())
    # generic strided, broadcast and vector paths
    ctx.eval(f.transpose(0, 1) * 2.0, f + ctx.var(np.zeros((8,), np.float32)), f * ctx.var(np.zeros((5, 1), np.float32)))


def test_jit_compile_error_is_reported(ctx):
    m = ctypes.c_void_p()
    st = S.lib.sage_module_get(ctx.h, b"this is not CUDA", ctypes.byref(m))
    assert st == 4 and b"error" in S.lib.sage_last_error(ctx.h)


def test_allocator_policy():
    c = S.Context(-1, mem_capacity_bytes=64 << 20)
    a = c.alloc(100)  # small pool: 2 MiB segment, 512 B block
    s = c.mem_stats()
    assert s["mem_total"] == 2 << 20 and s["mem_used"] == 512 and s["num_device_allocs"] == 1
    b = c.alloc(3 << 20)  # large pool: 20 MiB segment
    assert c.mem_stats()["mem_total"] == (2 << 20) + (20 << 20)
    pa, pb = S.lib.sage_buf_ptr(a), S.lib.sage_buf_ptr(b)
    c.free(b)
    b2 = c.alloc(3 << 20)
    assert S.lib.sage_buf_ptr(b2) == pb and c.mem_stats()["num_device_allocs"] == 2  # reused, no new device allocation
    c3 = c.alloc(5 << 20)  # carved from the same 20 MiB segment (best fit + split)
    assert c.mem_stats()["num_device_allocs"] == 2
    with pytest.raises(S.SageError) as e:
        c.alloc(60 << 20)
    assert e.value.code == 2
    need, total = ctypes.c_uint64(), ctypes.c_uint64()
    S.lib.sage_last_oom(c.h, ctypes.byref(need), ctypes.byref(total))
    assert total.value == c.mem_stats()["mem_total"] and need.value > 0
    for buf in (a, b2, c3):
        c.free(buf)
    assert c.mem_stats()["mem_used"] == 0
    S.lib.sage_release_cached(c.h)
    assert c.mem_stats()["mem_total"] == 0  # merged back into whole segments and returned
    assert pa is not None
    c.close()


def test_allocator_reference_mode_without_cache():
    c = S.Context(-1, use_cache=0, mem_capacity_bytes=1000 << 20)  # the reference's shipped configuration
    bufs = [c.alloc(1 << 20) for _ in range(3)]
    assert c.mem_stats()["num_device_allocs"] == 3 and c.mem_stats()["mem_total"] == 3 << 20
    for b in bufs:
        c.free(b)
    assert c.mem_stats()["mem_total"] == 0
    c.close()


def test_oom_evicts_and_recomputes():
    """Program::exec's out-of-memory path (src/session.rs:259-331): with a tight cap the evaluator drops
    intermediates and finishes instead of failing."""
    n = 1 << 20  # 4 MiB tensors
    cap = 44 << 20  # room for two 20 MiB segments (ten 4 MiB blocks) + the 2 MiB small pool
    c = S.Context(-1, mem_capacity_bytes=cap)
    x = c.var(np.zeros((n,), np.float32))
    a = [x * float(i + 2) + 1.0 for i in range(12)]          # twelve 4 MiB states ...
    s = [v.sum([0], True) for v in a]                        # ... each needed early (its own sum) ...
    z = s[0]
    for v in s[1:]:
        z = z + v
    t = [(v * z.expand([n])).sum([0], True) for v in a]      # ... and again late, one at a time
    out = s[0] * 0.0
    for v, w in zip(t, s):
        out = out + v + v * 2.0 + w                           # t_i and s_i have two consumers: they are states
    c.trace_begin()
    c.eval(out)
    assert c.mem_stats()["mem_peak"] <= cap
    # more than 12 + 12 + 12 map/reduce launches means some states were evicted and recomputed
    assert len([k for k in c.trace() if k == "sage_map"]) > 24
    c.close()


def test_bert_base_plan():
    """The whole BERT-base graph compiles; the launch list is what the GPU will run."""
    c = S.Context(-1)
    model = S.Bert()
    params = model.params()
    assert len(params) == 2 + 2 + 12 * (8 + 2 + 4 + 2) + 2
    assert params[0].extents == (30522, 768) and params[1].extents == (512, 768) and params[-2].extents == (768, 2)
    for p in params:
        c.set(p, np.zeros(p.extents, np.float32))
    ids = c.var(np.zeros((32, 128), np.uint32))
    mask = c.var(np.ones((32, 128), np.float32))
    logits = model.pass_(ids, mask)
    assert logits.extents == (32, 2)
    c.trace_begin()
    c.eval(logits)
    t = c.trace()
    # scores, scale + mask, softmax and probabilities x values of a layer are one fused attention launch
    assert t.count("layernorm_rows") == 25 and t.count("softmax_rows") == 0 and t.count("attention_tc_3xtf32") == 12
    gemms = [k for k in t if k.startswith("gemm")]
    assert len(gemms) == 12 * 4 + 1  # per layer: grouped Q/K/V, output, FFN up, FFN down; + classifier
    k0, _ = c.launch_count()
    c.clear()
    c.eval(logits)
    # same program replayed; the tf32 splits of the 72 weight matrices are cached on their storages
    assert c.programs_compiled() == 1 and c.launch_count()[0] - k0 == len(t) - 72
    # Only the weights go through a split pass: every activation a GEMM reads gets its tf32 planes
    # from the kernel that produces it (GEMM epilogue, attention, layer norm).
    assert t.count("split_tf32") == 72 and t.count("gemm_tc_3xtf32") == 48
    # bias / residual / relu / scale+mask maps and the head split / merge copies are folded into the
    # GEMMs, the extended mask (1 - mask) * -1e5 into the attention kernel's expression (an elementwise map
    # commutes with the expand that follows it); what is left is the embedding sum and the classifier's two maps
    assert t.count("sage_map") == 1 + 2
    d = c.describe()
    # the three projections of a layer input are one grouped launch, read back as three slabs;
    # "=planes": the only reader is a GEMM, so the fp32 result is not stored at all
    assert d.count("slab(gemm_grouped=planes(") == 36
    # scale + mask is the expression between the score product and the softmax; head merge = the store pattern
    assert d.count("attention{((x0 / sg_lit(0x41000000u)) + (((-x1) + sg_lit(0x3f800000u)) * sg_lit(0xc7c35000u)))}[store]=planes") == 12
    assert d.count("gemm{(((float)((x0 + x1) > sg_lit(0x00000000u))) * (x0 + x1))}=planes") == 12  # FFN up: bias + relu
    assert d.count("gemm{((x0 + x1) + x2)}") == 24                           # output / FFN down: bias + residual
    assert d.count("softmax") == 0 and d.count("layer_norm+planes") == 24  # layer norm also feeds the residual
    # pattern_fusion bit 3 keeps the attention block as separate kernels: two batched products around a row softmax
    c9 = S.Context(-1, pattern_fusion=9)
    m9 = S.Bert(num_layers=1)
    for p in m9.params():
        c9.set(p, np.zeros(p.extents, np.float32))
    c9.trace_begin()
    c9.eval(m9.pass_(c9.var(np.zeros((32, 128), np.uint32)), c9.var(np.ones((32, 128), np.float32))))
    t9, d9 = c9.trace(), c9.describe()
    assert t9.count("softmax_rows") == 1 and "attention_tc_3xtf32" not in t9 and t9.count("gemm_tc_3xtf32") == 6
    assert "gemm_batched[store]=planes" in d9 and "gemm_batched{((x0 / sg_lit(0x41000000u)) + (((-x1) + sg_lit(" in d9 and "softmax=planes" in d9
    c9.close()
    # pattern_fusion bit 1: the softmax moves into the scores GEMM's epilogue (L = 128 keys fit one tile)
    c3 = S.Context(-1, pattern_fusion=3)
    m3 = S.Bert(num_layers=1)
    for p in m3.params():
        c3.set(p, np.zeros(p.extents, np.float32))
    c3.trace_begin()
    c3.eval(m3.pass_(c3.var(np.zeros((32, 128), np.uint32)), c3.var(np.ones((32, 128), np.float32))))
    assert "softmax_rows" not in c3.trace() and "|softmax=planes" in c3.describe()
    c3.close()
    assert c.mem_stats()["mem_peak"] < 3 << 30
    c.close()


def test_bert_plan_without_pattern_fusion_is_the_reference_decomposition():
    """pattern_fusion = 0: no composites, no GEMM lowering — every operator of the reference's graph is
    its own kernel (the evaluator of src/session.rs with map fusion only)."""
    c = S.Context(-1, pattern_fusion=0)
    model = S.Bert(num_vocabs=64, embed_dim=64, num_heads=2, seq_len=64, ffn_dim=128, num_layers=1, num_classes=3)
    for p in model.params():
        c.set(p, np.zeros(p.extents, np.float32))
    logits = model.pass_(c.var(np.zeros((4, 64), np.uint32)), c.var(np.ones((4, 64), np.float32)))
    c.trace_begin()
    c.eval(logits)
    t = c.trace()
    d = c.describe()
    assert "layernorm_rows" not in t and "softmax_rows" not in t
    assert "[store]" not in d and "+planes" not in d and "gemm{" not in d and "gemm_batched{" not in d
    # every operand goes through a split pass (the layer input once for its three readers Q, K, V)
    assert t.count("gemm_tc_3xtf32") == 8 and t.count("split_tf32") == 2 * 8 - 2
    c.close()


def test_resnet18_plan():
    c = S.Context(-1)
    model = S.ResNet18(3, 1000)
    params = model.params()
    assert params[0].extents == (7, 7, 3, 64) and params[-2].extents == (512, 1000)
    for p in params:
        c.set(p, np.zeros(p.extents, np.float32))
    x = c.var(np.zeros((2, 224, 224, 3), np.float32))
    y = model.pass_(x)
    assert y.extents == (2, 1000)
    c.trace_begin()
    c.eval(y)
    t = c.trace()
    assert t.count("max_pool2d") == 1 and t.count("avg_pool2d") == 1
    assert len([k for k in t if k.startswith("gemm")]) == 21
    c.close()


def test_training_step_plan(ctx):
    """examples/train.rs on a planning context: one cached program evaluates the loss, the accuracy and the
    gradients of all 42 parameters of ResNet d18(1, 10); Adam::update (src/optim.rs:134-177) is two launches
    of the multi-parameter kernel (32 slots each); weight-gradient GEMMs with a long K are split over K."""
    batch = 128
    model = S.ResNet18(1, 10)
    for p in model.params():
        ctx.set(p, np.zeros(p.extents, np.float32))
    xin, lin = S.Var.empty([batch, 28, 28, 1]), S.Var.empty([batch, 1], S.U32)
    ctx.set(xin, np.zeros((batch, 28, 28, 1), np.float32))
    ctx.set(lin, np.zeros((batch, 1), np.uint32))
    logits = model.pass_(xin)
    loss = S.softmax_cross_entropy(logits, lin).mean([0], False)
    acc = S.accuracy(logits, lin)
    assert acc.extents == (1,) and acc.dtype == S.F32
    grads = S.grad_param(loss, model)
    assert len(grads) == 42 and all(g.extents == p.extents for p, g in grads.items())
    opt = S.Adam(1e-4)
    opt.init(ctx)
    ctx.eval(*grads.values(), loss, acc)
    n = ctx.programs_compiled()
    ctx.trace_begin()
    opt.update(grads, ctx)
    assert ctx.trace() == ["adam_update", "adam_update"]
    ctx.clear()
    ctx.trace_begin()
    ctx.eval(*grads.values(), loss, acc)
    assert ctx.programs_compiled() == n                       # the step's program is compiled once
    t = ctx.trace()
    assert t.count("reduce_cols") >= 21 and "col2im" in t    # bias gradients, input gradients of the convolutions
    # gradients that the session has not evaluated are evaluated by update() itself (optim.rs:56-59)
    ctx.clear()
    ctx.trace_begin()
    opt.update(grads, ctx)
    assert ctx.trace()[-2:] == ["adam_update", "adam_update"] and len(ctx.trace()) > 100
    # Sgd: one rule, no state; a parameter that is not a data variable is refused (optim.rs:52-54)
    w = ctx.var(np.ones((4, 4), np.float32))
    y = (w * w).sum([0, 1], False)
    ctx.trace_begin()
    S.Sgd(0.1).update({w: w.grad(y)}, ctx)
    assert ctx.trace()[-1] == "sgd_update"
    with pytest.raises(S.SageError):
        S.Sgd(0.1).update({w * 2.0: w.grad(y)}, ctx)


def test_allocator_garbage_collects_old_cached_segments():
    """Pool::garbage_collect (src/session/memory.rs:410-452): nothing happens below 80 % use; above it, whole
    cached segments of the large pool go back to the device, oldest first (age = how many searches of the pool
    a block sat through), until 20 % of the capacity is reclaimed.  Pool::alloc runs it when no cached block
    fits (:336-341), before it tries to grow."""
    MiB = 1 << 20
    c = S.Context(-1, mem_capacity_bytes=250 * MiB)  # threshold 200 MiB in use, target 50 MiB

    def gc():
        r, runs, total = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        assert S.lib.sage_garbage_collect(c.h, ctypes.byref(r), ctypes.byref(runs), ctypes.byref(total)) == 0
        return r.value, runs.value, total.value
    old = c.alloc(12 * MiB)
    c.free(old)                                     # cached; every later search of the large pool ages it
    held = [c.alloc(20 * MiB) for _ in range(3)]    # 3 searches
    young = [c.alloc(14 * MiB), c.alloc(16 * MiB)]
    for b in young:
        c.free(b)                                   # two younger cached segments
    s = c.mem_stats()
    assert s["mem_total"] == (12 + 60 + 14 + 16) * MiB and s["mem_used"] == 60 * MiB
    assert gc() == (0, 0, 0)                        # 60 of 250 MiB in use: below the threshold
    held += [c.alloc(20 * MiB) for _ in range(7)]   # none of the cached segments fits: the pool grows to 242 MiB
    assert c.mem_stats()["mem_used"] == 200 * MiB and c.mem_stats()["mem_total"] == 242 * MiB
    r, runs, total = gc()
    # 80 % in use.  The first pass frees what is at least of average age (the old 12 MiB segment), the second the two
    # younger ones; 42 < 50 MiB, but nothing is left
    assert r == (12 + 14 + 16) * MiB and runs == 1 and total == r
    assert c.mem_stats()["mem_total"] == 200 * MiB
    # inside alloc: when no cached block fits, old cached segments are collected before the pool grows
    c.free(held.pop())                              # a whole 20 MiB segment is cached, 180 MiB in use
    held.append(c.alloc(30 * MiB))                  # does not fit it; below the threshold: no collection, grows
    assert c.mem_stats()["mem_total"] == 230 * MiB
    held.append(c.alloc(21 * MiB))                  # 210 MiB in use: the cached 20 MiB go back, then 22 MiB are added
    assert c.mem_stats()["mem_total"] == 232 * MiB
    assert gc() == (0, 2, total + 20 * MiB)         # that collection ran inside alloc; nothing is left to collect
    for b in held:
        c.free(b)
    c.close()


def test_bert_training_plan():
    """One training step of Bert (4 layers here, base width) on a planning context: LayerNorm's backward pass and the
    softmax backward pieces run as generated row programs between the GEMMs, weight gradients are cut into K
    slices, and after the first step (which splits the weights once) no tf32 split pass is left: every GEMM
    operand's planes are written by the kernel that produces it or kept up to date by the optimizer."""
    layers = 4
    model = S.Bert(num_layers=layers)
    c = S.Context(-1)
    for p in model.params():
        c.set(p, np.zeros(p.extents, np.float32))
    ids, mask, lab = c.var(np.zeros((32, 128), np.uint32)), c.var(np.ones((32, 128), np.float32)), c.var(np.zeros((32, 1), np.uint32))
    loss = S.softmax_cross_entropy(model.pass_(ids, mask), lab).mean([0], False)
    grads = S.grad_param(loss, model)
    opt = S.Adam(1e-4)
    opt.init(c)
    counts = []
    for step in range(2):
        c.trace_begin()
        c.eval(*grads.values(), loss)
        opt.update(grads, c)
        c.clear()
        t = c.trace()
        counts.append({k: t.count(k) for k in ("sage_row_program", "split_tf32", "gemm_tc_3xtf32", "adam_update", "layernorm_rows",
                                               "reduce_slices", "reduce_cols")})
    first, steady = counts
    # LayerNorm backward (2 per layer + the embedding's) and two softmax backward pieces per layer
    assert steady["sage_row_program"] == first["sage_row_program"] == (2 * layers + 1) + 2 * layers
    assert first["split_tf32"] == 6 * layers and steady["split_tf32"] == 0                              # the weights, once
    assert steady["gemm_tc_3xtf32"] == 24 * layers and steady["layernorm_rows"] == 2 * layers + 1
    # the six weight gradients of a layer are cut over K and summed by the slice kernel; the six bias gradients are
    # column sums, one launch each
    assert steady["reduce_slices"] == 6 * layers and steady["reduce_cols"] == 6 * layers
    d = c.describe()
    assert "row_program[4096x768" in d and "row_program[49152x128" in d
    c.close()


def test_program_cache_is_bounded_and_least_recently_used():
    """A loop that builds a fresh graph per step (a new input Var per batch) must not grow the session: compiled
    programs are kept up to a limit, least recently used dropped first, and a dropped program lets go of the
    tensors only it kept alive."""
    ctx = S.Context(-1)
    try:
        w = ctx.var(np.ones((64, 64), np.float32))
        _, limit = ctx.programs_cached()
        assert 8 <= limit <= 64
        first = (ctx.var(np.zeros((256, 64), np.float32)).matmul(w) + 1.0)
        ctx.eval(first)
        used = []
        for i in range(3 * limit):
            x = ctx.var(np.zeros((256, 64), np.float32))      # a fresh leaf: a new program every time
            y = S.relu(x.matmul(w) + 1.0)
            ctx.eval(y)
            ctx.clear()
            del x, y
            if i % 7 == 0:                                    # keep `first` recent: it must survive
                before = ctx.programs_compiled()
                ctx.eval(first)
                ctx.clear()
                assert ctx.programs_compiled() == before
            used.append(ctx.mem_stats()["mem_used"])
            assert ctx.programs_cached()[0] <= limit
        assert ctx.programs_cached()[0] == limit
        assert max(used[limit + 2:]) <= max(used[:limit + 2])  # memory in use stops growing once the cache is full
        ctx.drop_programs()
        assert ctx.programs_cached()[0] == 0
        before = ctx.programs_compiled()
        ctx.eval(first)
        assert ctx.programs_compiled() == before + 1
    finally:
        ctx.close()
