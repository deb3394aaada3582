// Matrix products.  Reference: src/ops/gemm.rs — matmul :30-51, matmul_batched :53-104, gemm
// :106-140, Gemm::compute_direct :176-250, gemm_batched :253-290, GemmBatched::compute_direct
// :338-421.  Operands are forced contiguous by organize(), so the leading dimension is the row
// length; C is row-major [M,N].  The reference zero-fills C before the kernel (gemm.rs:179); with
// beta = 0 that fill has no effect on the result and is dropped here.
#include "graph.h"

namespace sage {
using namespace ops;

struct GemmOp : Operator {
    bool ta, tb, batched;
    const char *name() const override { return batched ? "gemm_batched" : "gemm"; }
    Cat cat() const override { return Cat::Contract; }

    std::vector<Var> grad(const std::vector<Var> &x, const Var &, const Var &gy) override {  // gemm.rs:150-163,304-328
        auto g = [&](const Var &a, const Var &b, bool t1, bool t2) { return batched ? gemm_batched(a, b, t1, t2) : gemm(a, b, t1, t2); };
        if (!ta && !tb) return {g(gy, x[1], false, true), g(x[0], gy, true, false)};
        if (!ta && tb) return {g(gy, x[1], false, false), g(gy, x[0], true, false)};
        if (ta && !tb) return {g(x[1], gy, false, true), g(x[0], gy, false, false)};
        return {g(x[1], gy, true, true), g(gy, x[0], true, true)};
    }

    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        const int o = batched ? 1 : 0;
        const Shape &a = x[0].desc.shape, &b = x[1].desc.shape;
        const int h_ax = ta ? 1 : 0, c_ax = ta ? 0 : 1, w_ax = tb ? 0 : 1;
        k::GemmArgs g;
        g.ta = ta;
        g.tb = tb;
        g.m = a.extents[h_ax + o];
        g.k = a.extents[c_ax + o];
        g.n = b.extents[w_ax + o];
        g.a = (const float *)x[0].ptr();
        g.b = (const float *)x[1].ptr();
        g.c = (float *)y->ptr();
        g.lda = a.strides[o];
        g.ldb = b.strides[o];
        g.ldc = g.n;
        g.batch = batched ? a.extents[0] : 1;
        g.stride_a = batched ? a.strides[0] : 0;
        g.stride_b = batched ? b.strides[0] : 0;
        g.stride_c = g.m * g.n;
        if (ctx.opts().gemm_backend == 1 || !k::gemm_tc_supported(g)) return k::gemm_simt(ctx, g);
        // Tensor-core path: each operand's hi/lo split is cached on its storage.
        std::shared_ptr<SplitCache> sa, sb;
        st = split_of(ctx, x[0], g.lda, g.stride_a, ta ? g.k : g.m, ta ? g.m : g.k, g.batch, &sa);
        if (st) return st;
        st = split_of(ctx, x[1], g.ldb, g.stride_b, tb ? g.n : g.k, tb ? g.k : g.n, g.batch, &sb);
        if (st) return st;
        return k::gemm_tcgen05_planes(ctx, g, sa->planes, sb->planes);
    }

    static sage_status split_of(Context &ctx, const Tensor &t, long long ld, long long batch_stride, long long rows, long long cols,
                                long long batches, std::shared_ptr<SplitCache> *out) {
        std::shared_ptr<SplitCache> &c = t.data->split;
        const long long off = t.desc.shape.offset;
        if (c && c->offset == off && c->ld == ld && c->batch_stride == batch_stride && c->planes.rows == rows && c->planes.cols == cols &&
            c->planes.batches == batches) {
            *out = c;
            return SAGE_OK;
        }
        auto fresh = std::make_shared<SplitCache>();
        fresh->alloc = ctx.allocator_ptr();
        fresh->offset = off;
        fresh->ld = ld;
        fresh->batch_stride = batch_stride;
        sage_status st = k::split_tf32(ctx, (const float *)t.ptr(), ld, batch_stride, (int)rows, (int)cols, (int)batches, &fresh->planes);
        if (st) return st;
        c = fresh;
        *out = fresh;
        return SAGE_OK;
    }
};

static void gemm_dims(const Array &e1, const Array &e2, size_t o, bool t1, bool t2, long long *h, long long *w) {
    const long long c1 = t1 ? e1[o] : e1[o + 1], c2 = t2 ? e2[o + 1] : e2[o];
    *h = t1 ? e1[o + 1] : e1[o];
    *w = t2 ? e2[o] : e2[o + 1];
    if (c1 != c2) shape_fail("gemm: inner dimensions differ");
}

Var ops::gemm(const Var &a0, const Var &b0, bool ta, bool tb) {
    Var a = a0.organize(), b = b0.organize();
    if (a.rank() != 2 || b.rank() != 2) shape_fail("gemm: operands must be rank 2");
    if (a.dtype() != b.dtype() || a.dtype() != SAGE_F32) shape_fail("gemm: operands must be float");
    long long h, w;
    gemm_dims(a.extents(), b.extents(), 0, ta, tb, &h, &w);
    auto op = std::make_shared<GemmOp>();
    op->ta = ta;
    op->tb = tb;
    op->batched = false;
    op->in = {a.desc, b.desc};
    op->out = TensorDesc(Array{h, w}, a.dtype());
    return Var::from_op(op, {a, b});
}

Var ops::gemm_batched(const Var &a0, const Var &b0, bool ta, bool tb) {
    Var a = a0.organize(), b = b0.organize();
    if (a.rank() != 3 || b.rank() != 3) shape_fail("gemm_batched: operands must be rank 3");
    if (a.extent(0) != b.extent(0)) shape_fail("gemm_batched: batch extents differ");
    if (a.dtype() != b.dtype() || a.dtype() != SAGE_F32) shape_fail("gemm_batched: operands must be float");
    long long h, w;
    gemm_dims(a.extents(), b.extents(), 1, ta, tb, &h, &w);
    auto op = std::make_shared<GemmOp>();
    op->ta = ta;
    op->tb = tb;
    op->batched = true;
    op->in = {a.desc, b.desc};
    op->out = TensorDesc(Array{a.extent(0), h, w}, a.dtype());
    return Var::from_op(op, {a, b});
}

Var ops::matmul(const Var &x1, const Var &x2) {  // gemm.rs:30-51
    Array ext(x1.extents().begin(), x1.extents().end() - 1);
    ext.insert(ext.end(), x2.extents().begin() + 1, x2.extents().end());
    Var a = view(x1, {x1.size() / x1.extent(-1), x1.extent(-1)});
    Var b = view(x2, {x2.extent(0), x2.size() / x2.extent(0)});
    return view(gemm(a, b, false, false), ext);
}

Var ops::matmul_batched(const Var &x1, const Var &x2) {  // gemm.rs:53-104
    Array batch_ext;
    for (int i = 0; i < std::min(x1.rank() - 2, x2.rank() - 2); ++i) {
        if (x1.extent(i) == x2.extent(i)) batch_ext.push_back(x1.extent(i));
        else break;
    }
    const int bl = (int)batch_ext.size();
    if (bl == 0) shape_fail("batch dim incorrect!");
    long long bs = 1;
    for (long long e : batch_ext) bs *= e;
    Array ext = batch_ext;
    ext.insert(ext.end(), x1.extents().begin() + bl, x1.extents().end() - 1);
    ext.insert(ext.end(), x2.extents().begin() + bl + 1, x2.extents().end());
    Var a = view(x1, {bs, x1.size() / (x1.extent(-1) * bs), x1.extent(-1)});
    Var b = view(x2, {bs, x2.extent(bl), x2.size() / (x2.extent(bl) * bs)});
    return view(gemm_batched(a, b, false, false), ext);
}

}  // namespace sage
