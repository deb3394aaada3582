// Convolution building blocks.  Reference: src/ops/conv.rs — conv_size :47-59, conv_2d :61-96,
// avg_pool_2d / max_pool_2d :143-165, batch_norm_2d :167-185, im2col :188-226 + kernel :289-374,
// col2im :229-264 + kernel :404-498.  Images are NHWC, filters [KH,KW,C,OC]; every two-element
// parameter is ordered [w, h].
#include "graph.h"

namespace sage {
using namespace ops;

static k::Window window(Pair ker, Pair stride, Pair pad, Pair dil) {
    return k::Window{(int)ker.w, (int)ker.h, (int)stride.w, (int)stride.h, (int)pad.w, (int)pad.h, (int)dil.w, (int)dil.h};
}

static long long conv_size(long long size, long long ker, long long stride, long long pad, long long dil) {
    return (size + 2 * pad - dil * (ker - 1) - 1) / stride + 1;
}

struct Im2colOp : Operator {
    Pair ker, stride, pad, dil, col;
    const char *name() const override { return "im2col"; }
    std::vector<Var> grad(const std::vector<Var> &x, const Var &, const Var &gy) override {
        return {col2im(gy, Pair{x[0].extent(2), x[0].extent(1)}, ker, stride, pad, dil)};
    }
    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        const Array &e = x[0].desc.shape.extents;
        return k::im2col(ctx, (const float *)x[0].ptr(), (float *)y->ptr(), e[0], e[1], e[2], e[3], col.h, col.w,
                         window(ker, stride, pad, dil));
    }
};

bool im2col_params(const Operator &op, k::Window *w, long long dims[6]) {
    const Im2colOp *o = dynamic_cast<const Im2colOp *>(&op);
    if (!o || o->in[0].dtype != SAGE_F32 || !o->in[0].shape.has_default_strides()) return false;
    *w = window(o->ker, o->stride, o->pad, o->dil);
    const Array &e = o->in[0].shape.extents;
    dims[0] = e[0];
    dims[1] = e[1];
    dims[2] = e[2];
    dims[3] = e[3];
    dims[4] = o->col.h;
    dims[5] = o->col.w;
    return true;
}

struct Col2imOp : Operator {
    Pair img, ker, stride, pad, dil;
    const char *name() const override { return "col2im"; }
    std::vector<Var> grad(const std::vector<Var> &, const Var &, const Var &gy) override {
        return {im2col(gy, ker, stride, pad, dil)};
    }
    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        const Array &e = x[0].desc.shape.extents;  // [N, col_h, col_w, KH, KW, C]
        return k::col2im(ctx, (const float *)x[0].ptr(), (float *)y->ptr(), e[0], img.h, img.w, e[5], e[1], e[2],
                         window(ker, stride, pad, dil));
    }
};

Var ops::im2col(const Var &x0, Pair ker, Pair stride, Pair pad, Pair dil) {
    Var x = x0.organize();
    if (x.rank() != 4) shape_fail("im2col: input must be [N,H,W,C]");
    if (x.dtype() != SAGE_F32) shape_fail("im2col: input must be float");
    Pair col{conv_size(x.extent(2), ker.w, stride.w, pad.w, dil.w), conv_size(x.extent(1), ker.h, stride.h, pad.h, dil.h)};
    if (col.w <= 0 || col.h <= 0) shape_fail("im2col: window larger than the padded image");
    auto op = std::make_shared<Im2colOp>();
    op->ker = ker;
    op->stride = stride;
    op->pad = pad;
    op->dil = dil;
    op->col = col;
    op->in = {x.desc};
    op->out = TensorDesc(Array{x.extent(0), col.h, col.w, ker.h, ker.w, x.extent(3)}, x.dtype());
    return Var::from_op(op, {x});
}

Var ops::col2im(const Var &x0, Pair img, Pair ker, Pair stride, Pair pad, Pair dil) {
    Var x = x0.organize();
    if (x.rank() != 6) shape_fail("col2im: input must be [N,OH,OW,KH,KW,C]");
    auto op = std::make_shared<Col2imOp>();
    op->img = img;
    op->ker = ker;
    op->stride = stride;
    op->pad = pad;
    op->dil = dil;
    op->in = {x.desc};
    op->out = TensorDesc(Array{x.extent(0), img.h, img.w, x.extent(5)}, x.dtype());
    return Var::from_op(op, {x});
}

Var ops::conv_2d(const Var &x, const Var &filter, Pair stride, Pair pad, Pair dil) {  // conv.rs:61-96
    if (filter.rank() != 4) shape_fail("conv_2d: filter must be [KH,KW,C,OC]");
    const long long kh = filter.extent(0), kw = filter.extent(1), cin = filter.extent(2), cout = filter.extent(3);
    Var col = im2col(x, Pair{kw, kh}, stride, pad, dil);
    if (col.extent(5) != cin) shape_fail("conv_2d: channel mismatch");
    const long long n = col.extent(0), ch = col.extent(1), cw = col.extent(2);
    Var c2 = view(col, {n * ch * cw, kh * kw * cin});
    Var f2 = view(filter, {kh * kw * cin, cout});
    return view(matmul(c2, f2), {n, ch, cw, cout});
}

// Pooling as one kernel: the same value as im2col followed by mean / max over [KH,KW], without the
// KH*KW-times larger intermediate.
struct Pool2dOp : Operator {
    bool is_max;
    Pair ker, stride, pad, dil;
    const char *name() const override { return is_max ? "max_pool2d" : "avg_pool2d"; }
    std::vector<Var> grad(const std::vector<Var> &, const Var &, const Var &) override {
        shape_fail("pool2d composite is not differentiated; grad walks the decomposed graph");
    }
    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        const Array &e = x[0].desc.shape.extents;
        const Array &o = out.shape.extents;
        return k::pool2d(ctx, is_max, (const float *)x[0].ptr(), (float *)y->ptr(), e[0], e[1], e[2], e[3], o[1], o[2],
                         window(ker, stride, pad, dil));
    }
};

static Var pool(const Var &x, Pair ker, Pair stride, Pair pad, Pair dil, bool is_max) {
    Var col = im2col(x, ker, stride, pad, dil);
    Var y = is_max ? reduce(col, {3, 4}, false, RMax) : mean(col, {3, 4}, false);
    const Var &src = col.origin->inputs[0];  // the organized image
    auto op = std::make_shared<Pool2dOp>();
    op->is_max = is_max;
    op->ker = ker;
    op->stride = stride;
    op->pad = pad;
    op->dil = dil;
    op->in = {src.desc};
    op->out = y.desc.pristine();
    y.origin->composite.reset(new Composite{op, {src}});
    return y;
}

Var ops::avg_pool_2d(const Var &x, Pair ker, Pair stride, Pair pad, Pair dil) { return pool(x, ker, stride, pad, dil, false); }
Var ops::max_pool_2d(const Var &x, Pair ker, Pair stride, Pair pad, Pair dil) { return pool(x, ker, stride, pad, dil, true); }

Var ops::batch_norm_2d(const Var &x, const Var &gamma, const Var &beta, const Var &mean_, const Var &var_, float eps) {
    Var xc = div(sub(x, mean_), unary_map(add(var_, eps), Sqrt));  // conv.rs:181-184
    return add(mul(gamma, xc), beta);
}

}  // namespace sage
