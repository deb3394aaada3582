// Layout and index operators.  Reference: src/ops/core.rs — zero-copy views (reshape :203-261,
// expand :263-322, permute :358-398, squeeze/unsqueeze :400-476, slice :478-523) and the kernels
// unslice :525-611, gather :613-719, scatter :721-834, concat :836-935.
#include <cuda_runtime.h>

#include "graph.h"

namespace sage {
using namespace ops;

enum ViewKind { VReshape, VExpand, VPermute, VSqueeze, VUnsqueeze, VSlice };

struct ViewOp : Operator {
    ViewKind kind;
    std::vector<int> perm;
    int axis = 0;
    long long start = 0, end = 0;

    const char *name() const override {
        static const char *n[] = {"reshape", "expand", "permute", "squeeze", "unsqueeze", "slice"};
        return n[kind];
    }
    Cat cat() const override { return kind == VExpand ? Cat::LayoutExpand : Cat::Other; }

    sage_status compute(const std::vector<Tensor> &x, Context &, Tensor *y) override {
        const Tensor &t = x[0];
        switch (kind) {
        case VReshape: {  // core.rs:246-260
            Shape s = out.shape;
            s.offset += t.desc.shape.offset;
            *y = t.with_shape(s);
            break;
        }
        case VExpand: *y = t.with_shape(t.desc.shape.expand(out.shape.extents)); break;
        case VPermute: *y = t.with_shape(t.desc.shape.permute(perm)); break;
        case VSqueeze: *y = t.with_shape(t.desc.shape.remove(axis)); break;
        case VUnsqueeze: *y = t.with_shape(t.desc.shape.insert(axis)); break;
        case VSlice: *y = t.with_shape(t.desc.shape.select_range(start, end - 1, axis)); break;
        }
        return SAGE_OK;
    }

    std::vector<Var> grad(const std::vector<Var> &x, const Var &, const Var &gy) override {
        const Var &x0 = x[0];
        switch (kind) {
        case VReshape: return {reshape(gy, in[0].shape)};  // core.rs:242-244
        case VExpand: {                                     // core.rs:292-313
            const int surplus = gy.rank() - x0.rank();
            std::vector<long long> axes;
            for (int i = 0; i < surplus; ++i) axes.push_back(i);
            for (int i = 0; i < x0.rank(); ++i)
                if (gy.extent(i + surplus) != x0.extent(i)) axes.push_back(i + surplus);
            return {view(reduce(gy, axes, false, Sum), in[0].shape.extents)};
        }
        case VPermute: {  // core.rs:387-390 applies the same permutation to gy
            std::vector<long long> p(perm.begin(), perm.end());
            return {permute(gy, p)};
        }
        case VSqueeze: return {unsqueeze(gy, axis)};
        case VUnsqueeze: return {squeeze(gy, axis)};
        case VSlice: return {unslice(gy, axis, start, x0.extent(axis))};
        }
        return {Var()};
    }
};

bool is_view_op(const Operator &op) { return dynamic_cast<const ViewOp *>(&op) != nullptr; }
bool is_reshape_op(const Operator &op) {
    const ViewOp *v = dynamic_cast<const ViewOp *>(&op);
    return v && v->kind == VReshape;
}

bool is_expand_op(const Operator &op) {
    const ViewOp *v = dynamic_cast<const ViewOp *>(&op);
    return v && v->kind == VExpand;
}
// An expand of `in` to `extents` as a bare operator (the evaluator builds these when it moves a map behind an expand).
std::shared_ptr<Operator> make_expand_op(const TensorDesc &in, const Array &extents) {
    auto op = std::make_shared<ViewOp>();
    op->kind = VExpand;
    op->in = {in};
    op->out = TensorDesc(in.shape.expand(extents), in.dtype);
    return op;
}

// 0 reshape, 1 expand, 2 permute, 3 squeeze, 4 unsqueeze, 5 slice; -1 when `op` is no view
int view_op_kind(const Operator &op) {
    const ViewOp *v = dynamic_cast<const ViewOp *>(&op);
    return v ? (int)v->kind : -1;
}

static Var make_view(ViewKind kind, const Var &x, const Shape &shape, std::function<void(ViewOp &)> fill = nullptr) {
    auto op = std::make_shared<ViewOp>();
    op->kind = kind;
    op->in = {x.desc};
    op->out = TensorDesc(shape, x.dtype());
    if (fill) fill(*op);
    return Var::from_op(op, {x});
}

Var ops::reshape(const Var &x0, const Shape &shape) {  // core.rs:213-236
    Var x = x0.organize();
    if (x.size() != shape.size()) shape_fail("incompatible size");
    return make_view(VReshape, x, shape);
}

Var ops::view(const Var &x, const Array &extents) { return reshape(x, Shape(infer_extents(extents, x.size()))); }

Var ops::expand(const Var &x, const Array &extents) {
    Array e = infer_extents(extents, 0);
    return make_view(VExpand, x, x.desc.shape.expand(e));
}

Var ops::permute(const Var &x, const std::vector<long long> &axes) {
    std::vector<int> p = to_axes(axes, x.rank());
    if ((int)p.size() != x.rank()) shape_fail("permute: wrong number of axes");
    return make_view(VPermute, x, x.desc.shape.permute(p), [&](ViewOp &o) { o.perm = p; });
}

Var ops::transpose(const Var &x, long long a1, long long a2) {  // core.rs:330-356
    const int r = x.rank(), i1 = to_axis(a1, r), i2 = to_axis(a2, r);
    std::vector<long long> axes(r);
    for (int i = 0; i < r; ++i) axes[i] = i == i1 ? i2 : i == i2 ? i1 : i;
    return permute(x, axes);
}

Var ops::squeeze(const Var &x, long long axis) {
    const int a = to_axis(axis, x.rank());
    if (x.extents()[a] != 1) shape_fail("only size=1 axes can be squeezed");
    return make_view(VSqueeze, x, x.desc.shape.remove(a), [&](ViewOp &o) { o.axis = a; });
}

Var ops::unsqueeze(const Var &x, long long axis) {
    const int a = to_axis(axis, x.rank() + 1);
    return make_view(VUnsqueeze, x, x.desc.shape.insert(a), [&](ViewOp &o) { o.axis = a; });
}

Var ops::slice(const Var &x, long long axis, long long start, long long end) {
    const int a = to_axis(axis, x.rank());
    if (end <= start) shape_fail("slice: empty range");
    return make_view(VSlice, x, x.desc.shape.select_range(start, end - 1, a), [&](ViewOp &o) {
        o.axis = a;
        o.start = start;
        o.end = end;
    });
}

// ---------------------------------------------------------------- unslice (core.rs:525-611)
struct UnsliceOp : Operator {
    int axis;
    long long start, end;
    const char *name() const override { return "unslice"; }
    std::vector<Var> grad(const std::vector<Var> &x, const Var &, const Var &gy) override {
        return {slice(gy, axis, start, start + x[0].extent(axis))};
    }
    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        ctx.note_memset();  // fill_zero, core.rs:577
        if (!ctx.dry()) {
            st = ctx.check_cuda(cudaMemsetAsync(y->ptr(), 0, (size_t)out.shape.size() * 4, ctx.stream()), "memset");
            if (st) return st;
        }
        Shape sub = y->desc.shape.select_range(start, start + x[0].desc.shape.extents[axis] - 1, axis);
        return k::strided_copy(ctx, (const uint32_t *)x[0].ptr(), x[0].dims(),
                               (uint32_t *)y->data->dev + sub.offset, sub.strides.data());
    }
};

Var ops::unslice(const Var &x, long long axis, long long start, long long end) {
    const int a = to_axis(axis, x.rank());
    if (end < start + x.extent(a)) shape_fail("unslice: range smaller than the input");
    Array e = x.extents();
    e[a] = end;
    auto op = std::make_shared<UnsliceOp>();
    op->axis = a;
    op->start = start;
    op->end = end;
    op->in = {x.desc};
    op->out = TensorDesc(e, x.dtype());
    return Var::from_op(op, {x});
}

// ---------------------------------------------------------------- gather / scatter (core.rs:613-834)
struct GatherOp : Operator {
    int axis;
    const char *name() const override { return "gather"; }
    std::vector<Var> grad(const std::vector<Var> &x, const Var &, const Var &gy) override {
        return {scatter(gy, x[1], axis, x[0].extents()), Var()};
    }
    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        return k::gather(ctx, (const uint32_t *)x[0].ptr(), x[0].desc.shape.strides.data(), (const uint32_t *)x[1].ptr(),
                         x[1].dims(), axis, (uint32_t *)y->ptr());
    }
};

Var ops::gather(const Var &x, const Var &ind, long long axis) {
    const int a = to_axis(axis, x.rank());
    if (x.rank() != ind.rank()) shape_fail("gather: x and index ranks differ");  // core.rs:623
    if (ind.dtype() == SAGE_F32) shape_fail("gather: index must be int or uint");
    auto op = std::make_shared<GatherOp>();
    op->axis = a;
    op->in = {x.desc, ind.desc};
    op->out = TensorDesc(ind.extents(), x.dtype());
    return Var::from_op(op, {x, ind});
}

struct ScatterOp : Operator {
    int axis;
    const char *name() const override { return "scatter"; }
    std::vector<Var> grad(const std::vector<Var> &x, const Var &, const Var &gy) override {
        return {gather(gy, x[1], axis), Var()};
    }
    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        if (x[0].desc.dtype != SAGE_F32) return ctx.fail(SAGE_ERR_UNSUPPORTED, "scatter: only float values");
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        ctx.note_memset();  // fill_zero, core.rs:782
        if (!ctx.dry()) {
            st = ctx.check_cuda(cudaMemsetAsync(y->ptr(), 0, (size_t)out.shape.size() * 4, ctx.stream()), "memset");
            if (st) return st;
        }
        return k::scatter_add(ctx, (const float *)x[0].ptr(), x[0].desc.shape.strides.data(), (const uint32_t *)x[1].ptr(),
                              x[1].dims(), axis, (float *)y->ptr(), y->desc.shape.strides.data());
    }
};

Var ops::scatter(const Var &x, const Var &ind, long long axis, const Array &extents) {
    const int a = to_axis(axis, x.rank());
    Array e = infer_extents(extents, 0);
    if ((int)e.size() != x.rank() || x.rank() != ind.rank()) shape_fail("scatter: rank mismatch");
    if (x.extents() != ind.extents()) shape_fail("scatter: values and index extents differ");
    auto op = std::make_shared<ScatterOp>();
    op->axis = a;
    op->in = {x.desc, ind.desc};
    op->out = TensorDesc(e, x.dtype());
    return Var::from_op(op, {x, ind});
}

// The axis of a gather (`scatter` false) or scatter operator, -1 when `op` is neither.
int index_op_axis(const Operator &op, bool scatter) {
    if (scatter) {
        const ScatterOp *s = dynamic_cast<const ScatterOp *>(&op);
        return s ? s->axis : -1;
    }
    const GatherOp *g = dynamic_cast<const GatherOp *>(&op);
    return g ? g->axis : -1;
}

// ---------------------------------------------------------------- concat (core.rs:836-935)
struct ConcatOp : Operator {
    int axis;
    const char *name() const override { return "concat"; }
    std::vector<Var> grad(const std::vector<Var> &x, const Var &, const Var &gy) override {
        std::vector<Var> g;
        long long i = 0;
        for (const Var &v : x) {
            g.push_back(slice(gy, axis, i, i + v.extent(axis)));
            i += v.extent(axis);
        }
        return g;
    }
    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        // The reference zero-fills first (core.rs:896); every element is overwritten below, so the
        // fill is dropped.
        long long i = 0;
        for (const Tensor &t : x) {
            const long long e = t.desc.shape.extents[axis];
            Shape sub = y->desc.shape.select_range(i, i + e - 1, axis);
            i += e;
            st = k::strided_copy(ctx, (const uint32_t *)t.ptr(), t.dims(), (uint32_t *)y->data->dev + sub.offset,
                                 sub.strides.data());
            if (st) return st;
        }
        return SAGE_OK;
    }
};

Var ops::concat(const std::vector<Var> &xs, long long axis) {
    if (xs.empty()) shape_fail("concat: no inputs");
    const int a = to_axis(axis, xs[0].rank());
    Array e = xs[0].extents();
    long long total = 0;
    for (const Var &v : xs) {
        if (v.rank() != xs[0].rank()) shape_fail("not in the same shape");
        for (int i = 0; i < v.rank(); ++i)
            if (i != a && v.extents()[i] != e[i]) shape_fail("not in the same shape");
        total += v.extent(a);
    }
    e[a] = total;
    auto op = std::make_shared<ConcatOp>();
    op->axis = a;
    for (const Var &v : xs) op->in.push_back(v.desc);
    op->out = TensorDesc(e, xs[0].dtype());
    return Var::from_op(op, xs);
}

// ---------------------------------------------------------------- uniform / normal (src/ops/rand.rs:21-140)
// The reference draws the two seeds from the thread's generator at every evaluation; here they belong to
// the operator, so an evaluation can be repeated.
struct RandOp : Operator {
    bool normal;
    unsigned seed_x, seed_y;
    const char *name() const override { return normal ? "normal" : "uniform"; }
    std::vector<Var> grad(const std::vector<Var> &, const Var &, const Var &) override { return {}; }
    sage_status compute(const std::vector<Tensor> &, Context &ctx, Tensor *y) override {
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        return k::rand_fill(ctx, normal, (float *)y->ptr(), out.shape.size(), seed_x, seed_y);
    }
};

static Var make_rand(bool normal, const Array &extents, unsigned seed_x, unsigned seed_y) {
    auto op = std::make_shared<RandOp>();
    op->normal = normal;
    op->seed_x = seed_x;
    op->seed_y = seed_y;
    op->out = TensorDesc(infer_extents(extents, 0), SAGE_F32);
    return Var::from_op(op, {});
}
Var ops::uniform(const Array &extents, unsigned seed_x, unsigned seed_y) { return make_rand(false, extents, seed_x, seed_y); }
Var ops::normal(const Array &extents, unsigned seed_x, unsigned seed_y) { return make_rand(true, extents, seed_x, seed_y); }

}  // namespace sage
