// Reduction operators.  Reference: src/ops/reduce.rs — reduce :203-325, mean :59-71, var :73-82,
// reduce_arg :327-431, reduced_extents :124-140.
#include "graph.h"

namespace sage {
using namespace ops;

static Array reduced_extents(const Array &extents, const std::vector<int> &axes, bool preserve) {
    Array out;
    for (int i = 0; i < (int)extents.size(); ++i) {
        const bool red = std::find(axes.begin(), axes.end(), i) != axes.end();
        if (!red) out.push_back(extents[i]);
        else if (preserve) out.push_back(1);
    }
    if (out.empty()) out.push_back(1);
    return out;
}

static k::Dims to_dims(const Shape &s) {
    k::Dims d;
    d.ndim = s.rank();
    for (int i = 0; i < d.ndim; ++i) {
        d.ext[i] = s.extents[i];
        d.str[i] = s.strides[i];
    }
    return d;
}

struct ReduceOp : Operator {
    Red kind;
    std::vector<int> axes;
    bool preserve;
    const char *name() const override {
        static const char *n[] = {"reduce_sum", "reduce_prod", "reduce_max", "reduce_min"};
        return n[kind];
    }
    Cat cat() const override { return Cat::Reduce; }

    std::vector<Var> grad(const std::vector<Var> &xs, const Var &y0, const Var &gy0) override {  // reduce.rs:236-256
        const Var &x = xs[0];
        Var y = y0, gy = gy0;
        if (!preserve) {
            Array e = reduced_extents(in[0].shape.extents, axes, true);
            y = view(y, e);
            gy = view(gy, e);
        }
        switch (kind) {
        case Sum: return {expand(gy, x.extents())};
        case Prod: return {div(mul(gy, y), x)};
        default: return {cond(binary_map(x, y, Eq), gy, scalar_f(0.0f, {1}))};
        }
    }

    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        Shape inner, outer;
        x[0].desc.shape.extract(axes, &inner, &outer);
        return k::reduce(ctx, x[0].desc.dtype, (int)kind, (const char *)x[0].data->dev + outer.offset * 4, to_dims(outer),
                         to_dims(inner), y->ptr());
    }
};

bool reduce_op_info(const Operator &op, int *kind, std::vector<int> *axes) {
    const ReduceOp *r = dynamic_cast<const ReduceOp *>(&op);
    if (!r) return false;
    *kind = (int)r->kind;
    *axes = r->axes;
    return true;
}

Var ops::reduce(const Var &x, const std::vector<long long> &axes_in, bool preserve, Red kind) {
    std::vector<int> axes = to_axes(axes_in, x.rank());
    auto op = std::make_shared<ReduceOp>();
    op->kind = kind;
    op->axes = axes;
    op->preserve = preserve;
    op->in = {x.desc};
    op->out = TensorDesc(reduced_extents(x.extents(), axes, preserve), x.dtype());
    return Var::from_op(op, {x});
}

Var ops::mean(const Var &x, const std::vector<long long> &axes_in, bool preserve) {  // reduce.rs:59-71
    std::vector<int> axes = to_axes(axes_in, x.rank());
    long long n = 1;
    for (int a : axes) n *= x.extents()[a];
    Var r = reduce(x, axes_in, preserve, Sum);
    return div(r, scalar_f((float)n, r.extents()));
}

Var ops::var(const Var &x, const std::vector<long long> &axes, bool preserve) {  // reduce.rs:73-82
    return sub(mean(unary_map(x, Square), axes, preserve), unary_map(mean(x, axes, preserve), Square));
}

struct ReduceArgOp : Operator {
    bool is_max;
    int axis;
    bool preserve;
    const char *name() const override { return is_max ? "argmax" : "argmin"; }
    std::vector<Var> grad(const std::vector<Var> &, const Var &, const Var &) override { return {Var()}; }
    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        if (x[0].desc.dtype != SAGE_F32) return ctx.fail(SAGE_ERR_UNSUPPORTED, "argmax/argmin: only float input");
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        Shape inner, outer;
        x[0].desc.shape.extract({axis}, &inner, &outer);
        return k::reduce_arg(ctx, is_max, (const float *)x[0].data->dev + outer.offset, to_dims(outer), inner.extents[0],
                             inner.strides[0], (uint32_t *)y->ptr());
    }
};

Var ops::reduce_arg(const Var &x, long long axis, bool preserve, bool is_max) {
    const int a = to_axis(axis, x.rank());
    auto op = std::make_shared<ReduceArgOp>();
    op->is_max = is_max;
    op->axis = a;
    op->preserve = preserve;
    op->in = {x.desc};
    op->out = TensorDesc(reduced_extents(x.extents(), {a}, preserve), SAGE_U32);
    return Var::from_op(op, {x});
}

}  // namespace sage
