// Composite neural-network functions.  Reference: src/ops/nn.rs — relu :33-40, softmax :42-56,
// log_sum_exp :58-68, softmax_cross_entropy :70-82, layer_norm :84-100.  Each builds the same
// decomposed graph as the reference (so grad() sees the same operators) and, where the reduced axes
// are the trailing axes of a contiguous input, tags the result with a Composite so the evaluator can
// run it as one kernel (kernels/rowops.cu).
#include "graph.h"

namespace sage {
using namespace ops;

sage_status storage_planes_attach(Context &ctx, Storage &st);  // ops_gemm.cc

enum RowKind { RSoftmax, RLse, RLayerNorm };

struct RowOp : Operator {
    RowKind kind;
    long long rows = 0, cols = 0;
    float eps = 0.f;
    const char *name() const override {
        static const char *n[] = {"softmax", "log_sum_exp", "layer_norm"};
        return n[kind];
    }
    std::vector<Var> grad(const std::vector<Var> &, const Var &, const Var &) override {
        shape_fail("row composites are not differentiated; grad walks the decomposed graph");
    }
    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        if (!x[0].desc.shape.has_default_strides())
            return ctx.fail(SAGE_ERR_INVALID, std::string(name()) + ": input is not contiguous");
        const bool emit = ctx.hint_emit_planes && kind != RLse, only = emit && ctx.hint_planes_only;
        ctx.hint_emit_planes = ctx.hint_planes_only = false;
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        const float *xp = (const float *)x[0].ptr();
        float *yp = (float *)y->ptr();
        float *hi = nullptr;
        long long plane = 0;
        if (emit) {  // a tensor-core GEMM reads y next: write its tf32 planes in the same pass
            st = storage_planes_attach(ctx, *y->data);
            if (st) return st;
            hi = y->data->split->planes.planes + y->desc.shape.offset;
            plane = y->data->split->plane;
            if (only) {
                yp = nullptr;
                y->data->planes_only = true;
            }
        }
        switch (kind) {
        case RSoftmax: return k::softmax_rows(ctx, xp, yp, rows, cols, hi, plane);
        case RLse: return k::lse_rows(ctx, xp, yp, rows, cols);
        case RLayerNorm:
            return k::layernorm_rows(ctx, xp, yp, rows, cols, (const float *)x[1].ptr(), x[1].desc.shape.size() == 1 ? 0 : 1,
                                     (const float *)x[2].ptr(), x[2].desc.shape.size() == 1 ? 0 : 1, eps, hi, plane);
        }
        return SAGE_ERR_INVALID;
    }
};

bool row_op_is_softmax(const Operator &op, long long *rows, long long *cols) {
    const RowOp *r = dynamic_cast<const RowOp *>(&op);
    if (!r || r->kind != RSoftmax) return false;
    *rows = r->rows;
    *cols = r->cols;
    return true;
}

bool row_op_emits_planes(const Operator &op) {
    const RowOp *r = dynamic_cast<const RowOp *>(&op);
    return r && r->kind != RLse;
}

// True when `axes` are exactly the last axes of x and x is float + contiguous; fills rows/cols.
static bool trailing(const Var &x, const std::vector<int> &axes, long long *rows, long long *cols) {
    if (x.dtype() != SAGE_F32 || !x.desc.shape.has_default_strides() || axes.empty()) return false;
    const int r = x.rank(), k = (int)axes.size();
    std::vector<bool> seen(r, false);
    for (int a : axes) {
        if (a < r - k || seen[a]) return false;
        seen[a] = true;
    }
    *rows = *cols = 1;
    for (int i = 0; i < r; ++i) (i < r - k ? *rows : *cols) *= x.extents()[i];
    return true;
}

static void tag(const Var &y, RowKind kind, const std::vector<Var> &inputs, long long rows, long long cols, float eps) {
    auto op = std::make_shared<RowOp>();
    op->kind = kind;
    op->rows = rows;
    op->cols = cols;
    op->eps = eps;
    for (const Var &v : inputs) op->in.push_back(v.desc);
    op->out = y.desc.pristine();
    y.origin->composite.reset(new Composite{op, inputs});
}

std::shared_ptr<Operator> make_relu_map(const TensorDesc &x);  // ops_map.cc

Var ops::relu(const Var &x) {  // nn.rs:33-40
    Var out = mul(unary_map(binary_map(x, scalar_f(0.0f, {1}), Gt), CastFloat), x);
    if (x.dtype() == SAGE_F32) out.origin->composite.reset(new Composite{make_relu_map(x.desc), {x}});
    return out;
}

Var ops::softmax(const Var &x, const std::vector<long long> &axes_in) {  // nn.rs:42-56
    std::vector<int> axes = to_axes(axes_in, x.rank());
    Var xm = reduce(x, axes_in, true, RMax);
    Var y = unary_map(sub(x, xm), Exp);
    Var s = reduce(y, axes_in, true, Sum);
    Var out = div(y, s);
    long long rows, cols;
    if (trailing(x, axes, &rows, &cols)) tag(out, RSoftmax, {x}, rows, cols, 0.f);
    return out;
}

Var ops::log_sum_exp(const Var &x, const std::vector<long long> &axes_in) {  // nn.rs:58-68
    std::vector<int> axes = to_axes(axes_in, x.rank());
    Var c = reduce(x, axes_in, true, RMax);
    Var out = add(unary_map(reduce(unary_map(sub(x, c), Exp), axes_in, true, Sum), Log), c);
    long long rows, cols;
    if (trailing(x, axes, &rows, &cols)) tag(out, RLse, {x}, rows, cols, 0.f);
    return out;
}

Var ops::softmax_cross_entropy(const Var &x1, const Var &x2) {  // nn.rs:70-82
    Var log_z = sub(x1, log_sum_exp(x1, {1}));
    Var log_p = gather(log_z, x2, 1);
    return neg(reduce(log_p, {1}, false, Sum));
}

Var ops::accuracy(const Var &logits, const Var &labels) {  // metric.rs:4-17
    Var top = reduce_arg(logits, 1, true, true);
    Var hits = reduce(binary_map(top, labels, Eq), {0}, false, Sum);
    return div(unary_map(hits, CastFloat), (float)top.size());
}

Var ops::layer_norm(const Var &x, const std::vector<long long> &axes_in, const Var &gamma, const Var &beta, float eps) {
    std::vector<int> axes = to_axes(axes_in, x.rank());  // nn.rs:84-100
    Var m = mean(x, axes_in, true);
    Var v = var(x, axes_in, true);
    Var xc = div(sub(x, m), unary_map(add(v, eps), Sqrt));
    Var out = add(mul(xc, gamma), beta);
    long long rows, cols;
    auto param_ok = [&](const Var &p) {
        return p.dtype() == SAGE_F32 && p.desc.shape.has_default_strides() && (p.size() == 1 || (p.rank() == 1 && p.size() == cols));
    };
    if (trailing(x, axes, &rows, &cols) && param_ok(gamma) && param_ok(beta) && out.extents() == x.extents())
        tag(out, RLayerNorm, {x, gamma, beta}, rows, cols, eps);
    return out;
}

}  // namespace sage
