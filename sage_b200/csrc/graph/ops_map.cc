// Elementwise map operators and their fusion.  Reference: src/ops/map.rs (op tables :92-196,
// map_fn :224-367, dtype rules :458-513, grads :937-968,1014-1042,1094-1099, compute :898-1175)
// and Operator::fuse (src/ops.rs:104-161).
#include <cmath>
#include <cstring>

#include "graph.h"

namespace sage {
using namespace ops;

static const char *kUnaryFn[kNumUnary] = {
    "",        "sg_abs",  "-",        "sg_recip", "sg_log",  "sg_exp",   "sg_sqrt", "sg_square", "sg_erf",  "sg_sign",
    "sg_ceil", "sg_floor", "sg_round", "sg_sin",  "sg_sinh", "sg_cos",   "sg_cosh", "sg_tan",    "sg_tanh", "sg_asin",
    "sg_asinh", "sg_acos", "sg_acosh", "sg_atan", "sg_atanh", "!",       "(int)",   "(float)"};
static const char *kBinaryInfix[kNumBinary] = {"+", "-", "/", "*", nullptr, nullptr, nullptr, nullptr,
                                               "&&", "||", "==", "!=", ">", ">=", "<", "<="};
static const char *kBinaryFn[kNumBinary] = {nullptr, nullptr, nullptr, nullptr, "sg_mod", "sg_pow", "sg_min", "sg_max",
                                            nullptr, nullptr, nullptr, nullptr, nullptr,  nullptr,  nullptr,  nullptr};

// VariadicMapOperator::map_fn, map.rs:304-367: every sub-expression is parenthesised once.
std::string map_expr_text(const MapExpr &e) {
    switch (e.kind) {
    case MapExpr::Input:
        return "x" + std::to_string(e.input);
    case MapExpr::Literal: {
        // The reference prints "(float)<decimal>" (map.rs:524); the exact bit pattern avoids a
        // decimal -> double -> float double rounding.
        char buf[48];
        if (e.lit_dtype == SAGE_F32) snprintf(buf, sizeof buf, "sg_lit(0x%08xu)", e.bits);
        else if (e.lit_dtype == SAGE_I32) snprintf(buf, sizeof buf, "((int)%d)", (int)e.bits);
        else snprintf(buf, sizeof buf, "((uint)%uu)", e.bits);
        return buf;
    }
    case MapExpr::Un: {
        const std::string a = map_expr_text(e.args[0]);
        if (e.op == Copy) return "(" + a + ")";
        if (e.op == Neg || e.op == Not || e.op == CastInt || e.op == CastFloat) return std::string("(") + kUnaryFn[e.op] + a + ")";
        return std::string("(") + kUnaryFn[e.op] + "(" + a + "))";
    }
    case MapExpr::Bin: {
        const std::string a = map_expr_text(e.args[0]), b = map_expr_text(e.args[1]);
        if (kBinaryInfix[e.op]) return "(" + a + " " + kBinaryInfix[e.op] + " " + b + ")";
        return std::string("(") + kBinaryFn[e.op] + "(" + a + ", " + b + "))";
    }
    case MapExpr::Tern:
        return "(" + map_expr_text(e.args[0]) + " ? " + map_expr_text(e.args[1]) + " : " + map_expr_text(e.args[2]) + ")";
    }
    return "";
}

sage_status storage_planes_attach(Context &ctx, Storage &st);  // ops_gemm.cc

struct MapOp : Operator {
    MapExpr expr;
    bool primitive = true;  // a single nullary/unary/binary/ternary op (differentiable); false once fused
    MapCache cache;
    std::string text;       // C expression, built on first use

    const char *name() const override { return in.empty() ? "nullary_map" : primitive ? "map" : "variadic"; }
    Cat cat() const override { return Cat::Map; }

    std::vector<Var> grad(const std::vector<Var> &x, const Var &y, const Var &gy) override;

    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        const bool emit = ctx.hint_emit_planes && out.dtype == SAGE_F32;
        ctx.hint_emit_planes = ctx.hint_planes_only = false;
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        float *hi = nullptr;
        long long plane = 0;
        if (emit) {  // a tensor-core GEMM reads y next: the kernel writes its tf32 planes as well
            st = storage_planes_attach(ctx, *y->data);
            if (st) return st;
            hi = y->data->split->planes.planes + y->desc.shape.offset;
            plane = y->data->split->plane;
        }
        if (text.empty()) text = map_expr_text(expr);
        std::vector<MapOperand> operands(x.size());
        for (size_t i = 0; i < x.size(); ++i) {
            operands[i].dtype = x[i].desc.dtype;
            operands[i].ptr = x[i].ptr();
            operands[i].view = x[i].dims();
        }
        return map_launch(ctx, text, operands, out.dtype, y->ptr(), out.shape.rank(), out.shape.extents.data(), &cache, hi, plane);
    }
};

bool map_op_emits_planes(const Operator &op) {
    const MapOp *m = dynamic_cast<const MapOp *>(&op);
    return m && m->out.dtype == SAGE_F32 && !m->in.empty();
}

const MapExpr *map_expr_of(const Operator &op) {
    const MapOp *m = dynamic_cast<const MapOp *>(&op);
    return m ? &m->expr : nullptr;
}

// expand(map(a, b, ..)) == map(expand(a), expand(b), ..): the same elementwise map over operands that are each
// expanded to `extents`.  Null when `op` is no map with operands.
std::shared_ptr<Operator> map_over_expanded(const Operator &op, const Array &extents) {
    const MapOp *m = dynamic_cast<const MapOp *>(&op);
    if (!m || m->in.empty()) return nullptr;
    auto f = std::make_shared<MapOp>();
    f->primitive = false;
    f->expr = m->expr;
    for (const TensorDesc &d : m->in) f->in.push_back(TensorDesc(d.shape.expand(extents), d.dtype));
    f->out = TensorDesc(extents, m->out.dtype);
    return f;
}

bool is_copy_map(const Operator &op) {  // organize(): y = x
    const MapOp *m = dynamic_cast<const MapOp *>(&op);
    return m && m->in.size() == 1 && m->expr.kind == MapExpr::Un && m->expr.op == Copy && m->expr.args[0].kind == MapExpr::Input &&
           m->out.dtype == m->in[0].dtype;
}

// The expression text with operand i renamed to x<remap[i]>.
std::string map_expr_text_remap(const MapExpr &e, const std::vector<int> &remap) {
    std::function<MapExpr(const MapExpr &)> walk = [&](const MapExpr &x) {
        MapExpr r = x;
        if (r.kind == MapExpr::Input) r.input = remap[r.input];
        for (auto &a : r.args) a = walk(a);
        return r;
    };
    return map_expr_text(walk(e));
}

static MapExpr input_expr(int i) {
    MapExpr e;
    e.kind = MapExpr::Input;
    e.input = i;
    return e;
}

// ---------------------------------------------------------------- constructors
static Var make_literal(uint32_t bits, int dtype, const Array &extents) {  // scalar, map.rs:517-531
    auto op = std::make_shared<MapOp>();
    op->out = TensorDesc(infer_extents(extents, 0), dtype);
    op->expr.kind = MapExpr::Literal;
    op->expr.bits = bits;
    op->expr.lit_dtype = dtype;
    return Var::from_op(op, {});
}

Var ops::scalar_f(float v, const Array &extents) {
    uint32_t bits;
    memcpy(&bits, &v, 4);
    return make_literal(bits, SAGE_F32, extents);
}

Var ops::scalar_i(int v, const Array &extents) { return make_literal((uint32_t)v, SAGE_I32, extents); }

Var ops::unary_map(const Var &x, Unary m) {  // map.rs:458-481
    int dt;
    switch (m) {
    case Sign: case Copy: case Abs: case Neg: dt = x.dtype(); break;
    case Not: dt = SAGE_U32; break;
    case CastInt: dt = SAGE_I32; break;
    default: dt = SAGE_F32; break;
    }
    auto op = std::make_shared<MapOp>();
    op->in = {x.desc};
    op->out = TensorDesc(x.extents(), dt);
    op->expr.kind = MapExpr::Un;
    op->expr.op = m;
    op->expr.args = {input_expr(0)};
    return Var::from_op(op, {x});
}

static void broadcast(Var *a, Var *b) {  // map.rs:412-429
    Array u = union_extents(a->extents(), b->extents());
    if (a->extents() != u) *a = expand(*a, u);
    if (b->extents() != u) *b = expand(*b, u);
}

Var ops::binary_map(const Var &x1, const Var &x2, Binary m) {  // map.rs:483-513
    Var a = x1, b = x2;
    broadcast(&a, &b);
    if (a.dtype() != b.dtype()) shape_fail("binary map: operand data types differ");
    const bool logic = m >= And;
    auto op = std::make_shared<MapOp>();
    op->in = {a.desc, b.desc};
    op->out = TensorDesc(a.extents(), logic ? (int)SAGE_U32 : a.dtype());
    op->expr.kind = MapExpr::Bin;
    op->expr.op = m;
    op->expr.args = {input_expr(0), input_expr(1)};
    return Var::from_op(op, {a, b});
}

Var ops::cond(const Var &c0, const Var &x1, const Var &x2) {  // map.rs:861-883, broadcast3 :431-456
    Var c = c0, a = x1, b = x2;
    Array u = union_extents(union_extents(c.extents(), a.extents()), union_extents(a.extents(), b.extents()));
    if (c.extents() != u) c = expand(c, u);
    if (a.extents() != u) a = expand(a, u);
    if (b.extents() != u) b = expand(b, u);
    if (a.dtype() != b.dtype()) shape_fail("cond: branch data types differ");
    if (c.dtype() != SAGE_U32) shape_fail("cond: condition must be uint");
    auto op = std::make_shared<MapOp>();
    op->in = {c.desc, a.desc, b.desc};
    op->out = a.desc.pristine();
    op->expr.kind = MapExpr::Tern;
    op->expr.args = {input_expr(0), input_expr(1), input_expr(2)};
    return Var::from_op(op, {c, a, b});
}

// relu(x) = float(x > 0) * x (nn.rs:33-40) as ONE single-input map: the same expression, so the same
// bits for every input (NaN, -inf and -0 included), but its operand is read once and the value
// below it need not be materialised for having two readers.
std::shared_ptr<Operator> make_relu_map(const TensorDesc &x) {
    auto op = std::make_shared<MapOp>();
    op->primitive = false;
    op->in = {x};
    op->out = x.pristine();
    MapExpr zero;
    zero.kind = MapExpr::Literal;
    zero.bits = 0;
    zero.lit_dtype = SAGE_F32;
    MapExpr gt;
    gt.kind = MapExpr::Bin;
    gt.op = Gt;
    gt.args = {input_expr(0), zero};
    MapExpr cast;
    cast.kind = MapExpr::Un;
    cast.op = CastFloat;
    cast.args = {gt};
    op->expr.kind = MapExpr::Bin;
    op->expr.op = Mul;
    op->expr.args = {cast, input_expr(0)};
    return op;
}

// ---------------------------------------------------------------- grads
std::vector<Var> MapOp::grad(const std::vector<Var> &x, const Var &y, const Var &gy) {
    if (!primitive) shape_fail("variadic map operators cannot be differentiated");  // map.rs:1137-1139
    auto U = [](const Var &v, Unary m) { return unary_map(v, m); };
    Var none;
    if (expr.kind == MapExpr::Literal) return {};
    if (expr.kind == MapExpr::Un) {  // map.rs:937-968
        const Var &a = x[0];
        auto zero = [&]() { return scalar_f(0.0f, a.extents()); };
        auto one_minus_sq = [&]() { return add(neg(U(a, Square)), 1.0f); };
        switch (expr.op) {
        case Copy: return {gy};
        case Abs: return {mul(U(a, Sign), gy)};
        case Neg: return {neg(gy)};
        case Recip: return {div(neg(gy), U(a, Square))};
        case Log: return {div(gy, a)};
        case Exp: return {mul(gy, y)};
        case Sqrt: return {div(gy, mul(y, 2.0f))};
        case Square: return {mul(mul(gy, a), 2.0f)};
        case Erf: return {div(mul(gy, 2.0f / std::sqrt((float)M_PI)), U(U(a, Square), Exp))};
        case Sign: case Ceil: case Floor: case Round: return {zero()};
        case Sin: return {mul(gy, U(a, Cos))};
        case Sinh: return {mul(gy, U(a, Cosh))};
        case Cos: return {mul(neg(gy), U(a, Sin))};
        case Cosh: return {mul(gy, U(a, Sinh))};
        case Tan: return {div(gy, U(U(a, Cos), Square))};
        case Tanh: return {div(gy, U(U(a, Cosh), Square))};
        case Asin: return {div(gy, U(one_minus_sq(), Sqrt))};
        case Asinh: return {div(gy, U(add(U(a, Square), 1.0f), Sqrt))};
        case Acos: return {div(neg(gy), U(one_minus_sq(), Sqrt))};
        case Acosh: return {div(gy, U(sub(U(a, Square), 1.0f), Sqrt))};
        case Atan: return {div(gy, add(U(a, Square), 1.0f))};
        case Atanh: return {div(gy, one_minus_sq())};
        case Not: return {none};
        case CastInt: case CastFloat: return {gy};
        }
        return {none};
    }
    if (expr.kind == MapExpr::Bin) {  // map.rs:1014-1042
        const Var &a = x[0], &b = x[1];
        auto F = [&](const Var &p, const Var &q, Binary m) { return U(binary_map(p, q, m), CastFloat); };
        switch (expr.op) {
        case Add: return {gy, gy};
        case Sub: return {gy, neg(gy)};
        case Div: return {div(gy, b), mul(gy, div(neg(a), U(b, Square)))};
        case Mul: return {mul(gy, b), mul(gy, a)};
        case Mod: return {gy, mul(neg(gy), U(div(a, b), Floor))};
        case Pow: return {mul(mul(gy, b), binary_map(a, sub(b, 1.0f), Pow)), mul(mul(gy, binary_map(a, b, Pow)), U(a, Log))};
        case Min: return {mul(gy, F(a, b, Lt)), mul(gy, F(a, b, Ge))};
        case Max: return {mul(gy, F(b, a, Lt)), mul(gy, F(b, a, Ge))};
        default: return {none, none};
        }
    }
    // cond: map.rs:1094-1099
    return {cond(x[0], gy, scalar_f(0.0f, {1})), cond(x[0], scalar_f(0.0f, {1}), gy), none};
}

// ---------------------------------------------------------------- fusion (Operator::fuse, ops.rs:104-161)
static MapExpr substitute(const MapExpr &e, int idx, const MapExpr &child, int child_arity) {
    if (e.kind == MapExpr::Input) {
        if (e.input == idx) {
            // child inputs are spliced in at position idx
            std::function<MapExpr(const MapExpr &)> shift = [&](const MapExpr &c) {
                MapExpr r = c;
                if (r.kind == MapExpr::Input) r.input += idx;
                for (auto &a : r.args) a = shift(a);
                return r;
            };
            return shift(child);
        }
        MapExpr r = e;
        if (e.input > idx) r.input += child_arity - 1;
        return r;
    }
    MapExpr r = e;
    for (auto &a : r.args) a = substitute(a, idx, child, child_arity);
    return r;
}

struct ExpandTag;  // defined in ops_core.cc
bool is_expand_op(const Operator &op);

std::shared_ptr<Operator> fuse_ops(const Operator &parent, const Operator &child, int idx) {
    const MapOp *p = dynamic_cast<const MapOp *>(&parent);
    const MapOp *c = dynamic_cast<const MapOp *>(&child);
    if (p && c) {  // map + map -> variadic map
        auto f = std::make_shared<MapOp>();
        f->primitive = false;
        for (int i = 0; i < (int)p->in.size(); ++i) {
            if (i == idx) f->in.insert(f->in.end(), c->in.begin(), c->in.end());
            else f->in.push_back(p->in[i]);
        }
        f->out = p->out.pristine();
        f->expr = substitute(p->expr, idx, c->expr, (int)c->in.size());
        return f;
    }
    if (c && is_expand_op(parent) && c->expr.kind == MapExpr::Literal) {  // expand(nullary literal) -> nullary literal
        auto f = std::make_shared<MapOp>();
        f->out = TensorDesc(parent.out.shape.extents, c->out.dtype);
        f->expr = c->expr;
        return f;
    }
    return nullptr;
}

}  // namespace sage
