// The lazy evaluator.  Reference: Context::eval (src/session/context.rs:96-117), Program::compile
// (src/session.rs:62-206: which values are materialised), Routine::compile (:514-610: postfix
// expansion + operator fusion), Program::exec (:208-468: demand-driven execution with
// out-of-memory eviction and recompute) and Routine::exec (:612-673).
//
// Differences, none of which change results:
//   * a compiled Program is cached per (targets, already-evaluated inputs) instead of being rebuilt
//     on every eval;
//   * where a Var carries a Composite tag (softmax / log_sum_exp / layer_norm / pooling) and pattern
//     fusion is on, the composite's inputs take the place of the decomposed sub-graph;
//   * an intermediate is released as soon as its last consumer routine has run (the reference keeps
//     every intermediate until exec returns unless it runs out of memory).
#include <chrono>

#include "graph.h"

namespace sage {

struct Node {
    bool is_data = false;
    Var var;                       // data leaf: an input of the routine
    std::shared_ptr<Operator> op;  // operation
    std::vector<Node> args;
};

struct Routine {
    std::vector<Var> inputs;
    Var output;
    Node root;
    double exec_time = 0.0;
};

struct Program {
    std::vector<Origin *> target_keys, x_keys;
    std::vector<Var> outputs;
    std::unordered_map<Origin *, Routine> routines;
    std::unordered_map<Origin *, int> consumers;  // how many routines read each state
    bool fusion = true, pattern = true;
};

Session::Session(Context *ctx) : ctx_(ctx) {}
Session::~Session() {}

void Session::clear() { data.clear(); }

bool Session::get(const Var &v, Tensor *out) const {
    auto it = data.find(v.key());
    if (it == data.end()) return false;
    *out = it->second.second;
    return true;
}

static const std::vector<Var> &children(const Var &v, bool pattern, std::shared_ptr<Operator> *op) {
    Origin *o = v.origin.get();
    if (pattern && o->composite) {
        if (op) *op = o->composite->op;
        return o->composite->inputs;
    }
    if (op) *op = o->op;
    return o->inputs;
}

// Routine::compile, session.rs:514-610: expand the sub-graph between the routine's inputs and its
// output into a tree (shared non-state nodes are expanded once per use) and fold it bottom-up with
// Operator::fuse.
static Node build(const Var &v, const std::unordered_set<Origin *> &inputs, bool fusion, bool pattern, bool is_root) {
    Node n;
    if (!is_root && inputs.count(v.key())) {
        n.is_data = true;
        n.var = v;
        return n;
    }
    if (!v.is_op()) shape_fail("uninitialized variable");
    std::shared_ptr<Operator> op;
    const std::vector<Var> &kids = children(v, pattern, &op);
    std::vector<Node> args;
    for (const Var &k : kids) args.push_back(build(k, inputs, fusion, pattern, false));
    std::vector<Node> folded;
    int offset = 0;
    for (int i = 0; i < (int)args.size(); ++i) {
        Node &a = args[i];
        if (!a.is_data && fusion) {
            std::shared_ptr<Operator> f = fuse_ops(*op, *a.op, i + offset);
            if (f) {
                offset += (int)a.op->in.size() - 1;
                op = f;
                for (Node &g : a.args) folded.push_back(std::move(g));
                continue;
            }
        }
        folded.push_back(std::move(a));
    }
    n.op = op;
    n.args = std::move(folded);
    return n;
}

// Program::compile, session.rs:62-206.
static std::unique_ptr<Program> compile(const std::vector<Var> &x, std::vector<Var> y, bool fusion, bool pattern) {
    std::unique_ptr<Program> p(new Program());
    p->fusion = fusion;
    p->pattern = pattern;
    std::stable_sort(y.begin(), y.end(), [](const Var &a, const Var &b) { return a.t_order() < b.t_order(); });
    std::unordered_set<Origin *> xset, yset;
    for (const Var &v : x) xset.insert(v.key());
    for (const Var &v : y) yset.insert(v.key());

    const size_t THRES = 5;
    std::unordered_map<Origin *, Var> nodes;
    std::vector<Var> stack;
    for (const Var &k : y) {
        stack.push_back(k);
        while (!stack.empty()) {
            Var v = stack.back();
            stack.pop_back();
            if (nodes.emplace(v.key(), v).second && !xset.count(v.key()) && v.is_op())
                for (const Var &c : children(v, pattern, nullptr)) stack.push_back(c);
        }
    }
    std::unordered_map<Origin *, size_t> edges;
    for (auto &kv : nodes)
        if (kv.second.is_op() && !xset.count(kv.first))
            for (const Var &c : children(kv.second, pattern, nullptr)) ++edges[c.key()];

    std::vector<Var> candidates;
    for (auto &kv : edges) {
        const Var &v = nodes[kv.first];
        if (kv.second >= 2 && v.is_op() && !xset.count(kv.first) && !yset.count(kv.first)) candidates.push_back(v);
    }
    for (const Var &v : y) candidates.push_back(v);
    std::stable_sort(candidates.begin(), candidates.end(), [](const Var &a, const Var &b) {
        return a.t_order() != b.t_order() ? a.t_order() < b.t_order() : a.key() < b.key();
    });

    std::unordered_map<Origin *, std::vector<Var>> states;
    std::vector<Var> state_order;
    for (const Var &node : candidates) {
        if (states.count(node.key())) continue;
        std::unordered_map<Origin *, Var> inputs;
        size_t num_ops = 0;
        bool complex_op = false;
        stack.push_back(node);
        bool first = true;
        while (!stack.empty()) {
            Var v = stack.back();
            stack.pop_back();
            ++num_ops;
            const bool root = first;
            first = false;
            if (!root && (v.is_data() || states.count(v.key()) || xset.count(v.key()))) {
                inputs.emplace(v.key(), v);
            } else if (v.is_op()) {
                std::shared_ptr<Operator> op;
                for (const Var &c : children(v, pattern, &op)) stack.push_back(c);
                const Cat c = op->cat();
                if (c == Cat::Contract || c == Cat::Reduce || c == Cat::Other) complex_op = true;
            } else {
                shape_fail("uninitialized variable");
            }
        }
        if (yset.count(node.key()) || complex_op || num_ops * inputs.size() > THRES) {
            std::vector<Var> in;
            for (auto &kv : inputs) in.push_back(kv.second);
            states[node.key()] = in;
            state_order.push_back(node);
        }
    }
    for (const Var &node : state_order) {
        Routine r;
        r.inputs = states[node.key()];
        r.output = node;
        std::unordered_set<Origin *> in_keys;
        for (const Var &v : r.inputs) {
            in_keys.insert(v.key());
            if (v.is_op()) ++p->consumers[v.key()];
        }
        r.root = build(node, in_keys, fusion, pattern, true);
        p->routines.emplace(node.key(), std::move(r));
    }
    p->outputs = y;
    return p;
}

// Routine::exec, session.rs:612-673 (a recursive walk instead of the flattened stack).
static sage_status run_node(const Node &n, Context &ctx, Session &s, const std::unordered_map<Origin *, Tensor> &temp,
                            Tensor *out) {
    if (n.is_data) {
        Origin *o = n.var.key();
        if (!n.var.is_op()) {
            if (!o->data.defined()) return ctx.fail(SAGE_ERR_INVALID, "uninitialized variable" + (o->name.empty() ? "" : " " + o->name));
            sage_status st = o->data.to_device(ctx);
            if (st) return st;
            *out = o->data;
            return SAGE_OK;
        }
        auto it = s.data.find(o);
        if (it != s.data.end()) {
            *out = it->second.second;
            return SAGE_OK;
        }
        auto jt = temp.find(o);
        if (jt == temp.end()) return ctx.fail(SAGE_ERR_INVALID, "internal: routine input not available");
        *out = jt->second;
        return SAGE_OK;
    }
    std::vector<Tensor> args(n.args.size());
    for (size_t i = 0; i < n.args.size(); ++i) {
        sage_status st = run_node(n.args[i], ctx, s, temp, &args[i]);
        if (st) return st;
    }
    for (size_t i = 0; i < args.size(); ++i)  // Operator::compute's spec check, ops.rs:163-178
        if (args[i].desc.shape.extents != n.op->in[i].shape.extents)
            return ctx.fail(SAGE_ERR_INVALID, std::string("operand extents differ from the operator's spec in ") + n.op->name());
    return n.op->compute(args, ctx, out);
}

// Program::exec, session.rs:208-468.
static sage_status exec(Program &p, Context &ctx, Session &s) {
    std::unordered_map<Origin *, Tensor> temp;
    std::unordered_map<Origin *, int> remaining = p.consumers;
    std::unordered_map<Origin *, int> lock;        // how many pending routines need each state
    std::unordered_set<Origin *> pending, outputs;
    for (const Var &v : p.outputs) outputs.insert(v.key());
    std::vector<Var> stack(p.outputs.begin(), p.outputs.end());
    auto available = [&](const Var &v) { return v.is_data() || s.data.count(v.key()) || temp.count(v.key()); };
    while (!stack.empty()) {
        Var v = stack.back();
        if (available(v)) {
            stack.pop_back();
            continue;
        }
        auto rit = p.routines.find(v.key());
        if (rit == p.routines.end()) return ctx.fail(SAGE_ERR_INVALID, "internal: no routine for a required state");
        Routine &f = rit->second;
        // Inputs of a routine that is waiting for its other inputs are locked against eviction
        // (session.rs:237-239), otherwise two inputs could evict each other for ever.
        if (pending.insert(v.key()).second)
            for (const Var &k : f.inputs) ++lock[k.key()];
        std::vector<Var> missing;
        for (const Var &k : f.inputs)
            if (!available(k)) missing.push_back(k);
        if (!missing.empty()) {
            for (const Var &k : missing) stack.push_back(k);
            continue;
        }
        Tensor out;
        for (;;) {
            auto t0 = std::chrono::steady_clock::now();
            sage_status st = run_node(f.root, ctx, s, temp, &out);
            f.exec_time = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if (st == SAGE_OK) break;
            if (st != SAGE_ERR_OOM) return st;
            // Out of memory: drop the intermediates that are cheapest to recompute per byte
            // (session.rs:259-331); they are rebuilt on demand when a later routine needs them.
            const uint64_t needed = ctx.allocator().oom_needed, start = ctx.allocator().mem_used();
            bool evicted = false;
            while (start - ctx.allocator().mem_used() < needed) {
                Origin *best = nullptr;
                double best_tpm = 0.0;
                for (auto &kv : temp) {
                    auto lk = lock.find(kv.first);
                    if (lk != lock.end() && lk->second > 0) continue;
                    auto r2 = p.routines.find(kv.first);
                    if (r2 == p.routines.end()) continue;
                    const double tpm = (r2->second.exec_time + 1.0) / ((double)r2->second.output.size() + 1.0);
                    if (!best || tpm < best_tpm) {
                        best = kv.first;
                        best_tpm = tpm;
                    }
                }
                if (!best) break;
                temp.erase(best);
                evicted = true;
            }
            ctx.allocator().release_cached();
            if (!evicted) return ctx.fail(SAGE_ERR_OOM, "out of memory and nothing left to evict");
        }
        for (const Var &k : f.inputs) --lock[k.key()];
        pending.erase(v.key());
        if (outputs.count(v.key())) s.data[v.key()] = std::make_pair(v, out);
        else temp[v.key()] = out;
        for (const Var &k : f.inputs) {
            auto it = remaining.find(k.key());
            if (it != remaining.end() && --it->second == 0) temp.erase(k.key());
        }
        stack.pop_back();
    }
    return SAGE_OK;
}

sage_status Session::eval(const std::vector<Var> &targets) {
    // Context::eval, context.rs:96-117: everything already evaluated is an input of the program.
    std::vector<Var> y;
    for (const Var &t : targets)
        if (t.is_op() && !data.count(t.key())) y.push_back(t);
    if (y.empty()) return SAGE_OK;
    std::vector<Var> x;
    {
        std::unordered_set<Origin *> seen;
        std::vector<Var> stack = y;
        while (!stack.empty()) {
            Var e = stack.back();
            stack.pop_back();
            if (!seen.insert(e.key()).second) continue;
            if (data.count(e.key())) x.push_back(e);
            else if (e.is_op())
                for (const Var &c : children(e, ctx_->opts().pattern_fusion != 0, nullptr)) stack.push_back(c);
        }
    }
    std::vector<Origin *> tk, xk;
    for (const Var &v : y) tk.push_back(v.key());
    for (const Var &v : x) xk.push_back(v.key());
    std::sort(xk.begin(), xk.end());
    Program *prog = nullptr;
    for (auto &c : cache_)
        if (c->target_keys == tk && c->x_keys == xk) prog = c.get();
    if (!prog) {
        std::unique_ptr<Program> p;
        try {
            p = compile(x, y, true, ctx_->opts().pattern_fusion != 0);
        } catch (const ShapeError &e) {
            return ctx_->fail(SAGE_ERR_INVALID, e.msg);
        }
        p->target_keys = tk;
        p->x_keys = xk;
        prog = p.get();
        cache_.push_back(std::move(p));
        ++programs_compiled;
    }
    last_ = prog;
    try {
        return exec(*prog, *ctx_, *this);
    } catch (const ShapeError &e) {
        return ctx_->fail(SAGE_ERR_INVALID, e.msg);
    }
}

static void describe_node(const Node &n, std::string *out) {
    if (n.is_data) {
        out->append(n.var.is_op() ? "state" : "data");
        return;
    }
    out->append(n.op->name());
    if (const MapExpr *e = map_expr_of(*n.op)) out->append("{" + map_expr_text(*e) + "}");
    out->push_back('(');
    for (size_t i = 0; i < n.args.size(); ++i) {
        if (i) out->push_back(',');
        describe_node(n.args[i], out);
    }
    out->push_back(')');
}

std::string Session::describe_last() const {
    std::string out;
    if (!last_) return out;
    std::vector<const Routine *> rs;
    for (auto &kv : last_->routines) rs.push_back(&kv.second);
    std::sort(rs.begin(), rs.end(), [](const Routine *a, const Routine *b) {
        return a->output.t_order() != b->output.t_order() ? a->output.t_order() < b->output.t_order() : a->output.key() < b->output.key();
    });
    for (const Routine *r : rs) {
        describe_node(r->root, &out);
        out.push_back('\n');
    }
    return out;
}

}  // namespace sage
