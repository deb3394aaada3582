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
#include <cuda_runtime.h>

#include <chrono>
#include <cstdlib>

#include "graph.h"
#include "rowfuse.h"

namespace sage {

struct Node {
    bool is_data = false;
    Var var;                       // data leaf: an input of the routine
    std::shared_ptr<Operator> op;  // operation
    std::vector<Node> args;
    bool emit_planes = false;      // a tensor-core GEMM reads the result: ask the operator for its tf32 planes
    std::shared_ptr<Node> shared;  // a node several parents read (a grouped GEMM): evaluated once per routine run,
                                   // and passed to `op` as its only operand
    bool visited = false;          // traversal mark for shared nodes
    bool planes_only = false;      // ... and that GEMM is the only reader: the fp32 result need not be stored
    int readers = 0, gemm_readers = 0;  // shared nodes: how many parents, how many of them GEMM operands
};

// ops_map.cc / ops_core.cc / ops_gemm.cc / ops_nn.cc
bool is_copy_map(const Operator &op);
std::shared_ptr<Operator> map_over_expanded(const Operator &op, const Array &extents);
std::shared_ptr<Operator> make_expand_op(const TensorDesc &in, const Array &extents);
bool is_expand_op(const Operator &op);
std::string map_expr_text_remap(const MapExpr &e, const std::vector<int> &remap);
bool is_view_op(const Operator &op);
bool is_reshape_op(const Operator &op);
bool is_gemm_op(const Operator &op);
bool gemm_runs_on_tc(const Operator &op, bool tc_enabled);
bool gemm_can_fuse(const Operator &op, bool tc_enabled);
std::shared_ptr<Operator> gemm_with_operand_view(const Operator &op, int idx, const TensorDesc &view, bool tc_enabled);
std::shared_ptr<Operator> gemm_with_epilogue(const Operator &op, const std::string &expr, const std::vector<TensorDesc> &aux,
                                             const TensorDesc &out);
std::shared_ptr<Operator> gemm_with_im2col(const Operator &op, const Operator &im2col_op, bool tc_enabled);
std::shared_ptr<Operator> gemm_with_store(const Operator &op, const Shape &view, const TensorDesc &out, bool tc_enabled);
bool row_op_emits_planes(const Operator &op);
bool row_op_is_softmax(const Operator &op, long long *rows, long long *cols);
std::shared_ptr<Operator> gemm_with_row_softmax(const Operator &op, long long rows, long long cols, const TensorDesc &out, bool tc_enabled);
std::shared_ptr<Operator> gemm_with_attention(const Operator &outer_op, const Operator &score_op, long long rows, long long cols, bool tc_enabled);
bool is_attention_op(const Operator &op);
bool is_grouped_gemm_op(const Operator &op);
bool gemm_operand_static_direct(const Operator &op, int idx);
bool gemm_group_key(const Operator &op, std::string *key);
std::shared_ptr<Operator> make_grouped_gemm(const std::vector<const Operator *> &members);
std::shared_ptr<Operator> make_slab(const Operator &grouped, int index, const TensorDesc &member_out);
std::string describe_gemm(const Operator &op);  // "{epilogue}" / "[store]" of a lowered GEMM, else empty

static bool row_programs_enabled() {
    static const bool on = [] {
        const char *e = getenv("SAGE_ROW_PROGRAM");
        return !e || atoi(e) != 0;
    }();
    return on;
}

// Device time of a routine's first execution, taken with a pair of events on the context's stream and
// read once the second event has completed.  The reference measures the host time of the enqueue
// (session.rs:667-668), which says little about an asynchronous device.
struct RoutineTimer {
    cudaEvent_t ev[2] = {nullptr, nullptr};
    ~RoutineTimer() {
        for (cudaEvent_t e : ev)
            if (e) cudaEventDestroy(e);
    }
};

struct Routine {
    std::vector<Var> inputs;
    Var output;
    Node root;
    double exec_time = 0.0;  // microseconds on the device (host enqueue time on a planning context)
    std::shared_ptr<RoutineTimer> timer;
    bool timed = false;
    // Reads the timer if the device has got that far; true when exec_time is final.
    bool resolve_time() {
        if (!timer) return true;
        if (cudaEventQuery(timer->ev[1]) != cudaSuccess) return false;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, timer->ev[0], timer->ev[1]) == cudaSuccess) exec_time = 1e3 * (double)ms;
        timer.reset();
        return true;
    }
    // A row group (rowfuse.h): several states of one [R, C] space computed by one generated kernel.  The
    // same routine is registered under every state in `row_outputs`; running it once yields them all.
    std::shared_ptr<RowProgram> row;
    std::vector<Var> row_outputs;
    std::shared_ptr<std::vector<char>> row_emit_shared;  // per output: a tensor-core GEMM reads it, write its tf32 planes too
};

struct Program {
    std::vector<Origin *> target_keys, x_keys;
    uint64_t key_hash = 0;  // of (target_keys, x_keys): compared before the lists
    std::vector<Var> outputs;
    std::unordered_map<Origin *, Routine> routines;
    std::unordered_map<Origin *, int> consumers;  // how many routines read each state
    bool fusion = true, pattern = true;
    std::shared_ptr<RowProgram> row;  // set: the whole program is one generated row kernel (rowfuse.h)
};

Session::Session(Context *ctx) : ctx_(ctx) {}
Session::~Session() {}

void Session::clear() { data.clear(); }

void Session::drop_programs() {
    last_ = nullptr;
    cache_.clear();
}

static uint64_t program_key_hash(const std::vector<Origin *> &targets, const std::vector<Origin *> &inputs) {
    uint64_t h = 0xcbf29ce484222325ull;  // FNV-1a over the two pointer lists and their lengths
    auto mix = [&](uint64_t v) {
        for (int i = 0; i < 8; ++i) {
            h ^= (v >> (8 * i)) & 0xff;
            h *= 0x100000001b3ull;
        }
    };
    mix(targets.size());
    for (Origin *o : targets) mix((uint64_t)(uintptr_t)o);
    mix(inputs.size());
    for (Origin *o : inputs) mix((uint64_t)(uintptr_t)o);
    return h;
}

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

// ------------------------------------------------------------------------------ GEMM lowering
// After a routine's tree is built, the operators around each tensor-core GEMM are folded into it
// (no counterpart in the reference, whose GEMM is a library call between generated kernels):
//   gemm(.. reshape(copy(view)) ..)        the operand is read through `view`; the copy goes away
//   map(.. reshape(gemm) .., aux ..)       the map's expression becomes the GEMM's epilogue
//   copy(permute(reshape(gemm)))           the permutation becomes the GEMM's store pattern
//   gemm(reshape(softmax(gemm{f}(q, k))), v)   one fused attention operator (scores and probabilities stay on chip)
// Every fold is checked against the static strides and declined when TMA or the epilogue's
// addressing cannot express it; what is declined simply stays a separate kernel.
static bool reshape_keeps_matrix(const Operator &op) {
    const Array &a = op.in[0].shape.extents, &b = op.out.shape.extents;
    const size_t ra = a.size(), rb = b.size();
    return ra >= 2 && rb >= 2 && a[ra - 1] == b[rb - 1] && a[ra - 2] == b[rb - 2];
}

// The fused attention kernel is used unless pattern_fusion bit 3 (value 8) or SAGE_ATTENTION=0 says otherwise.
static bool attention_enabled() {
    static const bool on = !(getenv("SAGE_ATTENTION") && atoi(getenv("SAGE_ATTENTION")) == 0);
    return on;
}

static void lower(Node &n, bool tc, bool softmax_in_gemm, bool attention) {
    if (n.is_data) return;
    for (Node &a : n.args) lower(a, tc, softmax_in_gemm, attention);
    if (is_gemm_op(*n.op) && tc && n.args.size() == 2) {
        // the column matrix of a convolution: made by the GEMM itself, as planes (this may also bring a product onto the
        // tensor cores whose K = KH * KW * C alone is too short for them: a few-channel first layer)
        Node *p = &n.args[0];
        while (!p->is_data && is_reshape_op(*p->op)) p = &p->args[0];
        if (!p->is_data && p != &n.args[0] && p->args.size() == 1) {
            std::shared_ptr<Operator> f = gemm_with_im2col(*n.op, *p->op, tc);
            if (f) {
                Node inner = std::move(p->args[0]);
                n.args[0] = std::move(inner);
                n.op = f;
            }
        }
    }
    // operands behind an organize() copy
    if (is_gemm_op(*n.op) && gemm_runs_on_tc(*n.op, tc)) {
        for (int idx = 0; idx < 2; ++idx) {
            Node *p = &n.args[idx];
            while (!p->is_data && is_reshape_op(*p->op) && reshape_keeps_matrix(*p->op)) p = &p->args[0];
            if (p->is_data || !is_copy_map(*p->op) || p->args.size() != 1) continue;
            std::shared_ptr<Operator> f = gemm_with_operand_view(*n.op, idx, p->op->in[0], tc);
            if (!f) continue;
            Node inner = std::move(p->args[0]);
            n.args[idx] = std::move(inner);
            n.op = f;
        }
        if (attention && n.args.size() == 2) {  // the probabilities of an attention block times the values
            Node *p = &n.args[0];
            while (!p->is_data && is_reshape_op(*p->op)) p = &p->args[0];
            long long rows = 0, cols = 0;
            if (!p->is_data && row_op_is_softmax(*p->op, &rows, &cols) && p->args.size() == 1) {
                Node *s = &p->args[0];
                while (!s->is_data && is_reshape_op(*s->op)) s = &s->args[0];
                if (!s->is_data && !s->shared && is_gemm_op(*s->op) && s->args.size() >= 2) {
                    std::shared_ptr<Operator> f = gemm_with_attention(*n.op, *s->op, rows, cols, tc);
                    if (f) {
                        std::vector<Node> score_args = std::move(s->args);
                        std::vector<Node> args;
                        args.push_back(std::move(score_args[0]));  // Q
                        args.push_back(std::move(n.args[1]));      // V
                        for (size_t i = 1; i < score_args.size(); ++i) args.push_back(std::move(score_args[i]));  // K, operands of f
                        n.op = f;
                        n.args = std::move(args);
                    }
                }
            }
        }
        return;
    }
    long long sm_rows, sm_cols;
    if (softmax_in_gemm && row_op_is_softmax(*n.op, &sm_rows, &sm_cols) && n.args.size() == 1) {  // softmax over a product's rows
        Node *p = &n.args[0];
        while (!p->is_data && is_reshape_op(*p->op)) p = &p->args[0];
        if (!p->is_data && is_gemm_op(*p->op)) {
            std::shared_ptr<Operator> f = gemm_with_row_softmax(*p->op, sm_rows, sm_cols, n.op->out, tc);
            if (f) {
                std::vector<Node> args = std::move(p->args);
                n.op = f;
                n.args = std::move(args);
            }
        }
        return;
    }
    if (!map_expr_of(*n.op)) return;
    // An operand that is expand(map(small operands)) — the extended attention mask, (1 - mask) * -1e5 broadcast over
    // heads and queries — would be a kernel and a tensor of its own.  An elementwise map commutes with expand, so the
    // small map is moved behind the expand and folded into this map: its operands become broadcast views.
    if (!is_copy_map(*n.op)) {
        for (size_t i = 0; i < n.args.size(); ++i) {
            Node &a = n.args[i];
            if (a.is_data || a.shared || !is_expand_op(*a.op) || a.args.size() != 1) continue;
            Node &c = a.args[0];
            if (c.is_data || c.shared || !map_expr_of(*c.op) || c.args.empty() || c.op->out.shape.size() * 16 > a.op->out.shape.size()) continue;
            const Array ext = a.op->out.shape.extents;
            std::shared_ptr<Operator> moved;
            try {
                moved = map_over_expanded(*c.op, ext);
            } catch (const ShapeError &) {
                moved = nullptr;
            }
            if (!moved) continue;
            std::shared_ptr<Operator> f = fuse_ops(*n.op, *moved, (int)i);
            if (!f) continue;
            std::vector<Node> args;
            for (size_t j = 0; j < n.args.size(); ++j) {
                if (j != i) {
                    args.push_back(std::move(n.args[j]));
                    continue;
                }
                for (size_t q = 0; q < c.args.size(); ++q) {  // each operand of the small map, expanded
                    Node e;
                    e.op = make_expand_op(c.op->in[q], ext);
                    e.args.push_back(std::move(c.args[q]));
                    args.push_back(std::move(e));
                }
            }
            n.op = f;
            n.args = std::move(args);
            i = (size_t)-1;  // operands moved: look again from the start
        }
    }
    const MapExpr *expr = map_expr_of(*n.op);
    if (is_copy_map(*n.op)) {  // a permuted copy of a product
        Node *p = &n.args[0];
        while (!p->is_data && is_view_op(*p->op)) p = &p->args[0];
        if (p != &n.args[0] && !p->is_data && is_gemm_op(*p->op)) {
            std::shared_ptr<Operator> f = gemm_with_store(*p->op, n.op->in[0].shape, n.op->out, tc);
            if (f) {
                std::vector<Node> args = std::move(p->args);
                n.op = f;
                n.args = std::move(args);
            }
        }
        return;
    }
    if (n.op->out.dtype != SAGE_F32) return;
    for (size_t j = 0; j < n.args.size(); ++j) {  // a map over a product
        Node *p = &n.args[j];
        while (!p->is_data && is_reshape_op(*p->op)) p = &p->args[0];
        if (p->is_data || !gemm_can_fuse(*p->op, tc) || p->op->out.shape.size() != n.op->out.shape.size()) continue;
        std::vector<int> remap(n.args.size());
        std::vector<TensorDesc> aux;
        int next = 1;
        for (size_t i = 0; i < n.args.size(); ++i) {
            remap[i] = i == j ? 0 : next++;
            if (i != j) aux.push_back(n.op->in[i]);
        }
        std::shared_ptr<Operator> f = gemm_with_epilogue(*p->op, map_expr_text_remap(*expr, remap), aux, n.op->out);
        if (!f) continue;
        std::vector<Node> args;
        args.push_back(std::move(p->args[0]));
        args.push_back(std::move(p->args[1]));
        for (size_t i = 0; i < n.args.size(); ++i)
            if (i != j) args.push_back(std::move(n.args[i]));
        n.op = f;
        n.args = std::move(args);
        return;
    }
}

// Which values a tensor-core GEMM reads (through views only): in-tree producers get emit_planes,
// states are collected so that their routine's root gets it.
static Node *skip_views(Node *p) {
    for (;;) {
        if (p->is_data) return p;
        if (p->shared) p = p->shared.get();  // a slab of a grouped product
        else if (is_view_op(*p->op)) p = &p->args[0];
        else return p;
    }
}
bool map_op_emits_planes(const Operator &op);
static bool can_emit_planes(const Operator &op, bool tc) {
    return gemm_runs_on_tc(op, tc) || row_op_emits_planes(op) || is_grouped_gemm_op(op) || (tc && map_op_emits_planes(op));
}

// GEMMs of one routine that multiply the same A (same leaf, same view) by different weights, with
// the same shape and epilogue, become one grouped launch; each member turns into a slab view of the
// shared node.  Members must take their weight (and bias) straight from data leaves, because the
// grouped operator keeps a concatenated copy of them.
static void collect_gemms(Node &n, std::vector<Node *> *out) {
    if (n.is_data) return;
    for (Node &a : n.args) collect_gemms(a, out);
    if (is_gemm_op(*n.op)) out->push_back(&n);
}

static void group_gemms(Node &root) {
    std::vector<Node *> gemms;
    collect_gemms(root, &gemms);
    std::unordered_map<std::string, std::vector<Node *>> by_key;
    std::vector<std::string> order;
    for (Node *g : gemms) {
        std::string key;
        if (!gemm_group_key(*g->op, &key)) continue;
        Node *a = skip_views(&g->args[0]);
        if (!a->is_data) continue;
        bool leaves = true;
        for (size_t i = 1; i < g->args.size(); ++i) {
            Node *w = skip_views(&g->args[i]);
            if (!w->is_data || w->var.is_op()) leaves = false;
        }
        if (!leaves) continue;
        char id[32];
        snprintf(id, sizeof id, "#%p", (void *)a->var.key());
        key += id;
        if (!by_key.count(key)) order.push_back(key);
        by_key[key].push_back(g);
    }
    for (const std::string &key : order) {
        std::vector<Node *> &members = by_key[key];
        if (members.size() < 2) continue;
        std::vector<const Operator *> ops;
        for (Node *m : members) ops.push_back(m->op.get());
        auto shared = std::make_shared<Node>();
        shared->op = make_grouped_gemm(ops);
        shared->args.push_back(std::move(members[0]->args[0]));
        for (Node *m : members) shared->args.push_back(std::move(m->args[1]));
        if (members[0]->args.size() > 2)
            for (Node *m : members) shared->args.push_back(std::move(m->args[2]));
        for (size_t i = 0; i < members.size(); ++i) {
            Node *m = members[i];
            std::shared_ptr<Operator> slab = make_slab(*shared->op, (int)i, m->op->out);
            m->op = slab;
            m->args.clear();
            m->shared = shared;
            ++shared->readers;
        }
    }
}

static void mark_plane_readers(Node &n, bool tc, std::unordered_set<Origin *> *states) {
    if (n.is_data) return;
    if (n.shared && !n.shared->visited) {
        n.shared->visited = true;
        mark_plane_readers(*n.shared, tc, states);
    }
    for (Node &a : n.args) mark_plane_readers(a, tc, states);
    const bool grouped = is_grouped_gemm_op(*n.op);
    if (!grouped && (!is_gemm_op(*n.op) || !gemm_runs_on_tc(*n.op, tc))) return;
    for (int idx = 0; idx < (grouped ? 1 : is_attention_op(*n.op) ? 3 : 2); ++idx) {
        Node *p = skip_views(&n.args[idx]);
        if (p->is_data) {
            if (p->var.is_op() && gemm_operand_static_direct(*n.op, idx)) states->insert(p->var.key());
        } else if (can_emit_planes(*p->op, tc)) {
            // Inside a routine's tree a node has one reader, so this GEMM is the only one — unless the
            // node is shared (a grouped product): then every slab must end in a GEMM operand.
            const bool direct = gemm_operand_static_direct(*n.op, idx);
            if (direct) p->emit_planes = true;
            if (p->readers > 0) {
                if (direct) ++p->gemm_readers;
                p->planes_only = p->gemm_readers == p->readers;
            } else {
                p->planes_only = direct;
            }
        }
    }
}

// ------------------------------------------------------------------------------ row groups
// States whose bodies stay inside one [R, C] row space (maps, axis-1 reductions, gather / scatter along
// the row) and that feed one another are merged into one generated kernel: the values between them
// never travel through DRAM.  `order` is topological; `inputs[k]` lists what state k reads.
struct RowGroupPlan {
    std::vector<int> members;  // indices into `order`
};

static std::vector<RowGroupPlan> plan_row_groups(const std::vector<Var> &order, const std::unordered_map<Origin *, std::vector<Var>> &inputs) {
    const int n = (int)order.size();
    std::vector<RowGroupPlan> plans;
    if (n < 1 || n > 4096) return plans;  // the legality test is quadratic in the number of states
    std::unordered_map<Origin *, int> index;
    for (int i = 0; i < n; ++i) index[order[i].key()] = i;
    const int words = (n + 63) / 64;
    std::vector<std::vector<uint64_t>> anc(n, std::vector<uint64_t>(words, 0));  // states that state i depends on
    std::vector<std::vector<int>> reads(n);
    std::vector<long long> R(n, 0), C(n, 0);
    std::vector<char> ok(n, 0), exchanges(n, 0);
    for (int i = 0; i < n; ++i) {
        const std::vector<Var> &in = inputs.at(order[i].key());
        for (const Var &v : in) {
            auto it = index.find(v.key());
            if (it == index.end()) continue;
            reads[i].push_back(it->second);
            anc[i][it->second / 64] |= 1ull << (it->second % 64);
            for (int w = 0; w < words; ++w) anc[i][w] |= anc[it->second][w];
        }
        if (auto probe = row_program_build(in, {order[i]}, false, false)) {
            ok[i] = 1;
            exchanges[i] = row_program_exchanges(*probe) > 0;
            row_program_space(*probe, &R[i], &C[i]);
        }
    }
    std::vector<int> group(n);
    std::vector<std::vector<int>> members(n);
    for (int i = 0; i < n; ++i) {
        group[i] = i;
        members[i] = {i};
    }
    auto in_set = [&](const std::vector<uint64_t> &set, int i) { return (set[i / 64] >> (i % 64)) & 1; };
    // May groups P and Q become one routine?  Not if some state outside them lies between them (it would
    // have to run both after and before the merged routine).
    auto legal = [&](int P, int Q) {
        std::vector<uint64_t> u(words, 0), au(words, 0);
        for (int g : {P, Q})
            for (int m : members[g]) {
                u[m / 64] |= 1ull << (m % 64);
                for (int w = 0; w < words; ++w) au[w] |= anc[m][w];
            }
        if (members[P].size() + members[Q].size() > 24) return false;  // keeps the register arrays of one kernel in hand
        for (int x = 0; x < n; ++x) {
            if (!in_set(au, x) || in_set(u, x)) continue;
            for (int w = 0; w < words; ++w)
                if (anc[x][w] & u[w]) return false;
        }
        return true;
    };
    for (int i = 0; i < n; ++i) {
        if (!ok[i]) continue;
        for (int j : reads[i]) {
            if (!ok[j] || R[j] != R[i] || C[j] != C[i]) continue;
            const int P = group[j], Q = group[i];
            if (P == Q || !legal(P, Q)) continue;
            for (int m : members[Q]) {
                group[m] = P;
                members[P].push_back(m);
            }
            members[Q].clear();
        }
    }
    // a state on its own is worth a generated kernel when its body reduces (it would otherwise run as
    // several kernels); a lone map chain already is one kernel, and a lone softmax / log_sum_exp /
    // layer_norm has its hand-written kernel (which also writes the tf32 planes a GEMM reads next)
    for (int g = 0; g < n; ++g)
        if (members[g].size() >= 2 || (members[g].size() == 1 && ok[g] && exchanges[g] && !order[g].origin->composite)) {
            RowGroupPlan plan;
            plan.members = members[g];
            std::sort(plan.members.begin(), plan.members.end());
            plans.push_back(plan);
        }
    return plans;
}

// Program::compile, session.rs:62-206.
static std::unique_ptr<Program> compile(const std::vector<Var> &x, std::vector<Var> y, bool fusion, bool pattern, bool tc, bool softmax_in_gemm,
                                        bool row_groups = false, bool attention = false) {
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
    // row groups: states replaced by one generated kernel each
    std::unordered_set<Origin *> grouped;
    if (pattern && row_groups) {
        std::unordered_map<Origin *, std::vector<Origin *>> readers;  // state -> states that read it
        for (const Var &node : state_order)
            for (const Var &in : states[node.key()]) readers[in.key()].push_back(node.key());
        for (const RowGroupPlan &plan : plan_row_groups(state_order, states)) {
            std::unordered_set<Origin *> inside;
            for (int m : plan.members) inside.insert(state_order[m].key());
            std::vector<Var> outs, leaves;
            std::unordered_set<Origin *> seen;
            for (int m : plan.members) {
                const Var &v = state_order[m];
                bool needed = yset.count(v.key()) != 0;
                for (Origin *r : readers[v.key()])
                    if (!inside.count(r)) needed = true;
                if (needed) outs.push_back(v);
                for (const Var &in : states[v.key()])
                    if (!inside.count(in.key()) && seen.insert(in.key()).second) leaves.push_back(in);
            }
            if (outs.empty()) continue;
            std::shared_ptr<RowProgram> row = row_program_build(leaves, outs, false, true);
            if (!row) continue;  // e.g. an output that is only a view of another value: leave the states as they are
            Routine r;
            r.inputs = leaves;
            r.output = outs[0];
            r.row = row;
            r.row_outputs = outs;
            r.row_emit_shared = std::make_shared<std::vector<char>>(outs.size(), 0);
            for (const Var &v : r.inputs)
                if (v.is_op()) ++p->consumers[v.key()];
            for (Origin *k : inside) grouped.insert(k);
            for (const Var &o : outs) p->routines.emplace(o.key(), r);
        }
    }
    for (const Var &node : state_order) {
        if (grouped.count(node.key())) continue;
        Routine r;
        r.inputs = states[node.key()];
        r.output = node;
        std::unordered_set<Origin *> in_keys;
        for (const Var &v : r.inputs) {
            in_keys.insert(v.key());
            if (v.is_op()) ++p->consumers[v.key()];
        }
        r.root = build(node, in_keys, fusion, pattern, true);
        if (pattern) {
            lower(r.root, tc, softmax_in_gemm, attention && tc && attention_enabled());
            if (tc) group_gemms(r.root);
        }
        p->routines.emplace(node.key(), std::move(r));
    }
    if (pattern) {
        std::unordered_set<Origin *> plane_states;
        for (auto &kv : p->routines)
            if (!kv.second.row) mark_plane_readers(kv.second.root, tc, &plane_states);
        for (Origin *key : plane_states) {
            // A state that is only a view of another state (reshape(state)) shares its storage, and planes
            // belong to the storage: ask the state that really produces the values.
            auto it = p->routines.find(key);
            for (int hops = 0; it != p->routines.end() && !it->second.row && hops < 8; ++hops) {
                Node *root = skip_views(&it->second.root);
                if (!root->is_data || !root->var.is_op()) break;
                it = p->routines.find(root->var.key());
            }
            if (it == p->routines.end()) continue;  // an input of the program: split on first use
            if (it->second.row) {                   // a row group: the generated kernel writes the planes of that output
                for (size_t i = 0; i < it->second.row_outputs.size(); ++i)
                    if (it->second.row_outputs[i].key() == it->first) (*it->second.row_emit_shared)[i] = 1;
                continue;
            }
            Node *root = skip_views(&it->second.root);
            if (!root->is_data && can_emit_planes(*root->op, tc)) root->emit_planes = true;
        }
    }
    p->outputs = y;
    return p;
}

// Routine::exec, session.rs:612-673 (a recursive walk instead of the flattened stack).
typedef std::unordered_map<const Node *, Tensor> SharedMemo;  // results of shared nodes during one routine run

static sage_status run_node(const Node &n, Context &ctx, Session &s, const std::unordered_map<Origin *, Tensor> &temp,
                            SharedMemo &memo, Tensor *out) {
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
        sage_status st = run_node(n.args[i], ctx, s, temp, memo, &args[i]);
        if (st) return st;
    }
    if (n.shared) {
        auto it = memo.find(n.shared.get());
        if (it == memo.end()) {
            Tensor t;
            sage_status st = run_node(*n.shared, ctx, s, temp, memo, &t);
            if (st) return st;
            it = memo.emplace(n.shared.get(), t).first;
        }
        args.insert(args.begin(), it->second);
    }
    for (size_t i = 0; i < args.size(); ++i)  // Operator::compute's spec check, ops.rs:163-178
        if (args[i].desc.shape.extents != n.op->in[i].shape.extents)
            return ctx.fail(SAGE_ERR_INVALID, std::string("operand extents differ from the operator's spec in ") + n.op->name());
    ctx.hint_emit_planes = n.emit_planes;
    ctx.hint_planes_only = n.emit_planes && n.planes_only;
    sage_status st = n.op->compute(args, ctx, out);
    ctx.hint_emit_planes = ctx.hint_planes_only = false;
    return st;
}

// Program::exec, session.rs:208-468.
static sage_status exec(Program &p, Context &ctx, Session &s) {
    for (auto &kv : p.routines) kv.second.resolve_time();  // timers of an earlier run whose events have completed
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
        std::vector<Tensor> row_outs;
        for (;;) {
            auto t0 = std::chrono::steady_clock::now();
            std::shared_ptr<RoutineTimer> timer;
            if (!f.timed && !ctx.dry()) {
                timer = std::make_shared<RoutineTimer>();
                if (cudaEventCreate(&timer->ev[0]) != cudaSuccess || cudaEventCreate(&timer->ev[1]) != cudaSuccess ||
                    cudaEventRecord(timer->ev[0], ctx.stream()) != cudaSuccess)
                    timer.reset();
            }
            SharedMemo memo;
            sage_status st;
            if (f.row) {
                st = row_program_run(*f.row, ctx, [&](const Var &k, Tensor *t) {
                    auto jt = temp.find(k.key());
                    if (jt != temp.end()) {
                        *t = jt->second;
                        return true;
                    }
                    return s.get(k, t);
                }, &row_outs, f.row_emit_shared.get());
            } else {
                st = run_node(f.root, ctx, s, temp, memo, &out);
            }
            if (timer && st == SAGE_OK && cudaEventRecord(timer->ev[1], ctx.stream()) == cudaSuccess) {
                f.timer = timer;
                f.timed = true;
            } else if (!f.timed) {
                f.exec_time = 1e6 * std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            }
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
                    r2->second.resolve_time();
                    // cost of recomputing per element kept (session.rs:301-302), with the device time in microseconds
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
        if (f.row) {  // every state of the group at once
            for (size_t i = 0; i < f.row_outputs.size(); ++i) {
                const Var &o = f.row_outputs[i];
                if (outputs.count(o.key())) s.data[o.key()] = std::make_pair(o, row_outs[i]);
                else temp[o.key()] = row_outs[i];
            }
        } else if (outputs.count(v.key())) {
            s.data[v.key()] = std::make_pair(v, out);
        } else {
            temp[v.key()] = out;
        }
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
    const uint64_t key_hash = program_key_hash(tk, xk);
    for (size_t i = cache_.size(); i-- > 0;) {
        Program *c = cache_[i].get();
        if (c->key_hash != key_hash || c->target_keys != tk || c->x_keys != xk || (c->row && !row_program_ready(*c->row, *this))) continue;
        prog = c;
        if (i + 1 != cache_.size()) std::rotate(cache_.begin() + (long)i, cache_.begin() + (long)i + 1, cache_.end());  // now the most recent
        break;
    }
    if (!prog) {
        std::unique_ptr<Program> p;
        try {
            // pattern_fusion bit 0: composites and whole-row programs; bit 2 keeps the row programs off
            // A lone softmax / log_sum_exp / layer_norm of evaluated data keeps its hand-written row kernel
            // (measured 0.85-0.98 of the HBM peak against 0.75-0.85 for the generated program).
            bool lone_composite = y.size() == 1 && y[0].origin->composite != nullptr;
            if (lone_composite)
                for (const Var &in : y[0].origin->composite->inputs)
                    if (in.is_op() && !data.count(in.key())) lone_composite = false;
            if ((ctx_->opts().pattern_fusion & 5) == 1 && row_programs_enabled() && !lone_composite) {
                std::vector<Var> held;
                for (auto &kv : data) held.push_back(kv.second.first);
                if (auto row = row_program_build(held, y)) {
                    p.reset(new Program());
                    p->outputs = y;
                    p->row = row;
                }
            }
            if (!p)
                p = compile(x, y, true, ctx_->opts().pattern_fusion != 0, ctx_->opts().gemm_backend != 1, (ctx_->opts().pattern_fusion & 2) != 0,
                            (ctx_->opts().pattern_fusion & 5) == 1 && row_programs_enabled(), (ctx_->opts().pattern_fusion & 8) == 0);
        } catch (const ShapeError &e) {
            return ctx_->fail(SAGE_ERR_INVALID, e.msg);
        }
        p->target_keys = tk;
        p->x_keys = xk;
        p->key_hash = key_hash;
        prog = p.get();
        if (cache_.size() >= kMaxPrograms) {
            if (last_ == cache_.front().get()) last_ = nullptr;
            cache_.erase(cache_.begin());  // the least recently used program and everything only it kept alive
        }
        cache_.push_back(std::move(p));
        ++programs_compiled;
    }
    last_ = prog;
    try {
        if (prog->row) return row_program_exec(*prog->row, *ctx_, *this);
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
    out->append(describe_gemm(*n.op));
    if (n.emit_planes) out->append(n.planes_only ? "=planes" : "+planes");
    out->push_back('(');
    if (n.shared) describe_node(*n.shared, out);
    for (size_t i = 0; i < n.args.size(); ++i) {
        if (i) out->push_back(',');
        describe_node(n.args[i], out);
    }
    out->push_back(')');
}

std::string Session::describe_last() const {
    std::string out;
    if (!last_) return out;
    if (last_->row) return row_program_describe(*last_->row);
    std::vector<const Routine *> rs;
    for (auto &kv : last_->routines) rs.push_back(&kv.second);
    std::sort(rs.begin(), rs.end(), [](const Routine *a, const Routine *b) {
        return a->output.t_order() != b->output.t_order() ? a->output.t_order() < b->output.t_order() : a->output.key() < b->output.key();
    });
    std::unordered_set<const RowProgram *> shown;
    for (const Routine *r : rs) {
        if (r->row) {
            if (shown.insert(r->row.get()).second) out.append(row_program_describe(*r->row));
            continue;
        }
        describe_node(r->root, &out);
        out.push_back('\n');
    }
    return out;
}

}  // namespace sage
