// Host-side restatement of sage's lazy graph for the hot path: Shape / Tensor / Var, the operator
// model with reverse-mode grad, and the session evaluator (state selection + map fusion).
// Reference: src/shape.rs, src/tensor.rs, src/var.rs, src/ops.rs, src/session.rs,
// src/session/context.rs.  The reference is Rust; no Rust toolchain exists where this library is
// built, so the same structures are written in C++ behind the C ABI of include/sage_graph.h.
#pragma once
#include <cstdint>
#include <algorithm>
#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../codegen/map_emit.h"
#include "../runtime/runtime.h"

namespace sage {

typedef std::vector<long long> Array;

struct ShapeError {
    std::string msg;
};
[[noreturn]] void shape_fail(const std::string &msg);  // throws ShapeError; caught at the C ABI

// ---------------------------------------------------------------- Shape (src/shape.rs:37-279)
struct Shape {
    Array extents, strides;
    long long offset = 0;

    Shape() {}
    explicit Shape(const Array &e) : extents(e), strides(default_strides(e)) {}
    Shape(const Array &e, const Array &s, long long off) : extents(e), strides(s), offset(off) {}

    static Array default_strides(const Array &extents);
    int rank() const { return (int)extents.size(); }
    long long size() const;
    bool has_default_strides() const;
    bool operator==(const Shape &o) const { return extents == o.extents && strides == o.strides && offset == o.offset; }
    void extract(const std::vector<int> &axes, Shape *inner, Shape *outer) const;  // nested = true
    Shape remove(int axis) const;
    Shape insert(int axis) const;
    Shape permute(const std::vector<int> &axes) const;
    Shape select_range(long long start, long long end_incl, int axis) const;
    Shape expand(const Array &extents) const;
};
Array union_extents(const Array &a, const Array &b);               // shape.rs:356-393
Array infer_extents(const Array &extents, long long size);         // shape.rs:400-441 (one -1)
int to_axis(long long axis, int bound);                            // shape.rs:517-545
std::vector<int> to_axes(const std::vector<long long> &axes, int bound);

struct TensorDesc {
    Shape shape;
    int dtype = SAGE_F32;
    TensorDesc() {}
    TensorDesc(const Array &extents, int dt) : shape(extents), dtype(dt) {}
    TensorDesc(const Shape &s, int dt) : shape(s), dtype(dt) {}
    TensorDesc pristine() const { return TensorDesc(shape.extents, dtype); }
};

// ---------------------------------------------------------------- Tensor (src/tensor.rs:106-110)
// Device memory returns to the allocator when the last handle drops (OpenClMemory, memory.rs:672-692).
// The tf32 hi/lo split of (a view of) a storage, kept next to it so that weights and activations
// read by several GEMMs are split once.  Dropped with the storage, or when the storage is rewritten.
// Two forms: `whole` planes mirror the storage element for element (hi at planes.planes[i], lo
// `plane` floats further), so any view of the storage is the same view of the planes; a compact
// split holds one strided view gathered into rows with a 16-byte pitch.
struct SplitCache {
    k::SplitPlanes planes;
    std::shared_ptr<Allocator> alloc;
    bool whole = false;
    long long plane = 0;     // whole: floats between the hi and the lo plane
    Shape view;              // compact: the view that was gathered
    ~SplitCache() {
        if (alloc && planes.block) alloc->free(planes.block);
    }
};

struct Storage {
    std::shared_ptr<SplitCache> split;       // whole-storage planes
    std::shared_ptr<SplitCache> split_view;  // last compact split of a view
    uint64_t version = 0;                    // bumped whenever the contents are rewritten
    bool planes_only = false;                // the fp32 buffer was never written: only `split` holds the value
    void drop_splits() {
        split.reset();
        split_view.reset();
        ++version;
    }
    Context *ctx = nullptr;  // identity only; never dereferenced by the destructor
    std::shared_ptr<Allocator> alloc;
    Block *block = nullptr;
    void *dev = nullptr;
    size_t bytes = 0;
    std::vector<uint8_t> host;  // host-resident data (Data::Host); uploaded on first use
    ~Storage();
};

struct Tensor {
    TensorDesc desc;
    std::shared_ptr<Storage> data;
    bool defined() const { return (bool)data; }
    bool on_device() const { return data && data->dev; }
    void *ptr() const { return static_cast<char *>(data->dev) + desc.shape.offset * 4; }
    Tensor with_shape(const Shape &s) const {
        Tensor t = *this;
        t.desc.shape = s;
        return t;
    }
    static sage_status uninit(Context &ctx, const TensorDesc &desc, Tensor *out);  // Tensor::uninit2, tensor.rs:195-210
    static Tensor from_host(const Array &extents, int dtype, const void *data);
    sage_status to_device(Context &ctx);                                          // tensor.rs:280-293
    k::Dims dims() const;
};

// ---------------------------------------------------------------- Var / Operator (src/var.rs, src/ops.rs)
struct Operator;
struct Origin;

struct Var {
    TensorDesc desc;
    std::shared_ptr<Origin> origin;

    bool defined() const { return (bool)origin; }
    const Array &extents() const { return desc.shape.extents; }
    long long extent(long long axis) const { return desc.shape.extents[to_axis(axis, rank())]; }
    int rank() const { return desc.shape.rank(); }
    long long size() const { return desc.shape.size(); }
    int dtype() const { return desc.dtype; }
    bool is_op() const;
    bool is_data() const { return !is_op(); }
    size_t t_order() const;
    Origin *key() const { return origin.get(); }
    bool operator==(const Var &o) const { return origin == o.origin; }

    static Var from_tensor(const Tensor &t);                    // Var::new, var.rs:153-164
    static Var empty(const Array &extents, int dtype);          // Var::empty, var.rs:166-175
    static Var from_op(std::shared_ptr<Operator> op, const std::vector<Var> &x);
    void set(const Tensor &t) const;                            // Var::set, var.rs:370-377
    Var organize() const;                                       // var.rs:506-512
};

enum class Cat { Map, Reduce, Contract, LayoutExpand, Other };  // ops.rs:23-30

struct Operator {
    std::vector<TensorDesc> in;
    TensorDesc out;
    virtual ~Operator() {}
    virtual const char *name() const = 0;
    virtual Cat cat() const { return Cat::Other; }
    // One entry per input; an undefined Var means "no gradient" (None).
    virtual std::vector<Var> grad(const std::vector<Var> &x, const Var &y, const Var &gy) = 0;
    virtual sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) = 0;
};

// Marks a Var as the output of a known composite (softmax, log_sum_exp, layer_norm, pooling) so the
// evaluator may run it as one kernel instead of walking the decomposed sub-graph below it.  The
// decomposed graph stays in place: grad() and evaluation with pattern fusion off use it.
struct Composite {
    std::shared_ptr<Operator> op;
    std::vector<Var> inputs;
};

struct Origin {
    std::shared_ptr<Operator> op;  // null for data
    std::vector<Var> inputs;
    size_t t_order = 0;
    Tensor data;                   // Origin::Data(RefCell<Option<Tensor>>)
    std::unique_ptr<Composite> composite;
    std::string name;
};

std::vector<Var> grad(const Var &y, const std::vector<Var> &xs);  // var.rs:56-103

// ---------------------------------------------------------------- Session (src/session.rs, context.rs)
struct Routine;
struct Program;

class Session {
public:
    explicit Session(Context *ctx);
    ~Session();
    Context &ctx() { return *ctx_; }
    // Context::eval, context.rs:96-117: evaluates the targets; results stay in `data`.
    sage_status eval(const std::vector<Var> &targets);
    void clear();  // Context::clear, context.rs:92-94
    bool get(const Var &v, Tensor *out) const;
    std::unordered_map<Origin *, std::pair<Var, Tensor>> data;  // Context::data
    // Kernel trace of the last compiled program, one routine per line (for tests / planning).
    std::string describe_last() const;
    uint64_t programs_compiled = 0;
    // Compiled programs are kept, least recently used first, up to this many.  A cached program keeps its whole
    // graph alive (leaf tensors, grouped weight copies, tf32 planes, generated kernels), so a loop that builds a
    // fresh graph per step would otherwise grow without bound; the reference recompiles on every eval
    // (context.rs:96-117) and keeps nothing.
    static constexpr size_t kMaxPrograms = 32;
    size_t programs_cached() const { return cache_.size(); }
    void drop_programs();  // forget every compiled program (and what it holds alive)

private:
    Context *ctx_;
    std::vector<std::unique_ptr<Program>> cache_;  // least recently used first
    Program *last_ = nullptr;
};

// ---------------------------------------------------------------- op constructors (free functions,
// named like the reference's src/ops/*.rs)
namespace ops {
// map.rs
enum Unary { Copy, Abs, Neg, Recip, Log, Exp, Sqrt, Square, Erf, Sign, Ceil, Floor, Round, Sin, Sinh, Cos, Cosh, Tan, Tanh,
             Asin, Asinh, Acos, Acosh, Atan, Atanh, Not, CastInt, CastFloat, kNumUnary };
enum Binary { Add, Sub, Div, Mul, Mod, Pow, Min, Max, And, Or, Eq, Ne, Gt, Ge, Lt, Le, kNumBinary };
Var scalar_f(float v, const Array &extents);
Var scalar_i(int v, const Array &extents);
Var unary_map(const Var &x, Unary m);
Var binary_map(const Var &a, const Var &b, Binary m);
Var cond(const Var &c, const Var &a, const Var &b);
inline Var operator_f(const Var &a, float b, Binary m) { return binary_map(a, scalar_f(b, {1}), m); }
// core.rs
Var reshape(const Var &x, const Shape &shape);
Var view(const Var &x, const Array &extents);
Var expand(const Var &x, const Array &extents);
Var permute(const Var &x, const std::vector<long long> &axes);
Var transpose(const Var &x, long long a1, long long a2);
Var squeeze(const Var &x, long long axis);
Var unsqueeze(const Var &x, long long axis);
Var slice(const Var &x, long long axis, long long start, long long end);
Var unslice(const Var &x, long long axis, long long start, long long end);
Var gather(const Var &x, const Var &ind, long long axis);
Var scatter(const Var &x, const Var &ind, long long axis, const Array &extents);
Var concat(const std::vector<Var> &xs, long long axis);
// reduce.rs
enum Red { Sum, Prod, RMax, RMin };
Var reduce(const Var &x, const std::vector<long long> &axes, bool preserve, Red kind);
Var mean(const Var &x, const std::vector<long long> &axes, bool preserve);
Var var(const Var &x, const std::vector<long long> &axes, bool preserve);
Var reduce_arg(const Var &x, long long axis, bool preserve, bool is_max);
// gemm.rs
Var gemm(const Var &a, const Var &b, bool ta, bool tb);
Var gemm_batched(const Var &a, const Var &b, bool ta, bool tb);
Var matmul(const Var &a, const Var &b);
Var matmul_batched(const Var &a, const Var &b);
// conv.rs ([w, h] ordered pairs)
struct Pair { long long w, h; };
Var im2col(const Var &x, Pair ker, Pair stride, Pair pad, Pair dil);
Var col2im(const Var &x, Pair img, Pair ker, Pair stride, Pair pad, Pair dil);
Var conv_2d(const Var &x, const Var &filter, Pair stride, Pair pad, Pair dil);
Var avg_pool_2d(const Var &x, Pair ker, Pair stride, Pair pad, Pair dil);
Var max_pool_2d(const Var &x, Pair ker, Pair stride, Pair pad, Pair dil);
Var batch_norm_2d(const Var &x, const Var &gamma, const Var &beta, const Var &mean, const Var &var, float eps);
// nn.rs
Var relu(const Var &x);
Var softmax(const Var &x, const std::vector<long long> &axes);
Var log_sum_exp(const Var &x, const std::vector<long long> &axes);
Var softmax_cross_entropy(const Var &x, const Var &labels);
Var layer_norm(const Var &x, const std::vector<long long> &axes, const Var &gamma, const Var &beta, float eps);
// metric.rs
Var accuracy(const Var &logits, const Var &labels);
// rand.rs (the seeds the reference draws per evaluation are arguments here)
Var uniform(const Array &extents, unsigned seed_x, unsigned seed_y);
Var normal(const Array &extents, unsigned seed_x, unsigned seed_y);
// arithmetic sugar (map.rs:1180-1370)
inline Var add(const Var &a, const Var &b) { return binary_map(a, b, Add); }
inline Var sub(const Var &a, const Var &b) { return binary_map(a, b, Sub); }
inline Var mul(const Var &a, const Var &b) { return binary_map(a, b, Mul); }
inline Var div(const Var &a, const Var &b) { return binary_map(a, b, Div); }
inline Var add(const Var &a, float b) { return operator_f(a, b, Add); }
inline Var sub(const Var &a, float b) { return operator_f(a, b, Sub); }
inline Var mul(const Var &a, float b) { return operator_f(a, b, Mul); }
inline Var div(const Var &a, float b) { return operator_f(a, b, Div); }
inline Var neg(const Var &a) { return unary_map(a, Neg); }
}  // namespace ops

// Map operator internals shared between ops_map.cc and session.cc (fusion).
struct MapExpr {
    enum Kind { Input, Literal, Un, Bin, Tern } kind = Input;
    int op = 0;       // ops::Unary / ops::Binary
    int input = 0;    // Input: operand index
    uint32_t bits = 0;  // Literal: raw 32-bit pattern
    int lit_dtype = SAGE_F32;
    std::vector<MapExpr> args;
};
struct MapOp;
std::shared_ptr<Operator> fuse_ops(const Operator &parent, const Operator &child, int idx);  // Operator::fuse, ops.rs:104-161
std::string map_expr_text(const MapExpr &e);
const MapExpr *map_expr_of(const Operator &op);

}  // namespace sage
