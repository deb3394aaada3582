// Shape, Tensor, Var and reverse-mode grad.  Reference: src/shape.rs, src/tensor.rs, src/var.rs.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <queue>

#include "graph.h"

namespace sage {

void shape_fail(const std::string &msg) { throw ShapeError{msg}; }

// ---------------------------------------------------------------- Shape
Array Shape::default_strides(const Array &extents) {  // shape.rs:45-54
    Array s(extents.size());
    long long p = 1;
    for (int i = (int)extents.size() - 1; i >= 0; --i) {
        s[i] = p;
        p *= extents[i];
    }
    return s;
}

long long Shape::size() const {
    long long p = 1;
    for (long long e : extents) p *= e;
    return p;
}

bool Shape::has_default_strides() const { return strides == default_strides(extents); }  // shape.rs:134-143

void Shape::extract(const std::vector<int> &axes, Shape *inner, Shape *outer) const {  // shape.rs:113-132
    inner->extents.clear();
    inner->strides.clear();
    inner->offset = 0;
    outer->extents.clear();
    outer->strides.clear();
    outer->offset = offset;
    for (int a : axes) {
        inner->extents.push_back(extents[a]);
        inner->strides.push_back(strides[a]);
    }
    for (int a = 0; a < rank(); ++a)
        if (std::find(axes.begin(), axes.end(), a) == axes.end()) {
            outer->extents.push_back(extents[a]);
            outer->strides.push_back(strides[a]);
        }
}

Shape Shape::remove(int axis) const {
    Shape s = *this;
    s.extents.erase(s.extents.begin() + axis);
    s.strides.erase(s.strides.begin() + axis);
    return s;
}

Shape Shape::insert(int axis) const {  // shape.rs:190-195: the new unit axis has stride 0
    Shape s = *this;
    s.extents.insert(s.extents.begin() + axis, 1);
    s.strides.insert(s.strides.begin() + axis, 0);
    return s;
}

Shape Shape::permute(const std::vector<int> &axes) const {
    Shape s;
    s.offset = offset;
    for (int a : axes) {
        s.extents.push_back(extents[a]);
        s.strides.push_back(strides[a]);
    }
    return s;
}

Shape Shape::select_range(long long start, long long end_incl, int axis) const {  // shape.rs:229-237
    if (extents[axis] <= end_incl) shape_fail("index out of bounds");
    Shape s = *this;
    s.offset += strides[axis] * start;
    s.extents[axis] = end_incl - start + 1;
    return s;
}

Shape Shape::expand(const Array &target) const {  // shape.rs:239-279
    if (target.size() < extents.size()) shape_fail("target shape must be larger than the broadcasted shape");
    Shape s = *this;
    for (size_t i = 0; i < target.size() - extents.size(); ++i) {
        s.extents.insert(s.extents.begin(), 1);
        s.strides.insert(s.strides.begin(), 0);
    }
    for (size_t i = 0; i < target.size(); ++i)
        if (s.extents[i] != target[i]) {
            if (s.extents[i] != 1) shape_fail("invalid broadcast... target shape should be larger.");
            s.extents[i] = target[i];
            s.strides[i] = 0;
        }
    return s;
}

Array union_extents(const Array &a, const Array &b) {
    if (a == b) return a;
    const Array &longer = a.size() > b.size() ? a : b;
    const Array &shorter = a.size() > b.size() ? b : a;
    Array u(longer.begin(), longer.begin() + (longer.size() - shorter.size()));
    u.insert(u.end(), shorter.begin(), shorter.end());
    for (size_t i = 0; i < u.size(); ++i)
        if (u[i] != longer[i]) {
            if (u[i] == 1) u[i] = longer[i];
            else if (longer[i] != 1) shape_fail("invalid broadcast");
        }
    return u;
}

Array infer_extents(const Array &extents, long long size) {
    Array out = extents;
    long long known = 1;
    int infer = -1;
    for (size_t i = 0; i < out.size(); ++i) {
        if (out[i] == -1) {
            if (infer >= 0) shape_fail("cannot infer the size");
            infer = (int)i;
        } else if (out[i] <= 0) {
            shape_fail("invalid shape extent " + std::to_string(out[i]));
        } else {
            known *= out[i];
        }
    }
    if (infer < 0) {
        if (size > 0 && known != size) shape_fail("size mismatch! expected " + std::to_string(size) + " but got " + std::to_string(known));
    } else {
        if (size == 0 || size % known != 0) shape_fail("cannot infer the size");
        out[infer] = size / known;
    }
    return out;
}

int to_axis(long long axis, int bound) {
    if (bound < 1) shape_fail("invalid index bound");
    long long a = axis < 0 ? axis + bound : axis;
    if (a < 0 || a >= bound) shape_fail("index out of range: " + std::to_string(axis));
    return (int)a;
}

std::vector<int> to_axes(const std::vector<long long> &axes, int bound) {
    std::vector<int> out;
    for (long long a : axes) out.push_back(to_axis(a, bound));
    return out;
}

// ---------------------------------------------------------------- Tensor
Storage::~Storage() {
    if (alloc && block) alloc->free(block);
}

sage_status Tensor::uninit(Context &ctx, const TensorDesc &desc, Tensor *out) {
    TensorDesc d = desc.pristine();
    Block *b = ctx.allocator().alloc((size_t)d.shape.size() * 4);
    if (!b) return ctx.fail(SAGE_ERR_OOM, "out of memory: needed " + std::to_string(ctx.allocator().oom_needed) +
                                              " more bytes, total " + std::to_string(ctx.allocator().oom_total));
    auto st = std::make_shared<Storage>();
    st->ctx = &ctx;
    st->alloc = ctx.allocator_ptr();
    st->block = b;
    st->dev = b->ptr;
    st->bytes = (size_t)d.shape.size() * 4;
    out->desc = d;
    out->data = st;
    return SAGE_OK;
}

Tensor Tensor::from_host(const Array &extents, int dtype, const void *data) {
    Tensor t;
    t.desc = TensorDesc(extents, dtype);
    auto st = std::make_shared<Storage>();
    st->bytes = (size_t)t.desc.shape.size() * 4;
    st->host.resize(st->bytes);
    if (data) memcpy(st->host.data(), data, st->bytes);
    t.data = st;
    return t;
}

// Uploads host-resident data once; every handle to the same storage sees the device copy.  (The
// reference panics when a kernel meets a host tensor, src/session/device.rs:259; BertEmbedding
// builds its position ids on the host, src/models/bert.rs:132, so the upload happens here.)
sage_status Tensor::to_device(Context &ctx) {
    if (on_device()) return SAGE_OK;
    Block *b = ctx.allocator().alloc(data->bytes);
    if (!b) return ctx.fail(SAGE_ERR_OOM, "out of memory uploading a host tensor");
    data->ctx = &ctx;
    data->alloc = ctx.allocator_ptr();
    data->block = b;
    data->dev = b->ptr;
    if (!ctx.dry()) {
        // the vector stays alive as long as the storage does, so an async copy is safe, but the
        // source is pageable, so this is a synchronous-staged copy anyway
        sage_status st = ctx.check_cuda(cudaMemcpyAsync(b->ptr, data->host.data(), data->bytes, cudaMemcpyHostToDevice, ctx.stream()), "upload");
        if (st) return st;
        cudaStreamSynchronize(ctx.stream());
    }
    data->host.clear();
    data->host.shrink_to_fit();
    return SAGE_OK;
}

k::Dims Tensor::dims() const {
    k::Dims d;
    d.ndim = desc.shape.rank();
    for (int i = 0; i < d.ndim; ++i) {
        d.ext[i] = desc.shape.extents[i];
        d.str[i] = desc.shape.strides[i];
    }
    return d;
}

// ---------------------------------------------------------------- Var
bool Var::is_op() const { return origin && origin->op; }
size_t Var::t_order() const { return origin ? origin->t_order : 0; }

Var Var::from_tensor(const Tensor &t) {
    Var v;
    v.desc = t.desc;
    v.origin = std::make_shared<Origin>();
    v.origin->data = t;
    return v;
}

Var Var::empty(const Array &extents, int dtype) {
    Var v;
    v.desc = TensorDesc(infer_extents(extents, 0), dtype);
    v.origin = std::make_shared<Origin>();
    return v;
}

Var Var::from_op(std::shared_ptr<Operator> op, const std::vector<Var> &x) {  // Operation::*, ops.rs:248-315
    Var v;
    v.desc = op->out;
    v.origin = std::make_shared<Origin>();
    v.origin->op = std::move(op);
    v.origin->inputs = x;
    size_t t = 0;
    for (const Var &i : x) t = std::max(t, i.t_order());
    v.origin->t_order = x.empty() ? 0 : t + 1;
    return v;
}

void Var::set(const Tensor &t) const {
    if (is_op()) shape_fail("can only assign tensor to the data variable");
    if (t.desc.shape.extents != desc.shape.extents) shape_fail("Var::set: extents differ from the variable's");
    origin->data = t;
}

Var Var::organize() const { return desc.shape.has_default_strides() ? *this : ops::unary_map(*this, ops::Copy); }

// ---------------------------------------------------------------- grad (var.rs:56-103)
std::vector<Var> grad(const Var &y, const std::vector<Var> &xs) {
    struct Ranked {
        size_t rank;
        uint64_t seq;
        Var v;
        bool operator<(const Ranked &o) const { return rank != o.rank ? rank < o.rank : seq > o.seq; }
    };
    std::priority_queue<Ranked> queue;  // max-heap on topological order
    std::unordered_map<Origin *, Var> grads;
    uint64_t seq = 0;
    grads[y.key()] = ops::scalar_f(1.0f, y.extents());
    queue.push({y.t_order(), seq++, y});
    while (!queue.empty()) {
        Var v = queue.top().v;
        queue.pop();
        Var gy = grads[v.key()];
        if (!v.is_op()) continue;
        const std::vector<Var> &x = v.origin->inputs;
        std::vector<Var> gx = v.origin->op->grad(x, v, gy);
        for (size_t i = 0; i < x.size() && i < gx.size(); ++i) {
            if (!gx[i].defined()) continue;
            if (gx[i].extents() != x[i].extents()) shape_fail(std::string("grad shape error in ") + v.origin->op->name());
            auto it = grads.find(x[i].key());
            if (it == grads.end()) {
                queue.push({x[i].t_order(), seq++, x[i]});
                grads[x[i].key()] = gx[i];
            } else {
                it->second = ops::add(gx[i], it->second);
            }
        }
    }
    std::vector<Var> out;
    for (const Var &x : xs) {
        auto it = grads.find(x.key());
        if (it == grads.end()) shape_fail("grad: the variable does not contribute to y");
        out.push_back(it->second);
    }
    return out;
}

}  // namespace sage
