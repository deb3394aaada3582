// extern "C" surface of include/sage_graph.h.
#include <cuda_runtime.h>

#include <cstring>

#include "../../../include/sage_graph.h"
#include "../graph/graph.h"
#include "../nn/nn.h"
#include "../nn/optim.h"

using namespace sage;

struct sage_session {
    Session *impl;
    sage_ctx *ctx;
};
struct sage_var {
    Var v;
};
struct sage_bert {
    nn::Bert *impl;
};
struct sage_model {
    std::shared_ptr<nn::Sequential> impl;
};

struct sage_optimizer {
    std::unique_ptr<nn::Optimizer> impl;
};

static thread_local std::string g_error;

template <typename F>
static sage_status guarded(F f) {
    try {
        return f();
    } catch (const ShapeError &e) {
        g_error = e.msg;
        return SAGE_ERR_INVALID;
    } catch (const std::exception &e) {
        g_error = e.what();
        return SAGE_ERR_INVALID;
    }
}

static Array arr(int32_t n, const int64_t *v) { return Array(v, v + n); }
static std::vector<long long> axes_of(int32_t n, const int64_t *v) { return std::vector<long long>(v, v + n); }
static sage_status ret(sage_var **out, const Var &v) {
    *out = new sage_var{v};
    return SAGE_OK;
}
static ops::Pair pr(const int32_t p[2]) { return ops::Pair{p[0], p[1]}; }

extern "C" {

const char *sage_graph_last_error(void) { return g_error.c_str(); }

sage_status sage_session_create(sage_ctx *ctx, sage_session **s) {
    if (!ctx || !ctx->impl) return SAGE_ERR_INVALID;
    *s = new sage_session{new Session(ctx->impl), ctx};
    return SAGE_OK;
}
sage_status sage_session_destroy(sage_session *s) {
    if (s) {
        delete s->impl;
        delete s;
    }
    return SAGE_OK;
}
sage_status sage_session_clear(sage_session *s) {
    s->impl->clear();
    return SAGE_OK;
}

static sage_status upload_into(Context &C, Tensor *t, const void *data, bool async) {
    if (C.dry()) return SAGE_OK;  // planning: the buffer exists, its contents are never read
    sage_status st = C.check_cuda(cudaMemcpyAsync(t->ptr(), data, (size_t)t->desc.shape.size() * 4, cudaMemcpyHostToDevice, C.stream()), "upload");
    if (st || async) return st;
    return C.check_cuda(cudaStreamSynchronize(C.stream()), "upload sync");
}

sage_status sage_var_from_host(sage_session *s, int32_t dtype, int32_t ndim, const int64_t *extents, const void *data, sage_var **out) {
    return guarded([&]() -> sage_status {
        Context &C = s->impl->ctx();
        C.make_current();
        Tensor t;
        sage_status st = Tensor::uninit(C, TensorDesc(infer_extents(arr(ndim, extents), 0), dtype), &t);
        if (st) return st;
        st = upload_into(C, &t, data, false);
        if (st) return st;
        return ret(out, Var::from_tensor(t));
    });
}

sage_status sage_var_from_host_lazy(int32_t dtype, int32_t ndim, const int64_t *extents, const void *data, sage_var **out) {
    return guarded([&]() -> sage_status { return ret(out, Var::from_tensor(Tensor::from_host(infer_extents(arr(ndim, extents), 0), dtype, data))); });
}

sage_status sage_var_empty(int32_t dtype, int32_t ndim, const int64_t *extents, sage_var **out) {
    return guarded([&]() -> sage_status { return ret(out, Var::empty(arr(ndim, extents), dtype)); });
}

sage_status sage_var_set(sage_session *s, sage_var *v, const void *data, int32_t async) {
    return guarded([&]() -> sage_status {
        Context &C = s->impl->ctx();
        C.make_current();
        if (v->v.is_op()) shape_fail("can only assign tensor to the data variable");
        Tensor &cur = v->v.origin->data;
        // Reuse the variable's buffer when it is exclusively owned, contiguous and of the right size.
        if (!(cur.defined() && cur.on_device() && cur.data.use_count() == 1 && cur.data->ctx == &C &&
              cur.desc.shape.has_default_strides() && cur.desc.shape.offset == 0 &&
              cur.desc.shape.extents == v->v.extents())) {
            Tensor t;
            sage_status st = Tensor::uninit(C, v->v.desc, &t);
            if (st) return st;
            cur = t;
        }
        cur.data->drop_splits();  // the buffer is being rewritten: any cached tf32 split is stale
        return upload_into(C, &cur, data, async != 0);
    });
}

sage_status sage_var_free(sage_var *v) {
    delete v;
    return SAGE_OK;
}

sage_status sage_var_info(const sage_var *v, int32_t *dtype, int32_t *ndim, int64_t *extents, int64_t *strides, int64_t *offset,
                          int32_t *is_op, uint64_t *t_order) {
    const Var &x = v->v;
    if (dtype) *dtype = x.dtype();
    if (ndim) *ndim = x.rank();
    for (int i = 0; i < x.rank() && i < SAGE_MAX_DIMS; ++i) {
        if (extents) extents[i] = x.desc.shape.extents[i];
        if (strides) strides[i] = x.desc.shape.strides[i];
    }
    if (offset) *offset = x.desc.shape.offset;
    if (is_op) *is_op = x.is_op();
    if (t_order) *t_order = x.t_order();
    return SAGE_OK;
}

sage_status sage_eval(sage_session *s, sage_var *const *targets, int32_t n) {
    std::vector<Var> t;
    for (int i = 0; i < n; ++i) t.push_back(targets[i]->v);
    s->impl->ctx().make_current();
    sage_status st = s->impl->eval(t);
    if (st) g_error = s->impl->ctx().last_error();
    return st;
}

static sage_status tensor_of(sage_session *s, const Var &v, Tensor *t) {
    Context &C = s->impl->ctx();
    C.make_current();
    if (v.is_op()) {
        if (!s->impl->get(v, t)) return C.fail(SAGE_ERR_INVALID, "variable has not been evaluated");
        return SAGE_OK;
    }
    if (!v.origin->data.defined()) return C.fail(SAGE_ERR_INVALID, "uninitialized variable");
    sage_status st = v.origin->data.to_device(C);
    if (st) return st;
    *t = v.origin->data;
    return SAGE_OK;
}

sage_status sage_var_read(sage_session *s, const sage_var *v, void *dst, size_t bytes) {
    return guarded([&]() -> sage_status {
        Context &C = s->impl->ctx();
        C.make_current();
        Tensor t;
        sage_status st = tensor_of(s, v->v, &t);
        if (st) {
            g_error = C.last_error();
            return st;
        }
        if ((size_t)t.desc.shape.size() * 4 != bytes) return C.fail(SAGE_ERR_INVALID, "read: byte count differs from the tensor's size");
        if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "read on a planning context");
        if (!t.desc.shape.has_default_strides()) {
            Tensor c;
            st = Tensor::uninit(C, t.desc, &c);
            if (st) return st;
            st = k::strided_copy(C, (const uint32_t *)t.ptr(), t.dims(), (uint32_t *)c.ptr(), c.desc.shape.strides.data());
            if (st) return st;
            t = c;
        }
        st = C.check_cuda(cudaMemcpyAsync(dst, t.ptr(), bytes, cudaMemcpyDeviceToHost, C.stream()), "download");
        if (st) return st;
        return C.check_cuda(cudaStreamSynchronize(C.stream()), "download sync");
    });
}

sage_status sage_var_buffer(sage_session *s, const sage_var *v, void **dev_ptr, size_t *bytes) {
    Tensor t;
    sage_status st = tensor_of(s, v->v, &t);
    if (st) return st;
    *dev_ptr = t.ptr();
    *bytes = (size_t)t.desc.shape.size() * 4;
    return SAGE_OK;
}

sage_status sage_grad(const sage_var *y, sage_var *const *xs, int32_t n, sage_var **out) {
    return guarded([&]() -> sage_status {
        std::vector<Var> x;
        for (int i = 0; i < n; ++i) x.push_back(xs[i]->v);
        std::vector<Var> g = grad(y->v, x);
        for (int i = 0; i < n; ++i) out[i] = new sage_var{g[i]};
        return SAGE_OK;
    });
}

sage_status sage_session_describe(sage_session *s, char *out, size_t out_len, size_t *needed) {
    std::string d = s->impl->describe_last();
    if (needed) *needed = d.size() + 1;
    if (out && out_len) {
        size_t n = d.size() < out_len - 1 ? d.size() : out_len - 1;
        memcpy(out, d.data(), n);
        out[n] = 0;
    }
    return SAGE_OK;
}

sage_status sage_session_stats(sage_session *s, uint64_t *programs_compiled) {
    *programs_compiled = s->impl->programs_compiled;
    return SAGE_OK;
}
sage_status sage_session_programs_cached(sage_session *s, uint64_t *count, uint64_t *limit) {
    if (count) *count = s->impl->programs_cached();
    if (limit) *limit = Session::kMaxPrograms;
    return SAGE_OK;
}
sage_status sage_session_drop_programs(sage_session *s) {
    s->impl->drop_programs();
    return SAGE_OK;
}

// ---------------------------------------------------------------- ops
#define OP(body) return guarded([&]() -> sage_status { return ret(out, body); })

sage_status sage_op_scalar_f32(float value, int32_t ndim, const int64_t *extents, sage_var **out) { OP(ops::scalar_f(value, arr(ndim, extents))); }
sage_status sage_op_scalar_i32(int32_t value, int32_t ndim, const int64_t *extents, sage_var **out) { OP(ops::scalar_i(value, arr(ndim, extents))); }
sage_status sage_op_unary(int32_t kind, const sage_var *x, sage_var **out) {
    if (kind < 0 || kind >= ops::kNumUnary) return SAGE_ERR_INVALID;
    OP(ops::unary_map(x->v, (ops::Unary)kind));
}
sage_status sage_op_binary(int32_t kind, const sage_var *a, const sage_var *b, sage_var **out) {
    if (kind < 0 || kind >= ops::kNumBinary) return SAGE_ERR_INVALID;
    OP(ops::binary_map(a->v, b->v, (ops::Binary)kind));
}
sage_status sage_op_cond(const sage_var *c, const sage_var *a, const sage_var *b, sage_var **out) { OP(ops::cond(c->v, a->v, b->v)); }

sage_status sage_op_view(const sage_var *x, int32_t ndim, const int64_t *extents, sage_var **out) { OP(ops::view(x->v, arr(ndim, extents))); }
sage_status sage_op_expand(const sage_var *x, int32_t ndim, const int64_t *extents, sage_var **out) { OP(ops::expand(x->v, arr(ndim, extents))); }
sage_status sage_op_permute(const sage_var *x, int32_t n, const int64_t *axes, sage_var **out) { OP(ops::permute(x->v, axes_of(n, axes))); }
sage_status sage_op_transpose(const sage_var *x, int64_t a1, int64_t a2, sage_var **out) { OP(ops::transpose(x->v, a1, a2)); }
sage_status sage_op_squeeze(const sage_var *x, int64_t axis, sage_var **out) { OP(ops::squeeze(x->v, axis)); }
sage_status sage_op_unsqueeze(const sage_var *x, int64_t axis, sage_var **out) { OP(ops::unsqueeze(x->v, axis)); }
sage_status sage_op_slice(const sage_var *x, int64_t axis, int64_t start, int64_t end, sage_var **out) { OP(ops::slice(x->v, axis, start, end)); }
sage_status sage_op_unslice(const sage_var *x, int64_t axis, int64_t start, int64_t end, sage_var **out) { OP(ops::unslice(x->v, axis, start, end)); }
sage_status sage_op_gather(const sage_var *x, const sage_var *ind, int64_t axis, sage_var **out) { OP(ops::gather(x->v, ind->v, axis)); }
sage_status sage_op_scatter(const sage_var *x, const sage_var *ind, int64_t axis, int32_t ndim, const int64_t *extents, sage_var **out) {
    OP(ops::scatter(x->v, ind->v, axis, arr(ndim, extents)));
}
sage_status sage_op_concat(sage_var *const *xs, int32_t n, int64_t axis, sage_var **out) {
    std::vector<Var> v;
    for (int i = 0; i < n; ++i) v.push_back(xs[i]->v);
    OP(ops::concat(v, axis));
}
sage_status sage_op_copy_organize(const sage_var *x, sage_var **out) { OP(x->v.organize()); }

sage_status sage_op_reduce(int32_t kind, const sage_var *x, int32_t naxes, const int64_t *axes, int32_t preserve, sage_var **out) {
    if (kind < 0 || kind > 3) return SAGE_ERR_INVALID;
    OP(ops::reduce(x->v, axes_of(naxes, axes), preserve != 0, (ops::Red)kind));
}
sage_status sage_op_mean(const sage_var *x, int32_t naxes, const int64_t *axes, int32_t preserve, sage_var **out) { OP(ops::mean(x->v, axes_of(naxes, axes), preserve != 0)); }
sage_status sage_op_var(const sage_var *x, int32_t naxes, const int64_t *axes, int32_t preserve, sage_var **out) { OP(ops::var(x->v, axes_of(naxes, axes), preserve != 0)); }
sage_status sage_op_reduce_arg(int32_t is_max, const sage_var *x, int64_t axis, int32_t preserve, sage_var **out) { OP(ops::reduce_arg(x->v, axis, preserve != 0, is_max != 0)); }

sage_status sage_op_gemm(const sage_var *a, const sage_var *b, int32_t ta, int32_t tb, sage_var **out) { OP(ops::gemm(a->v, b->v, ta != 0, tb != 0)); }
sage_status sage_op_gemm_batched(const sage_var *a, const sage_var *b, int32_t ta, int32_t tb, sage_var **out) { OP(ops::gemm_batched(a->v, b->v, ta != 0, tb != 0)); }
sage_status sage_op_matmul(const sage_var *a, const sage_var *b, sage_var **out) { OP(ops::matmul(a->v, b->v)); }
sage_status sage_op_matmul_batched(const sage_var *a, const sage_var *b, sage_var **out) { OP(ops::matmul_batched(a->v, b->v)); }

sage_status sage_op_im2col(const sage_var *x, const sage_window *w, sage_var **out) { OP(ops::im2col(x->v, pr(w->ker), pr(w->stride), pr(w->pad), pr(w->dil))); }
sage_status sage_op_col2im(const sage_var *x, int64_t img_w, int64_t img_h, const sage_window *w, sage_var **out) {
    OP(ops::col2im(x->v, ops::Pair{img_w, img_h}, pr(w->ker), pr(w->stride), pr(w->pad), pr(w->dil)));
}
sage_status sage_op_conv_2d(const sage_var *x, const sage_var *filter, const sage_window *w, sage_var **out) {
    OP(ops::conv_2d(x->v, filter->v, pr(w->stride), pr(w->pad), pr(w->dil)));
}
sage_status sage_op_pool_2d(int32_t is_max, const sage_var *x, const sage_window *w, sage_var **out) {
    OP(is_max ? ops::max_pool_2d(x->v, pr(w->ker), pr(w->stride), pr(w->pad), pr(w->dil))
              : ops::avg_pool_2d(x->v, pr(w->ker), pr(w->stride), pr(w->pad), pr(w->dil)));
}
sage_status sage_op_batch_norm_2d(const sage_var *x, const sage_var *gamma, const sage_var *beta, const sage_var *mean, const sage_var *var,
                                  float eps, sage_var **out) {
    OP(ops::batch_norm_2d(x->v, gamma->v, beta->v, mean->v, var->v, eps));
}

sage_status sage_op_relu(const sage_var *x, sage_var **out) { OP(ops::relu(x->v)); }
sage_status sage_op_softmax(const sage_var *x, int32_t naxes, const int64_t *axes, sage_var **out) { OP(ops::softmax(x->v, axes_of(naxes, axes))); }
sage_status sage_op_log_sum_exp(const sage_var *x, int32_t naxes, const int64_t *axes, sage_var **out) { OP(ops::log_sum_exp(x->v, axes_of(naxes, axes))); }
sage_status sage_op_softmax_cross_entropy(const sage_var *x, const sage_var *labels, sage_var **out) { OP(ops::softmax_cross_entropy(x->v, labels->v)); }
sage_status sage_op_layer_norm(const sage_var *x, int32_t naxes, const int64_t *axes, const sage_var *gamma, const sage_var *beta, float eps,
                               sage_var **out) {
    OP(ops::layer_norm(x->v, axes_of(naxes, axes), gamma->v, beta->v, eps));
}

sage_status sage_op_uniform(int32_t ndim, const int64_t *extents, uint32_t seed_x, uint32_t seed_y, sage_var **out) {
    OP(ops::uniform(arr(ndim, extents), seed_x, seed_y));
}
sage_status sage_op_normal(int32_t ndim, const int64_t *extents, uint32_t seed_x, uint32_t seed_y, sage_var **out) {
    OP(ops::normal(arr(ndim, extents), seed_x, seed_y));
}
sage_status sage_op_accuracy(const sage_var *logits, const sage_var *labels, sage_var **out) { OP(ops::accuracy(logits->v, labels->v)); }

// conv_2d over caller-owned buffers (declared in sage_cuda.h; lives here because the lowering to an implicit
// GEMM is part of the graph evaluator).  The operands are wrapped as tensors that do not own their memory.
static Tensor borrow(sage_ctx *ctx, const sage_tensor *t) {
    Tensor out;
    Array e(t->extents, t->extents + t->ndim), st(t->strides, t->strides + t->ndim);
    out.desc = TensorDesc(Shape(e, st, t->offset), t->dtype);
    auto s = std::make_shared<Storage>();
    s->ctx = ctx->impl;
    s->dev = t->buf->ptr;
    s->bytes = t->buf->size;
    out.data = s;  // no allocator, no block: nothing is freed when the handle drops
    return out;
}

sage_status sage_conv2d_nhwc(sage_ctx *ctx, const sage_tensor *x, const sage_tensor *filter, const sage_window *w, const sage_tensor *y) {
    if (!ctx || !ctx->impl || !x || !filter || !w || !y || !x->buf || !filter->buf || !y->buf) return SAGE_ERR_INVALID;
    Context &C = *ctx->impl;
    sage_status st = guarded([&]() -> sage_status {
        if (x->ndim != 4 || filter->ndim != 4 || y->ndim != 4) shape_fail("conv2d: x, filter and y must have rank 4");
        if (x->dtype != SAGE_F32 || filter->dtype != SAGE_F32 || y->dtype != SAGE_F32) shape_fail("conv2d: f32 only");
        Session session(&C);
        Var xv = Var::from_tensor(borrow(ctx, x)), fv = Var::from_tensor(borrow(ctx, filter));
        Var out = ops::conv_2d(xv, fv, pr(w->stride), pr(w->pad), pr(w->dil));
        Array ye(y->extents, y->extents + 4);
        if (out.extents() != ye) shape_fail("conv2d: y does not have the extents of the result");
        long long run = 1;
        for (int i = 3; i >= 0; --i) {
            if (y->extents[i] != 1 && y->strides[i] != run) shape_fail("conv2d: y must be contiguous");
            run *= y->extents[i];
        }
        sage_status e = session.eval({out});
        if (e) return e;
        Tensor t;
        if (!session.get(out, &t)) return C.fail(SAGE_ERR_INVALID, "internal: conv2d result missing");
        if (C.dry()) return SAGE_OK;
        return C.check_cuda(cudaMemcpyAsync(static_cast<char *>(y->buf->ptr) + y->offset * 4, t.ptr(), (size_t)out.size() * 4, cudaMemcpyDeviceToDevice,
                                            C.stream()),
                            "conv2d result copy");
    });
    if (st == SAGE_ERR_INVALID && !g_error.empty() && C.last_error().empty()) C.fail(st, g_error);
    return st;
}

// ---------------------------------------------------------------- optimizers
sage_status sage_sgd_create(float lr, sage_optimizer **out) {
    *out = new sage_optimizer{std::unique_ptr<nn::Optimizer>(new nn::Sgd(lr))};
    return SAGE_OK;
}
sage_status sage_adam_create(float lr, sage_optimizer **out) {
    *out = new sage_optimizer{std::unique_ptr<nn::Optimizer>(new nn::Adam(lr))};
    return SAGE_OK;
}
sage_status sage_optimizer_set_weight_decay(sage_optimizer *o, float weight_decay) {
    if (auto *a = dynamic_cast<nn::Adam *>(o->impl.get())) a->weight_decay = weight_decay;
    else if (auto *g = dynamic_cast<nn::Sgd *>(o->impl.get())) g->weight_decay = weight_decay;
    return SAGE_OK;
}
sage_status sage_optimizer_destroy(sage_optimizer *o) {
    delete o;
    return SAGE_OK;
}
sage_status sage_optimizer_init(sage_optimizer *o, sage_session *s) {
    return guarded([&]() -> sage_status { return o->impl->init(*s->impl); });
}
sage_status sage_optimizer_update(sage_optimizer *o, sage_session *s, sage_var *const *params, sage_var *const *grads, int32_t n) {
    return guarded([&]() -> sage_status {
        std::vector<Var> p, g;
        for (int i = 0; i < n; ++i) {
            p.push_back(params[i]->v);
            g.push_back(grads[i]->v);
        }
        return o->impl->update(p, g, *s->impl);
    });
}

// ---------------------------------------------------------------- models
void sage_bert_config_base(sage_bert_config *c) {
    c->embed_dim = 768;
    c->num_vocabs = 30522;
    c->max_num_tokens = 512;
    c->hidden_dim = 3072;
    c->num_layers = 12;
    c->num_heads = 12;
    c->num_classes = 2;
    c->gelu = 0;
    c->layer_norm_eps = 1e-05f;
}

sage_status sage_bert_create(const sage_bert_config *c, sage_bert **out) {
    return guarded([&]() -> sage_status {
        nn::BertConfig k;
        k.embed_dim = c->embed_dim;
        k.num_vocabs = c->num_vocabs;
        k.max_num_tokens = c->max_num_tokens;
        k.hidden_dim = c->hidden_dim;
        k.num_layers = c->num_layers;
        k.num_heads = c->num_heads;
        k.num_classes = c->num_classes;
        k.gelu = c->gelu;
        k.layer_norm_eps = c->layer_norm_eps;
        if (k.embed_dim % k.num_heads) shape_fail("embed_dim must be a multiple of num_heads");
        *out = new sage_bert{new nn::Bert(k)};
        return SAGE_OK;
    });
}
sage_status sage_bert_destroy(sage_bert *b) {
    if (b) {
        delete b->impl;
        delete b;
    }
    return SAGE_OK;
}
static sage_status fill_params(const std::vector<Var> &p, sage_var **out, int32_t cap, int32_t *count) {
    *count = (int32_t)p.size();
    for (int i = 0; i < (int)p.size() && i < cap; ++i) out[i] = new sage_var{p[i]};
    return SAGE_OK;
}
sage_status sage_bert_params(sage_bert *b, sage_var **out, int32_t cap, int32_t *count) {
    std::vector<Var> p;
    b->impl->params(&p);
    return fill_params(p, out, cap, count);
}
sage_status sage_bert_pass(sage_bert *b, const sage_var *ids, const sage_var *mask, sage_var **out) { OP(b->impl->pass(ids->v, mask->v)); }

sage_status sage_resnet18_create(int64_t chan_input, int64_t num_classes, sage_model **out) {
    return guarded([&]() -> sage_status {
        *out = new sage_model{nn::resnet18(chan_input, num_classes)};
        return SAGE_OK;
    });
}
sage_status sage_resnet18_bn_create(int64_t chan_input, int64_t num_classes, sage_model **out) {
    return guarded([&]() -> sage_status {
        *out = new sage_model{nn::resnet18(chan_input, num_classes, true)};
        return SAGE_OK;
    });
}
sage_status sage_densenet_create(int64_t chan_input, int64_t num_classes, int64_t depth, int64_t growth_rate, sage_model **out) {
    return guarded([&]() -> sage_status {
        *out = new sage_model{nn::densenet(chan_input, num_classes, depth, growth_rate)};
        return SAGE_OK;
    });
}
sage_status sage_mobilenet_v2_create(int64_t chan_in, int64_t num_classes, sage_model **out) {
    return guarded([&]() -> sage_status {
        *out = new sage_model{nn::mobilenet_v2(chan_in, num_classes)};
        return SAGE_OK;
    });
}
sage_status sage_model_destroy(sage_model *m) {
    delete m;
    return SAGE_OK;
}
sage_status sage_model_params(sage_model *m, sage_var **out, int32_t cap, int32_t *count) {
    std::vector<Var> p;
    m->impl->params(&p);
    return fill_params(p, out, cap, count);
}
sage_status sage_model_buffers(sage_model *m, sage_var **out, int32_t cap, int32_t *count) {
    std::vector<Var> p;
    m->impl->buffers(&p);
    return fill_params(p, out, cap, count);
}
sage_status sage_model_pass(sage_model *m, const sage_var *x, sage_var **out) { OP(m->impl->pass(x->v)); }

}  // extern "C"
