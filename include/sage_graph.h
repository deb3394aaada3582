/*
 * sage_graph.h — C ABI of the lazy-graph layer that sits on top of sage_cuda.h.
 *
 * In the reference this layer is Rust (src/var.rs, the files under src/ops, src/session.rs,
 * src/layers.rs, the files under src/models) and stays as it is when a `backend::cuda` binds
 * sage_cuda.h.  No Rust toolchain exists where this library is built, so the same
 * layer is restated in C++ and exported here, one entry point per reference
 * function (cited by file:line inside ingim/sage), so that tests and benchmarks
 * can build and evaluate "the same graph" the reference would.
 *
 * Every function returns a sage_status (sage_cuda.h).  Graph construction has no
 * context, so its error text is per-thread: sage_graph_last_error().
 * A sage_var is a handle to a Var (a shared reference to its origin, like Rc<Origin>
 * in src/var.rs:34-42); free each handle with sage_var_free.
 */
#ifndef SAGE_GRAPH_H
#define SAGE_GRAPH_H

#include "sage_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sage_session sage_session; /* Context's evaluated-data cache + program cache */
typedef struct sage_var sage_var;
typedef struct sage_bert sage_bert;
typedef struct sage_model sage_model; /* a Sequential (ResNet) */

const char *sage_graph_last_error(void);

/* Context::new / Context::data / Context::clear — src/session/context.rs:25-52,92-94 */
sage_status sage_session_create(sage_ctx *ctx, sage_session **s);
sage_status sage_session_destroy(sage_session *s);
sage_status sage_session_clear(sage_session *s);

/* Var::new(Tensor::new(..).to_device(ctx)) — src/var.rs:153-164, src/tensor.rs:280-293 */
sage_status sage_var_from_host(sage_session *s, int32_t dtype, int32_t ndim, const int64_t *extents, const void *data, sage_var **out);
/* Var::new(host tensor): uploaded on first use (the reference panics instead, src/session/device.rs:259) */
sage_status sage_var_from_host_lazy(int32_t dtype, int32_t ndim, const int64_t *extents, const void *data, sage_var **out);
/* Var::empty — src/var.rs:166-175 */
sage_status sage_var_empty(int32_t dtype, int32_t ndim, const int64_t *extents, sage_var **out);
/* Var::set(Tensor::new(..).to_device(ctx)) — src/var.rs:370-377.  async != 0: `data` must be pinned
 * host memory that stays valid until the stream reaches the copy; the device buffer is reused
 * when the variable already owns one of the right size. */
sage_status sage_var_set(sage_session *s, sage_var *v, const void *data, int32_t async);
sage_status sage_var_free(sage_var *v);
sage_status sage_var_info(const sage_var *v, int32_t *dtype, int32_t *ndim, int64_t *extents /*[SAGE_MAX_DIMS]*/,
                          int64_t *strides /*[SAGE_MAX_DIMS]*/, int64_t *offset, int32_t *is_op, uint64_t *t_order);

/* Var::eval / Context::eval — src/var.rs:338-352, src/session/context.rs:96-117 */
sage_status sage_eval(sage_session *s, sage_var *const *targets, int32_t n);
/* tensor.to_host() — src/tensor.rs:295-309: contiguous row-major copy of an evaluated (or data)
 * variable; blocks until the stream has finished (the reference's only sync point). */
sage_status sage_var_read(sage_session *s, const sage_var *v, void *dst, size_t bytes);
/* Device address + buffer of an evaluated variable (for the multi-GPU output gather). */
sage_status sage_var_buffer(sage_session *s, const sage_var *v, void **dev_ptr, size_t *bytes);
/* grad(y, xs) — src/var.rs:56-103 */
sage_status sage_grad(const sage_var *y, sage_var *const *xs, int32_t n, sage_var **out);
/* One line per routine of the last compiled program: the fused kernels and what feeds them. */
sage_status sage_session_describe(sage_session *s, char *out, size_t out_len, size_t *needed);
sage_status sage_session_stats(sage_session *s, uint64_t *programs_compiled);
/* Compiled programs are cached per (targets, evaluated inputs), at most `limit` of them, least recently used
 * dropped first; a cached program keeps its graph's tensors alive.  The reference recompiles on every eval
 * (src/session/context.rs:96-117) and keeps nothing, so it has no counterpart for these two. */
sage_status sage_session_programs_cached(sage_session *s, uint64_t *count, uint64_t *limit);
sage_status sage_session_drop_programs(sage_session *s);

/* ---- map ops, src/ops/map.rs.  Kinds follow the reference's enums (UnaryMap :92-130, BinaryMap :151-172). */
enum { SAGE_U_COPY, SAGE_U_ABS, SAGE_U_NEG, SAGE_U_RECIP, SAGE_U_LOG, SAGE_U_EXP, SAGE_U_SQRT, SAGE_U_SQUARE, SAGE_U_ERF,
       SAGE_U_SIGN, SAGE_U_CEIL, SAGE_U_FLOOR, SAGE_U_ROUND, SAGE_U_SIN, SAGE_U_SINH, SAGE_U_COS, SAGE_U_COSH, SAGE_U_TAN,
       SAGE_U_TANH, SAGE_U_ASIN, SAGE_U_ASINH, SAGE_U_ACOS, SAGE_U_ACOSH, SAGE_U_ATAN, SAGE_U_ATANH, SAGE_U_NOT,
       SAGE_U_INT, SAGE_U_FLOAT };
enum { SAGE_B_ADD, SAGE_B_SUB, SAGE_B_DIV, SAGE_B_MUL, SAGE_B_MOD, SAGE_B_POW, SAGE_B_MIN, SAGE_B_MAX, SAGE_B_AND, SAGE_B_OR,
       SAGE_B_EQ, SAGE_B_NE, SAGE_B_GT, SAGE_B_GE, SAGE_B_LT, SAGE_B_LE };
sage_status sage_op_scalar_f32(float value, int32_t ndim, const int64_t *extents, sage_var **out); /* scalar, map.rs:517-531 */
sage_status sage_op_scalar_i32(int32_t value, int32_t ndim, const int64_t *extents, sage_var **out);
sage_status sage_op_unary(int32_t kind, const sage_var *x, sage_var **out);                        /* unary_map, map.rs:458-481 */
sage_status sage_op_binary(int32_t kind, const sage_var *a, const sage_var *b, sage_var **out);    /* binary_map, map.rs:483-513 */
sage_status sage_op_cond(const sage_var *c, const sage_var *a, const sage_var *b, sage_var **out); /* cond, map.rs:861-883 */

/* ---- layout / index ops, src/ops/core.rs */
sage_status sage_op_view(const sage_var *x, int32_t ndim, const int64_t *extents, sage_var **out);     /* :203-211 (-1 = infer) */
sage_status sage_op_expand(const sage_var *x, int32_t ndim, const int64_t *extents, sage_var **out);   /* :263-281 */
sage_status sage_op_permute(const sage_var *x, int32_t n, const int64_t *axes, sage_var **out);        /* :358-377 */
sage_status sage_op_transpose(const sage_var *x, int64_t a1, int64_t a2, sage_var **out);              /* :330-356 */
sage_status sage_op_squeeze(const sage_var *x, int64_t axis, sage_var **out);                          /* :400-419 */
sage_status sage_op_unsqueeze(const sage_var *x, int64_t axis, sage_var **out);                        /* :439-458 */
sage_status sage_op_slice(const sage_var *x, int64_t axis, int64_t start, int64_t end, sage_var **out);   /* :478-500 */
sage_status sage_op_unslice(const sage_var *x, int64_t axis, int64_t start, int64_t end, sage_var **out); /* :525-551 */
sage_status sage_op_gather(const sage_var *x, const sage_var *ind, int64_t axis, sage_var **out);      /* :613-640 */
sage_status sage_op_scatter(const sage_var *x, const sage_var *ind, int64_t axis, int32_t ndim, const int64_t *extents, sage_var **out); /* :721-749 */
sage_status sage_op_concat(sage_var *const *xs, int32_t n, int64_t axis, sage_var **out);              /* :836-876 */
sage_status sage_op_copy_organize(const sage_var *x, sage_var **out);                                  /* Var::organize, var.rs:506-512 */

/* ---- reductions, src/ops/reduce.rs (kind: sage_reduce_kind) */
sage_status sage_op_reduce(int32_t kind, const sage_var *x, int32_t naxes, const int64_t *axes, int32_t preserve, sage_var **out); /* :203-224 */
sage_status sage_op_mean(const sage_var *x, int32_t naxes, const int64_t *axes, int32_t preserve, sage_var **out);  /* :59-71 */
sage_status sage_op_var(const sage_var *x, int32_t naxes, const int64_t *axes, int32_t preserve, sage_var **out);   /* :73-82 */
sage_status sage_op_reduce_arg(int32_t is_max, const sage_var *x, int64_t axis, int32_t preserve, sage_var **out);  /* :327-348 */

/* ---- contractions, src/ops/gemm.rs */
sage_status sage_op_gemm(const sage_var *a, const sage_var *b, int32_t ta, int32_t tb, sage_var **out);          /* :106-140 */
sage_status sage_op_gemm_batched(const sage_var *a, const sage_var *b, int32_t ta, int32_t tb, sage_var **out);  /* :253-290 */
sage_status sage_op_matmul(const sage_var *a, const sage_var *b, sage_var **out);                                /* :30-51 */
sage_status sage_op_matmul_batched(const sage_var *a, const sage_var *b, sage_var **out);                        /* :53-104 */

/* ---- convolution, src/ops/conv.rs (window pairs are [w, h]) */
sage_status sage_op_im2col(const sage_var *x, const sage_window *w, sage_var **out);                              /* :188-226 */
sage_status sage_op_col2im(const sage_var *x, int64_t img_w, int64_t img_h, const sage_window *w, sage_var **out); /* :229-264 */
sage_status sage_op_conv_2d(const sage_var *x, const sage_var *filter, const sage_window *w /* ker ignored */, sage_var **out); /* :61-96 */
sage_status sage_op_pool_2d(int32_t is_max, const sage_var *x, const sage_window *w, sage_var **out);             /* :143-165 */
sage_status sage_op_batch_norm_2d(const sage_var *x, const sage_var *gamma, const sage_var *beta, const sage_var *mean,
                                  const sage_var *var, float eps, sage_var **out);                                /* :167-185 */

/* ---- composites, src/ops/nn.rs */
sage_status sage_op_relu(const sage_var *x, sage_var **out);                                                      /* :33-40 */
sage_status sage_op_softmax(const sage_var *x, int32_t naxes, const int64_t *axes, sage_var **out);               /* :42-56 */
sage_status sage_op_log_sum_exp(const sage_var *x, int32_t naxes, const int64_t *axes, sage_var **out);           /* :58-68 */
sage_status sage_op_softmax_cross_entropy(const sage_var *x, const sage_var *labels, sage_var **out);             /* :70-82 */
sage_status sage_op_layer_norm(const sage_var *x, int32_t naxes, const int64_t *axes, const sage_var *gamma,
                               const sage_var *beta, float eps, sage_var **out);                                  /* :84-100 */

/* ---- random tensors, src/ops/rand.rs:21-140.  The reference takes two 32-bit seeds from the thread's generator at
 * every evaluation; here the caller gives them, so results can be reproduced.  uniform: [0, 1]; normal: Box-Muller. */
sage_status sage_op_uniform(int32_t ndim, const int64_t *extents, uint32_t seed_x, uint32_t seed_y, sage_var **out);
sage_status sage_op_normal(int32_t ndim, const int64_t *extents, uint32_t seed_x, uint32_t seed_y, sage_var **out);

/* ---- metric, src/ops/metric.rs:4-17: share of rows whose argmax(logits, 1) equals the label */
sage_status sage_op_accuracy(const sage_var *logits, const sage_var *labels, sage_var **out);

/* ---- optimizers, src/optim.rs.  One in-place launch updates every parameter (and the optimizer's
 * moments); the arithmetic per element is the reference's, in the reference's order.
 * Sgd::new(lr) — optim.rs:28-40; Adam::new(lr) — optim.rs:112-125 (beta1 0.9, beta2 0.999, eps 1e-08). */
typedef struct sage_optimizer sage_optimizer;
sage_status sage_sgd_create(float lr, sage_optimizer **out);
sage_status sage_adam_create(float lr, sage_optimizer **out);
/* The private fields of the reference's structs (optim.rs:14-26, 97-110); Sgd's momentum stays 0 (with
 * any other value the reference's update panics, optim.rs:68-69, and this one returns SAGE_ERR_UNSUPPORTED). */
sage_status sage_optimizer_set_weight_decay(sage_optimizer *o, float weight_decay);
sage_status sage_optimizer_destroy(sage_optimizer *o);
/* Optimizer::init — optim.rs:9,43-46,128-132: forgets the moments, step count back to 1 */
sage_status sage_optimizer_init(sage_optimizer *o, sage_session *s);
/* Optimizer::update(&grads, ctx) — optim.rs:11,48-93,134-177.  grads[i] = d loss / d params[i]
 * (sage_grad); a gradient that the session has not evaluated yet is evaluated first, like the
 * reference does (with its "inefficient" warning, optim.rs:56-59). */
sage_status sage_optimizer_update(sage_optimizer *o, sage_session *s, sage_var *const *params, sage_var *const *grads, int32_t n);

/* ---- models.  Bert — src/models/bert.rs:57-139; config fields mirror BertConfig (:8-55). */
typedef struct {
    int64_t embed_dim, num_vocabs, max_num_tokens, hidden_dim, num_layers, num_heads, num_classes;
    int32_t gelu;          /* 0 = ReLU feed-forward (the reference) ; 1 = erf-GELU variant */
    float layer_norm_eps;  /* the reference's LayerNorm::pass always uses 1e-05 (src/layers.rs:586-589) */
} sage_bert_config;
void sage_bert_config_base(sage_bert_config *c); /* BertConfig::base, bert.rs:42-54 */
sage_status sage_bert_create(const sage_bert_config *c, sage_bert **out);
sage_status sage_bert_destroy(sage_bert *b);
/* Parameter::params traversal order (bert.rs:90-94,121-125,212-216,325-331).  Fills up to `cap`
 * handles (each to be freed by the caller) and returns the total count. */
sage_status sage_bert_params(sage_bert *b, sage_var **out, int32_t cap, int32_t *count);
sage_status sage_bert_pass(sage_bert *b, const sage_var *token_ids, const sage_var *attn_mask, sage_var **logits); /* bert.rs:72-81 */

/* ResNet::new(ResNetConfig::d18(chan_input, num_classes)) — src/models/resnet.rs:20-28,74-104 */
sage_status sage_resnet18_create(int64_t chan_input, int64_t num_classes, sage_model **out);
/* The same graph with the BatchNorm2d layers the reference has commented out (resnet.rs:80,167,170; layer:
 * src/layers.rs:479-546) put back: inference normalisation by running statistics, eps 1e-05. */
sage_status sage_resnet18_bn_create(int64_t chan_input, int64_t num_classes, sage_model **out);
/* DenseNet::new(DenseNetConfig::d121 / d169 / d201(chan_input, num_classes)) — src/models/densenet.rs:20-107:
 * (depth, growth_rate) = (121, 12), (169, 24), (201, 12) */
sage_status sage_densenet_create(int64_t chan_input, int64_t num_classes, int64_t depth, int64_t growth_rate, sage_model **out);
/* MobileNetV2::new(MobileNetV2Config::new(chan_in, num_classes)) — src/models/mobilenet.rs:27-80 */
sage_status sage_mobilenet_v2_create(int64_t chan_in, int64_t num_classes, sage_model **out);
sage_status sage_model_destroy(sage_model *m);
sage_status sage_model_params(sage_model *m, sage_var **out, int32_t cap, int32_t *count);
/* State that Parameter::params does not list: BatchNorm2d's running_mean / running_var (layers.rs:486-490), in
 * traversal order.  Same calling convention as sage_model_params. */
sage_status sage_model_buffers(sage_model *m, sage_var **out, int32_t cap, int32_t *count);
sage_status sage_model_pass(sage_model *m, const sage_var *x, sage_var **out); /* Layer::pass, resnet.rs:138-142 */

#ifdef __cplusplus
}
#endif
#endif /* SAGE_GRAPH_H */
