// extern "C" surface of include/sage_cuda.h.
#include <cuda_runtime.h>

#include <cstring>

#include "../codegen/map_emit.h"
#include "../kernels/kernels.h"
#include "../runtime/runtime.h"

using namespace sage;

#define CTX_OR_FAIL(c)                    \
    if (!(c) || !(c)->impl) return SAGE_ERR_INVALID; \
    Context &C = *(c)->impl;                         \
    C.make_current()

static void *tensor_ptr(const sage_tensor *t) { return static_cast<char *>(t->buf->ptr) + t->offset * 4; }

static k::Dims tensor_dims(const sage_tensor *t) {
    k::Dims d;
    d.ndim = t->ndim;
    for (int i = 0; i < t->ndim; ++i) {
        d.ext[i] = t->extents[i];
        d.str[i] = t->strides[i];
    }
    return d;
}

static bool contiguous(const sage_tensor *t) {
    long long s = 1;
    for (int i = t->ndim - 1; i >= 0; --i) {
        if (t->extents[i] != 1 && t->strides[i] != s) return false;
        s *= t->extents[i];
    }
    return true;
}

static long long tensor_size(const sage_tensor *t) {
    long long s = 1;
    for (int i = 0; i < t->ndim; ++i) s *= t->extents[i];
    return s;
}

extern "C" {

sage_status sage_device_count(int32_t *count) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    *count = n;
    return SAGE_OK;
}

sage_status sage_device_name(int32_t index, char *name, size_t name_len) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, index) != cudaSuccess) {
        cudaGetLastError();
        return SAGE_ERR_NO_DEVICE;
    }
    strncpy(name, p.name, name_len);
    if (name_len) name[name_len - 1] = 0;
    return SAGE_OK;
}

void sage_ctx_opts_default(sage_ctx_opts *o) {
    o->mem_capacity_bytes = 0;
    o->use_cache = 1;
    o->ref_compat = 1;
    o->pattern_fusion = 1;
    o->gemm_backend = 0;
}

sage_status sage_ctx_create(int32_t device, const sage_ctx_opts *opts, sage_ctx **ctx) {
    sage_ctx_opts o;
    sage_ctx_opts_default(&o);
    if (opts) o = *opts;
    Context *c = nullptr;
    sage_status st = Context::create(device, o, &c);
    if (st) return st;
    *ctx = new sage_ctx{c};
    return SAGE_OK;
}

sage_status sage_ctx_destroy(sage_ctx *ctx) {
    if (!ctx) return SAGE_OK;
    delete ctx->impl;
    delete ctx;
    return SAGE_OK;
}

sage_status sage_sync(sage_ctx *ctx) {
    CTX_OR_FAIL(ctx);
    if (C.dry()) return SAGE_OK;
    return C.check_cuda(cudaStreamSynchronize(C.stream()), "sync");
}

const char *sage_last_error(sage_ctx *ctx) { return (ctx && ctx->impl) ? ctx->impl->last_error().c_str() : "invalid context"; }

sage_status sage_status_word(sage_ctx *ctx, uint32_t *word) {
    CTX_OR_FAIL(ctx);
    *word = 0;
    if (C.dry()) return SAGE_OK;
    sage_status st = C.check_cuda(cudaMemcpyAsync(word, C.status_word_dev, 4, cudaMemcpyDeviceToHost, C.stream()), "status word");
    if (st) return st;
    st = C.check_cuda(cudaStreamSynchronize(C.stream()), "sync");
    if (st) return st;
    if (*word) cudaMemsetAsync(C.status_word_dev, 0, 4, C.stream());
    return SAGE_OK;
}

sage_status sage_selftest_bounded_wait(sage_ctx *ctx) {
    CTX_OR_FAIL(ctx);
    return k::bounded_wait_selftest(C);
}

void *sage_ctx_stream(sage_ctx *ctx) { return (ctx && ctx->impl) ? (void *)ctx->impl->stream() : nullptr; }

// ---------------------------------------------------------------- memory
sage_status sage_alloc(sage_ctx *ctx, size_t bytes, sage_buf **buf) {
    CTX_OR_FAIL(ctx);
    Block *b = C.allocator().alloc(bytes);
    if (!b) return C.fail(SAGE_ERR_OOM, "out of memory");
    *buf = new sage_buf{b, b->ptr, bytes, &C};
    return SAGE_OK;
}

sage_status sage_free(sage_ctx *ctx, sage_buf *buf) {
    CTX_OR_FAIL(ctx);
    if (!buf) return SAGE_OK;
    if (buf->block) C.allocator().free(buf->block);
    delete buf;
    return SAGE_OK;
}

sage_status sage_last_oom(sage_ctx *ctx, uint64_t *needed, uint64_t *total) {
    CTX_OR_FAIL(ctx);
    *needed = C.allocator().oom_needed;
    *total = C.allocator().oom_total;
    return SAGE_OK;
}

sage_status sage_mem_stats(sage_ctx *ctx, sage_mem_stats_t *s) {
    CTX_OR_FAIL(ctx);
    s->capacity = C.allocator().capacity();
    s->mem_total = C.allocator().mem_total();
    s->mem_used = C.allocator().mem_used();
    s->mem_peak = C.allocator().mem_peak();
    s->num_device_allocs = C.allocator().num_device_allocs();
    return SAGE_OK;
}

sage_status sage_release_cached(sage_ctx *ctx) {
    CTX_OR_FAIL(ctx);
    C.allocator().release_cached();
    return SAGE_OK;
}
sage_status sage_garbage_collect(sage_ctx *ctx, uint64_t *reclaimed, uint64_t *runs_total, uint64_t *reclaimed_total) {
    if (!ctx || !ctx->impl) return SAGE_ERR_INVALID;
    Allocator &a = ctx->impl->allocator();
    const uint64_t r = a.garbage_collect();
    if (reclaimed) *reclaimed = r;
    if (runs_total) *runs_total = a.gc_runs;
    if (reclaimed_total) *reclaimed_total = a.gc_reclaimed;
    return SAGE_OK;
}

sage_status sage_upload(sage_ctx *ctx, sage_buf *dst, size_t off, const void *src, size_t bytes) {
    CTX_OR_FAIL(ctx);
    if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "upload on a planning context");
    if (off + bytes > dst->size) return C.fail(SAGE_ERR_INVALID, "upload past the end of the buffer");
    sage_status st = C.check_cuda(cudaMemcpyAsync((char *)dst->ptr + off, src, bytes, cudaMemcpyHostToDevice, C.stream()), "upload");
    if (st) return st;
    return C.check_cuda(cudaStreamSynchronize(C.stream()), "upload sync");
}

sage_status sage_upload_async(sage_ctx *ctx, sage_buf *dst, size_t off, const void *src, size_t bytes) {
    CTX_OR_FAIL(ctx);
    if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "upload on a planning context");
    if (off + bytes > dst->size) return C.fail(SAGE_ERR_INVALID, "upload past the end of the buffer");
    return C.check_cuda(cudaMemcpyAsync((char *)dst->ptr + off, src, bytes, cudaMemcpyHostToDevice, C.stream()), "upload");
}

sage_status sage_download(sage_ctx *ctx, const sage_buf *src, size_t off, void *dst, size_t bytes) {
    CTX_OR_FAIL(ctx);
    if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "download on a planning context");
    if (off + bytes > src->size) return C.fail(SAGE_ERR_INVALID, "download past the end of the buffer");
    sage_status st = C.check_cuda(cudaMemcpyAsync(dst, (const char *)src->ptr + off, bytes, cudaMemcpyDeviceToHost, C.stream()), "download");
    if (st) return st;
    return C.check_cuda(cudaStreamSynchronize(C.stream()), "download sync");
}

sage_status sage_memset(sage_ctx *ctx, sage_buf *buf, size_t off, int32_t value, size_t bytes) {
    CTX_OR_FAIL(ctx);
    if (off + bytes > buf->size) return C.fail(SAGE_ERR_INVALID, "memset past the end of the buffer");
    C.note_memset();
    if (C.dry()) return SAGE_OK;
    return C.check_cuda(cudaMemsetAsync((char *)buf->ptr + off, value, bytes, C.stream()), "memset");
}

void *sage_buf_ptr(const sage_buf *buf) { return buf ? buf->ptr : nullptr; }
size_t sage_buf_size(const sage_buf *buf) { return buf ? buf->size : 0; }

sage_status sage_host_alloc(size_t bytes, void **ptr) {
    if (cudaMallocHost(ptr, bytes) != cudaSuccess) {
        cudaGetLastError();
        return SAGE_ERR_DEVICE;
    }
    return SAGE_OK;
}

sage_status sage_host_free(void *ptr) {
    cudaFreeHost(ptr);
    return SAGE_OK;
}

// ---------------------------------------------------------------- JIT
sage_status sage_module_get(sage_ctx *ctx, const char *src, sage_module **module) {
    CTX_OR_FAIL(ctx);
    Module *m = nullptr;
    sage_status st = C.module_get(src, &m);
    if (st) return st;
    *module = new sage_module{m};  // thin handle; the module itself lives in the context's cache
    return SAGE_OK;
}

sage_status sage_launch(sage_ctx *ctx, sage_module *module, const char *name, const uint32_t grid[3], const uint32_t block[3],
                        uint32_t smem, const sage_arg *args, int32_t nargs) {
    CTX_OR_FAIL(ctx);
    std::vector<void *> ptrs(nargs);
    std::vector<int64_t> store(nargs);
    std::vector<void *> params(nargs);
    for (int i = 0; i < nargs; ++i) {
        switch (args[i].kind) {
        case SAGE_ARG_BUF:
            ptrs[i] = args[i].buf ? args[i].buf->ptr : nullptr;
            params[i] = &ptrs[i];
            break;
        case SAGE_ARG_I32: case SAGE_ARG_U32: {
            int32_t v = (int32_t)args[i].i;
            memcpy(&store[i], &v, 4);
            params[i] = &store[i];
            break;
        }
        case SAGE_ARG_I64:
            store[i] = args[i].i;
            params[i] = &store[i];
            break;
        case SAGE_ARG_F32:
            memcpy(&store[i], &args[i].f, 4);
            params[i] = &store[i];
            break;
        case SAGE_ARG_BYTES:
            params[i] = const_cast<void *>(args[i].bytes);
            break;
        default:
            return C.fail(SAGE_ERR_INVALID, "unknown argument kind");
        }
    }
    return C.launch(module->impl, name, grid, block, smem, params.data());
}

// ---------------------------------------------------------------- op-level entry points
sage_status sage_map(sage_ctx *ctx, const char *expr, const sage_tensor *x, int32_t nx, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (!contiguous(y)) return C.fail(SAGE_ERR_INVALID, "map: output must be contiguous");
    std::vector<MapOperand> in(nx);
    for (int i = 0; i < nx; ++i) {
        if (x[i].ndim != y->ndim) return C.fail(SAGE_ERR_INVALID, "map: operand rank differs from the output's");
        in[i].dtype = x[i].dtype;
        in[i].ptr = tensor_ptr(&x[i]);
        in[i].view = tensor_dims(&x[i]);
    }
    long long ext[SAGE_MAX_DIMS];
    for (int i = 0; i < y->ndim; ++i) ext[i] = y->extents[i];
    return map_launch(C, expr, in, y->dtype, tensor_ptr(y), y->ndim, ext, nullptr);
}

static void split_axes(const sage_tensor *x, const int32_t *axes, int naxes, k::Dims *outer, k::Dims *inner) {
    outer->ndim = inner->ndim = 0;
    for (int a = 0; a < naxes; ++a) {
        inner->ext[inner->ndim] = x->extents[axes[a]];
        inner->str[inner->ndim++] = x->strides[axes[a]];
    }
    for (int i = 0; i < x->ndim; ++i) {
        bool red = false;
        for (int a = 0; a < naxes; ++a) red |= axes[a] == i;
        if (!red) {
            outer->ext[outer->ndim] = x->extents[i];
            outer->str[outer->ndim++] = x->strides[i];
        }
    }
}

sage_status sage_reduce(sage_ctx *ctx, int32_t kind, const sage_tensor *x, const int32_t *axes, int32_t naxes, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (!contiguous(y)) return C.fail(SAGE_ERR_INVALID, "reduce: output must be contiguous");
    k::Dims outer, inner;
    split_axes(x, axes, naxes, &outer, &inner);
    if (outer.size() != tensor_size(y)) return C.fail(SAGE_ERR_INVALID, "reduce: output size does not match the kept axes");
    return k::reduce(C, x->dtype, kind, tensor_ptr(x), outer, inner, tensor_ptr(y));
}

sage_status sage_reduce_arg(sage_ctx *ctx, int32_t is_max, const sage_tensor *x, int32_t axis, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (x->dtype != SAGE_F32) return C.fail(SAGE_ERR_UNSUPPORTED, "reduce_arg: only float input");
    k::Dims outer, inner;
    split_axes(x, &axis, 1, &outer, &inner);
    if (outer.size() != tensor_size(y)) return C.fail(SAGE_ERR_INVALID, "reduce_arg: output size does not match the kept axes");
    return k::reduce_arg(C, is_max != 0, (const float *)tensor_ptr(x), outer, inner.ext[0], inner.str[0], (uint32_t *)tensor_ptr(y));
}

sage_status sage_softmax(sage_ctx *ctx, const sage_tensor *x, int64_t rows, int64_t inner, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (!contiguous(x) || !contiguous(y) || tensor_size(x) != rows * inner) return C.fail(SAGE_ERR_INVALID, "softmax: bad layout");
    return k::softmax_rows(C, (const float *)tensor_ptr(x), (float *)tensor_ptr(y), rows, inner);
}

sage_status sage_log_sum_exp(sage_ctx *ctx, const sage_tensor *x, int64_t rows, int64_t inner, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (!contiguous(x) || !contiguous(y) || tensor_size(x) != rows * inner || tensor_size(y) != rows)
        return C.fail(SAGE_ERR_INVALID, "log_sum_exp: bad layout");
    return k::lse_rows(C, (const float *)tensor_ptr(x), (float *)tensor_ptr(y), rows, inner);
}

sage_status sage_layer_norm(sage_ctx *ctx, const sage_tensor *x, int64_t rows, int64_t inner, const sage_tensor *gamma,
                            const sage_tensor *beta, float eps, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (!contiguous(x) || !contiguous(y) || tensor_size(x) != rows * inner) return C.fail(SAGE_ERR_INVALID, "layer_norm: bad layout");
    const long long gs = tensor_size(gamma), bs = tensor_size(beta);
    if ((gs != 1 && gs != inner) || (bs != 1 && bs != inner)) return C.fail(SAGE_ERR_INVALID, "layer_norm: gamma/beta size");
    return k::layernorm_rows(C, (const float *)tensor_ptr(x), (float *)tensor_ptr(y), rows, inner, (const float *)tensor_ptr(gamma),
                             gs == 1 ? 0 : 1, (const float *)tensor_ptr(beta), bs == 1 ? 0 : 1, eps);
}

sage_status sage_gather(sage_ctx *ctx, const sage_tensor *x, const sage_tensor *ind, int32_t axis, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (x->ndim != ind->ndim || !contiguous(y) || tensor_size(y) != tensor_size(ind)) return C.fail(SAGE_ERR_INVALID, "gather: bad shapes");
    long long xs[SAGE_MAX_DIMS];
    for (int i = 0; i < x->ndim; ++i) xs[i] = x->strides[i];
    return k::gather(C, (const uint32_t *)tensor_ptr(x), xs, (const uint32_t *)tensor_ptr(ind), tensor_dims(ind), axis,
                     (uint32_t *)tensor_ptr(y));
}

sage_status sage_scatter(sage_ctx *ctx, const sage_tensor *x, const sage_tensor *ind, int32_t axis, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (x->ndim != ind->ndim || x->ndim != y->ndim || !contiguous(y) || x->dtype != SAGE_F32)
        return C.fail(SAGE_ERR_INVALID, "scatter: bad shapes");
    C.note_memset();
    if (!C.dry()) {
        sage_status st = C.check_cuda(cudaMemsetAsync(tensor_ptr(y), 0, (size_t)tensor_size(y) * 4, C.stream()), "memset");
        if (st) return st;
    }
    long long xs[SAGE_MAX_DIMS], ys[SAGE_MAX_DIMS];
    for (int i = 0; i < x->ndim; ++i) {
        xs[i] = x->strides[i];
        ys[i] = y->strides[i];
    }
    return k::scatter_add(C, (const float *)tensor_ptr(x), xs, (const uint32_t *)tensor_ptr(ind), tensor_dims(ind), axis,
                          (float *)tensor_ptr(y), ys);
}

sage_status sage_unslice(sage_ctx *ctx, const sage_tensor *x, int32_t axis, int64_t start, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (x->ndim != y->ndim || !contiguous(y)) return C.fail(SAGE_ERR_INVALID, "unslice: bad shapes");
    C.note_memset();
    if (!C.dry()) {
        sage_status st = C.check_cuda(cudaMemsetAsync(tensor_ptr(y), 0, (size_t)tensor_size(y) * 4, C.stream()), "memset");
        if (st) return st;
    }
    long long ys[SAGE_MAX_DIMS];
    for (int i = 0; i < y->ndim; ++i) ys[i] = y->strides[i];
    return k::strided_copy(C, (const uint32_t *)tensor_ptr(x), tensor_dims(x), (uint32_t *)tensor_ptr(y) + start * y->strides[axis], ys);
}

sage_status sage_concat(sage_ctx *ctx, const sage_tensor *xs, int32_t nx, int32_t axis, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (!contiguous(y)) return C.fail(SAGE_ERR_INVALID, "concat: output must be contiguous");
    long long ys[SAGE_MAX_DIMS];
    for (int i = 0; i < y->ndim; ++i) ys[i] = y->strides[i];
    long long at = 0;
    for (int q = 0; q < nx; ++q) {
        sage_status st = k::strided_copy(C, (const uint32_t *)tensor_ptr(&xs[q]), tensor_dims(&xs[q]),
                                         (uint32_t *)tensor_ptr(y) + at * y->strides[axis], ys);
        if (st) return st;
        at += xs[q].extents[axis];
    }
    return SAGE_OK;
}

sage_status sage_gemm(sage_ctx *ctx, int32_t ta, int32_t tb, int64_t m, int64_t n, int64_t kk, const sage_buf *a, int64_t a_off,
                      int64_t lda, const sage_buf *b, int64_t b_off, int64_t ldb, sage_buf *c, int64_t c_off, int64_t ldc) {
    CTX_OR_FAIL(ctx);
    k::GemmArgs g{ta != 0, tb != 0, m, n, kk, (const float *)a->ptr + a_off, lda, 0, (const float *)b->ptr + b_off, ldb, 0,
                  (float *)c->ptr + c_off, ldc, 0, 1};
    return k::gemm(C, g);
}

sage_status sage_gemm_strided_batched(sage_ctx *ctx, int32_t ta, int32_t tb, int64_t m, int64_t n, int64_t kk, const sage_buf *a,
                                      int64_t a_off, int64_t lda, int64_t sa, const sage_buf *b, int64_t b_off, int64_t ldb,
                                      int64_t sb, sage_buf *c, int64_t c_off, int64_t ldc, int64_t sc, int64_t batch) {
    CTX_OR_FAIL(ctx);
    k::GemmArgs g{ta != 0, tb != 0, m, n, kk, (const float *)a->ptr + a_off, lda, sa, (const float *)b->ptr + b_off, ldb, sb,
                  (float *)c->ptr + c_off, ldc, sc, batch};
    return k::gemm(C, g);
}

static k::Window to_window(const sage_window *w) {
    return k::Window{w->ker[0], w->ker[1], w->stride[0], w->stride[1], w->pad[0], w->pad[1], w->dil[0], w->dil[1]};
}

sage_status sage_im2col(sage_ctx *ctx, const sage_tensor *x, const sage_window *w, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (x->ndim != 4 || y->ndim != 6 || !contiguous(x) || !contiguous(y)) return C.fail(SAGE_ERR_INVALID, "im2col: bad layout");
    return k::im2col(C, (const float *)tensor_ptr(x), (float *)tensor_ptr(y), x->extents[0], x->extents[1], x->extents[2],
                     x->extents[3], y->extents[1], y->extents[2], to_window(w));
}

sage_status sage_col2im(sage_ctx *ctx, const sage_tensor *x, const sage_window *w, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (x->ndim != 6 || y->ndim != 4 || !contiguous(x) || !contiguous(y)) return C.fail(SAGE_ERR_INVALID, "col2im: bad layout");
    return k::col2im(C, (const float *)tensor_ptr(x), (float *)tensor_ptr(y), y->extents[0], y->extents[1], y->extents[2],
                     y->extents[3], x->extents[1], x->extents[2], to_window(w));
}

sage_status sage_pool2d(sage_ctx *ctx, int32_t is_max, const sage_tensor *x, const sage_window *w, const sage_tensor *y) {
    CTX_OR_FAIL(ctx);
    if (x->ndim != 4 || y->ndim != 4 || !contiguous(x) || !contiguous(y)) return C.fail(SAGE_ERR_INVALID, "pool2d: bad layout");
    return k::pool2d(C, is_max != 0, (const float *)tensor_ptr(x), (float *)tensor_ptr(y), x->extents[0], x->extents[1],
                     x->extents[2], x->extents[3], y->extents[1], y->extents[2], to_window(w));
}

// ---------------------------------------------------------------- multi-GPU
sage_status sage_ipc_export(sage_ctx *ctx, sage_buf *buf, uint8_t handle[64], uint64_t *offset) {
    CTX_OR_FAIL(ctx);
    if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "ipc on a planning context");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    void *base = buf->block ? buf->block->segment : buf->ptr;
    sage_status st = C.check_cuda(cudaIpcGetMemHandle(&h, base), "cudaIpcGetMemHandle");
    if (st) return st;
    *offset = (uint64_t)((char *)buf->ptr - (char *)base);
    memcpy(handle, &h, 64);
    return SAGE_OK;
}

sage_status sage_ipc_open(sage_ctx *ctx, const uint8_t handle[64], void **peer_ptr) {
    CTX_OR_FAIL(ctx);
    if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "ipc on a planning context");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    return C.check_cuda(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

sage_status sage_ipc_close(sage_ctx *ctx, void *peer_ptr) {
    CTX_OR_FAIL(ctx);
    return C.check_cuda(cudaIpcCloseMemHandle(peer_ptr), "cudaIpcCloseMemHandle");
}

sage_status sage_peer_write_ptr(sage_ctx *ctx, void *peer_ptr, size_t peer_off, const void *src_dev, size_t bytes) {
    CTX_OR_FAIL(ctx);
    if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "peer copy on a planning context");
    return C.check_cuda(cudaMemcpyAsync((char *)peer_ptr + peer_off, src_dev, bytes, cudaMemcpyDeviceToDevice, C.stream()), "peer copy");
}

sage_status sage_peer_write(sage_ctx *ctx, void *peer_ptr, size_t peer_off, const sage_buf *src, size_t src_off, size_t bytes) {
    CTX_OR_FAIL(ctx);
    if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "peer copy on a planning context");
    return C.check_cuda(cudaMemcpyAsync((char *)peer_ptr + peer_off, (const char *)src->ptr + src_off, bytes, cudaMemcpyDeviceToDevice,
                                        C.stream()), "peer copy");
}

// ---------------------------------------------------------------- introspection
sage_status sage_launch_count(sage_ctx *ctx, uint64_t *kernels, uint64_t *memsets) {
    CTX_OR_FAIL(ctx);
    *kernels = C.kernel_launches;
    *memsets = C.memset_launches;
    return SAGE_OK;
}

sage_status sage_trace_begin(sage_ctx *ctx) {
    CTX_OR_FAIL(ctx);
    C.tracing = true;
    C.trace.clear();
    return SAGE_OK;
}

sage_status sage_timer_start(sage_ctx *ctx) {
    CTX_OR_FAIL(ctx);
    if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "timer on a planning context");
    if (!C.timer_events[0]) {
        cudaEvent_t a, b;
        if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return C.fail(SAGE_ERR_DEVICE, "cudaEventCreate");
        C.timer_events[0] = a;
        C.timer_events[1] = b;
    }
    return C.check_cuda(cudaEventRecord((cudaEvent_t)C.timer_events[0], C.stream()), "event record");
}

sage_status sage_timer_stop(sage_ctx *ctx, float *ms) {
    CTX_OR_FAIL(ctx);
    if (C.dry() || !C.timer_events[0]) return C.fail(SAGE_ERR_INVALID, "timer was not started");
    sage_status st = C.check_cuda(cudaEventRecord((cudaEvent_t)C.timer_events[1], C.stream()), "event record");
    if (st) return st;
    st = C.check_cuda(cudaEventSynchronize((cudaEvent_t)C.timer_events[1]), "event sync");
    if (st) return st;
    return C.check_cuda(cudaEventElapsedTime(ms, (cudaEvent_t)C.timer_events[0], (cudaEvent_t)C.timer_events[1]), "event elapsed");
}

sage_status sage_profile_begin(sage_ctx *ctx) {
    CTX_OR_FAIL(ctx);
    C.profile_begin();
    return SAGE_OK;
}

sage_status sage_profile_end(sage_ctx *ctx, char *out, size_t out_len, size_t *needed) {
    CTX_OR_FAIL(ctx);
    static thread_local std::string last;
    if (C.profiling) last = C.profile_end();  // a second call with a larger buffer re-reads the same text
    if (needed) *needed = last.size() + 1;
    if (out && out_len) {
        size_t n = last.size() < out_len - 1 ? last.size() : out_len - 1;
        memcpy(out, last.data(), n);
        out[n] = 0;
    }
    return SAGE_OK;
}

sage_status sage_trace_get(sage_ctx *ctx, char *out, size_t out_len, size_t *needed) {
    CTX_OR_FAIL(ctx);
    if (needed) *needed = C.trace.size() + 1;
    if (out && out_len) {
        size_t n = C.trace.size() < out_len - 1 ? C.trace.size() : out_len - 1;
        memcpy(out, C.trace.data(), n);
        out[n] = 0;
    }
    return SAGE_OK;
}

}  // extern "C"
