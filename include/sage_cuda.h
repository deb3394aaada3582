/*
 * sage_cuda.h — C ABI of the B200 (sm_100a) CUDA backend for sage's hot path.
 *
 * This is the device boundary: it stands where sage's concrete OpenCL layer
 * stands today (there is no Backend trait in the reference; every op's
 * compute() calls Context / Device / Buffer / KernelProgram / Kernel directly).
 * Each entry point below names the reference call it replaces, by file:line
 * inside ingim/sage.  A Rust `backend::cuda` module binds these 1:1 through
 * `extern "C"`; the Python package sage_b200 binds the same symbols via ctypes.
 *
 * Conventions
 *  - every function returns a sage_status; 0 is success; nothing aborts or throws
 *  - sizes are in BYTES unless the name says elements; tensor offsets/strides are
 *    in ELEMENTS (4-byte elements: float / int / uint), like the reference's Shape
 *  - one sage_ctx owns one device, one in-order stream and one allocator and is
 *    single-threaded, like the reference's Context + cl_queue
 *  - all launches are asynchronous on the context's stream; sage_download and
 *    sage_sync are the only blocking calls (Buffer::read is the reference's only
 *    synchronisation point, src/session/device.rs:111-129)
 *  - there is no CPU fallback: without a CUDA device every compute entry point
 *    returns SAGE_ERR_NO_DEVICE
 */
#ifndef SAGE_CUDA_H
#define SAGE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t sage_status;
enum {
    SAGE_OK = 0,
    SAGE_ERR_INVALID = 1,   /* bad argument / shape error (reference: Error::Shape, src/error.rs:5-13) */
    SAGE_ERR_OOM = 2,       /* reference: Error::Memory(OutOfMemory{mem_needed, mem_total}), src/session/memory.rs:45-54 */
    SAGE_ERR_DEVICE = 3,    /* CUDA runtime/driver failure (reference: Error::Device) */
    SAGE_ERR_COMPILE = 4,   /* NVRTC rejected generated source (reference: clBuildProgram failure) */
    SAGE_ERR_NO_DEVICE = 5, /* context has no GPU (planning context) and the call needs one */
    SAGE_ERR_TIMEOUT = 6,   /* a bounded device-side wait ran out; see sage_status_word */
    SAGE_ERR_UNSUPPORTED = 7
};

/* Element types the reference can actually store (all 4 bytes: src/session/device.rs:73-81,
 * src/tensor/data.rs:13-30). */
typedef enum { SAGE_F32 = 0, SAGE_I32 = 1, SAGE_U32 = 2 } sage_dtype;

typedef struct sage_ctx sage_ctx;
typedef struct sage_buf sage_buf;
typedef struct sage_module sage_module;

#define SAGE_MAX_DIMS 8

/* A strided operand: the reference's Tensor = buffer + Shape{extents,strides,offset}
 * (src/tensor.rs:106-110, src/shape.rs:37-43).  Strides/offset in elements; stride 0 = broadcast. */
typedef struct {
    sage_buf *buf;
    int32_t dtype; /* sage_dtype */
    int32_t ndim;
    int64_t extents[SAGE_MAX_DIMS];
    int64_t strides[SAGE_MAX_DIMS];
    int64_t offset;
} sage_tensor;

/* ------------------------------------------------------------------ devices / contexts */

/* Device::get_list / get_first_gpu — src/session/device.rs:26-43 */
sage_status sage_device_count(int32_t *count);
sage_status sage_device_name(int32_t index, char *name, size_t name_len);

typedef struct {
    uint64_t mem_capacity_bytes; /* 0 = 90 % of the device's free memory.  Reference: hard-coded
                                    1000 MiB, src/session/context.rs:49 */
    int32_t use_cache;           /* 1 = caching allocator (default); 0 = the reference's shipped
                                    setting: one device allocation per tensor */
    int32_t ref_compat;          /* 1 (default) = reduce accumulators start at 0 like the reference
                                    (src/ops/reduce.rs:276-285); 0 = true identities */
    int32_t pattern_fusion;      /* 1 (default) = softmax / log_sum_exp / layer_norm / pooling run as
                                    single kernels; 0 = op-by-op like the reference */
    int32_t gemm_backend;        /* 0 = auto (tcgen05 3xTF32 where shapes allow), 1 = SIMT fp32 only */
} sage_ctx_opts;

void sage_ctx_opts_default(sage_ctx_opts *opts);

/* Context::with_device(idx) — src/session/context.rs:43-52 (+ Device::new, device.rs:45-71;
 * Allocator::new, memory.rs:178-182).  device = -1 creates a PLANNING context: graph
 * compilation, code generation (real NVRTC), allocator bookkeeping and launch recording
 * work, nothing is computed, and data movement returns SAGE_ERR_NO_DEVICE. */
sage_status sage_ctx_create(int32_t device, const sage_ctx_opts *opts, sage_ctx **ctx);
sage_status sage_ctx_destroy(sage_ctx *ctx);
sage_status sage_sync(sage_ctx *ctx);
/* Human-readable description of the last failure on this context ("" if none). */
const char *sage_last_error(sage_ctx *ctx);
/* Device-side status word: kernels with bounded waits set bits here instead of trapping.
 * Reads (and clears) it after synchronising the stream. */
sage_status sage_status_word(sage_ctx *ctx, uint32_t *word);
/* Self-test of the bounded waits (no counterpart in the reference, whose kernels never wait on one
 * another): enqueues a kernel that waits, with the tensor-core GEMM's own bounded wait, on a
 * barrier nothing arrives on.  The wait gives up after its limit (about one second), the kernel
 * sets bits 0x140 in the status word and returns normally; the context stays usable. */
sage_status sage_selftest_bounded_wait(sage_ctx *ctx);
/* The context's CUDA stream as an opaque cudaStream_t (for event timing by the caller). */
void *sage_ctx_stream(sage_ctx *ctx);

/* ------------------------------------------------------------------ memory */

/* Context::alloc → Allocator::alloc → Device::alloc_buffer —
 * src/session/context.rs:119-137, memory.rs:200-208,336-363, device.rs:73-89 */
sage_status sage_alloc(sage_ctx *ctx, size_t bytes, sage_buf **buf);
/* Drop for OpenClMemory → Pool::free — src/session/memory.rs:685-692,365-408.
 * Stream-ordered: the block may be handed to the next allocation without a sync. */
sage_status sage_free(sage_ctx *ctx, sage_buf *buf);
/* OutOfMemory{mem_needed, mem_total} of the last SAGE_ERR_OOM — memory.rs:45-54 */
sage_status sage_last_oom(sage_ctx *ctx, uint64_t *needed_bytes, uint64_t *total_bytes);

typedef struct {
    uint64_t capacity; /* Allocator::capacity  — memory.rs:184-186 */
    uint64_t mem_total;/* reserved from the device — memory.rs:188-190 */
    uint64_t mem_used; /* live tensors — memory.rs:196-198 */
    uint64_t mem_peak; /* peak reserved — memory.rs:192-194 */
    uint64_t num_device_allocs; /* cudaMalloc calls so far (new: shows the cache working) */
} sage_mem_stats_t;
sage_status sage_mem_stats(sage_ctx *ctx, sage_mem_stats_t *stats);
/* Pool::release_cached_blocks — memory.rs:454-474: return every fully-free segment to the device. */
sage_status sage_release_cached(sage_ctx *ctx);
/* Pool::garbage_collect — memory.rs:410-452: when 80 % of the capacity is in use, whole cached segments go
 * back to the device, oldest first (age = searches of the pool a block sat through), until 20 % of the
 * capacity is reclaimed.  Runs by itself inside sage_alloc when no cached block fits; this entry point runs
 * it on demand.  `reclaimed` = bytes freed by this call; `runs_total` / `reclaimed_total` = since creation. */
sage_status sage_garbage_collect(sage_ctx *ctx, uint64_t *reclaimed, uint64_t *runs_total, uint64_t *reclaimed_total);

/* Buffer::write / Buffer::read (blocking) — src/session/device.rs:111-147 */
sage_status sage_upload(sage_ctx *ctx, sage_buf *dst, size_t dst_offset, const void *src, size_t bytes);
sage_status sage_download(sage_ctx *ctx, const sage_buf *src, size_t src_offset, void *dst, size_t bytes);
/* Asynchronous upload from (ideally pinned) host memory; ordered on the context's stream. */
sage_status sage_upload_async(sage_ctx *ctx, sage_buf *dst, size_t dst_offset, const void *src, size_t bytes);
/* Buffer::fill — src/session/device.rs:149-164 (Tensor::fill_zero, tensor.rs:212-223) */
sage_status sage_memset(sage_ctx *ctx, sage_buf *buf, size_t offset, int32_t byte_value, size_t bytes);
/* Raw device address of a buffer (for interop and for the multi-GPU gather). */
void *sage_buf_ptr(const sage_buf *buf);
size_t sage_buf_size(const sage_buf *buf);
/* Pinned host staging memory for the end-to-end path (no reference counterpart: OpenCL
 * enqueue_write_buffer stages internally). */
sage_status sage_host_alloc(size_t bytes, void **ptr);
sage_status sage_host_free(void *ptr);

/* ------------------------------------------------------------------ JIT modules + launch */

/* Context::get_program(src) / CachedAccess::load_program → KernelProgram::new —
 * src/session/context.rs:62-90,158-180, device.rs:201-213.  Cached by source text. */
sage_status sage_module_get(sage_ctx *ctx, const char *cuda_src, sage_module **module);

typedef enum { SAGE_ARG_BUF = 0, SAGE_ARG_I32 = 1, SAGE_ARG_U32 = 2, SAGE_ARG_F32 = 3, SAGE_ARG_I64 = 4, SAGE_ARG_BYTES = 5 } sage_arg_kind;
typedef struct {
    int32_t kind;
    sage_buf *buf;     /* SAGE_ARG_BUF: passed as the buffer's base device pointer */
    int64_t i;         /* I32 / U32 / I64 */
    float f;           /* F32 */
    const void *bytes; /* SAGE_ARG_BYTES: by-value struct parameter */
    size_t nbytes;
} sage_arg;

/* KernelProgram::kernel(name) + Kernel::{arg_tensor,arg,global_work_size,local_work_size,launch}
 * — src/session/device.rs:215-318.  Asynchronous. */
sage_status sage_launch(sage_ctx *ctx, sage_module *module, const char *kernel_name,
                        const uint32_t grid[3], const uint32_t block[3], uint32_t smem_bytes,
                        const sage_arg *args, int32_t nargs);

/* ------------------------------------------------------------------ op-level entry points
 * NaryOperator::compute / VariadicOperator::compute — src/ops.rs:79-101.  `y` must be a
 * contiguous tensor the caller allocated (every compute() in the reference returns a fresh
 * contiguous tensor). */

/* Map kernels: {Nullary,Unary,Binary,Ternary,Variadic}MapOperator::compute —
 * src/ops/map.rs:898-921,970-998,1044-1078,1101-1120,1141-1175.  `expr` is the element
 * expression in C syntax over x0..x{n-1} (what map_fn() returns, map.rs:224-367), e.g.
 * "((x0 * x1) + (x2 * 3.14f))". */
sage_status sage_map(sage_ctx *ctx, const char *expr, const sage_tensor *x, int32_t nx, const sage_tensor *y);

typedef enum { SAGE_RED_SUM = 0, SAGE_RED_PROD = 1, SAGE_RED_MAX = 2, SAGE_RED_MIN = 3 } sage_reduce_kind;
/* ReduceOperator::compute — src/ops/reduce.rs:258-325 */
sage_status sage_reduce(sage_ctx *ctx, int32_t kind, const sage_tensor *x, const int32_t *axes, int32_t naxes, const sage_tensor *y);
/* ReduceArgOperator::compute — src/ops/reduce.rs:372-431 (is_max: argmax else argmin; y is uint) */
sage_status sage_reduce_arg(sage_ctx *ctx, int32_t is_max, const sage_tensor *x, int32_t axis, const sage_tensor *y);

/* Fused composites over the trailing `inner` elements of each row of a contiguous x:
 * softmax / log_sum_exp — src/ops/nn.rs:42-68; layer_norm — nn.rs:84-100 with
 * mean/var of src/ops/reduce.rs:59-82.  gamma/beta hold 1 element (the reference's
 * LayerNorm, src/layers.rs:563-564) or `inner` elements. */
sage_status sage_softmax(sage_ctx *ctx, const sage_tensor *x, int64_t rows, int64_t inner, const sage_tensor *y);
sage_status sage_log_sum_exp(sage_ctx *ctx, const sage_tensor *x, int64_t rows, int64_t inner, const sage_tensor *y);
sage_status sage_layer_norm(sage_ctx *ctx, const sage_tensor *x, int64_t rows, int64_t inner,
                            const sage_tensor *gamma, const sage_tensor *beta, float eps, const sage_tensor *y);

/* Gather::compute / Scatter::compute / Unslice::compute / Concat::compute —
 * src/ops/core.rs:655-718,764-833,571-610,892-934 */
sage_status sage_gather(sage_ctx *ctx, const sage_tensor *x, const sage_tensor *ind, int32_t axis, const sage_tensor *y);
sage_status sage_scatter(sage_ctx *ctx, const sage_tensor *x, const sage_tensor *ind, int32_t axis, const sage_tensor *y);
sage_status sage_unslice(sage_ctx *ctx, const sage_tensor *x, int32_t axis, int64_t start, const sage_tensor *y);
sage_status sage_concat(sage_ctx *ctx, const sage_tensor *xs, int32_t nx, int32_t axis, const sage_tensor *y);

/* Gemm::compute_direct — src/ops/gemm.rs:176-250 (kernel: src/ops/kernels/matmul_direct.opencl:514-771).
 * Row-major C[M,N] = op(A)·op(B); offsets and leading dimensions in elements. */
sage_status sage_gemm(sage_ctx *ctx, int32_t trans_a, int32_t trans_b, int64_t m, int64_t n, int64_t k,
                      const sage_buf *a, int64_t a_off, int64_t lda,
                      const sage_buf *b, int64_t b_off, int64_t ldb,
                      sage_buf *c, int64_t c_off, int64_t ldc);
/* GemmBatched::compute_direct — src/ops/gemm.rs:338-421 (matmul_direct.opencl:857-927) */
sage_status sage_gemm_strided_batched(sage_ctx *ctx, int32_t trans_a, int32_t trans_b, int64_t m, int64_t n, int64_t k,
                                      const sage_buf *a, int64_t a_off, int64_t lda, int64_t stride_a,
                                      const sage_buf *b, int64_t b_off, int64_t ldb, int64_t stride_b,
                                      sage_buf *c, int64_t c_off, int64_t ldc, int64_t stride_c, int64_t batch);

/* No counterpart in the reference (which allocates a fresh buffer in every compute()).
 * The same tensor-core GEMM as sage_gemm for callers that may not allocate device memory —
 * a host whose HBM was partitioned in advance by another runtime, or a latency-critical loop
 * that must not meet cudaMalloc's device-wide synchronisation.  The hi/lo operand split goes
 * into a fixed 32 MiB array inside the library's device image instead of the context's
 * allocator, and the call performs no cudaMalloc / cudaFree / pool allocation at all.
 * Limits: m >= 64, n >= 32, k >= 32, and 8 bytes x (rows_a x pitch(cols_a) + rows_b x pitch(cols_b))
 * <= 32 MiB (pitch = contiguous extent rounded up to 4); otherwise SAGE_ERR_UNSUPPORTED /
 * SAGE_ERR_INVALID with a message naming the limit.  The first call on a device resolves the
 * array's address; make it before any stream capture.  All calls share the array (it keeps the
 * previous call's contents; every byte a call reads is rewritten by that call first), so calls
 * that overlap on one GPU race and must be serialised by the caller. */
sage_status sage_gemm_noalloc(sage_ctx *ctx, int32_t trans_a, int32_t trans_b, int64_t m, int64_t n, int64_t k,
                              const sage_buf *a, int64_t a_off, int64_t lda,
                              const sage_buf *b, int64_t b_off, int64_t ldb,
                              sage_buf *c, int64_t c_off, int64_t ldc);

typedef struct {
    /* every pair is ordered [w, h] like the reference's SizedExtent<2> arguments
     * (src/ops/conv.rs:83,205-209,359-368) */
    int32_t ker[2], stride[2], pad[2], dil[2];
} sage_window;
/* Im2col::compute — src/ops/conv.rs:289-374.  x [N,H,W,C] contiguous → y [N,OH,OW,KH,KW,C]. */
sage_status sage_im2col(sage_ctx *ctx, const sage_tensor *x, const sage_window *w, const sage_tensor *y);
/* Col2im::compute — src/ops/conv.rs:404-498 */
sage_status sage_col2im(sage_ctx *ctx, const sage_tensor *x, const sage_window *w, const sage_tensor *y);
/* max_pool_2d / avg_pool_2d = im2col + reduce over [KH,KW] — src/ops/conv.rs:143-165, without
 * materialising the column tensor.  is_max: 1 max, 0 mean.  Padded taps count as zeros. */
sage_status sage_pool2d(sage_ctx *ctx, int32_t is_max, const sage_tensor *x, const sage_window *w, const sage_tensor *y);
/* conv_2d — src/ops/conv.rs:61-96: x [N,H,W,C] and filter [KH,KW,C,OC] (any strides) -> y [N,OH,OW,OC]
 * contiguous, OH = (H + 2 pad - dil (KH - 1) - 1) / stride + 1 (:47-59); `w.ker` is ignored (the filter's
 * extents give it).  The reference materialises im2col(x) and calls its GEMM; here the product runs as an
 * implicit GEMM on the tensor cores when C % 32 == 0, otherwise the GEMM builds its column planes on the fly. */
sage_status sage_conv2d_nhwc(sage_ctx *ctx, const sage_tensor *x, const sage_tensor *filter, const sage_window *w, const sage_tensor *y);

/* ------------------------------------------------------------------ multi-GPU (no reference counterpart:
 * the reference has no multi-device code).  Batch shards are independent; the only exchange
 * is a peer copy of the outputs into one GPU's memory over NVLink. */
/* The handle names the device allocation the buffer was carved from; `offset` is the buffer's
 * byte offset inside it (add it to the pointer sage_ipc_open returns). */
sage_status sage_ipc_export(sage_ctx *ctx, sage_buf *buf, uint8_t handle[64], uint64_t *offset);
sage_status sage_ipc_open(sage_ctx *ctx, const uint8_t handle[64], void **peer_ptr);
sage_status sage_ipc_close(sage_ctx *ctx, void *peer_ptr);
/* Asynchronous copy local buffer → peer pointer (+ byte offset) on the context's stream. */
sage_status sage_peer_write(sage_ctx *ctx, void *peer_ptr, size_t peer_offset, const sage_buf *src, size_t src_offset, size_t bytes);
/* Same, from a raw device address of this context's GPU (e.g. the one sage_var_buffer returns). */
sage_status sage_peer_write_ptr(sage_ctx *ctx, void *peer_ptr, size_t peer_offset, const void *src_dev, size_t bytes);

/* ------------------------------------------------------------------ introspection (planning + tests) */
/* Number of kernels / memsets this context has launched (or recorded, on a planning context). */
sage_status sage_launch_count(sage_ctx *ctx, uint64_t *kernels, uint64_t *memsets);
/* Start/stop recording kernel names; sage_trace_get copies a '\n'-separated list. */
sage_status sage_trace_begin(sage_ctx *ctx);
sage_status sage_trace_get(sage_ctx *ctx, char *out, size_t out_len, size_t *needed);
/* Device time per kernel name.  Between begin and end a CUDA event is recorded on the context's
 * stream in front of every launch; end synchronises and copies "name launches total_ms" lines,
 * largest first.  (The reference only has host wall time around asynchronous enqueues,
 * src/session.rs:619,667-676.) */
/* A pair of CUDA events on the context's stream: start records one, stop records the other,
 * waits for it and returns the device time between them in milliseconds. */
sage_status sage_timer_start(sage_ctx *ctx);
sage_status sage_timer_stop(sage_ctx *ctx, float *milliseconds);
sage_status sage_profile_begin(sage_ctx *ctx);
sage_status sage_profile_end(sage_ctx *ctx, char *out, size_t out_len, size_t *needed);

#ifdef __cplusplus
}
#endif
#endif /* SAGE_CUDA_H */
