// Host launchers of the hand-written (non-JIT) CUDA kernels.  Pointers are raw device
// addresses with the tensor's element offset already applied; strides are in elements.
#pragma once
#include <cstdint>

#include "../runtime/runtime.h"

namespace sage {
namespace k {

constexpr int kMaxDims = SAGE_MAX_DIMS;

struct Dims {  // extents + strides of a (sub)space, row-major order of traversal
    int ndim = 0;
    long long ext[kMaxDims] = {0};
    long long str[kMaxDims] = {0};
    long long size() const {
        long long p = 1;
        for (int i = 0; i < ndim; ++i) p *= ext[i];
        return p;
    }
};

// reduce.cu — ReduceOperator / ReduceArgOperator (src/ops/reduce.rs:258-325, 372-431)
sage_status reduce(Context &ctx, int dtype, int kind, const void *x, const Dims &outer, const Dims &inner, void *y);
sage_status reduce_arg(Context &ctx, bool is_max, const float *x, const Dims &outer, long long inner_ext,
                       long long inner_str, uint32_t *y);

// rowops.cu — softmax / log_sum_exp / layer_norm over contiguous rows (src/ops/nn.rs:42-100)
// `hi` (optional): also write the tf32 hi / lo planes of y, laid out like y, lo `plane` floats after hi.
sage_status softmax_rows(Context &ctx, const float *x, float *y, long long rows, long long cols, float *hi = nullptr,
                         long long plane = 0);
sage_status lse_rows(Context &ctx, const float *x, float *y, long long rows, long long cols);
sage_status layernorm_rows(Context &ctx, const float *x, float *y, long long rows, long long cols, const float *gamma,
                           int gamma_stride, const float *beta, int beta_stride, float eps, float *hi = nullptr, long long plane = 0);

// index.cu — gather / scatter / strided copy (src/ops/core.rs:571-934)
sage_status gather(Context &ctx, const uint32_t *x, const long long *x_str, const uint32_t *ind, const Dims &ind_dims,
                   int axis, uint32_t *y);
sage_status scatter_add(Context &ctx, const float *x, const long long *x_str, const uint32_t *ind, const Dims &ind_dims,
                        int axis, float *y, const long long *y_str);
// y[translate(g, dims.ext, y_str)] = x[translate(g, dims.ext, dims.str)]
sage_status strided_copy(Context &ctx, const uint32_t *x, const Dims &dims, uint32_t *y, const long long *y_str);

// Uniform::compute / Normal::compute (src/ops/rand.rs:50-140) with the two 32-bit seeds given by the caller.
sage_status rand_fill(Context &ctx, bool normal, float *y, long long n, unsigned seed_x, unsigned seed_y);

// conv.cu — im2col / col2im / direct pooling (src/ops/conv.rs:143-165, 289-498)
struct Window {
    int ker_w, ker_h, stride_w, stride_h, pad_w, pad_h, dil_w, dil_h;
};
sage_status im2col(Context &ctx, const float *img, float *col, long long n, long long img_h, long long img_w,
                   long long chan, long long col_h, long long col_w, const Window &w);
// im2col writing the fp32 column tensor (`col`, row pitch K, may be null) and / or its tf32 planes
// (`hi`, lo `plane` floats further, row pitch `pitch` >= K and a multiple of 4, may be null).
sage_status im2col_planes(Context &ctx, const float *img, long long n, long long img_h, long long img_w, long long chan,
                          long long col_h, long long col_w, const Window &w, float *col, float *hi, long long plane, int pitch);
sage_status col2im(Context &ctx, const float *col, float *img, long long n, long long img_h, long long img_w,
                   long long chan, long long col_h, long long col_w, const Window &w);
// Convolutions with C <= 4: the image as tf32 planes [n, hp, wp, 4] (channels padded to 4, `pad_h` / `pad_w` zero rows /
// columns in front, the rest behind), and the filter [kh, kw, c, oc] as planes [kh * 32, oc] with row ky * 32 + kx * 4 + c.
// plane = 0: write plain fp32 instead of the two planes.
sage_status pack_small_c_image(Context &ctx, const float *img, long long n, long long h, long long w, long long c, long long hp, long long wp,
                               int pad_h, int pad_w, float *hi, long long plane);
sage_status pack_small_c_filter(Context &ctx, const float *filt, int kh, int kw, int c, int oc, float *hi, long long plane);
sage_status pool2d(Context &ctx, bool is_max, const float *img, float *out, long long n, long long img_h,
                   long long img_w, long long chan, long long out_h, long long out_w, const Window &w);

// gemm_simt.cu / gemm_tcgen05.cu — Gemm / GemmBatched (src/ops/gemm.rs:176-250, 338-421)
struct GemmArgs {
    bool ta, tb;
    long long m, n, k;
    const float *a;
    long long lda, stride_a;
    const float *b;
    long long ldb, stride_b;
    float *c;
    long long ldc, stride_c;
    long long batch;
};
// An operand split for 3xTF32: [2 planes (hi, lo)][batches][rows][pitch] floats, rows x cols as the
// operand lies in memory (cols contiguous), pitch = cols rounded up to 4.
struct SplitPlanes {
    Block *block = nullptr;
    float *planes = nullptr;
    int rows = 0, cols = 0, pitch = 0, batches = 0;
};
bool gemm_tc_supported(const GemmArgs &g);
sage_status split_tf32(Context &ctx, const float *src, long long ld, long long batch_stride, int rows, int cols, int batches,
                       SplitPlanes *out);
void free_split(Context &ctx, SplitPlanes *s);
// The same split into caller-provided device memory of split_tf32_bytes(...) bytes; allocates nothing.
size_t split_tf32_bytes(int rows, int cols, int batches);
sage_status split_tf32_into(Context &ctx, const float *src, long long ld, long long batch_stride, int rows, int cols, int batches,
                            float *dst, SplitPlanes *out);
// `a` / `b` are the splits of g.a / g.b (as stored); g.a / g.b themselves are not read.  With `no_split_k` the
// product runs as one pass over K whatever its shape, so neither the allocator nor a second kernel is reached.
sage_status gemm_tcgen05_planes(Context &ctx, const GemmArgs &g, const SplitPlanes &a, const SplitPlanes &b, bool no_split_k = false);

// ---- the general form of the tensor-core GEMM, used by the evaluator's fused GEMM operator.
// A split operand as the tensor core reads it: `rows` x `cols` with cols contiguous, rows `ld` floats
// apart, batch index = b1 * nb0 + b0 at b0 * sb0 + b1 * sb1 floats.  `hi` points at the first
// element of the tf32 high parts; the low parts lie `plane` floats further.  hi must be 16-byte
// aligned and ld, sb0, sb1, plane multiples of 4 (TMA strides are multiples of 16 bytes).
struct TcOperand {
    const float *hi = nullptr;
    long long plane = 0, ld = 0;
    long long rows = 0, cols = 0;
    long long nb0 = 1, nb1 = 1, sb0 = 0, sb1 = 0;
    bool bcast = false;  // one matrix shared by every batch of the GEMM (nb0 = nb1 = 1)
};
bool tc_operand_ok(const TcOperand &o);
// An extra operand of the epilogue expression: element (batch, row, col) of the output reads
// ptr[b0 * s0 + b1 * s1 + row * sr + col * sc] with the output's batch decomposition; sc is 0 or 1.
struct TcAuxArg {
    const float *ptr = nullptr;
    long long s0 = 0, s1 = 0, sr = 0;
    int sc = 0;
};
// Implicit-GEMM convolution: A (one row per output pixel, K over (tap, channel)) is read by im2col-mode
// TMA from the tf32 planes of a contiguous NHWC image; needs C % 32 == 0.
struct TcConv {
    bool on = false;
    const float *hi = nullptr;  // hi plane of the image; lo `plane` floats further
    long long plane = 0;
    long long n = 0, h = 0, w = 0, c = 0, out_h = 0, out_w = 0;
    Window win{};
    // Element strides between pixels, rows and images; 0 = the dense NHWC ones (c, w * c, h * w * c).  A pixel stride
    // below c makes neighbouring pixels overlap (the C <= 4 layout: 32-float windows 4 * stride floats apart).
    long long sw = 0, sh = 0, sn = 0;
    bool raw = false;  // `hi` points at plain fp32 (no lo plane): the kernel splits each tile in shared memory
};
struct TcGemm {
    TcConv conv;             // when conv.on, `a` is ignored
    bool a_kmajor = true, b_kmajor = false;  // is K the contiguous axis of the operand as stored
    long long m = 0, n = 0, k = 0, batch = 1;
    TcOperand a, b;
    float *c = nullptr;      // fp32 result (may be null when only planes are wanted)
    float *c_hi = nullptr;   // hi plane of the result, laid out like c (may be null)
    long long c_plane = 0;   // floats from the hi to the lo plane
    long long ldc = 0, sc0 = 0, sc1 = 0, nbc0 = 1;  // result (batch, row, col) at b0 * sc0 + b1 * sc1 + row * ldc + col
    int naux = 0;
    TcAuxArg aux[3];
    std::string epilogue;    // C expression over x0 (the product) and x1..x3 (aux); empty = x0
    bool row_softmax = false;  // store softmax over each output row of the expression; needs n <= 256 (one tile per row)
    int force_bn = 0;          // tile width chosen by the caller (64 / 128 / 192 / 256); 0 = the launcher's own choice
    bool no_split_k = false;   // never cut K into slices: the launch then needs no scratch from the allocator
};
// Fused attention: O[batch] = softmax_rows(f(Q[batch] K[batch]^T)) V[batch] in one launch (kernels/attn_tc_device.inc).
// Q is lq x d, K is lk x d, V is lk x d per batch, each given as the tensor core reads it: `q` and `k` with rows =
// tokens, cols = head columns when `*_kmajor` (the head columns are contiguous), else stored transposed (rows = head
// columns, cols = tokens); `v` with rows = keys, cols = head columns when NOT `v_kmajor`, else stored transposed.
// `epilogue` is f over x0 (the score) and x1.. (aux, addressed like a GEMM epilogue operand of the lq x lk score
// matrix, batch cut by `nbe0`).  The result goes to o / o_hi exactly like TcGemm's c / c_hi.  d <= 64.
struct TcAttn {
    long long lq = 0, lk = 0, d = 0, batch = 1;
    TcOperand q, k, v;
    bool q_kmajor = true, k_kmajor = true, v_kmajor = false;
    float *o = nullptr, *o_hi = nullptr;
    long long o_plane = 0, ldo = 0, so0 = 0, so1 = 0, nbo0 = 1;
    int naux = 0;
    TcAuxArg aux[3];
    long long nbe0 = 1;
    std::string epilogue;  // empty = x0
};
bool attention_tc_shape_ok(long long lq, long long lk, long long d, long long batch);
sage_status attention_tc_run(Context &ctx, const TcAttn &a);
bool gemm_tc_shape_ok(long long m, long long n, long long k, long long batch);
sage_status gemm_tc_run(Context &ctx, const TcGemm &g);
// How many K slices gemm_tc_run would cut this product into (0 = none).  Only products without an epilogue are
// cut; a caller with an epilogue may ask for the plain product and apply the epilogue to the sum itself.
int gemm_tc_split_plan(Context &ctx, const TcGemm &g);
// hi/lo split of `n` consecutive floats into planes laid out like the source (dst_hi[i], dst_hi[plane + i]).
sage_status split_tf32_flat(Context &ctx, const float *src, long long n, float *dst_hi, long long plane);
// hi/lo split of a strided 4-level view (b1, b0, row, col) into compact planes owned by `out`.
struct SplitView {
    long long nb1 = 1, nb0 = 1, rows = 0, cols = 0;
    long long sb1 = 0, sb0 = 0, ld = 0, col_stride = 1;
};
sage_status split_tf32_view(Context &ctx, const float *src, const SplitView &v, SplitPlanes *out);
// Launches a kernel whose bounded wait runs out (nothing arrives on its barrier): ~1 s, then status bit 0x140.
sage_status bounded_wait_selftest(Context &ctx);
sage_status gemm_simt(Context &ctx, const GemmArgs &g);
// Returns SAGE_ERR_UNSUPPORTED when the shape/alignment cannot go through TMA; the caller
// then uses gemm_simt.
sage_status gemm_tcgen05(Context &ctx, const GemmArgs &g);
sage_status gemm(Context &ctx, const GemmArgs &g);  // picks per ctx.opts().gemm_backend

// optim.cu — Sgd::update / Adam::update (src/optim.rs:42-94, 125-178), many parameters per launch.
// A slot: parameter `p` (n contiguous floats, updated in place), gradient `g`, Adam's moments `m`, `v`
// (updated in place; null for Sgd), and optionally the parameter's whole-storage tf32 planes (`hi`, lo
// `plane` floats further) which receive the split of the new value.  `first` = this parameter's first
// update: Adam stores zero moments then.  `vec` is filled in by the launcher.
constexpr int kOptSlots = 32;
struct OptSlot {
    float *p = nullptr;
    const float *g = nullptr;
    float *m = nullptr, *v = nullptr;
    float *hi = nullptr;
    long long plane = 0, n = 0;
    int first = 0, vec = 0;
};
struct OptSgd {
    float lr = 0.f, weight_decay = 0.f;
};
struct OptAdam {
    float lr = 0.f, beta1 = 0.9f, beta2 = 0.999f, one_minus_beta1 = 0.f, one_minus_beta2 = 0.f, eps = 1e-08f, weight_decay = 0.f;
    float corr1 = 1.f, corr2 = 1.f;  // -(beta1 ^ t) + 1 and -(beta2 ^ t) + 1 for this step's t
};
sage_status sgd_update(Context &ctx, const OptSlot *slots, int count, const OptSgd &k);
sage_status adam_update(Context &ctx, const OptSlot *slots, int count, const OptAdam &k);

}  // namespace k
}  // namespace sage
