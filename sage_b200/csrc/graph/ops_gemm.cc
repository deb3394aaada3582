// Matrix products.  Reference: src/ops/gemm.rs — matmul :30-51, matmul_batched :53-104, gemm
// :106-140, Gemm::compute_direct :176-250, gemm_batched :253-290, GemmBatched::compute_direct
// :338-421.  As in the reference the graph forces operands contiguous with organize() and C is
// row-major [M,N]; the reference zero-fills C before the kernel (gemm.rs:179), which has no effect
// with beta = 0 and is dropped here.
//
// What the evaluator may change when it lowers a routine (session.cc; the graph that grad() sees is
// never touched):
//   * an operand that is an organize() copy of a strided view (head split, transposed keys) is read
//     through the view itself: TMA addresses the view, the copy kernel disappears;
//   * the elementwise map that consumes the product (bias, residual, scale + mask, relu ...) becomes
//     the GEMM's epilogue expression;
//   * a permuted copy of the product (head merge) becomes the GEMM's store pattern;
//   * the product's tf32 hi/lo planes are written by the epilogue when another GEMM reads it next;
//   * gemm(softmax(gemm{f}(Q, K)), V) — the attention block of src/models/bert.rs:250-280 — becomes ONE operator
//     that runs the fused attention kernel: scores and probabilities never exist in memory.
#include <cuda_runtime.h>

#include <cstdlib>

#include "graph.h"

namespace sage {
using namespace ops;

// ------------------------------------------------------------------------------ tf32 planes of a storage
sage_status storage_planes_attach(Context &ctx, Storage &st) {  // allocate only; the caller's kernel fills them
    if (st.split) return SAGE_OK;
    auto c = std::make_shared<SplitCache>();
    c->alloc = ctx.allocator_ptr();
    c->whole = true;
    const size_t bytes = (st.bytes + 511) / 512 * 512;
    c->plane = (long long)(bytes / 4);
    c->planes.block = ctx.allocator().alloc(2 * bytes);
    if (!c->planes.block) return ctx.fail(SAGE_ERR_OOM, "out of memory for tf32 planes");
    c->planes.planes = reinterpret_cast<float *>(c->planes.block->ptr);
    st.split = c;
    return SAGE_OK;
}

static sage_status storage_planes(Context &ctx, Storage &st) {  // planes of existing data: run the split pass
    if (st.split) return SAGE_OK;
    sage_status s = storage_planes_attach(ctx, st);
    if (s) return s;
    s = k::split_tf32_flat(ctx, (const float *)st.dev, (long long)(st.bytes / 4), st.split->planes.planes, st.split->plane);
    if (s) st.split.reset();
    return s;
}

// ------------------------------------------------------------------------------ operand views
// A GEMM operand is a tensor view of rank >= 2: the last two axes are the matrix, the axes before
// them the batch.  `levels` collapses the batch axes into at most two (extent, stride) pairs,
// innermost first; false when that is not possible.
struct BatchLevels {
    long long n[2] = {1, 1}, s[2] = {0, 0};
};
static bool collapse_batch(const Shape &sh, int nbatch_axes, BatchLevels *out) {
    std::vector<std::pair<long long, long long>> lv;  // outermost first
    for (int i = 0; i < nbatch_axes; ++i) {
        const long long e = sh.extents[i], s = sh.strides[i];
        if (e == 1) continue;
        if (!lv.empty() && lv.back().second == s * e) lv.back() = {lv.back().first * e, s};
        else lv.push_back({e, s});
    }
    if (lv.size() > 2) return false;
    *out = BatchLevels();
    if (lv.size() == 1) {
        out->n[0] = lv[0].first;
        out->s[0] = lv[0].second;
    } else if (lv.size() == 2) {
        out->n[1] = lv[0].first;
        out->s[1] = lv[0].second;
        out->n[0] = lv[1].first;
        out->s[0] = lv[1].second;
    }
    return true;
}

// Can TMA read this view straight from whole-storage planes?  `swapped` = the row axis is the
// contiguous one (the matrix lies transposed in memory).
static bool view_direct(const Shape &sh, bool *swapped, BatchLevels *bl) {
    const int r = sh.rank();
    if (r < 2 || !collapse_batch(sh, r - 2, bl)) return false;
    const long long R = sh.extents[r - 2], C = sh.extents[r - 1], sR = sh.strides[r - 2], sC = sh.strides[r - 1];
    long long ld;
    if (sC == 1 || C == 1) {
        *swapped = false;
        ld = R == 1 ? (C + 3) / 4 * 4 : sR;
    } else if (sR == 1 || R == 1) {
        *swapped = true;
        ld = sC;
    } else {
        return false;
    }
    if (ld <= 0 || ld % 4 || sh.offset % 4) return false;
    for (int l = 0; l < 2; ++l)
        if (bl->n[l] > 1 && (bl->s[l] <= 0 || bl->s[l] % 4)) return false;
    return true;
}

bool gemm_operand_view_ok(const Shape &sh) {
    bool sw;
    BatchLevels bl;
    return view_direct(sh, &sw, &bl);
}

// Fills `op` for tensor `t`; *swapped tells whether the matrix lies transposed in memory.  Keeps the
// planes alive through *hold.
static sage_status make_operand(Context &ctx, const Tensor &t, k::TcOperand *op, bool *swapped, std::shared_ptr<SplitCache> *hold) {
    const Shape &sh = t.desc.shape;
    const int r = sh.rank();
    BatchLevels bl;
    Storage &st = *t.data;
    // A view that covers a small part of a large allocation is gathered instead of splitting it all.
    const bool small_part = !st.split && (unsigned long long)sh.size() * 16 < st.bytes;
    if (view_direct(sh, swapped, &bl) && !small_part) {
        sage_status s = storage_planes(ctx, st);
        if (s) return s;
        *hold = st.split;
        const long long R = sh.extents[r - 2], C = sh.extents[r - 1];
        op->hi = st.split->planes.planes + sh.offset;
        op->plane = st.split->plane;
        op->rows = *swapped ? C : R;
        op->cols = *swapped ? R : C;
        op->ld = *swapped ? sh.strides[r - 1] : (R == 1 ? (C + 3) / 4 * 4 : sh.strides[r - 2]);
        if (op->rows == 1) op->ld = (op->cols + 3) / 4 * 4;
        op->nb0 = bl.n[0];
        op->nb1 = bl.n[1];
        op->sb0 = bl.s[0];
        op->sb1 = bl.s[1];
        return SAGE_OK;
    }
    // Gather the view into compact planes (any strides; one pass instead of organize() + split).
    if (st.planes_only) return ctx.fail(SAGE_ERR_INVALID, "internal: a planes-only tensor reached an operand TMA cannot address");
    if (!collapse_batch(sh, r - 2, &bl)) return ctx.fail(SAGE_ERR_UNSUPPORTED, "gemm: batch axes of an operand do not collapse to two levels");
    *swapped = false;
    std::shared_ptr<SplitCache> &c = st.split_view;
    if (!(c && c->view == sh)) {
        auto fresh = std::make_shared<SplitCache>();
        fresh->alloc = ctx.allocator_ptr();
        fresh->view = sh;
        k::SplitView v;
        v.nb0 = bl.n[0];
        v.nb1 = bl.n[1];
        v.sb0 = bl.s[0];
        v.sb1 = bl.s[1];
        v.rows = sh.extents[r - 2];
        v.cols = sh.extents[r - 1];
        v.ld = sh.strides[r - 2];
        v.col_stride = sh.strides[r - 1];
        sage_status s = k::split_tf32_view(ctx, (const float *)t.ptr(), v, &fresh->planes);
        if (s) return s;
        c = fresh;
    }
    *hold = c;
    const k::SplitPlanes &p = c->planes;
    op->hi = p.planes;
    op->ld = p.pitch;
    op->rows = p.rows;
    op->cols = p.cols;
    op->nb0 = p.batches;
    op->nb1 = 1;
    op->sb0 = (long long)p.rows * p.pitch;
    op->sb1 = 0;
    op->plane = (long long)p.batches * p.rows * p.pitch;
    return SAGE_OK;
}

// ------------------------------------------------------------------------------ the operator
// Axis groups of the epilogue's index space.
enum { GBatchHi = 0, GBatchLo = 1, GRow = 2, GCol = 3 };

// SAGE_CONV_RAW=1 (read at every use; off by default): convolutions read the image as plain fp32 and split every tile
// into its tf32 planes inside the SM (TcConv::raw) instead of reading whole-image planes.  It halves the bytes operand
// A moves from L2 into shared memory, but measured on B200 the four split warps do not keep up with the MMAs:
// 56 x 56 x 64 -> 64 at batch 256: 717 -> 1311 us; 28 x 28 x 128: 388 -> 656 us; the 3-channel first layer 1301 -> 2229 us.
static bool conv_raw_enabled() {
    const char *e = getenv("SAGE_CONV_RAW");
    return e && atoi(e) != 0;
}

struct GemmOp : Operator {
    bool ta = false, tb = false, batched = false;
    // ---- set by the evaluator's lowering; the defaults describe the plain operator
    bool lowered = false;           // operands are views [batch axes..., rows, cols]; m/n/k/batch below are valid
    long long m = 0, n = 0, k = 0, batch = 1;
    std::string epilogue;           // C expression over x0 (the product) and x1.. (inputs 2..)
    Array epi_ext;                  // extents of the epilogue operands (the fused map's index space)
    std::vector<int> epi_group;     // per axis of epi_ext: GBatchHi .. GCol
    bool conv = false;              // operand A is the im2col of input 0 ([N,H,W,C]), made on the fly as tf32 planes
    k::Window win{};
    long long img[6] = {0, 0, 0, 0, 0, 0};  // N, H, W, C, OH, OW
    bool row_softmax = false;       // the stored value is softmax over the last axis of the (epilogue of the) product
    bool folded = false;            // result stored through (ldc, sc0, sc1, nbc0) instead of row-major [batch, M, N]
    long long ldc = 0, sc0 = 0, sc1 = 0, nbc0 = 1;
    // Fused attention: the operator is softmax_rows(f(Q K^T)) V.  in = {Q, V, K, operands of f...}; m = queries,
    // n = head columns, k = keys; ta / tb keep describing the outer product (P V), score_ta / score_tb the inner
    // one (Q K); `epilogue`, `epi_ext` and `epi_group` are f and its index space (that of the score matrix).
    bool attn = false, score_ta = false, score_tb = false;

    const char *name() const override { return attn ? "attention" : batched ? "gemm_batched" : "gemm"; }
    Cat cat() const override { return Cat::Contract; }
    int first_aux() const { return attn ? 3 : 2; }
    int naux() const { return (int)in.size() - first_aux(); }

    std::vector<Var> grad(const std::vector<Var> &x, const Var &, const Var &gy) override {  // gemm.rs:150-163,304-328
        if (lowered) shape_fail("a lowered gemm is not differentiated");
        auto g = [&](const Var &a, const Var &b, bool t1, bool t2) { return batched ? gemm_batched(a, b, t1, t2) : gemm(a, b, t1, t2); };
        if (!ta && !tb) return {g(gy, x[1], false, true), g(x[0], gy, true, false)};
        if (!ta && tb) return {g(gy, x[1], false, false), g(gy, x[0], true, false)};
        if (ta && !tb) return {g(x[1], gy, false, true), g(x[0], gy, false, false)};
        return {g(x[1], gy, true, true), g(gy, x[0], true, true)};
    }

    // Implicit GEMM needs 32-channel K-blocks; images below 128 KiB take the explicit path (im2col-mode
    // tensor maps over very small tensors are avoided).
    // Opt-in: narrow products (at most 128 output channels) read the image as plain fp32 and split it per tile in
    // shared memory.  Wider ones always keep whole-image planes (their kernels have no registers to spare for four more warps).
    bool conv_raw() const { return conv_raw_enabled() && n <= 128; }
    bool conv_implicit() const { return conv && img[3] % 32 == 0 && img[0] * img[1] * img[2] * img[3] * 4 >= 131072; }
    // At most 4 input channels (the first convolution of an image model): the image is re-laid with 4-float pixels so
    // that the taps of a filter row are contiguous, and runs as an implicit GEMM over overlapping 32-float windows
    // (kernels/conv.cu: pack_small_c_*); needs undilated columns, a window at most 8 wide and enough output pixels.
    bool conv_small_c() const {
        return conv && img[3] >= 1 && img[3] <= 4 && win.dil_w == 1 && win.ker_w >= 1 && win.ker_w <= 8 && n % 4 == 0 && img[0] * img[4] * img[5] >= 512;
    }
    struct PackedFilter {  // the filter as the B operand of that GEMM, kept until the filter is rewritten
        const Storage *key = nullptr;
        uint64_t version = 0;
        std::shared_ptr<Allocator> alloc;
        Block *block = nullptr;
        ~PackedFilter() {
            if (alloc && block) alloc->free(block);
        }
    };
    std::shared_ptr<PackedFilter> packed_filter;

    void dims_from_inputs() {  // m, n, k, batch from in[0] / in[1] (last two axes = matrix)
        const Shape &a = in[0].shape, &b = in[1].shape;
        const int ra = a.rank(), rb = b.rank();
        m = ta ? a.extents[ra - 1] : a.extents[ra - 2];
        k = ta ? a.extents[ra - 2] : a.extents[ra - 1];
        n = tb ? b.extents[rb - 2] : b.extents[rb - 1];
        batch = 1;
        for (int i = 0; i < ra - 2; ++i) batch *= a.extents[i];
    }

    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        const bool emit = ctx.hint_emit_planes, only = emit && ctx.hint_planes_only;
        ctx.hint_emit_planes = ctx.hint_planes_only = false;
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        if (!lowered) dims_from_inputs();
        if (attn) return compute_attention(x, ctx, y, emit, only);
        if (!lowered && (ctx.opts().gemm_backend == 1 || !k::gemm_tc_shape_ok(m, n, k, batch))) {
            const int o = batched ? 1 : 0;
            const Shape &a = x[0].desc.shape, &b = x[1].desc.shape;
            k::GemmArgs g;
            g.ta = ta;
            g.tb = tb;
            g.m = m;
            g.k = k;
            g.n = n;
            g.a = (const float *)x[0].ptr();
            g.b = (const float *)x[1].ptr();
            g.c = (float *)y->ptr();
            g.lda = a.strides[o];
            g.ldb = b.strides[o];
            g.ldc = n;
            g.batch = batch;
            g.stride_a = batched ? a.strides[0] : 0;
            g.stride_b = batched ? b.strides[0] : 0;
            g.stride_c = m * n;
            return k::gemm_simt(ctx, g);
        }
        k::TcGemm g;
        g.m = m;
        g.n = n;
        g.k = k;
        g.batch = batch;
        std::shared_ptr<SplitCache> hold_a, hold_b;
        bool sw_a = false, sw_b = false;
        Block *col_block = nullptr;  // conv: the column matrix (or the channel-padded image) exists only as tf32 planes, only for this launch
        bool small_c = false;
        if (conv && (!x[0].desc.shape.has_default_strides() || ta)) return ctx.fail(SAGE_ERR_INVALID, "internal: conv gemm needs a contiguous image");
        if (conv_implicit() && x[0].desc.shape.offset % 4 == 0) {
            // implicit GEMM: im2col-mode TMA reads the image's tf32 planes, nothing is materialised (with SAGE_CONV_RAW=1:
            // the plain fp32 image, split per tile inside the SM)
            g.conv.on = true;
            if (conv_raw() && !x[0].data->planes_only) {
                g.conv.hi = (const float *)x[0].ptr();
                g.conv.plane = 0;
                g.conv.raw = true;
            } else {
                st = storage_planes(ctx, *x[0].data);
                if (st) return st;
                hold_a = x[0].data->split;
                g.conv.hi = hold_a->planes.planes + x[0].desc.shape.offset;
                g.conv.plane = hold_a->plane;
            }
            g.conv.n = img[0];
            g.conv.h = img[1];
            g.conv.w = img[2];
            g.conv.c = img[3];
            g.conv.out_h = img[4];
            g.conv.out_w = img[5];
            g.conv.win = win;
        } else if (conv_small_c() && x[1].desc.shape.has_default_strides()) {
            if (x[0].data->planes_only) return ctx.fail(SAGE_ERR_INVALID, "internal: a planes-only image reached the channel-padding path");
            const long long N = img[0], H = img[1], W = img[2], C = img[3], OH = img[4], OW = img[5];
            // a row holds the left padding, the image, and enough behind it for the last pixel's 32-float window
            const long long wp = std::max(W + 2 * win.pad_w, (OW - 1) * win.stride_w + 8);
            const long long hp = std::max(H + 2 * win.pad_h, (OH - 1) * win.stride_h + (long long)(win.ker_h - 1) * win.dil_h + 1);
            const bool raw = conv_raw();  // plain fp32, split per tile inside the SM
            const long long plane = raw ? 0 : N * hp * wp * 4;
            col_block = ctx.allocator().alloc((size_t)(N * hp * wp * 4) * (raw ? 1 : 2) * sizeof(float));
            if (!col_block) return ctx.fail(SAGE_ERR_OOM, "out of memory for the channel-padded image");
            float *hi = reinterpret_cast<float *>(col_block->ptr);
            st = k::pack_small_c_image(ctx, (const float *)x[0].ptr(), N, H, W, C, hp, wp, win.pad_h, win.pad_w, hi, plane);
            if (st) {
                ctx.allocator().free(col_block);
                return st;
            }
            g.conv.on = true;
            g.conv.hi = hi;
            g.conv.plane = plane;
            g.conv.raw = raw;
            g.conv.n = N;
            g.conv.h = hp;
            g.conv.w = OW;          // window positions along a row, 4 * stride_w floats apart
            g.conv.c = 32;          // a window: the (up to) 8 taps x 4 channels of one filter row
            g.conv.out_h = OH;
            g.conv.out_w = OW;
            g.conv.sw = 4 * win.stride_w;
            g.conv.sh = 4 * wp;
            g.conv.sn = 4 * hp * wp;
            g.conv.win = k::Window{1, win.ker_h, 1, win.stride_h, 0, 0, 1, win.dil_h};
            g.k = (long long)win.ker_h * 32;
            small_c = true;
        } else if (conv) {
            if (x[0].data->planes_only) return ctx.fail(SAGE_ERR_INVALID, "internal: a planes-only image reached the explicit im2col path");
            if (!k::gemm_tc_shape_ok(m, n, k, batch)) return ctx.fail(SAGE_ERR_UNSUPPORTED, "conv_2d: a strided filter with so short a window is not supported");
            const int pitch = (int)((k + 3) / 4 * 4);
            const long long plane = m * pitch;
            col_block = ctx.allocator().alloc((size_t)plane * 2 * sizeof(float));
            if (!col_block) return ctx.fail(SAGE_ERR_OOM, "out of memory for the convolution's column planes");
            float *hi = reinterpret_cast<float *>(col_block->ptr);
            st = k::im2col_planes(ctx, (const float *)x[0].ptr(), img[0], img[1], img[2], img[3], img[4], img[5], win, nullptr, hi, plane, pitch);
            if (st) {
                ctx.allocator().free(col_block);
                return st;
            }
            g.a.hi = hi;
            g.a.plane = plane;
            g.a.ld = pitch;
            g.a.rows = m;
            g.a.cols = k;
        } else {
            st = make_operand(ctx, x[0], &g.a, &sw_a, &hold_a);
            if (st) return st;
        }
        struct FreeCol {  // stream-ordered: the block may be reused by launches enqueued after the GEMM
            Context &c;
            Block *b;
            ~FreeCol() {
                if (b) c.allocator().free(b);
            }
        } free_col{ctx, col_block};
        if (small_c) {
            const Storage *key = x[1].data.get();
            if (!packed_filter || packed_filter->key != key || packed_filter->version != key->version) {
                auto pf = std::make_shared<PackedFilter>();
                pf->alloc = ctx.allocator_ptr();
                pf->key = key;
                pf->version = key->version;
                const long long fplane = (long long)win.ker_h * 32 * n;
                pf->block = ctx.allocator().alloc((size_t)fplane * 2 * sizeof(float));
                if (!pf->block) return ctx.fail(SAGE_ERR_OOM, "out of memory for the re-laid filter");
                st = k::pack_small_c_filter(ctx, (const float *)x[1].ptr(), win.ker_h, win.ker_w, (int)img[3], (int)n, reinterpret_cast<float *>(pf->block->ptr), fplane);
                if (st) return st;
                packed_filter = pf;
            }
            g.b.hi = reinterpret_cast<const float *>(packed_filter->block->ptr);
            g.b.plane = (long long)win.ker_h * 32 * n;
            g.b.ld = n;
            g.b.rows = (long long)win.ker_h * 32;
            g.b.cols = n;
            if (tb) return ctx.fail(SAGE_ERR_INVALID, "internal: a convolution's filter operand is not transposed");
        } else {
            st = make_operand(ctx, x[1], &g.b, &sw_b, &hold_b);
            if (st) return st;
        }
        // A lies as [M,K] (K contiguous) unless transposed; B as [K,N] (N contiguous) unless transposed.
        g.a_kmajor = (!ta) != sw_a;
        g.b_kmajor = tb != sw_b;
        if (g.a.nb0 * g.a.nb1 != batch || g.b.nb0 * g.b.nb1 != batch) {
            // a batch of one on one side (or levels merged differently) still addresses every batch
            if (g.a.nb0 * g.a.nb1 != batch || g.b.nb0 * g.b.nb1 != batch)
                return ctx.fail(SAGE_ERR_INVALID, "gemm: operand batch extents differ from the operator's");
        }
        g.c = (float *)y->ptr();
        if (folded) {
            g.ldc = ldc;
            g.sc0 = sc0;
            g.sc1 = sc1;
            g.nbc0 = nbc0;
        } else {
            g.ldc = n;
            g.sc0 = m * n;
            g.sc1 = 0;
            g.nbc0 = batch;
        }
        if (emit) {
            st = storage_planes_attach(ctx, *y->data);
            if (st) return st;
            g.c_hi = y->data->split->planes.planes + y->desc.shape.offset;
            g.c_plane = y->data->split->plane;
            if (only) {
                g.c = nullptr;
                y->data->planes_only = true;
            }
        }
        g.naux = naux();
        g.epilogue = epilogue;
        g.row_softmax = row_softmax;
        // the epilogue's batch decomposition: the axes of epi_ext tagged batch low / high
        long long e_nb0 = batch;
        if (g.naux > 0) {
            e_nb0 = 1;
            bool any_hi = false;
            for (size_t d = 0; d < epi_ext.size(); ++d) {
                if (epi_group[d] == GBatchLo) e_nb0 *= epi_ext[d];
                if (epi_group[d] == GBatchHi && epi_ext[d] > 1) any_hi = true;
            }
            if (!any_hi && e_nb0 != batch) return ctx.fail(SAGE_ERR_INVALID, "internal: gemm epilogue batch groups do not cover the batch");
            if (folded && nbc0 != e_nb0 && batch > 1) return ctx.fail(SAGE_ERR_INVALID, "internal: gemm epilogue and store pattern split the batch differently");
            if (!folded) g.nbc0 = e_nb0, g.sc0 = m * n, g.sc1 = m * n * e_nb0;
        }
        for (int i = 0; i < g.naux; ++i) {
            st = aux_strides(ctx, x[2 + i], &g.aux[i]);
            if (st) return st;
        }
        // An epilogue cannot be applied before the K slices of a split product are summed.  Where the cost model
        // wants slices (few output tiles, long K: a convolution of a small feature map at a small batch), the
        // plain product goes to scratch and the epilogue runs as a generated map kernel over the sum.
        if (!g.epilogue.empty() && !g.row_softmax && !g.conv.on && !folded && batch == 1 && g.c && epi_ext == out.shape.extents) {
            k::TcGemm raw = g;
            raw.epilogue.clear();
            raw.naux = 0;
            raw.c_hi = nullptr;
            raw.ldc = n;
            raw.sc0 = m * n;
            raw.sc1 = 0;
            raw.nbc0 = 1;
            if (k::gemm_tc_split_plan(ctx, raw) >= 2) {
                Block *sum = ctx.allocator().alloc((size_t)(m * n) * sizeof(float));
                if (sum) {
                    raw.c = reinterpret_cast<float *>(sum->ptr);
                    st = k::gemm_tc_run(ctx, raw);
                    if (!st) {
                        std::vector<MapOperand> operands(1 + (size_t)g.naux);
                        operands[0].dtype = SAGE_F32;
                        operands[0].ptr = raw.c;
                        operands[0].view = Tensor().with_shape(Shape(out.shape.extents)).dims();
                        for (int i = 0; i < g.naux; ++i) {
                            operands[1 + i].dtype = x[2 + i].desc.dtype;
                            operands[1 + i].ptr = x[2 + i].ptr();
                            operands[1 + i].view = x[2 + i].dims();
                        }
                        st = map_launch(ctx, epilogue, operands, SAGE_F32, y->ptr(), out.shape.rank(), out.shape.extents.data(), &epi_cache, g.c_hi,
                                        g.c_plane);
                    }
                    ctx.allocator().free(sum);  // stream-ordered
                    return st;
                }
            }
        }
        return k::gemm_tc_run(ctx, g);
    }
    MapCache epi_cache;  // the epilogue as a map kernel, for products that are cut into K slices

    // Strides of an epilogue operand per axis group (batch high, batch low, row, column) and the number of
    // low-batch steps, from the operand's run-time shape.
    sage_status aux_strides(Context &ctx, const Tensor &t, k::TcAuxArg *out) const {
        const Shape &sh = t.desc.shape;
        if (sh.extents != epi_ext) return ctx.fail(SAGE_ERR_INVALID, "internal: gemm epilogue operand extents changed");
        long long gs[4] = {0, 0, 0, 0};
        bool seen[4] = {false, false, false, false};
        for (int d = (int)epi_ext.size() - 1; d >= 0; --d) {  // innermost axis of each group gives its stride
            if (epi_ext[d] == 1) continue;
            const int grp = epi_group[d];
            if (!seen[grp]) {
                seen[grp] = true;
                gs[grp] = sh.strides[d];
            }
        }
        if (!epilogue_operand_ok(sh, epi_ext, epi_group)) return ctx.fail(SAGE_ERR_INVALID, "internal: gemm epilogue operand is not addressable");
        out->ptr = (const float *)t.ptr();
        out->s1 = gs[GBatchHi];
        out->s0 = gs[GBatchLo];
        out->sr = gs[GRow];
        out->sc = (int)gs[GCol];
        return SAGE_OK;
    }

    sage_status compute_attention(const std::vector<Tensor> &x, Context &ctx, Tensor *y, bool emit, bool only) {
        k::TcAttn a;
        a.lq = m;
        a.lk = k;
        a.d = n;
        a.batch = batch;
        std::shared_ptr<SplitCache> hold_q, hold_k, hold_v;
        bool sw_q = false, sw_k = false, sw_v = false;
        sage_status st = make_operand(ctx, x[0], &a.q, &sw_q, &hold_q);
        if (!st) st = make_operand(ctx, x[2], &a.k, &sw_k, &hold_k);
        if (!st) st = make_operand(ctx, x[1], &a.v, &sw_v, &hold_v);
        if (st) return st;
        a.q_kmajor = (!score_ta) != sw_q;  // Q lies as [queries, head columns] unless transposed
        a.k_kmajor = score_tb != sw_k;     // K as operand B of Q K: [head columns, keys] unless transposed
        a.v_kmajor = tb != sw_v;           // V as operand B of P V: [keys, head columns] unless transposed
        if (a.q.nb0 * a.q.nb1 != batch || a.k.nb0 * a.k.nb1 != batch || a.v.nb0 * a.v.nb1 != batch)
            return ctx.fail(SAGE_ERR_INVALID, "attention: operand batch extents differ from the operator's");
        a.o = (float *)y->ptr();
        if (folded) {
            a.ldo = ldc;
            a.so0 = sc0;
            a.so1 = sc1;
            a.nbo0 = nbc0;
        } else {
            a.ldo = n;
            a.so0 = m * n;
            a.so1 = 0;
            a.nbo0 = batch;
        }
        if (emit) {
            st = storage_planes_attach(ctx, *y->data);
            if (st) return st;
            a.o_hi = y->data->split->planes.planes + y->desc.shape.offset;
            a.o_plane = y->data->split->plane;
            if (only) {
                a.o = nullptr;
                y->data->planes_only = true;
            }
        }
        a.naux = naux();
        a.epilogue = epilogue;
        a.nbe0 = batch;
        if (a.naux > 0) {
            a.nbe0 = 1;
            bool any_hi = false;
            for (size_t d = 0; d < epi_ext.size(); ++d) {
                if (epi_group[d] == GBatchLo) a.nbe0 *= epi_ext[d];
                if (epi_group[d] == GBatchHi && epi_ext[d] > 1) any_hi = true;
            }
            if (!any_hi && a.nbe0 != batch) return ctx.fail(SAGE_ERR_INVALID, "internal: attention expression batch groups do not cover the batch");
        }
        for (int i = 0; i < a.naux; ++i) {
            st = aux_strides(ctx, x[3 + i], &a.aux[i]);
            if (st) return st;
        }
        return k::attention_tc_run(ctx, a);
    }

    // Each group's axes must step through the operand like one axis (or not at all), and the
    // column group with stride 0 or 1.
    static bool epilogue_operand_ok(const Shape &sh, const Array &ext, const std::vector<int> &group) {
        for (int grp = 0; grp < 4; ++grp) {
            long long inner_stride = 0, span = 1;
            bool first = true;
            for (int d = (int)ext.size() - 1; d >= 0; --d) {
                if (group[d] != grp || ext[d] == 1) continue;
                if (first) {
                    inner_stride = sh.strides[d];
                    first = false;
                } else if (sh.strides[d] != inner_stride * span) {
                    return false;
                }
                span *= ext[d];
            }
            if (grp == GCol && inner_stride != 0 && inner_stride != 1) return false;
            if (inner_stride < 0) return false;
        }
        return true;
    }
};

// ------------------------------------------------------------------------------ lowering helpers (used by session.cc)
static const GemmOp *as_gemm(const Operator &op) { return dynamic_cast<const GemmOp *>(&op); }

bool gemm_runs_on_tc(const Operator &op, bool tc_enabled) {
    const GemmOp *g = as_gemm(op);
    if (!g || !tc_enabled) return false;
    if (g->lowered) return true;
    GemmOp probe = *g;
    probe.dims_from_inputs();
    return k::gemm_tc_shape_ok(probe.m, probe.n, probe.k, probe.batch);
}

// A GEMM that runs on the tensor cores and has not been given an epilogue or a store pattern yet.
bool gemm_can_fuse(const Operator &op, bool tc_enabled) {
    const GemmOp *g = as_gemm(op);
    return g && g->epilogue.empty() && !g->folded && g->naux() == 0 && gemm_runs_on_tc(op, tc_enabled);
}

static std::shared_ptr<GemmOp> lowered_clone(const GemmOp &g) {
    auto c = std::make_shared<GemmOp>(g);
    if (!c->lowered) {
        c->dims_from_inputs();
        c->lowered = true;
    }
    return c;
}

// Operand `idx` (0 or 1) read through `view` (rank >= 2: batch axes, then the matrix as organize()
// would have copied it) instead of through a contiguous copy.  Null when TMA cannot address it.
std::shared_ptr<Operator> gemm_with_operand_view(const Operator &op, int idx, const TensorDesc &view, bool tc_enabled) {
    const GemmOp *g = as_gemm(op);
    if (!g || idx < 0 || idx > 1 || view.dtype != SAGE_F32 || !gemm_runs_on_tc(op, tc_enabled)) return nullptr;
    if (g->conv && idx == 0) return nullptr;  // input 0 is the image, which im2col reads contiguous
    auto c = lowered_clone(*g);
    const Shape &old = c->in[idx].shape, &sh = view.shape;
    const int r = sh.rank(), ro = old.rank();
    if (r < 2 || sh.extents[r - 2] != old.extents[ro - 2] || sh.extents[r - 1] != old.extents[ro - 1]) return nullptr;
    long long b = 1;
    for (int i = 0; i < r - 2; ++i) b *= sh.extents[i];
    if (b != c->batch || !gemm_operand_view_ok(sh)) return nullptr;
    c->in[idx] = view;
    return c;
}

// Axis groups of `ext` (contiguous in the product's [batch, M, N] order).  False when an axis
// straddles the row / column / batch boundaries.
static bool classify_axes(const Array &ext, const Array &gstride, long long m, long long n, long long batch, std::vector<int> *group) {
    group->assign(ext.size(), GCol);
    long long total = 1;
    int innermost_batch = -1;
    long long innermost_batch_stride = 0;
    for (size_t d = 0; d < ext.size(); ++d) {
        total *= ext[d];
        if (ext[d] == 1) continue;
        const long long s = gstride[d];
        if (s >= m * n) {
            if (s % (m * n)) return false;
            (*group)[d] = GBatchHi;
            if (innermost_batch < 0 || s < innermost_batch_stride) {
                innermost_batch = (int)d;
                innermost_batch_stride = s;
            }
        } else if (s >= n) {
            if (s % n || s * ext[d] > m * n) return false;
            (*group)[d] = GRow;
        } else {
            if (s < 1 || s * ext[d] > n) return false;
            (*group)[d] = GCol;
        }
    }
    if (innermost_batch >= 0) (*group)[innermost_batch] = GBatchLo;
    return total == batch * m * n;
}

// The map `expr` over (product, aux...) becomes the epilogue.  `aux` are the map's other operands
// with the strides they will have at run time; `out` is the map's output.
std::shared_ptr<Operator> gemm_with_epilogue(const Operator &op, const std::string &expr, const std::vector<TensorDesc> &aux,
                                             const TensorDesc &out) {
    const GemmOp *g = as_gemm(op);
    if (!g || aux.size() > 3 || out.dtype != SAGE_F32) return nullptr;
    auto c = lowered_clone(*g);
    const Array &ext = out.shape.extents;
    if (!classify_axes(ext, Shape::default_strides(ext), c->m, c->n, c->batch, &c->epi_group)) return nullptr;
    for (const TensorDesc &a : aux)
        if (a.dtype != SAGE_F32 || a.shape.extents != ext || !GemmOp::epilogue_operand_ok(a.shape, ext, c->epi_group)) return nullptr;
    c->epi_ext = ext;
    c->epilogue = expr;
    c->in.resize(2);
    for (const TensorDesc &a : aux) c->in.push_back(a);
    c->out = out.pristine();
    return c;
}

// A contiguous copy of `view` (a permuted / reshaped view of the product: extents + strides into
// the product's row-major [batch, M, N] result) becomes the store pattern.
std::shared_ptr<Operator> gemm_with_store(const Operator &op, const Shape &view, const TensorDesc &out, bool tc_enabled) {
    const GemmOp *g = as_gemm(op);
    if (!g || g->folded || view.offset != 0 || !gemm_runs_on_tc(op, tc_enabled)) return nullptr;
    auto c = lowered_clone(*g);
    const Array &ext = view.extents;
    const Array dst = Shape::default_strides(ext);
    std::vector<int> group;
    if (!classify_axes(ext, view.strides, c->m, c->n, c->batch, &group)) return nullptr;
    // per group, walking the axes from the smallest product-stride up: both the product strides and
    // the destination strides must chain like one axis
    std::vector<int> order;
    for (size_t d = 0; d < ext.size(); ++d)
        if (ext[d] > 1) order.push_back((int)d);
    std::sort(order.begin(), order.end(), [&](int a, int b) { return view.strides[a] < view.strides[b]; });
    long long expect_src = 1;
    long long gdst[4] = {0, 0, 0, 0}, gspan[4] = {1, 1, 1, 1};
    bool seen[4] = {false, false, false, false};
    for (int d : order) {
        if (view.strides[d] != expect_src) return nullptr;  // the view must enumerate the product exactly once
        expect_src *= ext[d];
        const int grp = group[d];
        if (!seen[grp]) {
            seen[grp] = true;
            gdst[grp] = dst[d];
        } else if (dst[d] != gdst[grp] * gspan[grp]) {
            return nullptr;
        }
        gspan[grp] *= ext[d];
    }
    if (seen[GCol] && gdst[GCol] != 1) return nullptr;
    if (gspan[GCol] != c->n || gspan[GRow] != c->m) return nullptr;
    if (!c->epilogue.empty() && !c->attn) {  // the epilogue operands and the store must cut the batch the same way
        long long e_nb0 = 1;
        for (size_t d = 0; d < c->epi_ext.size(); ++d)
            if (c->epi_group[d] == GBatchLo) e_nb0 *= c->epi_ext[d];
        if (c->batch > 1 && e_nb0 != gspan[GBatchLo]) return nullptr;
    }
    c->folded = true;
    c->ldc = gdst[GRow];
    c->sc0 = gdst[GBatchLo];
    c->sc1 = gdst[GBatchHi];
    c->nbc0 = gspan[GBatchLo];
    c->out = out.pristine();
    return c;
}

// softmax over the last axis of a product whose rows fit one tile (n <= 256): computed by the GEMM's
// epilogue warps before the store, so neither the scores nor a softmax kernel touch memory.
// Opt-in (pattern_fusion bit 1): on the BERT-base step it measured slower than the separate row
// kernel (5700 vs 5910 sequences/s) — the score tiles have only two K-blocks, so the barrier rounds
// and the exponentials of the epilogue are not hidden behind any MMA work.
std::shared_ptr<Operator> gemm_with_row_softmax(const Operator &op, long long rows, long long cols, const TensorDesc &out, bool tc_enabled) {
    const GemmOp *g = as_gemm(op);
    if (!g || g->folded || g->row_softmax || g->conv || !gemm_runs_on_tc(op, tc_enabled)) return nullptr;
    auto c = lowered_clone(*g);
    if (c->n > 256 || cols != c->n || rows != c->batch * c->m || out.dtype != SAGE_F32) return nullptr;
    c->row_softmax = true;
    c->out = out.pristine();
    return c;
}

// gemm(softmax_rows(score), V) where score = gemm{f}(Q, K) on the tensor cores: one fused attention operator.
// `rows` x `cols` is the softmax's row space.  Null when the shapes do not fit the kernel (head columns <= 64,
// softmax over exactly the keys) or an operand is something TMA cannot read.
std::shared_ptr<Operator> gemm_with_attention(const Operator &outer_op, const Operator &score_op, long long rows, long long cols, bool tc_enabled) {
    const GemmOp *o = as_gemm(outer_op), *s = as_gemm(score_op);
    if (!o || !s || !tc_enabled || o->attn || s->attn || o->conv || s->conv || o->folded || s->folded || o->row_softmax || s->row_softmax) return nullptr;
    if (!o->epilogue.empty() || o->naux() != 0 || o->ta || s->naux() > 3) return nullptr;
    if (!gemm_runs_on_tc(outer_op, tc_enabled) || !gemm_runs_on_tc(score_op, tc_enabled)) return nullptr;
    auto c = lowered_clone(*o);
    auto sc = lowered_clone(*s);
    if (c->batch != sc->batch || c->m != sc->m || c->k != sc->n || cols != sc->n || rows != sc->batch * sc->m) return nullptr;
    if (!k::attention_tc_shape_ok(c->m, c->k, c->n, c->batch) || sc->k != c->n) return nullptr;  // queries and values share the head width here
    for (const TensorDesc &d : {sc->in[0], sc->in[1], c->in[1]})
        if (d.dtype != SAGE_F32 || !gemm_operand_view_ok(d.shape)) return nullptr;
    c->attn = true;
    c->score_ta = sc->ta;
    c->score_tb = sc->tb;
    c->epilogue = sc->epilogue;
    c->epi_ext = sc->epi_ext;
    c->epi_group = sc->epi_group;
    const TensorDesc v = c->in[1];
    c->in = {sc->in[0], v, sc->in[1]};
    for (int i = 0; i < sc->naux(); ++i) c->in.push_back(sc->in[2 + i]);
    return c;
}

bool is_attention_op(const Operator &op) {
    const GemmOp *g = as_gemm(op);
    return g && g->attn;
}

bool is_gemm_op(const Operator &op) { return as_gemm(op) != nullptr; }

// gemm(reshape(im2col(x)), W): the column matrix is never stored as fp32 — the GEMM makes its tf32
// planes straight from the image (one pass instead of im2col + split, a third of the traffic).
bool im2col_params(const Operator &op, k::Window *w, long long dims[6]);  // ops_conv.cc
std::shared_ptr<Operator> gemm_with_im2col(const Operator &op, const Operator &im2col_op, bool tc_enabled) {
    const GemmOp *g = as_gemm(op);
    k::Window w;
    long long d[6];
    if (!g || g->ta || g->conv || !tc_enabled || !im2col_params(im2col_op, &w, d)) return nullptr;
    auto c = lowered_clone(*g);
    if (c->batch != 1 || c->m != d[0] * d[4] * d[5] || c->k != (long long)w.ker_h * w.ker_w * d[3]) return nullptr;
    c->conv = true;
    c->win = w;
    for (int i = 0; i < 6; ++i) c->img[i] = d[i];
    // With at most 4 channels the contraction the tensor cores see is KH x 32 long, whatever KH * KW * C is (a 3 x 3
    // window over one channel has K = 9, below what the tiled path takes)
    const bool as_small_c = c->conv_small_c() && !g->tb && k::gemm_tc_shape_ok(c->m, c->n, (long long)w.ker_h * 32, 1);
    if (!as_small_c && !k::gemm_tc_shape_ok(c->m, c->n, c->k, c->batch)) return nullptr;
    c->in[0] = im2col_op.in[0];
    return c;
}

// Will operand `idx` be read straight from whole-storage planes (never through the fp32 buffer)?
bool is_grouped_gemm_op(const Operator &op);
bool gemm_operand_static_direct(const Operator &op, int idx) {
    if (is_grouped_gemm_op(op)) return idx == 0 && gemm_operand_view_ok(op.in[0].shape);
    const GemmOp *g = as_gemm(op);
    if (g && g->conv && idx == 0) return g->conv_implicit() && !g->conv_raw();  // planes only when the kernel does not split the image itself
    return g && idx >= 0 && idx < (g->attn ? 3 : 2) && gemm_operand_view_ok(g->in[idx].shape);
}

std::string describe_gemm(const Operator &op) {
    const GemmOp *g = as_gemm(op);
    if (!g) return "";
    std::string s;
    if (g->attn) return "{" + (g->epilogue.empty() ? std::string("x0") : g->epilogue) + "}" + (g->folded ? "[store]" : "");
    if (g->conv) s += g->conv_implicit() ? "<implicit conv>" : g->conv_small_c() ? "<implicit conv, channels padded to 4>" : "<im2col>";
    if (!g->epilogue.empty()) s += "{" + g->epilogue + "}";
    if (g->row_softmax) s += "|softmax";
    if (g->folded) s += "[store]";
    return s;
}

// ------------------------------------------------------------------------------ grouped GEMM
// Several GEMMs that read the same A (the query / key / value projections of one layer input) run as
// ONE batched launch: batch g multiplies A by weight g and writes slab g of a [G, M, N] result.  A is
// a broadcast operand; the G weights (and biases) are copied once into one allocation so that the
// batch is a constant stride, and copied again only when a weight is rewritten (Storage::version).
// No counterpart in the reference; the evaluator forms groups when it lowers a routine.
struct GroupedGemmOp : Operator {
    int groups = 0;
    bool ta = false, tb = false, has_bias = false;
    long long m = 0, n = 0, k = 0;
    std::string epilogue;  // over x0 (product) and, with has_bias, x1 (the bias row)

    struct Concat {
        std::vector<std::pair<const Storage *, uint64_t>> key;
        std::shared_ptr<Allocator> alloc;
        Block *block = nullptr;
        ~Concat() {
            if (alloc && block) alloc->free(block);
        }
    };
    std::unique_ptr<Concat> weights, biases;

    const char *name() const override { return "gemm_grouped"; }
    Cat cat() const override { return Cat::Contract; }
    std::vector<Var> grad(const std::vector<Var> &, const Var &, const Var &) override {
        shape_fail("a grouped gemm is not differentiated; grad walks the separate gemms");
    }

    static bool same_key(const Concat *c, const std::vector<Tensor> &x, int first, int count) {
        if (!c || (int)c->key.size() != count) return false;
        for (int i = 0; i < count; ++i)
            if (c->key[i].first != x[first + i].data.get() || c->key[i].second != x[first + i].data->version) return false;
        return true;
    }

    sage_status compute(const std::vector<Tensor> &x, Context &ctx, Tensor *y) override {
        const bool emit = ctx.hint_emit_planes, only = emit && ctx.hint_planes_only;
        ctx.hint_emit_planes = ctx.hint_planes_only = false;
        sage_status st = Tensor::uninit(ctx, out, y);
        if (st) return st;
        const long long wsize = k * n;
        // ---- weights: [G] planes of K x N (or N x K), hi plane then lo plane
        if (!same_key(weights.get(), x, 1, groups)) {
            std::unique_ptr<Concat> c(new Concat());
            c->alloc = ctx.allocator_ptr();
            c->block = ctx.allocator().alloc((size_t)groups * wsize * 2 * sizeof(float));
            if (!c->block) return ctx.fail(SAGE_ERR_OOM, "out of memory for the grouped gemm's weights");
            float *hi = reinterpret_cast<float *>(c->block->ptr), *lo = hi + groups * wsize;
            for (int i = 0; i < groups; ++i) {
                const Tensor &w = x[1 + i];
                if (!w.desc.shape.has_default_strides()) return ctx.fail(SAGE_ERR_INVALID, "internal: grouped gemm weight is not contiguous");
                st = storage_planes(ctx, *w.data);
                if (st) return st;
                const SplitCache &sp = *w.data->split;
                const float *src = sp.planes.planes + w.desc.shape.offset;
                if (!ctx.dry()) {
                    st = ctx.check_cuda(cudaMemcpyAsync(hi + i * wsize, src, wsize * 4, cudaMemcpyDeviceToDevice, ctx.stream()), "grouped gemm weights");
                    if (st) return st;
                    st = ctx.check_cuda(cudaMemcpyAsync(lo + i * wsize, src + sp.plane, wsize * 4, cudaMemcpyDeviceToDevice, ctx.stream()), "grouped gemm weights");
                    if (st) return st;
                }
                c->key.push_back({w.data.get(), w.data->version});
            }
            weights = std::move(c);
        }
        if (has_bias && !same_key(biases.get(), x, 1 + groups, groups)) {
            std::unique_ptr<Concat> c(new Concat());
            c->alloc = ctx.allocator_ptr();
            c->block = ctx.allocator().alloc((size_t)groups * n * sizeof(float));
            if (!c->block) return ctx.fail(SAGE_ERR_OOM, "out of memory for the grouped gemm's biases");
            for (int i = 0; i < groups; ++i) {
                const Tensor &b = x[1 + groups + i];  // a broadcast view of a contiguous [N] vector
                if (b.desc.shape.strides.back() != 1) return ctx.fail(SAGE_ERR_INVALID, "internal: grouped gemm bias is not a row vector");
                if (!ctx.dry()) {
                    st = ctx.check_cuda(cudaMemcpyAsync(reinterpret_cast<float *>(c->block->ptr) + i * n, b.ptr(), n * 4, cudaMemcpyDeviceToDevice, ctx.stream()),
                                        "grouped gemm biases");
                    if (st) return st;
                }
                c->key.push_back({b.data.get(), b.data->version});
            }
            biases = std::move(c);
        }
        k::TcGemm g;
        g.m = m;
        g.n = n;
        g.k = k;
        g.batch = groups;
        std::shared_ptr<SplitCache> hold_a;
        bool sw_a = false;
        st = make_operand(ctx, x[0], &g.a, &sw_a, &hold_a);
        if (st) return st;
        if (g.a.nb0 * g.a.nb1 != 1) return ctx.fail(SAGE_ERR_INVALID, "internal: grouped gemm operand has a batch");
        g.a.bcast = true;
        g.a_kmajor = (!ta) != sw_a;
        g.b_kmajor = tb;
        g.b.hi = reinterpret_cast<const float *>(weights->block->ptr);
        g.b.plane = groups * wsize;
        g.b.rows = tb ? n : k;
        g.b.cols = tb ? k : n;
        g.b.ld = g.b.cols;
        g.b.nb0 = groups;
        g.b.sb0 = wsize;
        g.c = (float *)y->ptr();
        g.ldc = n;
        g.sc0 = m * n;
        g.nbc0 = groups;
        if (emit) {
            st = storage_planes_attach(ctx, *y->data);
            if (st) return st;
            g.c_hi = y->data->split->planes.planes + y->desc.shape.offset;
            g.c_plane = y->data->split->plane;
            if (only) {
                g.c = nullptr;
                y->data->planes_only = true;
            }
        }
        g.epilogue = epilogue;
        if (has_bias) {
            g.naux = 1;
            g.aux[0].ptr = reinterpret_cast<const float *>(biases->block->ptr);
            g.aux[0].s0 = n;
            g.aux[0].sc = 1;
        }
        return k::gemm_tc_run(ctx, g);
    }
};

// Slab i of a grouped product, shaped like the member GEMM's own result.
struct SlabOp : Operator {
    int index = 0;
    const char *name() const override { return "slab"; }
    std::vector<Var> grad(const std::vector<Var> &, const Var &, const Var &) override { shape_fail("slab is not differentiated"); }
    sage_status compute(const std::vector<Tensor> &x, Context &, Tensor *y) override {
        Shape s(out.shape.extents);
        s.offset = x[0].desc.shape.offset + (long long)index * out.shape.size();
        *y = x[0].with_shape(s);
        return SAGE_OK;
    }
};

bool is_slab_op(const Operator &op) { return dynamic_cast<const SlabOp *>(&op) != nullptr; }
bool is_grouped_gemm_op(const Operator &op) { return dynamic_cast<const GroupedGemmOp *>(&op) != nullptr; }

// Can this lowered GEMM join a group?  Fills a key that is equal for GEMMs that may share a launch
// (same A view, same shape and transposes, same epilogue text); the caller adds A's identity.
bool gemm_group_key(const Operator &op, std::string *key) {
    const GemmOp *g = as_gemm(op);
    if (!g || !g->lowered || g->attn || g->folded || g->conv || g->row_softmax || g->batch != 1 || g->naux() > 1) return false;
    if (g->n % 4 || g->k % 4 || !g->in[1].shape.has_default_strides() || g->in[1].shape.rank() != 2) return false;
    if (g->naux() == 1) {  // the one epilogue operand must be a row vector broadcast over the rows
        const Shape &b = g->in[2].shape;
        for (int d = 0; d < b.rank(); ++d) {
            const bool last = d == b.rank() - 1;
            if (b.extents[d] > 1 && b.strides[d] != (last ? 1 : 0)) return false;
        }
        if (b.extents.back() != g->n) return false;
    }
    const Shape &a = g->in[0].shape;
    std::string s = std::to_string(g->m) + "x" + std::to_string(g->n) + "x" + std::to_string(g->k) + (g->ta ? "T" : "N") + (g->tb ? "T" : "N") + "|" +
                    g->epilogue + "|" + std::to_string(g->naux()) + "|";
    for (int d = 0; d < a.rank(); ++d) s += std::to_string(a.extents[d]) + ":" + std::to_string(a.strides[d]) + ",";
    s += "@" + std::to_string(a.offset);
    *key = s;
    return true;
}

std::shared_ptr<Operator> make_grouped_gemm(const std::vector<const Operator *> &members) {
    const GemmOp *g0 = as_gemm(*members[0]);
    auto op = std::make_shared<GroupedGemmOp>();
    op->groups = (int)members.size();
    op->ta = g0->ta;
    op->tb = g0->tb;
    op->has_bias = g0->naux() == 1;
    op->m = g0->m;
    op->n = g0->n;
    op->k = g0->k;
    op->epilogue = g0->epilogue;
    op->in.push_back(g0->in[0]);
    for (const Operator *m : members) op->in.push_back(m->in[1]);
    if (op->has_bias)
        for (const Operator *m : members) op->in.push_back(m->in[2]);
    op->out = TensorDesc(Array{(long long)members.size(), g0->m, g0->n}, SAGE_F32);
    return op;
}

std::shared_ptr<Operator> make_slab(const Operator &grouped, int index, const TensorDesc &member_out) {
    auto op = std::make_shared<SlabOp>();
    op->index = index;
    op->in = {grouped.out};
    op->out = member_out.pristine();
    return op;
}

// ------------------------------------------------------------------------------ constructors
static void gemm_dims(const Array &e1, const Array &e2, size_t o, bool t1, bool t2, long long *h, long long *w) {
    const long long c1 = t1 ? e1[o] : e1[o + 1], c2 = t2 ? e2[o + 1] : e2[o];
    *h = t1 ? e1[o + 1] : e1[o];
    *w = t2 ? e2[o] : e2[o + 1];
    if (c1 != c2) shape_fail("gemm: inner dimensions differ");
}

Var ops::gemm(const Var &a0, const Var &b0, bool ta, bool tb) {
    Var a = a0.organize(), b = b0.organize();
    if (a.rank() != 2 || b.rank() != 2) shape_fail("gemm: operands must be rank 2");
    if (a.dtype() != b.dtype() || a.dtype() != SAGE_F32) shape_fail("gemm: operands must be float");
    long long h, w;
    gemm_dims(a.extents(), b.extents(), 0, ta, tb, &h, &w);
    auto op = std::make_shared<GemmOp>();
    op->ta = ta;
    op->tb = tb;
    op->batched = false;
    op->in = {a.desc, b.desc};
    op->out = TensorDesc(Array{h, w}, a.dtype());
    return Var::from_op(op, {a, b});
}

Var ops::gemm_batched(const Var &a0, const Var &b0, bool ta, bool tb) {
    Var a = a0.organize(), b = b0.organize();
    if (a.rank() != 3 || b.rank() != 3) shape_fail("gemm_batched: operands must be rank 3");
    if (a.extent(0) != b.extent(0)) shape_fail("gemm_batched: batch extents differ");
    if (a.dtype() != b.dtype() || a.dtype() != SAGE_F32) shape_fail("gemm_batched: operands must be float");
    long long h, w;
    gemm_dims(a.extents(), b.extents(), 1, ta, tb, &h, &w);
    auto op = std::make_shared<GemmOp>();
    op->ta = ta;
    op->tb = tb;
    op->batched = true;
    op->in = {a.desc, b.desc};
    op->out = TensorDesc(Array{a.extent(0), h, w}, a.dtype());
    return Var::from_op(op, {a, b});
}

Var ops::matmul(const Var &x1, const Var &x2) {  // gemm.rs:30-51
    Array ext(x1.extents().begin(), x1.extents().end() - 1);
    ext.insert(ext.end(), x2.extents().begin() + 1, x2.extents().end());
    Var a = view(x1, {x1.size() / x1.extent(-1), x1.extent(-1)});
    Var b = view(x2, {x2.extent(0), x2.size() / x2.extent(0)});
    return view(gemm(a, b, false, false), ext);
}

Var ops::matmul_batched(const Var &x1, const Var &x2) {  // gemm.rs:53-104
    Array batch_ext;
    for (int i = 0; i < std::min(x1.rank() - 2, x2.rank() - 2); ++i) {
        if (x1.extent(i) == x2.extent(i)) batch_ext.push_back(x1.extent(i));
        else break;
    }
    const int bl = (int)batch_ext.size();
    if (bl == 0) shape_fail("batch dim incorrect!");
    long long bs = 1;
    for (long long e : batch_ext) bs *= e;
    Array ext = batch_ext;
    ext.insert(ext.end(), x1.extents().begin() + bl, x1.extents().end() - 1);
    ext.insert(ext.end(), x2.extents().begin() + bl + 1, x2.extents().end());
    Var a = view(x1, {bs, x1.size() / (x1.extent(-1) * bs), x1.extent(-1)});
    Var b = view(x2, {bs, x2.extent(bl), x2.size() / (x2.extent(bl) * bs)});
    return view(gemm_batched(a, b, false, false), ext);
}

}  // namespace sage
