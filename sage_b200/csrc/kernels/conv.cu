// im2col / col2im / direct pooling for NHWC images.
//
// Reference: Im2col::compute (src/ops/conv.rs:289-374) gives each (y, x, c) of the column grid to a
// work-item that loops over the batch and the taps; Col2im::compute (:404-498) is the inverse
// gather-sum.  Here one thread produces one output element with the channel innermost, so both the
// image reads and the column writes coalesce.  pool2d evaluates max/avg pooling
// (conv.rs:143-165: im2col, then a reduction over [KH,KW]) straight from the image without
// materialising the KH*KW-times larger column tensor.  Padded taps count as zeros, and with
// ref_compat the max starts from 0 like the reference's reduce accumulator.
#include <cuda_runtime.h>

#include "kernels.h"

namespace sage {
namespace k {

struct ConvP {
    long long n, img_h, img_w, chan, col_h, col_w;
    Window w;
};

__global__ void __launch_bounds__(256) im2col_kernel(const float *__restrict__ img, float *__restrict__ col, ConvP p,
                                                     long long total) {
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total;
         g += (long long)gridDim.x * blockDim.x) {
        long long r = g;
        const long long c = r % p.chan; r /= p.chan;
        const long long kx = r % p.w.ker_w; r /= p.w.ker_w;
        const long long ky = r % p.w.ker_h; r /= p.w.ker_h;
        const long long ox = r % p.col_w; r /= p.col_w;
        const long long oy = r % p.col_h; r /= p.col_h;
        const long long n = r;
        const long long iy = oy * p.w.stride_h - p.w.pad_h + ky * p.w.dil_h;
        const long long ix = ox * p.w.stride_w - p.w.pad_w + kx * p.w.dil_w;
        float v = 0.f;
        if (ix >= 0 && ix < p.img_w && iy >= 0 && iy < p.img_h) v = img[((n * p.img_h + iy) * p.img_w + ix) * p.chan + c];
        col[g] = v;
    }
}

// Follows the reference's tap test literally, including dilation_h applied to the x tap and
// dilation_w to the y tap (conv.rs:462-464); identical whenever both dilations are equal.
__global__ void __launch_bounds__(256) col2im_kernel(const float *__restrict__ col, float *__restrict__ img, ConvP p,
                                                     long long total) {
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total;
         g += (long long)gridDim.x * blockDim.x) {
        long long r = g;
        const long long c = r % p.chan; r /= p.chan;
        const long long img_x = r % p.img_w; r /= p.img_w;
        const long long img_y = r % p.img_h; r /= p.img_h;
        const long long n = r;
        const long long xp = img_x + p.w.pad_w, yp = img_y + p.w.pad_h;
        const long long ker_ew = (p.w.ker_w - 1) * p.w.dil_w + 1, ker_eh = (p.w.ker_h - 1) * p.w.dil_h + 1;
        const long long xs = xp < ker_ew ? 0 : (xp - ker_ew) / p.w.stride_w + 1;
        const long long ys = yp < ker_eh ? 0 : (yp - ker_eh) / p.w.stride_h + 1;
        const long long xe = min(xp / p.w.stride_w + 1, p.col_w);
        const long long ye = min(yp / p.w.stride_h + 1, p.col_h);
        const long long col_b = n * p.col_h * p.col_w * p.w.ker_h * p.w.ker_w * p.chan;
        float val = 0.f;
        for (long long cx = xs; cx < xe; ++cx)
            for (long long cy = ys; cy < ye; ++cy) {
                long long kx = xp - cx * p.w.stride_w, ky = yp - cy * p.w.stride_h;
                if (kx % p.w.dil_h == 0 && ky % p.w.dil_w == 0) {
                    kx /= p.w.dil_h;
                    ky /= p.w.dil_w;
                    val += col[col_b + (((cy * p.col_w + cx) * p.w.ker_h + ky) * p.w.ker_w + kx) * p.chan + c];
                }
            }
        img[g] = val;
    }
}

__global__ void __launch_bounds__(256) pool2d_kernel(const float *__restrict__ img, float *__restrict__ out, ConvP p,
                                                     long long total, int is_max, int ref_compat) {
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total;
         g += (long long)gridDim.x * blockDim.x) {
        long long r = g;
        const long long c = r % p.chan; r /= p.chan;
        const long long ox = r % p.col_w; r /= p.col_w;
        const long long oy = r % p.col_h; r /= p.col_h;
        const long long n = r;
        float acc = is_max ? (ref_compat ? 0.f : -INFINITY) : 0.f;
        // reduce over axes [3,4] = [KH,KW]: the first listed axis (KH) is the inner loop
        for (int kx = 0; kx < p.w.ker_w; ++kx)
            for (int ky = 0; ky < p.w.ker_h; ++ky) {
                const long long iy = oy * p.w.stride_h - p.w.pad_h + (long long)ky * p.w.dil_h;
                const long long ix = ox * p.w.stride_w - p.w.pad_w + (long long)kx * p.w.dil_w;
                float v = 0.f;
                if (ix >= 0 && ix < p.img_w && iy >= 0 && iy < p.img_h)
                    v = img[((n * p.img_h + iy) * p.img_w + ix) * p.chan + c];
                acc = is_max ? fmaxf(acc, v) : acc + v;
            }
        if (!is_max) acc = acc / (float)(p.w.ker_w * p.w.ker_h);
        out[g] = acc;
    }
}

static unsigned grid_for(Context &ctx, long long n) {
    long long blocks = (n + 255) / 256;
    long long cap = (long long)ctx.sm_count * 32;
    return (unsigned)(blocks < cap ? blocks : cap);
}

sage_status im2col(Context &ctx, const float *img, float *col, long long n, long long img_h, long long img_w,
                   long long chan, long long col_h, long long col_w, const Window &w) {
    ConvP p{n, img_h, img_w, chan, col_h, col_w, w};
    long long total = n * col_h * col_w * w.ker_h * w.ker_w * chan;
    ctx.note_launch("im2col");
    if (ctx.dry() || total == 0) return SAGE_OK;
    im2col_kernel<<<grid_for(ctx, total), 256, 0, ctx.stream()>>>(img, col, p, total);
    return ctx.check_cuda(cudaGetLastError(), "im2col launch");
}

sage_status col2im(Context &ctx, const float *col, float *img, long long n, long long img_h, long long img_w,
                   long long chan, long long col_h, long long col_w, const Window &w) {
    ConvP p{n, img_h, img_w, chan, col_h, col_w, w};
    long long total = n * img_h * img_w * chan;
    ctx.note_launch("col2im");
    if (ctx.dry() || total == 0) return SAGE_OK;
    col2im_kernel<<<grid_for(ctx, total), 256, 0, ctx.stream()>>>(col, img, p, total);
    return ctx.check_cuda(cudaGetLastError(), "col2im launch");
}

sage_status pool2d(Context &ctx, bool is_max, const float *img, float *out, long long n, long long img_h,
                   long long img_w, long long chan, long long out_h, long long out_w, const Window &w) {
    ConvP p{n, img_h, img_w, chan, out_h, out_w, w};
    long long total = n * out_h * out_w * chan;
    ctx.note_launch(is_max ? "max_pool2d" : "avg_pool2d");
    if (ctx.dry() || total == 0) return SAGE_OK;
    pool2d_kernel<<<grid_for(ctx, total), 256, 0, ctx.stream()>>>(img, out, p, total, is_max ? 1 : 0, ctx.opts().ref_compat);
    return ctx.check_cuda(cudaGetLastError(), "pool2d launch");
}

}  // namespace k
}  // namespace sage
