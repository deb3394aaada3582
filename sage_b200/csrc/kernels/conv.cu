// im2col / col2im / direct pooling for NHWC images.
//
// Reference: Im2col::compute (src/ops/conv.rs:289-374) gives each (y, x, c) of the column grid to a
// work-item that loops over the batch and the taps; Col2im::compute (:404-498) is the inverse
// gather-sum.  Here im2col gives a warp to each output pixel (see im2col_kernel) and can write the
// tf32 hi / lo planes of the column matrix for the tensor-core GEMM in the same pass; convolutions
// whose channel count is a multiple of 32 do not come here at all (the GEMM loads image tiles with
// im2col-mode TMA).  pool2d evaluates max/avg pooling
// (conv.rs:143-165: im2col, then a reduction over [KH,KW]) straight from the image without
// materialising the KH*KW-times larger column tensor.  Padded taps count as zeros, and with
// ref_compat the max starts from 0 like the reference's reduce accumulator.
#include <cuda.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "gemm_tc_device.inc"  // split_tf32_value

namespace sage {
namespace k {

struct ConvP {
    long long n, img_h, img_w, chan, col_h, col_w;
    Window w;
};

// One warp per output pixel: the K = KH*KW*C values of a column row are contiguous in the output and
// C-contiguous runs in the image, so with C % 4 == 0 the lanes move 16-byte chunks and both sides
// coalesce; index arithmetic is 32-bit per chunk and once per pixel.  Outputs: the fp32 column
// tensor (row pitch K) and / or the tf32 hi / lo planes of it (row pitch `pitch` >= K, a multiple of
// 4; pad columns are written as zeros) for the tensor-core GEMM that consumes it.
struct ColOut {
    float *col;       // may be null
    float *hi;        // may be null; lo = hi + plane
    long long plane;
    int pitch;
};

__device__ __forceinline__ void split_pair(float x, float *hi, float *lo) { sage_tc::split_tf32_value(x, hi, lo); }

__global__ void __launch_bounds__(256) im2col_kernel(const float *__restrict__ img, ColOut o, ConvP p, long long pixels) {
    const int lane = threadIdx.x & 31;
    const long long pix = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pix >= pixels) return;
    const unsigned per_img = (unsigned)(p.col_h * p.col_w);
    const long long n = pix / per_img;
    const unsigned r = (unsigned)(pix - n * per_img);
    const int oy = (int)(r / (unsigned)p.col_w), ox = (int)(r % (unsigned)p.col_w);
    const int iy0 = oy * p.w.stride_h - p.w.pad_h, ix0 = ox * p.w.stride_w - p.w.pad_w;
    const int C = (int)p.chan, K = p.w.ker_h * p.w.ker_w * C;
    const float *im = img + n * p.img_h * p.img_w * C;
    if ((C & 3) == 0) {
        const int c4n = C >> 2, chunks = K >> 2;
        for (int ch = lane; ch < chunks; ch += 32) {
            const int tap = ch / c4n, c = (ch - tap * c4n) << 2;
            const int ky = tap / p.w.ker_w, kx = tap - ky * p.w.ker_w;
            const int iy = iy0 + ky * p.w.dil_h, ix = ix0 + kx * p.w.dil_w;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ix >= 0 && ix < p.img_w && iy >= 0 && iy < p.img_h)
                v = __ldg(reinterpret_cast<const float4 *>(im + ((long long)iy * p.img_w + ix) * C + c));
            if (o.col) *reinterpret_cast<float4 *>(o.col + pix * K + (ch << 2)) = v;
            if (o.hi) {
                float4 h, l;
                split_pair(v.x, &h.x, &l.x);
                split_pair(v.y, &h.y, &l.y);
                split_pair(v.z, &h.z, &l.z);
                split_pair(v.w, &h.w, &l.w);
                float *d = o.hi + pix * o.pitch + (ch << 2);
                *reinterpret_cast<float4 *>(d) = h;
                *reinterpret_cast<float4 *>(d + o.plane) = l;
            }
        }
    } else {
        const int width = o.hi ? o.pitch : K;
        for (int kk = lane; kk < width; kk += 32) {
            float v = 0.f;
            if (kk < K) {
                const int tap = kk / C, c = kk - tap * C;
                const int ky = tap / p.w.ker_w, kx = tap - ky * p.w.ker_w;
                const int iy = iy0 + ky * p.w.dil_h, ix = ix0 + kx * p.w.dil_w;
                if (ix >= 0 && ix < p.img_w && iy >= 0 && iy < p.img_h) v = __ldg(im + ((long long)iy * p.img_w + ix) * C + c);
                if (o.col) o.col[pix * K + kk] = v;
            }
            if (o.hi) {
                float h, l;
                split_pair(v, &h, &l);
                o.hi[pix * o.pitch + kk] = h;
                o.hi[pix * o.pitch + kk + o.plane] = l;
            }
        }
    }
}

// Planes of the column matrix when C is not a multiple of 4 (the first convolution of a network: C = 1 or 3,
// K = 49 or 147).  A thread owns 4 consecutive entries of a row (one 16-byte store into each plane), so a
// warp writes 512 contiguous bytes per plane; where an entry comes from (tap, channel) is looked up in a
// table in shared memory, built once per block, instead of being divided out per element.
constexpr int kTapTable = 1024;
__global__ void __launch_bounds__(256) im2col_quads_kernel(const float *__restrict__ img, ColOut o, ConvP p, long long quads) {
    __shared__ int tab_off[kTapTable];   // element offset of entry kk from the pixel's first tap, -1 beyond K
    __shared__ int tab_yx[kTapTable];    // (ky * dil_h) << 16 | (kx * dil_w)
    const int C = (int)p.chan, K = p.w.ker_h * p.w.ker_w * C;
    for (int kk = threadIdx.x; kk < o.pitch; kk += 256) {
        if (kk < K) {
            const int tap = kk / C, c = kk - tap * C;
            const int ky = tap / p.w.ker_w, kx = tap - ky * p.w.ker_w;
            tab_off[kk] = (ky * p.w.dil_h * (int)p.img_w + kx * p.w.dil_w) * C + c;
            tab_yx[kk] = ((ky * p.w.dil_h) << 16) | (kx * p.w.dil_w);
        } else {
            tab_off[kk] = -1;
            tab_yx[kk] = 0;
        }
    }
    __syncthreads();
    const int per_row = o.pitch >> 2;
    const unsigned per_img = (unsigned)(p.col_h * p.col_w);
    for (long long q = (long long)blockIdx.x * 256 + threadIdx.x; q < quads; q += (long long)gridDim.x * 256) {
        const long long pix = q / per_row;
        const int k0 = (int)(q - pix * per_row) << 2;
        const long long n = pix / per_img;
        const unsigned r = (unsigned)(pix - n * per_img);
        const int oy = (int)(r / (unsigned)p.col_w), ox = (int)(r % (unsigned)p.col_w);
        const int iy0 = oy * p.w.stride_h - p.w.pad_h, ix0 = ox * p.w.stride_w - p.w.pad_w;
        const float *base = img + (n * p.img_h * p.img_w + (long long)iy0 * p.img_w + ix0) * C;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int off = tab_off[k0 + i], yx = tab_yx[k0 + i];
            const int iy = iy0 + (yx >> 16), ix = ix0 + (yx & 0xffff);
            v[i] = (off >= 0 && ix >= 0 && ix < p.img_w && iy >= 0 && iy < p.img_h) ? __ldg(base + off) : 0.f;
        }
        float4 h, l;
        split_pair(v[0], &h.x, &l.x);
        split_pair(v[1], &h.y, &l.y);
        split_pair(v[2], &h.z, &l.z);
        split_pair(v[3], &h.w, &l.w);
        float *d = o.hi + pix * o.pitch + k0;
        *reinterpret_cast<float4 *>(d) = h;
        *reinterpret_cast<float4 *>(d + o.plane) = l;
        if (o.col) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (k0 + i < K) o.col[pix * K + k0 + i] = v[i];
        }
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

// The same gather with 32-bit index arithmetic and four channels per thread (C % 4 == 0): one 64-bit division per
// thread instead of a dozen per element, 16-byte loads and stores.  Same tap test, same order of accumulation.
__global__ void __launch_bounds__(256) col2im_quads_kernel(const float *__restrict__ col, float *__restrict__ img, ConvP p, long long total) {
    const int cn = (int)(p.chan >> 2), W = (int)p.img_w, H = (int)p.img_h, CW = (int)p.col_w, CH = (int)p.col_h;
    const int sw = p.w.stride_w, sh = p.w.stride_h, dw = p.w.dil_w, dh = p.w.dil_h, kw = p.w.ker_w, kh = p.w.ker_h;
    const int ker_ew = (kw - 1) * dw + 1, ker_eh = (kh - 1) * dh + 1;
    const unsigned per_img = (unsigned)(H * W);
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (long long)gridDim.x * blockDim.x) {
        const long long pix = g / cn;
        const int c = (int)(g - pix * cn) << 2;
        const long long n = pix / per_img;
        const unsigned r = (unsigned)(pix - n * per_img);
        const int img_y = (int)(r / (unsigned)W), img_x = (int)(r - (unsigned)img_y * (unsigned)W);
        const int xp = img_x + p.w.pad_w, yp = img_y + p.w.pad_h;
        const int xs = xp < ker_ew ? 0 : (xp - ker_ew) / sw + 1, ys = yp < ker_eh ? 0 : (yp - ker_eh) / sh + 1;
        const int xe = min(xp / sw + 1, CW), ye = min(yp / sh + 1, CH);
        const float *cb = col + n * (long long)CH * CW * kh * kw * p.chan + c;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int cx = xs; cx < xe; ++cx)
            for (int cy = ys; cy < ye; ++cy) {
                int kx = xp - cx * sw, ky = yp - cy * sh;
                if (kx % dh == 0 && ky % dw == 0) {  // the reference's test (conv.rs:462-464), dilations crossed as there
                    kx /= dh;
                    ky /= dw;
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(cb + ((((long long)cy * CW + cx) * kh + ky) * kw + kx) * p.chan));
                    val.x += v.x;
                    val.y += v.y;
                    val.z += v.z;
                    val.w += v.w;
                }
            }
        *reinterpret_cast<float4 *>(img + (pix * p.chan + c)) = val;
    }
}

// One thread per output pixel and group of 4 channels when C % 4 == 0 (16-byte loads, one 64-bit
// division per thread), else one thread per element.
template <int VEC>
__global__ void __launch_bounds__(256) pool2d_kernel(const float *__restrict__ img, float *__restrict__ out, ConvP p,
                                                     long long total, int is_max, int ref_compat) {
    const unsigned cn = (unsigned)(p.chan / VEC);
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total;
         g += (long long)gridDim.x * blockDim.x) {
        const long long pix = g / cn;
        const int c = (int)(g - pix * cn) * VEC;
        const unsigned per_img = (unsigned)(p.col_h * p.col_w);
        const long long n = pix / per_img;
        const unsigned r = (unsigned)(pix - n * per_img);
        const int oy = (int)(r / (unsigned)p.col_w), ox = (int)(r % (unsigned)p.col_w);
        const float init = is_max ? (ref_compat ? 0.f : -INFINITY) : 0.f;
        float acc[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] = init;
        // reduce over axes [3,4] = [KH,KW]: the first listed axis (KH) is the inner loop
        for (int kx = 0; kx < p.w.ker_w; ++kx)
            for (int ky = 0; ky < p.w.ker_h; ++ky) {
                const int iy = oy * p.w.stride_h - p.w.pad_h + ky * p.w.dil_h;
                const int ix = ox * p.w.stride_w - p.w.pad_w + kx * p.w.dil_w;
                float v[VEC];
#pragma unroll
                for (int j = 0; j < VEC; ++j) v[j] = 0.f;
                if (ix >= 0 && ix < p.img_w && iy >= 0 && iy < p.img_h) {
                    const float *src = img + ((n * p.img_h + iy) * p.img_w + ix) * p.chan + c;
                    if (VEC == 4) {
                        const float4 t = __ldg(reinterpret_cast<const float4 *>(src));
                        v[0] = t.x; v[1 % VEC] = t.y; v[2 % VEC] = t.z; v[3 % VEC] = t.w;
                    } else {
                        v[0] = __ldg(src);
                    }
                }
#pragma unroll
                for (int j = 0; j < VEC; ++j) acc[j] = is_max ? fmaxf(acc[j], v[j]) : acc[j] + v[j];
            }
        if (!is_max) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[j] = acc[j] / (float)(p.w.ker_w * p.w.ker_h);
        }
        float *dst = out + pix * p.chan + c;
        if (VEC == 4) *reinterpret_cast<float4 *>(dst) = make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
        else dst[0] = acc[0];
    }
}

static unsigned grid_for(Context &ctx, long long n) {
    long long blocks = (n + 255) / 256;
    long long cap = (long long)ctx.sm_count * 32;
    return (unsigned)(blocks < cap ? blocks : cap);
}

sage_status im2col_planes(Context &ctx, const float *img, long long n, long long img_h, long long img_w, long long chan,
                          long long col_h, long long col_w, const Window &w, float *col, float *hi, long long plane, int pitch) {
    ConvP p{n, img_h, img_w, chan, col_h, col_w, w};
    const long long pixels = n * col_h * col_w;
    ctx.note_launch("im2col");
    if (ctx.dry() || pixels == 0) return SAGE_OK;
    if (col_h * col_w > 0x7fffffffLL || img_h > 0x7fffffffLL || img_w > 0x7fffffffLL || (long long)w.ker_h * w.ker_w * chan > 0x7fffffffLL ||
        (pixels + 7) / 8 > 0x7fffffffLL)
        return ctx.fail(SAGE_ERR_UNSUPPORTED, "im2col: extents beyond 2^31");
    const bool vec = chan % 4 == 0;
    if (vec && ((col && reinterpret_cast<uintptr_t>(col) % 16) || reinterpret_cast<uintptr_t>(img) % 16 ||
                (hi && (reinterpret_cast<uintptr_t>(hi) % 16 || plane % 4 || pitch % 4))))
        return ctx.fail(SAGE_ERR_INVALID, "im2col: unaligned buffer");
    ColOut o{col, hi, plane, pitch};
    if (!vec && hi && pitch % 4 == 0 && pitch <= kTapTable && reinterpret_cast<uintptr_t>(hi) % 16 == 0 && plane % 4 == 0 &&
        img_w * (long long)w.ker_h * w.dil_h * chan < (1LL << 30) && w.ker_w * w.dil_w < 65536) {
        const long long quads = pixels * (pitch / 4);
        im2col_quads_kernel<<<grid_for(ctx, quads), 256, 0, ctx.stream()>>>(img, o, p, quads);
        return ctx.check_cuda(cudaGetLastError(), "im2col launch");
    }
    im2col_kernel<<<(unsigned)((pixels + 7) / 8), 256, 0, ctx.stream()>>>(img, o, p, pixels);
    return ctx.check_cuda(cudaGetLastError(), "im2col launch");
}

// ---- convolutions with at most 4 input channels (the first layer of an image model: C = 3 or 1).
// A channel run of 12 bytes is below TMA's 16-byte granularity, so the image is first re-laid as tf32 planes of
// [N, H + pad, W + pad, 4] — channels padded to 4, the spatial padding written as zeros.  In that layout the KW taps of one
// filter row are KW * 4 CONTIGUOUS floats, so one output pixel's operand row for tap row ky is a 32-float (128-byte)
// window starting 4 * stride_w floats after its left neighbour's: an "image" of 32-channel pixels that overlap.  The
// implicit-GEMM kernel then runs a (1 x KH) convolution over it; the column matrix is never written.
__global__ void __launch_bounds__(256) pack_small_c_kernel(const float *__restrict__ img, float4 *__restrict__ hi, float4 *__restrict__ lo, long long n,
                                                           int h, int w, int c, int hp, int wp, int pad_h, int pad_w) {
    const long long total = n * hp * (long long)wp;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (long long)gridDim.x * blockDim.x) {
        const int x = (int)(g % wp) - pad_w;
        const long long r = g / wp;
        const int y = (int)(r % hp) - pad_h;
        const long long b = r / hp;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (x >= 0 && x < w && y >= 0 && y < h) {
            const float *s = img + ((b * h + y) * (long long)w + x) * c;
            for (int i = 0; i < c; ++i) v[i] = s[i];
        }
        if (!lo) {  // plain fp32: the GEMM splits each tile itself
            hi[g] = make_float4(v[0], v[1], v[2], v[3]);
            continue;
        }
        float4 a, d;
        sage_tc::split_tf32_value(v[0], &a.x, &d.x);
        sage_tc::split_tf32_value(v[1], &a.y, &d.y);
        sage_tc::split_tf32_value(v[2], &a.z, &d.z);
        sage_tc::split_tf32_value(v[3], &a.w, &d.w);
        hi[g] = a;
        lo[g] = d;
    }
}

// The filter [KH, KW, C, OC] as the matching B operand [KH * 32, OC]: row ky * 32 + kx * 4 + c; rows of padded
// channels and of the window's unused tail are zero, so whatever the overlapping operand rows hold there is ignored.
__global__ void __launch_bounds__(256) pack_small_c_filter_kernel(const float *__restrict__ f, float *__restrict__ hi, float *__restrict__ lo,
                                                                  int kh, int kw, int c, int oc) {
    const long long total = (long long)kh * 32 * oc;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (long long)gridDim.x * blockDim.x) {
        const int o = (int)(g % oc), row = (int)(g / oc), ky = row / 32, r = row % 32, kx = r / 4, cc = r % 4;
        const float v = (kx < kw && cc < c) ? f[(((long long)ky * kw + kx) * c + cc) * oc + o] : 0.f;
        sage_tc::split_tf32_value(v, &hi[g], &lo[g]);
    }
}

sage_status pack_small_c_image(Context &ctx, const float *img, long long n, long long h, long long w, long long c, long long hp, long long wp,
                               int pad_h, int pad_w, float *hi, long long plane) {
    ctx.note_launch("pack_small_c");
    if (ctx.dry()) return SAGE_OK;
    if (c < 1 || c > 4 || plane % 4 || reinterpret_cast<uintptr_t>(hi) % 16 || h > 0x7fffffffLL || w > 0x7fffffffLL || hp > 0x7fffffffLL || wp > 0x7fffffffLL)
        return ctx.fail(SAGE_ERR_INVALID, "pack_small_c: bad arguments");
    const long long total = n * hp * wp;
    pack_small_c_kernel<<<grid_for(ctx, total), 256, 0, ctx.stream()>>>(img, reinterpret_cast<float4 *>(hi), plane ? reinterpret_cast<float4 *>(hi + plane) : nullptr, n, (int)h, (int)w,
                                                                        (int)c, (int)hp, (int)wp, pad_h, pad_w);
    return ctx.check_cuda(cudaGetLastError(), "pack_small_c launch");
}

sage_status pack_small_c_filter(Context &ctx, const float *filt, int kh, int kw, int c, int oc, float *hi, long long plane) {
    ctx.note_launch("pack_small_c_filter");
    if (ctx.dry()) return SAGE_OK;
    if (kw * 4 > 32 || c > 4) return ctx.fail(SAGE_ERR_INVALID, "pack_small_c_filter: window too wide");
    pack_small_c_filter_kernel<<<grid_for(ctx, (long long)kh * 32 * oc), 256, 0, ctx.stream()>>>(filt, hi, hi + plane, kh, kw, c, oc);
    return ctx.check_cuda(cudaGetLastError(), "pack_small_c_filter launch");
}

sage_status im2col(Context &ctx, const float *img, float *col, long long n, long long img_h, long long img_w,
                   long long chan, long long col_h, long long col_w, const Window &w) {
    return im2col_planes(ctx, img, n, img_h, img_w, chan, col_h, col_w, w, col, nullptr, 0, 0);
}

sage_status col2im(Context &ctx, const float *col, float *img, long long n, long long img_h, long long img_w,
                   long long chan, long long col_h, long long col_w, const Window &w) {
    ConvP p{n, img_h, img_w, chan, col_h, col_w, w};
    long long total = n * img_h * img_w * chan;
    ctx.note_launch("col2im");
    if (ctx.dry() || total == 0) return SAGE_OK;
    if (chan % 4 == 0 && reinterpret_cast<uintptr_t>(col) % 16 == 0 && reinterpret_cast<uintptr_t>(img) % 16 == 0 && img_h * img_w <= 0x7fffffffLL &&
        col_h * col_w <= 0x7fffffffLL && w.dil_w >= 1 && w.dil_h >= 1) {
        col2im_quads_kernel<<<grid_for(ctx, total / 4), 256, 0, ctx.stream()>>>(col, img, p, total / 4);
        return ctx.check_cuda(cudaGetLastError(), "col2im launch");
    }
    col2im_kernel<<<grid_for(ctx, total), 256, 0, ctx.stream()>>>(col, img, p, total);
    return ctx.check_cuda(cudaGetLastError(), "col2im launch");
}

sage_status pool2d(Context &ctx, bool is_max, const float *img, float *out, long long n, long long img_h,
                   long long img_w, long long chan, long long out_h, long long out_w, const Window &w) {
    ConvP p{n, img_h, img_w, chan, out_h, out_w, w};
    long long total = n * out_h * out_w * chan;
    ctx.note_launch(is_max ? "max_pool2d" : "avg_pool2d");
    if (ctx.dry() || total == 0) return SAGE_OK;
    const bool vec = chan % 4 == 0 && reinterpret_cast<uintptr_t>(img) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                     out_h * out_w <= 0x7fffffffLL;
    if (vec) pool2d_kernel<4><<<grid_for(ctx, total / 4), 256, 0, ctx.stream()>>>(img, out, p, total / 4, is_max ? 1 : 0, ctx.opts().ref_compat);
    else pool2d_kernel<1><<<grid_for(ctx, total), 256, 0, ctx.stream()>>>(img, out, p, total, is_max ? 1 : 0, ctx.opts().ref_compat);
    return ctx.check_cuda(cudaGetLastError(), "pool2d launch");
}

}  // namespace k
}  // namespace sage
