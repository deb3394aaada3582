/*
 * CPU oracle for the sage hot path.  TEST INFRASTRUCTURE ONLY: nothing in the
 * product (the sage_b200 package or libsagecuda.so) links, loads or calls this
 * file.  It restates, loop nest for loop nest, what the reference's generated
 * OpenCL kernels compute, so the CUDA kernels can be compared against it.
 *
 * Every tensor operand is (base pointer, element offset, extents[], strides[])
 * with strides in ELEMENTS, exactly like the reference's Shape
 * (src/shape.rs:37-43).  All element types are 4 bytes wide (float / int /
 * uint), which is also all the reference can store (src/session/device.rs:73-81).
 *
 * Parity status: pinned against the reference's own known-answer vectors
 * (tests/golden/reference_vectors.json, checked by tests/test_oracle_golden.py).
 * layer_norm, matmul_batched and the model graphs have no vector in the
 * reference: for those, parity is unpinned and the oracle is the only arbiter.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define O_MAX_DIMS 8

enum { O_SUM = 0, O_PROD = 1, O_MAX = 2, O_MIN = 3 };
enum { O_F32 = 0, O_I32 = 1, O_U32 = 2 };

/* src/ops/core.rs:113-175 (translate_id): decompose a linear id over a
 * contiguous reference space and re-compose it with the operand's strides. */
static inline int64_t translate(int64_t gid, int ndim, const int64_t *ext,
                                const int64_t *str, int64_t off) {
    int64_t idx = off;
    for (int i = ndim - 1; i >= 0; --i) {
        int64_t c = gid % ext[i];
        gid /= ext[i];
        idx += c * str[i];
    }
    return idx;
}

static inline int64_t prod(int n, const int64_t *e) {
    int64_t p = 1;
    for (int i = 0; i < n; ++i) p *= e[i];
    return p;
}

/* Strided read into a contiguous buffer: the index half of every map kernel
 * (src/ops/map.rs:369-410).  Works for any 4-byte element type. */
void o_strided_read(const uint32_t *x, int ndim, const int64_t *ext,
                    const int64_t *str, int64_t off, uint32_t *y) {
    int64_t n = prod(ndim, ext);
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n; ++g) y[g] = x[translate(g, ndim, ext, str, off)];
}

/* src/ops/reduce.rs:258-325.  One "work-item" per output element; accumulator
 * starts at 0 for every op; the FIRST listed reduced axis is the innermost
 * loop.  outer_* describe the kept axes (they index the output), inner_* the
 * reduced ones in the order the caller listed them. */
#define REDUCE_BODY(T, MAXF, MINF)                                              \
    int64_t n_out = prod(outer_ndim, outer_ext);                                \
    int64_t n_in = prod(inner_ndim, inner_ext);                                 \
    _Pragma("omp parallel for schedule(static)")                                \
    for (int64_t g = 0; g < n_out; ++g) {                                       \
        int64_t base = translate(g, outer_ndim, outer_ext, outer_str, outer_off);\
        T acc = 0;                                                              \
        int64_t c[O_MAX_DIMS] = {0};                                            \
        for (int64_t it = 0; it < n_in; ++it) {                                 \
            int64_t idx = base;                                                 \
            for (int a = 0; a < inner_ndim; ++a) idx += c[a] * inner_str[a];    \
            T v = ((const T *)x)[idx];                                          \
            switch (op) {                                                       \
            case O_SUM: acc = acc + v; break;                                   \
            case O_PROD: acc = acc * v; break;                                  \
            case O_MAX: acc = MAXF(acc, v); break;                              \
            default: acc = MINF(acc, v); break;                                 \
            }                                                                   \
            /* odometer: axis 0 of the reduced list runs fastest */             \
            for (int a = 0; a < inner_ndim; ++a) {                              \
                if (++c[a] < inner_ext[a]) break;                               \
                c[a] = 0;                                                       \
            }                                                                   \
        }                                                                       \
        ((T *)y)[g] = acc;                                                      \
    }

#define IMAX(a, b) ((a) > (b) ? (a) : (b))
#define IMIN(a, b) ((a) < (b) ? (a) : (b))

void o_reduce(const void *x, int dtype, int op, int outer_ndim,
              const int64_t *outer_ext, const int64_t *outer_str,
              int64_t outer_off, int inner_ndim, const int64_t *inner_ext,
              const int64_t *inner_str, void *y) {
    if (dtype == O_F32) {
        REDUCE_BODY(float, fmaxf, fminf)
    } else if (dtype == O_I32) {
        REDUCE_BODY(int32_t, IMAX, IMIN)
    } else {
        REDUCE_BODY(uint32_t, IMAX, IMIN)
    }
}

/* src/ops/reduce.rs:372-431.  best = x[outer]; strict compare, first extremum
 * wins, NaN never wins; uint output. */
void o_reduce_arg(const float *x, int is_max, int outer_ndim,
                  const int64_t *outer_ext, const int64_t *outer_str,
                  int64_t outer_off, int64_t inner_ext, int64_t inner_str,
                  uint32_t *y) {
    int64_t n_out = prod(outer_ndim, outer_ext);
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_out; ++g) {
        int64_t base = translate(g, outer_ndim, outer_ext, outer_str, outer_off);
        float best = x[base];
        uint32_t arg = 0;
        for (int64_t i = 0; i < inner_ext; ++i) {
            float v = x[base + i * inner_str];
            if (is_max ? (best < v) : (best > v)) {
                arg = (uint32_t)i;
                best = v;
            }
        }
        y[g] = arg;
    }
}

/* src/ops/core.rs:655-718.  Output is contiguous with the index tensor's
 * extents; the coordinate along `axis` is replaced by the gathered index. */
void o_gather(const uint32_t *x, int ndim, const int64_t *x_str, int64_t x_off,
              const uint32_t *ind, const int64_t *ind_ext,
              const int64_t *ind_str, int64_t ind_off, int axis, uint32_t *y) {
    int64_t n = prod(ndim, ind_ext);
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n; ++g) {
        int64_t t = ind[translate(g, ndim, ind_ext, ind_str, 0) + ind_off];
        int64_t idx = x_off, rem = g;
        int64_t c[O_MAX_DIMS];
        for (int i = ndim - 1; i >= 0; --i) {
            c[i] = rem % ind_ext[i];
            rem /= ind_ext[i];
        }
        for (int i = 0; i < ndim; ++i) idx += (i == axis ? t : c[i]) * x_str[i];
        y[g] = x[idx];
    }
}

/* src/ops/core.rs:764-833.  y is zero-filled and contiguous with `y_ext`;
 * one work-item per INDEX element; the work-item id is decomposed with the
 * index tensor's own strides (which equals a row-major unravel only when the
 * index tensor is contiguous: callers pass contiguous indices); the update is
 * a plain read-modify-write, so duplicate indices are undefined in the
 * reference.  Here work-items run in ascending order, which gives the
 * "last writer adds" result a sequential device would. */
void o_scatter(const float *x, int ndim, const int64_t *x_str, int64_t x_off,
               const uint32_t *ind, const int64_t *ind_ext,
               const int64_t *ind_str, int64_t ind_off, int axis,
               const int64_t *y_ext, float *y) {
    int64_t y_str[O_MAX_DIMS];
    int64_t p = 1;
    for (int i = ndim - 1; i >= 0; --i) {
        y_str[i] = p;
        p *= y_ext[i];
    }
    memset(y, 0, sizeof(float) * (size_t)p);
    int64_t n = prod(ndim, ind_ext);
    for (int64_t g = 0; g < n; ++g) {
        int64_t t = ind[translate(g, ndim, ind_ext, ind_str, 0) + ind_off];
        int64_t idx_in = x_off, idx_out = 0, rem = g;
        for (int i = 0; i < ndim; ++i) {
            int64_t c = ind_str[i] ? rem / ind_str[i] : 0;
            rem -= c * ind_str[i];
            idx_in += c * x_str[i];
            idx_out += (i == axis ? t : c) * y_str[i];
        }
        y[idx_out] += x[idx_in];
    }
}

/* src/ops/gemm.rs:176-250 + src/ops/kernels/matmul_direct.opencl:514-709:
 * C[i,j] = sum_{p=0..k-1} A'(i,p) * B'(p,j), accumulated in fp32 in increasing
 * p (alpha = 1, beta = 0).  `use_fma` selects whether each multiply-add is
 * contracted, since an OpenCL compiler may do either. */
static void gemm_one(int ta, int tb, int64_t m, int64_t n, int64_t k,
                     const float *A, int64_t lda, const float *B, int64_t ldb,
                     float *C, int64_t ldc, int use_fma) {
    /* B'(p,j) as a row-major [k,n] panel, so the j loop is unit-stride. */
    const float *Bp = B;
    int64_t ldbp = ldb;
    float *bt = NULL;
    if (tb) {
        bt = (float *)malloc(sizeof(float) * (size_t)(k * n));
#pragma omp parallel for schedule(static)
        for (int64_t p = 0; p < k; ++p)
            for (int64_t j = 0; j < n; ++j) bt[p * n + j] = B[j * ldb + p];
        Bp = bt;
        ldbp = n;
    }
    enum { IB = 8, JB = 512 };
    int64_t n_ib = (m + IB - 1) / IB;
    /* Blocking only changes which outputs are in flight together; each output
     * still sees p = 0..k-1 in order, like one reference work-item. */
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t bi = 0; bi < n_ib; ++bi) {
        int64_t i0 = bi * IB, i1 = IMIN(i0 + IB, m);
        for (int64_t j0 = 0; j0 < n; j0 += JB) {
            int64_t j1 = IMIN(j0 + JB, n);
            for (int64_t i = i0; i < i1; ++i)
                for (int64_t j = j0; j < j1; ++j) C[i * ldc + j] = 0.0f;
            for (int64_t p = 0; p < k; ++p) {
                const float *b = Bp + p * ldbp;
                for (int64_t i = i0; i < i1; ++i) {
                    float a = ta ? A[p * lda + i] : A[i * lda + p];
                    float *c = C + i * ldc;
                    if (use_fma) {
                        for (int64_t j = j0; j < j1; ++j) c[j] = fmaf(a, b[j], c[j]);
                    } else {
                        /* built with -ffp-contract=off: separate multiply and add */
                        for (int64_t j = j0; j < j1; ++j) c[j] = c[j] + a * b[j];
                    }
                }
            }
        }
    }
    free(bt);
}

void o_gemm(int ta, int tb, int64_t m, int64_t n, int64_t k, const float *A,
            int64_t a_off, int64_t lda, const float *B, int64_t b_off,
            int64_t ldb, float *C, int64_t c_off, int64_t ldc, int use_fma) {
    gemm_one(ta, tb, m, n, k, A + a_off, lda, B + b_off, ldb, C + c_off, ldc, use_fma);
}

/* src/ops/gemm.rs:338-421 + matmul_direct.opencl:857-927 */
void o_gemm_batched(int ta, int tb, int64_t batch, int64_t m, int64_t n,
                    int64_t k, const float *A, int64_t a_off, int64_t lda,
                    int64_t a_bs, const float *B, int64_t b_off, int64_t ldb,
                    int64_t b_bs, float *C, int64_t c_off, int64_t ldc,
                    int64_t c_bs, int use_fma) {
    for (int64_t b = 0; b < batch; ++b)
        gemm_one(ta, tb, m, n, k, A + a_off + b * a_bs, lda, B + b_off + b * b_bs,
                 ldb, C + c_off + b * c_bs, ldc, use_fma);
}

/* src/ops/conv.rs:289-374.  img [N,H,W,C] -> col [N,OH,OW,KH,KW,C], zero pad. */
void o_im2col(const float *img, float *col, int64_t batch, int64_t chan,
              int64_t img_w, int64_t img_h, int64_t col_w, int64_t col_h,
              int64_t ker_w, int64_t ker_h, int64_t stride_w, int64_t stride_h,
              int64_t pad_w, int64_t pad_h, int64_t dil_w, int64_t dil_h) {
    int64_t gsz = col_w * col_h * chan;
#pragma omp parallel for schedule(static)
    for (int64_t gid = 0; gid < gsz; ++gid) {
        for (int64_t n = 0; n < batch; ++n) {
            int64_t off_img_b = n * img_h * img_w * chan;
            int64_t off_col_b = n * col_h * col_w * ker_h * ker_w * chan;
            int64_t c = gid % chan;
            int64_t col_x = (gid / chan) % col_w;
            int64_t col_y = gid / (chan * col_w);
            int64_t bx = col_x * stride_w - pad_w, by = col_y * stride_h - pad_h;
            for (int64_t ky = 0; ky < ker_h; ++ky)
                for (int64_t kx = 0; kx < ker_w; ++kx) {
                    int64_t iy = by + ky * dil_h, ix = bx + kx * dil_w;
                    int64_t oc = off_col_b +
                                 (((col_y * col_w + col_x) * ker_h + ky) * ker_w + kx) * chan;
                    float v = 0;
                    if (ix >= 0 && ix < img_w && iy >= 0 && iy < img_h)
                        v = img[off_img_b + (iy * img_w + ix) * chan + c];
                    col[oc + c] = v;
                }
        }
    }
}

/* src/ops/conv.rs:404-498, including the reference's use of dilation_h for the
 * x tap and dilation_w for the y tap (:462-464). */
void o_col2im(const float *col, float *img, int64_t batch, int64_t chan,
              int64_t img_w, int64_t img_h, int64_t col_w, int64_t col_h,
              int64_t ker_w, int64_t ker_h, int64_t stride_w, int64_t stride_h,
              int64_t pad_w, int64_t pad_h, int64_t dil_w, int64_t dil_h) {
    int64_t gsz = img_w * img_h * chan;
#pragma omp parallel for schedule(static)
    for (int64_t gid = 0; gid < gsz; ++gid) {
        for (int64_t n = 0; n < batch; ++n) {
            int64_t off_img_b = n * img_h * img_w * chan;
            int64_t off_col_b = n * col_h * col_w * ker_h * ker_w * chan;
            int64_t c = gid % chan;
            int64_t img_x = (gid / chan) % img_w;
            int64_t img_y = gid / (chan * img_w);
            int64_t xp = img_x + pad_w, yp = img_y + pad_h;
            int64_t ker_ew = (ker_w - 1) * dil_w + 1, ker_eh = (ker_h - 1) * dil_h + 1;
            int64_t xs = xp < ker_ew ? 0 : (xp - ker_ew) / stride_w + 1;
            int64_t ys = yp < ker_eh ? 0 : (yp - ker_eh) / stride_h + 1;
            int64_t xe = IMIN(xp / stride_w + 1, col_w);
            int64_t ye = IMIN(yp / stride_h + 1, col_h);
            float val = 0;
            for (int64_t cx = xs; cx < xe; ++cx)
                for (int64_t cy = ys; cy < ye; ++cy) {
                    int64_t kx = xp - cx * stride_w, ky = yp - cy * stride_h;
                    if (kx % dil_h == 0 && ky % dil_w == 0) {
                        kx /= dil_h;
                        ky /= dil_w;
                        val += col[off_col_b +
                                   (((cy * col_w + cx) * ker_h + ky) * ker_w + kx) * chan + c];
                    }
                }
            img[off_img_b + (img_y * img_w + img_x) * chan + c] = val;
        }
    }
}

/* The number of OpenMP threads the loops above use from now on.  A launcher may start the process with
 * OMP_NUM_THREADS=1 (torch.distributed.run does); the timed CPU baseline sets what it wants explicitly. */
void o_set_num_threads(int n) {
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
}

int o_num_threads(void) {
    int n = 1;
#pragma omp parallel
    {
#pragma omp master
        {
#ifdef _OPENMP
            extern int omp_get_num_threads(void);
            n = omp_get_num_threads();
#endif
        }
    }
    return n;
}
