// softmax / log_sum_exp / layer_norm over contiguous rows, one kernel each.
//
// The reference builds these from 4-7 separate kernels with a DRAM round trip between each
// (src/ops/nn.rs:42-100 over src/ops/reduce.rs:59-82).  The arithmetic below is the same
// composition, evaluated per row with the row held in registers:
//   softmax     m = max_j x_j ; e_j = exp(x_j - m) ; y_j = e_j / sum_j e_j
//   log_sum_exp c = max_j x_j ; y = log(sum_j exp(x_j - c)) + c
//   layer_norm  mean = sum(x)/C ; var = sum(x^2)/C - mean^2 ; y = (x-mean)/sqrt(var+eps)*gamma + beta
// With ref_compat the two max reductions start from 0 like the reference's accumulator
// (reduce.rs:283), i.e. m = max(0, max_j x_j).
//
// A warp owns a row when it fits in registers (cols <= 2048, cols % 4 == 0): lanes read float4
// chunks `lane + 32*i`, so each pass over HBM is one coalesced read and one coalesced write.
// Other shapes use a CTA per row that re-reads the row (L2-resident) per pass.
#include <cuda.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "launch.h"
#include "gemm_tc_device.inc"  // split_tf32_value

namespace sage {
namespace k {

enum { ROW_SOFTMAX = 0, ROW_LSE = 1, ROW_LN = 2 };

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

struct RowParams {
    const float *x;
    float *y;
    long long rows, cols;
    const float *gamma, *beta;
    int gamma_stride, beta_stride;
    float eps;
    int ref_compat;
    float *hi;        // when set: also write the tf32 hi / lo planes of y (softmax, layer_norm), laid out like y
    long long plane;  // floats from the hi to the lo plane
};

__device__ __forceinline__ void row_store4(const RowParams &p, long long at, float4 o) {
    if (p.y) *reinterpret_cast<float4 *>(p.y + at) = o;  // y is null when only the planes are wanted
    if (p.hi) {
        float4 h, l;
        sage_tc::split_tf32_value(o.x, &h.x, &l.x);
        sage_tc::split_tf32_value(o.y, &h.y, &l.y);
        sage_tc::split_tf32_value(o.z, &h.z, &l.z);
        sage_tc::split_tf32_value(o.w, &h.w, &l.w);
        *reinterpret_cast<float4 *>(p.hi + at) = h;
        *reinterpret_cast<float4 *>(p.hi + p.plane + at) = l;
    }
}
__device__ __forceinline__ void row_store1(const RowParams &p, long long at, float o) {
    if (p.y) p.y[at] = o;
    if (p.hi) {
        float h, l;
        sage_tc::split_tf32_value(o, &h, &l);
        p.hi[at] = h;
        p.hi[p.plane + at] = l;
    }
}

// V = float4 chunks per lane; the row has cols/4 <= 32*V chunks.
template <int MODE, int V>
__global__ void __launch_bounds__(256) row_warp_kernel(RowParams p) {
    grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= p.rows) return;
    const int chunks = (int)(p.cols >> 2);
    const float4 *xr = reinterpret_cast<const float4 *>(p.x + row * p.cols);
    float4 v[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) v[i] = __ldg(xr + c);
    }
    if (MODE == ROW_LN) {
        // scale and shift: 16 bytes at a time when they are plain vectors (the same for every row: L1 hits)
        const bool vec_gb = p.gamma_stride == 1 && p.beta_stride == 1 && ((reinterpret_cast<unsigned long long>(p.gamma) | reinterpret_cast<unsigned long long>(p.beta)) & 15ull) == 0;
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i)
            if (lane + 32 * i < chunks) {
                s1 += (v[i].x + v[i].y) + (v[i].z + v[i].w);
                s2 += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
            }
        s1 = warp_sum(s1);
        s2 = warp_sum(s2);
        const float n = (float)p.cols;
        const float mean = s1 / n;
        const float var = s2 / n - mean * mean;
        const float denom = sqrtf(var + p.eps);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int c = lane + 32 * i;
            if (c < chunks) {
                const int e = c * 4;
                float4 g, b;
                if (vec_gb) {
                    g = __ldg(reinterpret_cast<const float4 *>(p.gamma) + c);
                    b = __ldg(reinterpret_cast<const float4 *>(p.beta) + c);
                } else {
                    g = make_float4(p.gamma[(e + 0) * p.gamma_stride], p.gamma[(e + 1) * p.gamma_stride], p.gamma[(e + 2) * p.gamma_stride],
                                    p.gamma[(e + 3) * p.gamma_stride]);
                    b = make_float4(p.beta[(e + 0) * p.beta_stride], p.beta[(e + 1) * p.beta_stride], p.beta[(e + 2) * p.beta_stride],
                                    p.beta[(e + 3) * p.beta_stride]);
                }
                float4 o;
                o.x = (v[i].x - mean) / denom * g.x + b.x;
                o.y = (v[i].y - mean) / denom * g.y + b.y;
                o.z = (v[i].z - mean) / denom * g.z + b.z;
                o.w = (v[i].w - mean) / denom * g.w + b.w;
                row_store4(p, row * p.cols + 4LL * c, o);
            }
        }
        return;
    }
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < V; ++i)
        if (lane + 32 * i < chunks) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    m = warp_max(m);
    if (p.ref_compat) m = fmaxf(0.f, m);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i)
        if (lane + 32 * i < chunks) {
            v[i].x = expf(v[i].x - m);
            v[i].y = expf(v[i].y - m);
            v[i].z = expf(v[i].z - m);
            v[i].w = expf(v[i].w - m);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    s = warp_sum(s);
    if constexpr (MODE == ROW_LSE) {
        if (lane == 0) p.y[row] = logf(s) + m;
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int c = lane + 32 * i;
            if (c < chunks) {
                float4 o;
                o.x = v[i].x / s;
                o.y = v[i].y / s;
                o.z = v[i].z / s;
                o.w = v[i].w / s;
                row_store4(p, row * p.cols + 4LL * c, o);
            }
        }
    }
}

__device__ __forceinline__ float block_reduce(float v, bool is_max, float *smem) {
    v = is_max ? warp_max(v) : warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // smem may still be read from a previous call
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    const int nw = blockDim.x >> 5;
    float r = lane < nw ? smem[lane] : (is_max ? -INFINITY : 0.f);
    r = is_max ? warp_max(r) : warp_sum(r);
    return r;
}

// Rows of 2049..16384 elements (multiple of 4): a CTA of 256 threads owns a row and keeps it in
// registers (V float4 chunks per thread), so HBM still sees one read and one write per element.
template <int MODE, int V>
__global__ void __launch_bounds__(256) row_cta_kernel(RowParams p) {
    grid_dependency_sync();
    __shared__ float smem[8];
    const long long row = blockIdx.x;
    const int chunks = (int)(p.cols >> 2);
    const float4 *xr = reinterpret_cast<const float4 *>(p.x + row * p.cols);
    float4 v[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < chunks) v[i] = __ldg(xr + c);
    }
    if (MODE == ROW_LN) {
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i)
            if (threadIdx.x + 256 * i < chunks) {
                s1 += (v[i].x + v[i].y) + (v[i].z + v[i].w);
                s2 += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
            }
        s1 = block_reduce(s1, false, smem);
        s2 = block_reduce(s2, false, smem);
        const float n = (float)p.cols;
        const float mean = s1 / n;
        const float var = s2 / n - mean * mean;
        const float denom = sqrtf(var + p.eps);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int c = threadIdx.x + 256 * i;
            if (c < chunks) {
                const int e = c * 4;
                float4 o;
                o.x = (v[i].x - mean) / denom * p.gamma[(e + 0) * p.gamma_stride] + p.beta[(e + 0) * p.beta_stride];
                o.y = (v[i].y - mean) / denom * p.gamma[(e + 1) * p.gamma_stride] + p.beta[(e + 1) * p.beta_stride];
                o.z = (v[i].z - mean) / denom * p.gamma[(e + 2) * p.gamma_stride] + p.beta[(e + 2) * p.beta_stride];
                o.w = (v[i].w - mean) / denom * p.gamma[(e + 3) * p.gamma_stride] + p.beta[(e + 3) * p.beta_stride];
                row_store4(p, row * p.cols + 4LL * c, o);
            }
        }
        return;
    }
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < V; ++i)
        if (threadIdx.x + 256 * i < chunks) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    m = block_reduce(m, true, smem);
    if (p.ref_compat) m = fmaxf(0.f, m);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i)
        if (threadIdx.x + 256 * i < chunks) {
            v[i].x = expf(v[i].x - m);
            v[i].y = expf(v[i].y - m);
            v[i].z = expf(v[i].z - m);
            v[i].w = expf(v[i].w - m);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    s = block_reduce(s, false, smem);
    if constexpr (MODE == ROW_LSE) {
        if (threadIdx.x == 0) p.y[row] = logf(s) + m;
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int c = threadIdx.x + 256 * i;
            if (c < chunks) row_store4(p, row * p.cols + 4LL * c, make_float4(v[i].x / s, v[i].y / s, v[i].z / s, v[i].w / s));
        }
    }
}

// Any row length: one CTA per row, the row is re-read per pass.
template <int MODE>
__global__ void __launch_bounds__(256) row_block_kernel(RowParams p) {
    grid_dependency_sync();
    __shared__ float smem[8];
    const long long row = blockIdx.x;
    const float *xr = p.x + row * p.cols;
    if (MODE == ROW_LN) {
        float s1 = 0.f, s2 = 0.f;
        for (long long j = threadIdx.x; j < p.cols; j += blockDim.x) {
            float v = xr[j];
            s1 += v;
            s2 += v * v;
        }
        s1 = block_reduce(s1, false, smem);
        s2 = block_reduce(s2, false, smem);
        const float n = (float)p.cols;
        const float mean = s1 / n;
        const float var = s2 / n - mean * mean;
        const float denom = sqrtf(var + p.eps);
        for (long long j = threadIdx.x; j < p.cols; j += blockDim.x)
            row_store1(p, row * p.cols + j, (xr[j] - mean) / denom * p.gamma[j * p.gamma_stride] + p.beta[j * p.beta_stride]);
        return;
    }
    float m = -INFINITY;
    for (long long j = threadIdx.x; j < p.cols; j += blockDim.x) m = fmaxf(m, xr[j]);
    m = block_reduce(m, true, smem);
    if (p.ref_compat) m = fmaxf(0.f, m);
    float s = 0.f;
    for (long long j = threadIdx.x; j < p.cols; j += blockDim.x) s += expf(xr[j] - m);
    s = block_reduce(s, false, smem);
    if constexpr (MODE == ROW_LSE) {
        if (threadIdx.x == 0) p.y[row] = logf(s) + m;
    } else {
        for (long long j = threadIdx.x; j < p.cols; j += blockDim.x) row_store1(p, row * p.cols + j, expf(xr[j] - m) / s);
    }
}

template <int MODE>
static sage_status launch_rows(Context &ctx, RowParams p, const char *name) {
    ctx.note_launch(name);
    if (ctx.dry() || p.rows == 0) return SAGE_OK;
    p.ref_compat = ctx.opts().ref_compat;
    cudaError_t err = cudaSuccess;
    const bool aligned = (reinterpret_cast<uintptr_t>(p.x) % 16 == 0) &&
                         (MODE == ROW_LSE || reinterpret_cast<uintptr_t>(p.y) % 16 == 0) &&
                         (!p.hi || (reinterpret_cast<uintptr_t>(p.hi) % 16 == 0 && p.plane % 4 == 0));
    if (p.cols % 4 == 0 && p.cols <= 2048 && aligned) {
        const int chunks = (int)(p.cols / 4);
        const int v = (chunks + 31) / 32;
        // a warp per row; with few rows per SM smaller blocks spread them more evenly ([4096, 768]: 12.1 -> 11.0 us)
        const int tpb = p.rows <= 64LL * ctx.sm_count ? 128 : 256;
        const unsigned blocks = (unsigned)((p.rows + tpb / 32 - 1) / (tpb / 32));
        cudaStream_t s = ctx.stream();
        if (v <= 1) err = launch_dependent(ctx.pdl, s, row_warp_kernel<MODE, 1>, dim3(blocks), dim3(tpb), 0, p);
        else if (v <= 2) err = launch_dependent(ctx.pdl, s, row_warp_kernel<MODE, 2>, dim3(blocks), dim3(tpb), 0, p);
        else if (v <= 4) err = launch_dependent(ctx.pdl, s, row_warp_kernel<MODE, 4>, dim3(blocks), dim3(tpb), 0, p);
        else if (v <= 8) err = launch_dependent(ctx.pdl, s, row_warp_kernel<MODE, 8>, dim3(blocks), dim3(tpb), 0, p);
        else err = launch_dependent(ctx.pdl, s, row_warp_kernel<MODE, 16>, dim3(blocks), dim3(tpb), 0, p);
    } else if (p.cols % 4 == 0 && p.cols <= 16384 && aligned && p.rows < (1LL << 31)) {
        const int v = (int)((p.cols / 4 + 255) / 256);
        const unsigned blocks = (unsigned)p.rows;
        cudaStream_t s = ctx.stream();
        if (v <= 4) err = launch_dependent(ctx.pdl, s, row_cta_kernel<MODE, 4>, dim3(blocks), dim3(256), 0, p);
        else if (v <= 8) err = launch_dependent(ctx.pdl, s, row_cta_kernel<MODE, 8>, dim3(blocks), dim3(256), 0, p);
        else err = launch_dependent(ctx.pdl, s, row_cta_kernel<MODE, 16>, dim3(blocks), dim3(256), 0, p);
    } else {
        err = launch_dependent(ctx.pdl, ctx.stream(), row_block_kernel<MODE>, dim3((unsigned)p.rows), dim3(256), 0, p);
    }
    return ctx.check_cuda(err, name);
}

sage_status softmax_rows(Context &ctx, const float *x, float *y, long long rows, long long cols, float *hi, long long plane) {
    RowParams p{x, y, rows, cols, nullptr, nullptr, 0, 0, 0.f, 1, hi, plane};
    return launch_rows<ROW_SOFTMAX>(ctx, p, "softmax_rows");
}

sage_status lse_rows(Context &ctx, const float *x, float *y, long long rows, long long cols) {
    RowParams p{x, y, rows, cols, nullptr, nullptr, 0, 0, 0.f, 1, nullptr, 0};
    return launch_rows<ROW_LSE>(ctx, p, "lse_rows");
}

sage_status layernorm_rows(Context &ctx, const float *x, float *y, long long rows, long long cols, const float *gamma,
                           int gamma_stride, const float *beta, int beta_stride, float eps, float *hi, long long plane) {
    RowParams p{x, y, rows, cols, gamma, beta, gamma_stride, beta_stride, eps, 1, hi, plane};
    return launch_rows<ROW_LN>(ctx, p, "layernorm_rows");
}

}  // namespace k
}  // namespace sage
