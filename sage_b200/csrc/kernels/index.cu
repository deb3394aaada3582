// gather / scatter / strided copy.  Pure data movement: results are bit-exact copies.
//
// Reference kernels: gather (src/ops/core.rs:674-705), scatter (:784-819), unslice (:591-600),
// concat (:917-924).  One thread per output (gather, copy) or per index (scatter) element;
// neighbouring threads walk the innermost axis, so accesses coalesce whenever that axis is
// contiguous in the operand (embedding rows, [N,C] logits).
#include <cuda_runtime.h>

#include "kernels.h"
#include "launch.h"

namespace sage {
namespace k {

struct IDims {
    int ndim;
    long long ext[kMaxDims];
    long long str[kMaxDims];   // index tensor / source strides
    long long str2[kMaxDims];  // second operand strides
};

// y[g] = x[ sum_{i != axis} c_i * x_str[i] + ind[...] * x_str[axis] ],  c = unravel(g, ind extents)
__global__ void __launch_bounds__(256) gather_kernel(const uint32_t *__restrict__ x, const uint32_t *__restrict__ ind,
                                                     uint32_t *__restrict__ y, IDims d, int axis, long long n) {
    grid_dependency_sync();
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (long long)gridDim.x * blockDim.x) {
        long long rem = g, ind_idx = 0, x_idx = 0;
#pragma unroll 1
        for (int i = d.ndim - 1; i >= 0; --i) {
            long long c = rem % d.ext[i];
            rem /= d.ext[i];
            ind_idx += c * d.str[i];
            if (i != axis) x_idx += c * d.str2[i];
        }
        long long t = ind[ind_idx];  // read as uint whatever the declared dtype (core.rs:684)
        y[g] = x[x_idx + t * d.str2[axis]];
    }
}

// y[ sum_{i != axis} c_i * y_str[i] + ind[...] * y_str[axis] ] += x[ sum c_i * x_str[i] ]
// The reference does a plain read-modify-write, which is only defined when no two work-items
// hit the same output.  atomicAdd gives the same bits in that case (0 + v == v) and the
// mathematically expected sum when indices repeat.
__global__ void __launch_bounds__(256) scatter_kernel(const float *__restrict__ x, const uint32_t *__restrict__ ind,
                                                      float *__restrict__ y, IDims d, IDims xs, int axis, long long n) {
    grid_dependency_sync();
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (long long)gridDim.x * blockDim.x) {
        long long rem = g, ind_idx = 0, x_idx = 0, y_idx = 0;
#pragma unroll 1
        for (int i = d.ndim - 1; i >= 0; --i) {
            long long c = rem % d.ext[i];
            rem /= d.ext[i];
            ind_idx += c * d.str[i];
            x_idx += c * xs.str[i];
            if (i != axis) y_idx += c * d.str2[i];
        }
        long long t = ind[ind_idx];
        atomicAdd(y + y_idx + t * d.str2[axis], x[x_idx]);
    }
}

__global__ void __launch_bounds__(256) strided_copy_kernel(const uint32_t *__restrict__ x, uint32_t *__restrict__ y,
                                                           IDims d, long long n) {
    grid_dependency_sync();
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n; g += (long long)gridDim.x * blockDim.x) {
        long long rem = g, xi = 0, yi = 0;
#pragma unroll 1
        for (int i = d.ndim - 1; i >= 0; --i) {
            long long c = rem % d.ext[i];
            rem /= d.ext[i];
            xi += c * d.str[i];
            yi += c * d.str2[i];
        }
        y[yi] = x[xi];
    }
}

static unsigned grid_for(Context &ctx, long long n) {
    long long blocks = (n + 255) / 256;
    long long cap = (long long)ctx.sm_count * 16;
    return (unsigned)(blocks < cap ? blocks : cap);
}

sage_status gather(Context &ctx, const uint32_t *x, const long long *x_str, const uint32_t *ind, const Dims &ind_dims,
                   int axis, uint32_t *y) {
    IDims d;
    d.ndim = ind_dims.ndim;
    for (int i = 0; i < d.ndim; ++i) {
        d.ext[i] = ind_dims.ext[i];
        d.str[i] = ind_dims.str[i];
        d.str2[i] = x_str[i];
    }
    long long n = ind_dims.size();
    ctx.note_launch("gather");
    if (ctx.dry() || n == 0) return SAGE_OK;
    launch_dependent(ctx.pdl, ctx.stream(), gather_kernel, dim3(grid_for(ctx, n)), dim3(256), 0, x, ind, y, d, axis, n);
    return ctx.check_cuda(cudaGetLastError(), "gather launch");
}

sage_status scatter_add(Context &ctx, const float *x, const long long *x_str, const uint32_t *ind, const Dims &ind_dims,
                        int axis, float *y, const long long *y_str) {
    IDims d, xs;
    d.ndim = xs.ndim = ind_dims.ndim;
    for (int i = 0; i < d.ndim; ++i) {
        d.ext[i] = ind_dims.ext[i];
        d.str[i] = ind_dims.str[i];
        d.str2[i] = y_str[i];
        xs.str[i] = x_str[i];
    }
    long long n = ind_dims.size();
    ctx.note_launch("scatter");
    if (ctx.dry() || n == 0) return SAGE_OK;
    launch_dependent(ctx.pdl, ctx.stream(), scatter_kernel, dim3(grid_for(ctx, n)), dim3(256), 0, x, ind, y, d, xs, axis, n);
    return ctx.check_cuda(cudaGetLastError(), "scatter launch");
}

sage_status strided_copy(Context &ctx, const uint32_t *x, const Dims &dims, uint32_t *y, const long long *y_str) {
    IDims d;
    d.ndim = dims.ndim;
    for (int i = 0; i < d.ndim; ++i) {
        d.ext[i] = dims.ext[i];
        d.str[i] = dims.str[i];
        d.str2[i] = y_str[i];
    }
    long long n = dims.size();
    ctx.note_launch("strided_copy");
    if (ctx.dry() || n == 0) return SAGE_OK;
    launch_dependent(ctx.pdl, ctx.stream(), strided_copy_kernel, dim3(grid_for(ctx, n)), dim3(256), 0, x, y, d, n);
    return ctx.check_cuda(cudaGetLastError(), "strided_copy launch");
}

}  // namespace k
}  // namespace sage
