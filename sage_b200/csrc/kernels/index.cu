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

// The same when the index does not vary along the last axis and x is contiguous along it (an embedding lookup: the
// index is a broadcast view, every output row is a row of the table): 16 bytes per thread and one unravelling per
// 16 bytes, in 32-bit arithmetic (the per-element kernel spends its time in 64-bit divisions: [4096, 768] rows of a
// table took 16 us).  `chunks_per_row` = ext[last] / 4; the caller has checked alignment and that n / 4 < 2^31.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint32_t *__restrict__ x, const uint32_t *__restrict__ ind,
                                                          uint32_t *__restrict__ y, IDims d, int axis, unsigned n_chunks, unsigned chunks_per_row) {
    grid_dependency_sync();
    for (unsigned g = blockIdx.x * blockDim.x + threadIdx.x; g < n_chunks; g += gridDim.x * blockDim.x) {
        unsigned rem = g / chunks_per_row;
        const unsigned chunk = g - rem * chunks_per_row;
        long long ind_idx = 0, x_idx = 0;
#pragma unroll 1
        for (int i = d.ndim - 2; i >= 0; --i) {
            const unsigned e = (unsigned)d.ext[i], q = rem / e, c = rem - q * e;
            rem = q;
            ind_idx += (long long)c * d.str[i];
            if (i != axis) x_idx += (long long)c * d.str2[i];
        }
        const long long t = ind[ind_idx];
        const uint4 v = *reinterpret_cast<const uint4 *>(x + x_idx + t * d.str2[axis] + 4u * chunk);
        *reinterpret_cast<uint4 *>(y + 4ll * g) = v;
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
    const int last = d.ndim - 1;
    bool rows = last >= 1 && axis != last && d.str[last] == 0 && d.str2[last] == 1 && d.ext[last] % 4 == 0 && n / 4 < (1ll << 31) &&
                reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
    for (int i = 0; i < last && rows; ++i)
        if ((d.ext[i] > 1 || i == axis) && d.str2[i] % 4 != 0) rows = false;  // every gathered row starts on a 16-byte boundary
    if (rows)
        launch_dependent(ctx.pdl, ctx.stream(), gather_rows_kernel, dim3(grid_for(ctx, n / 4)), dim3(256), 0, x, ind, y, d, axis, (unsigned)(n / 4),
                         (unsigned)(d.ext[last] / 4));
    else
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

// ---------------------------------------------------------------- random fills (src/ops/rand.rs:40-140)
// The reference's generator: one xorshift-style mix of two 32-bit seeds per element (rand.rs:40-48), the
// product with 2.3283064e-10 taken in double precision as OpenCL C does for an unsuffixed literal.
__device__ __forceinline__ float xorshift128(unsigned seed_x, unsigned seed_y) {
    const unsigned t = seed_x ^ (seed_x << 11);
    const unsigned rndint = seed_y ^ (seed_y >> 19) ^ (t ^ (t >> 8));
    return (float)((double)rndint * 2.3283064e-10);
}

__global__ void __launch_bounds__(256) rand_uniform_kernel(float *__restrict__ y, unsigned seed_x, unsigned seed_y, long long n) {
    grid_dependency_sync();
    for (long long g = (long long)blockIdx.x * 256 + threadIdx.x; g < n; g += (long long)gridDim.x * 256)
        y[g] = xorshift128(seed_x + (unsigned)g, seed_y + (unsigned)g);  // rand.rs:69-72
}

// Box-Muller on pairs (rand.rs:108-121); theta is formed in double like `2 * M_PI * u2` in OpenCL C.  The
// reference writes y[2 gid + 1] even when the tensor has an odd number of elements; here that store is skipped.
__global__ void __launch_bounds__(256) rand_normal_kernel(float *__restrict__ y, unsigned seed_x, unsigned seed_y, long long n) {
    grid_dependency_sync();
    const long long pairs = (n + 1) / 2;
    for (long long g = (long long)blockIdx.x * 256 + threadIdx.x; g < pairs; g += (long long)gridDim.x * 256) {
        const float u1 = xorshift128(seed_x + (unsigned)g * 2u, seed_y);
        const float u2 = xorshift128(seed_x + (unsigned)g * 2u + 1u, seed_y);
        const float rsq = -2.f * logf(u1);
        const float theta = (float)(2.0 * 3.14159265358979323846 * (double)u2);
        const float r = sqrtf(rsq);
        y[2 * g] = r * cosf(theta);
        if (2 * g + 1 < n) y[2 * g + 1] = r * sinf(theta);
    }
}

sage_status rand_fill(Context &ctx, bool normal, float *y, long long n, unsigned seed_x, unsigned seed_y) {
    ctx.note_launch(normal ? "rand_normal" : "rand_uniform");
    if (ctx.dry() || n == 0) return SAGE_OK;
    const long long work = normal ? (n + 1) / 2 : n;
    if (normal)
        launch_dependent(ctx.pdl, ctx.stream(), rand_normal_kernel, dim3(grid_for(ctx, work)), dim3(256), 0, y, seed_x, seed_y, n);
    else
        launch_dependent(ctx.pdl, ctx.stream(), rand_uniform_kernel, dim3(grid_for(ctx, work)), dim3(256), 0, y, seed_x, seed_y, n);
    return ctx.check_cuda(cudaGetLastError(), "rand launch");
}

}  // namespace k
}  // namespace sage
