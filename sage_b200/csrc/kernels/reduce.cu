// Reductions: sum / prod / max / min over arbitrary axes, argmax / argmin over one axis.
//
// Reference: ReduceOperator::compute (src/ops/reduce.rs:258-325) gives each OUTPUT element to one
// work-item that loops serially over the reduced axes; a last-axis reduction is then fully
// uncoalesced.  Here a GROUP of G threads owns one output:
//   G = 1    adjacent threads own adjacent outputs   -> coalesced when a kept axis is contiguous
//   G = 32   a warp strides over the reduced run     -> coalesced when a reduced axis is contiguous
//   G = 256  a whole CTA per output for long runs
// partial results meet through warp shuffles and a shared-memory tree.
//
// Accumulator start: the reference initialises the accumulator to 0 for all four ops
// (reduce.rs:283), so max returns max(0, ...), min returns min(0, ...) and prod returns 0.  With
// ref_compat the group result is combined with that 0 once at the end, which is the same value.
#include <cuda_runtime.h>

#include <algorithm>

#include "kernels.h"
#include "launch.h"

namespace sage {
namespace k {

struct RDims {
    int ndim;
    long long ext[kMaxDims];
    long long str[kMaxDims];
};

template <typename T>
struct Ops {
    __device__ static T identity(int kind);
    __device__ static T apply(int kind, T a, T b);
};

template <>
struct Ops<float> {
    __device__ static float identity(int kind) {
        return kind == 0 ? 0.f : kind == 1 ? 1.f : kind == 2 ? -INFINITY : INFINITY;
    }
    __device__ static float apply(int kind, float a, float b) {
        return kind == 0 ? a + b : kind == 1 ? a * b : kind == 2 ? fmaxf(a, b) : fminf(a, b);
    }
};
template <>
struct Ops<int> {
    __device__ static int identity(int kind) { return kind == 0 ? 0 : kind == 1 ? 1 : kind == 2 ? INT_MIN : INT_MAX; }
    __device__ static int apply(int kind, int a, int b) {
        return kind == 0 ? a + b : kind == 1 ? a * b : kind == 2 ? max(a, b) : min(a, b);
    }
};
template <>
struct Ops<unsigned> {
    __device__ static unsigned identity(int kind) { return kind == 0 ? 0u : kind == 1 ? 1u : kind == 2 ? 0u : UINT_MAX; }
    __device__ static unsigned apply(int kind, unsigned a, unsigned b) {
        return kind == 0 ? a + b : kind == 1 ? a * b : kind == 2 ? max(a, b) : min(a, b);
    }
};

__device__ __forceinline__ long long translate(long long g, const RDims &d) {
    long long idx = 0;
#pragma unroll 1
    for (int i = d.ndim - 1; i >= 0; --i) {
        long long c = g % d.ext[i];
        g /= d.ext[i];
        idx += c * d.str[i];
    }
    return idx;
}

template <typename T>
__device__ __forceinline__ T shfl_down_t(T v, int off) {
    return __shfl_down_sync(0xffffffffu, v, off);
}

// G threads per output.  blockDim.x is a multiple of G (and of 32).
template <typename T, int G>
__global__ void __launch_bounds__(256) reduce_kernel(const T *__restrict__ x, T *__restrict__ y, RDims outer, RDims inner,
                                                     long long n_out, long long n_in, int kind, int ref_compat) {
    grid_dependency_sync();
    __shared__ T smem[8];
    const int groups_per_block = blockDim.x / G;
    long long out = (long long)blockIdx.x * groups_per_block + threadIdx.x / G;
    const int lane = threadIdx.x % G;
    // (For G == 256 every thread of the CTA shares `out`, so the early exit is uniform.)
    if (out >= n_out) return;
    const T *base = x + translate(out, outer);
    T acc = Ops<T>::identity(kind);
    if (inner.ndim == 1) {
        const long long s = inner.str[0];
        long long it = lane;
        // 4 independent loads in flight per thread
        T a1 = acc, a2 = acc, a3 = acc;
        for (; it + 3LL * G < n_in; it += 4LL * G) {
            T v0 = base[it * s], v1 = base[(it + G) * s], v2 = base[(it + 2LL * G) * s], v3 = base[(it + 3LL * G) * s];
            acc = Ops<T>::apply(kind, acc, v0);
            a1 = Ops<T>::apply(kind, a1, v1);
            a2 = Ops<T>::apply(kind, a2, v2);
            a3 = Ops<T>::apply(kind, a3, v3);
        }
        for (; it < n_in; it += G) acc = Ops<T>::apply(kind, acc, base[it * s]);
        acc = Ops<T>::apply(kind, Ops<T>::apply(kind, acc, a1), Ops<T>::apply(kind, a2, a3));
    } else {
        for (long long it = lane; it < n_in; it += G) acc = Ops<T>::apply(kind, acc, base[translate(it, inner)]);
    }
    if (G >= 32) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc = Ops<T>::apply(kind, acc, shfl_down_t(acc, off));
    }
    if (G == 256) {
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) smem[warp] = acc;
        __syncthreads();
        if (threadIdx.x < 8) {
            acc = smem[threadIdx.x];
#pragma unroll
            for (int off = 4; off > 0; off >>= 1) acc = Ops<T>::apply(kind, acc, __shfl_down_sync(0xffu, acc, off));
        }
    }
    if (lane == 0) {
        if (ref_compat) acc = Ops<T>::apply(kind, (T)0, acc);
        y[out] = acc;
    }
}

// Contiguous reduced run, 16-byte aligned rows: each thread reads 128-bit vectors, four in flight.
template <typename T, int G>
__global__ void __launch_bounds__(256) reduce_vec_kernel(const T *__restrict__ x, T *__restrict__ y, RDims outer, long long n_out,
                                                         long long n_in, int kind, int ref_compat) {
    grid_dependency_sync();
    struct alignas(16) V4 {
        T v[4];
    };
    __shared__ T smem[8];
    const int groups_per_block = blockDim.x / G;
    long long out = (long long)blockIdx.x * groups_per_block + threadIdx.x / G;
    const int lane = threadIdx.x % G;
    if (out >= n_out) return;
    const V4 *base = reinterpret_cast<const V4 *>(x + translate(out, outer));
    const long long nv = n_in >> 2;
    T a0 = Ops<T>::identity(kind), a1 = a0, a2 = a0, a3 = a0;
    long long it = lane;
    for (; it + 3LL * G < nv; it += 4LL * G) {
        const V4 p0 = base[it], p1 = base[it + G], p2 = base[it + 2LL * G], p3 = base[it + 3LL * G];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            a0 = Ops<T>::apply(kind, a0, p0.v[j]);
            a1 = Ops<T>::apply(kind, a1, p1.v[j]);
            a2 = Ops<T>::apply(kind, a2, p2.v[j]);
            a3 = Ops<T>::apply(kind, a3, p3.v[j]);
        }
    }
    for (; it < nv; it += G) {
        const V4 p0 = base[it];
#pragma unroll
        for (int j = 0; j < 4; ++j) a0 = Ops<T>::apply(kind, a0, p0.v[j]);
    }
    T acc = Ops<T>::apply(kind, Ops<T>::apply(kind, a0, a1), Ops<T>::apply(kind, a2, a3));
    if (G >= 2) {  // lane 0 of a group of G <= 32 lanes only ever takes in lanes of its own group
#pragma unroll
        for (int off = (G >= 32 ? 16 : G / 2); off > 0; off >>= 1) acc = Ops<T>::apply(kind, acc, shfl_down_t(acc, off));
    }
    if (G == 256) {
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) smem[warp] = acc;
        __syncthreads();
        if (threadIdx.x < 8) {
            acc = smem[threadIdx.x];
#pragma unroll
            for (int off = 4; off > 0; off >>= 1) acc = Ops<T>::apply(kind, acc, __shfl_down_sync(0xffu, acc, off));
        }
    }
    if (lane == 0) {
        if (ref_compat) acc = Ops<T>::apply(kind, (T)0, acc);
        y[out] = acc;
    }
}

// Puts the reduced axis with the smallest non-zero stride last (fastest) and merges axes that
// form one run, so that a group's lanes read neighbouring addresses.  The order of a parallel
// reduction is free, so this does not change what is computed.
static RDims canonical_inner(const Dims &in) {
    int order[kMaxDims];
    int n = 0;
    for (int i = 0; i < in.ndim; ++i)
        if (in.ext[i] > 1) order[n++] = i;
    // sort by stride descending
    for (int i = 0; i < n; ++i)
        for (int j = i + 1; j < n; ++j)
            if (in.str[order[j]] > in.str[order[i]]) {
                int t = order[i];
                order[i] = order[j];
                order[j] = t;
            }
    RDims r;
    r.ndim = 0;
    for (int i = 0; i < n; ++i) {
        long long e = in.ext[order[i]], s = in.str[order[i]];
        if (r.ndim > 0 && r.str[r.ndim - 1] == s * e) {
            r.ext[r.ndim - 1] *= e;
            r.str[r.ndim - 1] = s;
        } else {
            r.ext[r.ndim] = e;
            r.str[r.ndim] = s;
            ++r.ndim;
        }
    }
    if (r.ndim == 0) {
        r.ndim = 1;
        r.ext[0] = 1;
        r.str[0] = 0;
    }
    return r;
}

// Column reduction: x is [rows, cols] with unit column stride and `pitch` elements between rows; y[c]
// combines x[r, c] over the rows.  A warp reads 32 * VEC consecutive columns of a row (128 or, with 16-byte
// loads, 512 contiguous bytes); the 8 warps of a block take rows 8 apart, four rows in flight each.  With
// gridDim.y > 1 the rows are cut into chunks: every block leaves its chunk's result in `partial`
// [chunks, cols], takes a ticket for its column tile, and the block that draws the last ticket of a tile
// combines the tile's partial rows the same way.  The order of combination depends on the launch geometry
// only, so results repeat bit for bit.  `tickets` (one word per column tile) is zero before the launch and
// is left zero by it.
template <typename T, int VEC, int U, bool COHERENT>
__device__ __forceinline__ void reduce_cols_pass(const T *x, long long r0, long long r1, long long pitch, long long col, long long cols,
                                                 int kind, T (*part)[32 * VEC + 1]) {
    struct alignas(sizeof(T) * VEC) Vec {
        T v[VEC];
    };
    auto load = [](const T *p) {
        Vec v;
        if (!COHERENT) {
            v = *reinterpret_cast<const Vec *>(p);
        } else if (VEC == 4) {  // written by other blocks of this launch: read through the L2
            const int4 raw = __ldcg(reinterpret_cast<const int4 *>(p));
            memcpy(&v, &raw, sizeof(v));
        } else {
            const int raw = __ldcg(reinterpret_cast<const int *>(p));
            memcpy(&v, &raw, sizeof(raw));
        }
        return v;
    };
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    T acc[U][VEC];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[u][e] = Ops<T>::identity(kind);
    if (col < cols) {
        const T *base = x + col;
        long long r = r0 + ty;
        for (; r + 8 * (U - 1) < r1; r += 8 * U) {  // U rows in flight per thread
            Vec v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = load(base + (r + 8 * u) * pitch);
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[u][e] = Ops<T>::apply(kind, acc[u][e], v[u].v[e]);
        }
        for (; r < r1; r += 8) {
            const Vec v = load(base + r * pitch);
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[0][e] = Ops<T>::apply(kind, acc[0][e], v.v[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
#pragma unroll
        for (int w = 1; w < U; w *= 2)  // pairwise: (0 1) (2 3) ..., then (01 23) ...
#pragma unroll
            for (int u = 0; u + w < U; u += 2 * w) acc[u][e] = Ops<T>::apply(kind, acc[u][e], acc[u + w][e]);
        part[ty][tx * VEC + e] = acc[0][e];
    }
}

// The 8 partial rows in shared memory are combined in a fixed order; 32 * VEC columns spread over the 256 threads.
template <typename T, int VEC>
__device__ __forceinline__ void reduce_cols_store(T (*part)[32 * VEC + 1], T *y, long long cols, int kind, int from_zero) {
    for (int c = threadIdx.x; c < 32 * VEC; c += 256) {
        const long long out_col = (long long)blockIdx.x * 32 * VEC + c;
        if (out_col >= cols) continue;
        T a = part[0][c];
#pragma unroll
        for (int i = 1; i < 8; ++i) a = Ops<T>::apply(kind, a, part[i][c]);
        if (from_zero) a = Ops<T>::apply(kind, (T)0, a);
        y[out_col] = a;
    }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256) reduce_cols_kernel(const T *__restrict__ x, T *__restrict__ y, long long rows, long long cols,
                                                          long long pitch, long long rows_per_chunk, int kind, int ref_compat, T *partial,
                                                          unsigned *tickets) {
    grid_dependency_sync();
    __shared__ T part[8][32 * VEC + 1];
    __shared__ int last_of_tile;
    const long long col = ((long long)blockIdx.x * 32 + (threadIdx.x & 31)) * VEC;  // VEC consecutive columns per lane (cols % VEC == 0)
    const long long r0 = (long long)blockIdx.y * rows_per_chunk;
    const long long r1 = r0 + rows_per_chunk < rows ? r0 + rows_per_chunk : rows;
    reduce_cols_pass<T, VEC, 4, false>(x, r0, r1, pitch, col, cols, kind, part);
    __syncthreads();
    if (gridDim.y == 1) {
        reduce_cols_store<T, VEC>(part, y, cols, kind, ref_compat);
        return;
    }
    // the accumulator rule (start from 0) is applied once, by the block that combines the chunks
    reduce_cols_store<T, VEC>(part, partial + (long long)blockIdx.y * cols, cols, kind, 0);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned drawn = atomicAdd(tickets + blockIdx.x, 1u);
        last_of_tile = drawn == gridDim.y - 1;
        if (last_of_tile) tickets[blockIdx.x] = 0;  // every other block of the tile has drawn: nobody reads it again
    }
    __syncthreads();
    if (!last_of_tile) return;
    __threadfence();
    reduce_cols_pass<T, VEC, 8, true>(partial, 0, (long long)gridDim.y, cols, col, cols, kind, part);
    __syncthreads();
    reduce_cols_store<T, VEC>(part, y, cols, kind, ref_compat);
}

// Few slices of a long run: y[i] = x[i] (+) x[i + pitch] (+) ... over `slices` < 64 rows (the partial products of a
// GEMM split over K, [S, m * n] -> [m * n]).  A thread owns four consecutive outputs and keeps up to eight 16-byte
// loads in flight; the slices are combined in index order, so the result repeats bit for bit.
template <typename T>
__global__ void __launch_bounds__(256) reduce_slices_kernel(const T *__restrict__ x, T *__restrict__ y, long long n_out, long long pitch,
                                                            int slices, int kind, int ref_compat) {
    grid_dependency_sync();
    struct alignas(16) V4 {
        T v[4];
    };
    const long long i = ((long long)blockIdx.x * 256 + threadIdx.x) * 4;
    if (i >= n_out) return;
    const T *base = x + i;
    V4 acc = *reinterpret_cast<const V4 *>(base);
    int s = 1;
    for (; s + 7 < slices; s += 8) {
        V4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const V4 *>(base + (long long)(s + u) * pitch);
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc.v[e] = Ops<T>::apply(kind, acc.v[e], v[u].v[e]);
    }
    for (; s < slices; ++s) {
        const V4 v = *reinterpret_cast<const V4 *>(base + (long long)s * pitch);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc.v[e] = Ops<T>::apply(kind, acc.v[e], v.v[e]);
    }
    if (ref_compat) {
#pragma unroll
        for (int e = 0; e < 4; ++e) acc.v[e] = Ops<T>::apply(kind, (T)0, acc.v[e]);
    }
    *reinterpret_cast<V4 *>(y + i) = acc;
}

template <typename T>
static sage_status launch_reduce_cols(Context &ctx, int kind, const T *x, long long rows, long long cols, long long pitch, T *y, int compat_in) {
    const int compat = compat_in < 0 ? ctx.opts().ref_compat : compat_in;
    // 16-byte loads (4 columns per lane) when the rows allow; the partial rows are read with pitch = cols
    const bool vec = cols % 4 == 0 && pitch % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && cols >= 256;
    const long long tiles = vec ? (cols + 127) / 128 : (cols + 31) / 32;
    auto kernel = vec ? reduce_cols_kernel<T, 4> : reduce_cols_kernel<T, 1>;
    // two blocks per SM, at least 64 rows each (measured: more and smaller chunks are slower, [4096, 3072] 9.3 -> 13.9 us
    // with eight blocks per SM, because the block that combines a tile's partial rows then has more of them to read)
    long long chunks = (2LL * ctx.sm_count + tiles - 1) / tiles;
    chunks = std::max(1LL, std::min(chunks, rows / 64));
    if (tiles > Context::kTickets) chunks = 1;  // so many column tiles fill the machine without cutting the rows
    ctx.note_launch("reduce_cols");
    if (ctx.dry()) return SAGE_OK;
    if (chunks == 1) {
        launch_dependent(ctx.pdl, ctx.stream(), kernel, dim3((unsigned)tiles, 1), dim3(256), 0, x, y, rows, cols, pitch, rows, kind, compat,
                         (T *)nullptr, (unsigned *)nullptr);
        return ctx.check_cuda(cudaGetLastError(), "reduce_cols launch");
    }
    const long long per = (rows + chunks - 1) / chunks;
    chunks = (rows + per - 1) / per;
    Block *scratch = ctx.allocator().alloc((size_t)(chunks * cols) * sizeof(T));
    if (!scratch) return ctx.fail(SAGE_ERR_OOM, "out of memory for the partial results of a column reduction");
    T *partial = reinterpret_cast<T *>(scratch->ptr);
    launch_dependent(ctx.pdl, ctx.stream(), kernel, dim3((unsigned)tiles, (unsigned)chunks), dim3(256), 0, x, y, rows, cols, pitch, per, kind,
                     compat, partial, ctx.tickets());
    sage_status st = ctx.check_cuda(cudaGetLastError(), "reduce_cols launch");
    ctx.allocator().free(scratch);  // stream-ordered: reused only by work enqueued after this launch
    return st;
}

template <typename T>
static sage_status launch_reduce(Context &ctx, int kind, const T *x, const Dims &outer_in, const Dims &inner_in, T *y, int compat_in = -1) {
    RDims outer;
    outer.ndim = outer_in.ndim;
    for (int i = 0; i < outer_in.ndim; ++i) {
        outer.ext[i] = outer_in.ext[i];
        outer.str[i] = outer_in.str[i];
    }
    if (outer.ndim == 0) {
        outer.ndim = 1;
        outer.ext[0] = 1;
        outer.str[0] = 0;
    }
    RDims inner = canonical_inner(inner_in);
    long long n_out = outer_in.size(), n_in = 1;
    for (int i = 0; i < inner.ndim; ++i) n_in *= inner.ext[i];
    if (n_out == 0) return SAGE_OK;
    const bool inner_contig = inner.str[inner.ndim - 1] == 1;
    // [rows, cols] -> [cols] (bias gradients, sums over the batch): the kept axis is the contiguous one
    if (outer_in.ndim == 1 && outer_in.str[0] == 1 && inner.ndim == 1 && inner.str[0] >= n_out && n_out >= 2 && n_in >= 64 && n_out <= (1LL << 31))
        return launch_reduce_cols<T>(ctx, kind, x, n_in, n_out, inner.str[0], y, compat_in);
    // [S, n] -> [n] with few slices S (the partial products of a GEMM split over K)
    if (outer_in.ndim == 1 && outer_in.str[0] == 1 && inner.ndim == 1 && inner.str[0] >= n_out && n_in >= 2 && n_in < 64 && n_out >= 4096 &&
        n_out % 4 == 0 && inner.str[0] % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
        ctx.note_launch("reduce_slices");
        if (ctx.dry()) return SAGE_OK;
        const int compat = compat_in < 0 ? ctx.opts().ref_compat : compat_in;
        launch_dependent(ctx.pdl, ctx.stream(), reduce_slices_kernel<T>, dim3((unsigned)((n_out / 4 + 255) / 256)), dim3(256), 0, x, y, n_out,
                         inner.str[0], (int)n_in, kind, compat);
        return ctx.check_cuda(cudaGetLastError(), "reduce_slices launch");
    }
    // Few outputs, each over a long run (a sum over a whole tensor, the gradient of a scalar parameter): one
    // CTA per output would leave the machine idle.  The run is cut into S equal chunks, a first launch
    // reduces every (output, chunk) pair into scratch [n_out, S], a second one reduces the S partials; the
    // order of combination is fixed.  The accumulator rule (start from 0) is applied by the second launch.
    if (inner.ndim == 1 && n_out * 4 <= ctx.sm_count && n_in >= (1LL << 16) && outer.ndim < kMaxDims) {
        long long want = std::min<long long>(4LL * ctx.sm_count / n_out, n_in / 4096), S = 0;
        for (long long c = want; c >= want / 2 && c >= 2; --c)
            if (n_in % c == 0) {
                S = c;
                break;
            }
        if (S >= 2) {
            Block *scratch = ctx.dry() ? nullptr : ctx.allocator().alloc((size_t)(n_out * S) * sizeof(T));
            if (scratch || ctx.dry()) {
                const long long chunk = n_in / S;
                Dims outer2 = outer_in, inner2;
                if (outer2.ndim == 0) {
                    outer2.ndim = 1;
                    outer2.ext[0] = 1;
                    outer2.str[0] = 0;
                }
                outer2.ext[outer2.ndim] = S;
                outer2.str[outer2.ndim] = chunk * inner.str[0];
                ++outer2.ndim;
                inner2.ndim = 1;
                inner2.ext[0] = chunk;
                inner2.str[0] = inner.str[0];
                T *partial = scratch ? reinterpret_cast<T *>(scratch->ptr) : nullptr;
                sage_status st = launch_reduce<T>(ctx, kind, x, outer2, inner2, partial, 0);
                if (!st) {
                    Dims outer3, inner3;
                    outer3.ndim = 1;
                    outer3.ext[0] = n_out;
                    outer3.str[0] = S;
                    inner3.ndim = 1;
                    inner3.ext[0] = S;
                    inner3.str[0] = 1;
                    st = launch_reduce<T>(ctx, kind, partial, outer3, inner3, y, compat_in);
                }
                if (scratch) ctx.allocator().free(scratch);
                return st;
            }
        }
    }
    int G = 1;
    if (inner_contig && n_in >= 64) G = (n_in >= 8192 || n_out < 2LL * ctx.sm_count) ? 256 : 32;
    // A column reduction with very few outputs would leave the GPU idle; a CTA per output is
    // uncoalesced but at least parallel.
    if (!inner_contig && n_out < 1024 && n_in >= 4096) G = 256;
    const int threads = 256;
    long long blocks = (n_out + (threads / G) - 1) / (threads / G);
    const int compat = compat_in < 0 ? ctx.opts().ref_compat : compat_in;
    ctx.note_launch(G == 1 ? "reduce_g1" : G == 32 ? "reduce_g32" : "reduce_g256");
    if (ctx.dry()) return SAGE_OK;
    bool vec = G > 1 && inner.ndim == 1 && inner_contig && n_in % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0;
    for (int i = 0; i < outer.ndim && vec; ++i)
        if (outer.ext[i] > 1 && outer.str[i] % 4 != 0) vec = false;
    // Many short rows (the row sums of a softmax gradient, [49152, 128]): eight lanes per row, every 16-byte load of a
    // lane in flight at once, instead of a warp per row with one load per lane.
    if (vec && G == 32 && n_in <= 512 && n_out >= 64LL * ctx.sm_count) {
        blocks = (n_out + 31) / 32;
        launch_dependent(ctx.pdl, ctx.stream(), reduce_vec_kernel<T, 8>, dim3((unsigned)blocks), dim3(threads), 0, x, y, outer, n_out, n_in, kind, compat);
        return ctx.check_cuda(cudaGetLastError(), "reduce launch");
    }
    if (vec) {
        if (G == 32)
            launch_dependent(ctx.pdl, ctx.stream(), reduce_vec_kernel<T, 32>, dim3((unsigned)blocks), dim3(threads), 0, x, y, outer, n_out, n_in, kind, compat);
        else
            launch_dependent(ctx.pdl, ctx.stream(), reduce_vec_kernel<T, 256>, dim3((unsigned)blocks), dim3(threads), 0, x, y, outer, n_out, n_in, kind, compat);
        return ctx.check_cuda(cudaGetLastError(), "reduce launch");
    }
    if (G == 1)
        launch_dependent(ctx.pdl, ctx.stream(), reduce_kernel<T, 1>, dim3((unsigned)blocks), dim3(threads), 0, x, y, outer, inner, n_out, n_in, kind, compat);
    else if (G == 32)
        launch_dependent(ctx.pdl, ctx.stream(), reduce_kernel<T, 32>, dim3((unsigned)blocks), dim3(threads), 0, x, y, outer, inner, n_out, n_in, kind, compat);
    else
        launch_dependent(ctx.pdl, ctx.stream(), reduce_kernel<T, 256>, dim3((unsigned)blocks), dim3(threads), 0, x, y, outer, inner, n_out, n_in, kind, compat);
    return ctx.check_cuda(cudaGetLastError(), "reduce launch");
}

sage_status reduce(Context &ctx, int dtype, int kind, const void *x, const Dims &outer, const Dims &inner, void *y) {
    if (dtype == SAGE_F32) return launch_reduce<float>(ctx, kind, (const float *)x, outer, inner, (float *)y);
    if (dtype == SAGE_I32) return launch_reduce<int>(ctx, kind, (const int *)x, outer, inner, (int *)y);
    return launch_reduce<unsigned>(ctx, kind, (const unsigned *)x, outer, inner, (unsigned *)y);
}

// ---------------------------------------------------------------------------------- argmax / argmin
// Reference (reduce.rs:396-421): best = x[outer]; for i in 0..extent: if best < x_i (max) or
// best > x_i (min) { arg = i; best = x_i }.  So the first extremum wins, a NaN never replaces
// anything, and a NaN at position 0 is never replaced.  The parallel form keeps (value, index)
// pairs and prefers the smaller index on ties; a NaN at i > 0 is treated as "never wins", and a
// NaN at 0 pins the answer to 0.  Results are bit-exact with the serial loop.
__device__ __forceinline__ bool better(bool is_max, float v, unsigned i, float bv, unsigned bi) {
    if (v != v) return false;    // NaN candidate never wins
    if (bv != bv) return true;   // placeholder NaN (no candidate yet) loses to anything real
    if (is_max ? (v > bv) : (v < bv)) return true;
    return v == bv && i < bi;
}

template <int G>
__global__ void __launch_bounds__(256) reduce_arg_kernel(const float *__restrict__ x, unsigned *__restrict__ y, RDims outer,
                                                         long long n_out, long long n_in, long long stride, int is_max) {
    grid_dependency_sync();
    long long out = (long long)blockIdx.x * (blockDim.x / G) + threadIdx.x / G;
    const int lane = threadIdx.x % G;
    if (out >= n_out) return;
    const float *base = x + translate(out, outer);
    float bv = __int_as_float(0x7fc00000);  // "nothing yet"
    unsigned bi = 0xffffffffu;
    for (long long it = lane; it < n_in; it += G) {
        float v = base[it * stride];
        if (better(is_max, v, (unsigned)it, bv, bi)) {
            bv = v;
            bi = (unsigned)it;
        }
    }
    if (G == 32) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            float ov = __shfl_down_sync(0xffffffffu, bv, off);
            unsigned oi = __shfl_down_sync(0xffffffffu, bi, off);
            if (oi != 0xffffffffu && better(is_max, ov, oi, bv, bi)) {
                bv = ov;
                bi = oi;
            }
        }
    }
    if (lane == 0) {
        float first = base[0];
        // NaN at position 0 is never displaced; no real candidate at all also yields 0.
        y[out] = (first != first || bi == 0xffffffffu) ? 0u : bi;
    }
}

sage_status reduce_arg(Context &ctx, bool is_max, const float *x, const Dims &outer_in, long long inner_ext,
                       long long inner_str, uint32_t *y) {
    RDims outer;
    outer.ndim = outer_in.ndim;
    for (int i = 0; i < outer_in.ndim; ++i) {
        outer.ext[i] = outer_in.ext[i];
        outer.str[i] = outer_in.str[i];
    }
    if (outer.ndim == 0) {
        outer.ndim = 1;
        outer.ext[0] = 1;
        outer.str[0] = 0;
    }
    long long n_out = outer_in.size();
    if (n_out == 0) return SAGE_OK;
    const int G = (inner_str == 1 && inner_ext >= 64) ? 32 : 1;
    const int threads = 256;
    long long blocks = (n_out + (threads / G) - 1) / (threads / G);
    ctx.note_launch(G == 1 ? "reduce_arg_g1" : "reduce_arg_g32");
    if (ctx.dry()) return SAGE_OK;
    if (G == 1)
        launch_dependent(ctx.pdl, ctx.stream(), reduce_arg_kernel<1>, dim3((unsigned)blocks), dim3(threads), 0, x, y, outer, n_out, inner_ext, inner_str, is_max);
    else
        launch_dependent(ctx.pdl, ctx.stream(), reduce_arg_kernel<32>, dim3((unsigned)blocks), dim3(threads), 0, x, y, outer, n_out, inner_ext, inner_str, is_max);
    return ctx.check_cuda(cudaGetLastError(), "reduce_arg launch");
}

}  // namespace k
}  // namespace sage
