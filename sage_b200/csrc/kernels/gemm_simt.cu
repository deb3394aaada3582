// fp32 SIMT GEMM: C[M,N] = op(A) * op(B), row-major, all four transpose modes, strided-batched.
//
// Reference: Gemm::compute_direct / GemmBatched::compute_direct (src/ops/gemm.rs:176-250,
// 338-421) launch the "XgemmDirect" kernel with 8x8x8 tiles and one output per thread
// (src/ops/kernels/matmul_direct.opencl:514-709).  This kernel computes the same fp32 products
// with per-output accumulation in increasing k (each thread walks k = 0..K-1 for its outputs, one
// fused multiply-add per step), using 128x128x16 tiles and 8x8 outputs per thread.  It serves
// shapes the tensor-core path cannot take (unaligned leading dimensions, tiny problems) and is
// the cross-check for that path in the tests.
#include <cuda_runtime.h>

#include "kernels.h"

namespace sage {
namespace k {

namespace {
constexpr int BM = 128, BN = 128, BK = 16;

struct GemmP {
    long long m, n, k;
    const float *a;
    long long lda, sa;
    const float *b;
    long long ldb, sb;
    float *c;
    long long ldc, sc;
    long long tiles_n, tiles_m, batch;  // the grid is one-dimensional: block = (batch * tiles_m + tile_m) * tiles_n + tile_n
};

template <bool TA, bool TB>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmP p) {
    __shared__ __align__(16) float As[BK][BM];
    __shared__ __align__(16) float Bs[BK][BN];
    const int t = threadIdx.x;
    // a one-dimensional grid: the y / z extents of a grid stop at 65535, which many small batches or a very tall
    // M would exceed
    const long long tile_n = blockIdx.x % p.tiles_n, rest = blockIdx.x / p.tiles_n;
    const long long tile_m = rest % p.tiles_m, bz = rest / p.tiles_m;
    const long long m0 = tile_m * BM, n0 = tile_n * BN;
    const float *A = p.a + bz * p.sa;
    const float *B = p.b + bz * p.sb;
    float *C = p.c + bz * p.sc;
    const int tx = t % 16, ty = t / 16;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    for (long long k0 = 0; k0 < p.k; k0 += BK) {
        // ---- stage A'(i,p) into As[p][i]
        if (!TA) {
            const int i = t / 2, pc = (t % 2) * 8;
            const long long gi = m0 + i;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const long long gp = k0 + pc + q;
                As[pc + q][i] = (gi < p.m && gp < p.k) ? A[gi * p.lda + gp] : 0.f;
            }
        } else {
            const int pp = t / 16, i0 = (t % 16) * 8;
            const long long gp = k0 + pp;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const long long gi = m0 + i0 + q;
                As[pp][i0 + q] = (gi < p.m && gp < p.k) ? A[gp * p.lda + gi] : 0.f;
            }
        }
        // ---- stage B'(p,j) into Bs[p][j]
        if (!TB) {
            const int pp = t / 16, j0 = (t % 16) * 8;
            const long long gp = k0 + pp;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const long long gj = n0 + j0 + q;
                Bs[pp][j0 + q] = (gj < p.n && gp < p.k) ? B[gp * p.ldb + gj] : 0.f;
            }
        } else {
            const int j = t / 2, pc = (t % 2) * 8;
            const long long gj = n0 + j;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const long long gp = k0 + pc + q;
                Bs[pc + q][j] = (gj < p.n && gp < p.k) ? B[gj * p.ldb + gp] : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int pp = 0; pp < BK; ++pp) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[pp][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&As[pp][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[pp][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[pp][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long gi = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (gi >= p.m) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long gj = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (gj < p.n) C[gi * p.ldc + gj] = acc[i][j];
        }
    }
}
// Few outputs, long K (a classifier head: 32 x 2 outputs, K = 768): one warp per output element,
// the lanes share K, so the tile kernel's single CTA walking K alone is avoided.
__global__ void __launch_bounds__(256) gemm_skinny_kernel(GemmP p, long long sai, long long sak, long long sbk, long long sbj) {
    const int lane = threadIdx.x & 31;
    const long long out = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long per_batch = p.m * p.n;
    if (out >= per_batch * p.batch) return;
    const long long bz = out / per_batch, rem = out % per_batch;
    const long long i = rem / p.n, j = rem % p.n;
    const float *A = p.a + bz * p.sa + i * sai;
    const float *B = p.b + bz * p.sb + j * sbj;
    float acc = 0.f;
    for (long long kk = lane; kk < p.k; kk += 32) acc = fmaf(A[kk * sak], B[kk * sbk], acc);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) p.c[bz * p.sc + i * p.ldc + j] = acc;
}
}  // namespace

sage_status gemm_simt(Context &ctx, const GemmArgs &g) {
    ctx.note_launch("gemm_simt");
    if (ctx.dry() || g.m == 0 || g.n == 0 || g.batch == 0) return SAGE_OK;
    GemmP p{g.m, g.n, g.k, g.a, g.lda, g.stride_a, g.b, g.ldb, g.stride_b, g.c, g.ldc, g.stride_c, (g.n + BN - 1) / BN, (g.m + BM - 1) / BM, g.batch};
    const long long grid_limit = 0x7fffffffLL;
    if (g.m * g.n <= 8192 && g.k >= 128 && (g.m * g.n * g.batch + 7) / 8 <= grid_limit) {
        const dim3 grid((unsigned)((g.m * g.n * g.batch + 7) / 8));
        gemm_skinny_kernel<<<grid, 256, 0, ctx.stream()>>>(p, g.ta ? 1 : g.lda, g.ta ? g.lda : 1, g.tb ? 1 : g.ldb, g.tb ? g.ldb : 1);
        return ctx.check_cuda(cudaGetLastError(), "gemm_skinny launch");
    }
    if (p.tiles_n * p.tiles_m > grid_limit / g.batch) return ctx.fail(SAGE_ERR_UNSUPPORTED, "gemm_simt: more than 2^31 tiles");
    const dim3 grid((unsigned)(p.tiles_n * p.tiles_m * g.batch));
    cudaStream_t s = ctx.stream();
    if (!g.ta && !g.tb) gemm_simt_kernel<false, false><<<grid, 256, 0, s>>>(p);
    else if (!g.ta && g.tb) gemm_simt_kernel<false, true><<<grid, 256, 0, s>>>(p);
    else if (g.ta && !g.tb) gemm_simt_kernel<true, false><<<grid, 256, 0, s>>>(p);
    else gemm_simt_kernel<true, true><<<grid, 256, 0, s>>>(p);
    return ctx.check_cuda(cudaGetLastError(), "gemm_simt launch");
}

}  // namespace k
}  // namespace sage
