// fp32 GEMM on the Blackwell tensor cores: tcgen05.mma (kind::tf32) with TMEM accumulators, operands
// staged by TMA into 128B-swizzled shared memory, 3xTF32 so results stay at fp32 accuracy.
//
// Reference: Gemm::compute_direct / GemmBatched::compute_direct (src/ops/gemm.rs:176-250, 338-421) run
// CLBlast's scalar "XgemmDirect" OpenCL kernel (src/ops/kernels/matmul_direct.opencl:514-709); the
// reference has no tensor-core path at all.  Same contract here: row-major C[M,N] = op(A) * op(B),
// all four transpose modes, strided batches, any M/N/K.
//
// 3xTF32.  Each fp32 operand is split once into hi = tf32(a) (round to nearest) and lo = a - hi, and
//   C = A_lo*B_hi + A_hi*B_lo + A_hi*B_hi
// The split is a separate pass (split_tf32_kernel) that also re-lays the operand out with a row pitch
// that is a multiple of 16 bytes, so TMA can read operands whose original leading dimension it could
// not (e.g. K = 147 of the first ResNet convolution).  Callers may keep the split of an operand
// (weights, activations read by several GEMMs) and pass it again.
//
// Accumulation.  The tensor core adds into its fp32 accumulator with truncation, which biases a
// long chain: measured on B200, 3072 chained MMAs (K = 8192) were ~17x less accurate than a plain
// fp32 loop.  So a chain is cut every kChunkKB K-blocks (128 k): each chunk accumulates in TMEM from
// zero, and the epilogue warps add the finished chunk into fp32 registers with round-to-nearest
// while the tensor core already works on the next chunk in the other TMEM buffer.
//
// Kernel structure (persistent: one CTA per SM walks over 128 x BN output tiles; 320 threads):
//   warp 0      one lane issues the TMA loads of a K-block (A_hi, A_lo, B_hi, B_lo) into a ring of stages
//   warp 1      allocates TMEM; one lane issues 4 k-steps x 3 tcgen05.mma per K-block, commits stages/chunks
//   warps 2-9   epilogue: tcgen05.ld each finished chunk (a TMEM lane = an output row; two warps share a
//               lane quarter and take half of the columns each), add it to registers, store C at tile end
// Hand-over by mbarriers: full/empty per shared-memory stage, tmem_full/tmem_empty per TMEM buffer.
// No cluster launch and no multicast: each CTA loads its own operands.
//
// Every wait is bounded: after ~1 s it records a timeout in the context's status word, and the CTA
// drains (waits, again bounded, for its loads in flight), frees its TMEM and returns.
#include <cuda.h>
#include <cuda_runtime.h>

#include "kernels.h"

namespace sage {
void *driver_symbol(const char *name);  // runtime/context.cc
namespace k {

namespace {
// A K-block is 32 k wide: K-major tiles are rows of 128 bytes (128-byte swizzle), MN-major tiles are
// 32 k-rows of 128 bytes.  BK = 16 (64-byte rows, twice the stages) was measured and is slower:
// the kernel is bound by the bytes each SM can take from L2 (~45 B/clk), not by load latency, and
// 16-wide K-blocks double the number of TMA operations for the same bytes.
constexpr int BM = 128, BK = 32;
constexpr int kThreads = 320;
constexpr int kEpiWarps = 8;
constexpr int kChunkKB = 128 / BK;  // K-blocks per accumulation chain (128 k)
constexpr long long kTimeoutCycles = 2000000000LL;  // ~1 s

struct TcParams {
    float *c;
    long long ldc, stride_c;
    int m, n, k;
    int stages;
    int a_kmajor, b_kmajor;
    int tiles_m, tiles_n, num_tiles;
    unsigned *status;  // device status word
};

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity) {
    const unsigned addr = smem_u32(bar);
    const long long t0 = clock64();
    for (;;) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
        if (clock64() - t0 > kTimeoutCycles) return false;
    }
}

__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, unsigned long long *bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma: start address, leading / stride byte offsets
// (all >> 4), descriptor version 1 (bits 46-47), layout type in bits 61-63: 2 = 128-byte swizzle
// (16-byte chunks, used for K-major tiles), 1 = 128-byte swizzle with a 32-byte base, the only
// layout the tensor core accepts for MN-major 32-bit (tf32) operands.
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes, unsigned layout_type) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr >> 4) & 0x3fff);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= 1ull << 46;
    d |= (unsigned long long)layout_type << 61;
    return d;
}

__device__ __forceinline__ void umma_tf32(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void flag_timeout(const TcParams &p, volatile int *abort_flag, unsigned where) {
    atomicOr(p.status, 0x100u | where);  // bit 8 = "a tcgen05 GEMM wait timed out", low bits = which wait
    *abort_flag = 1;
}

// Loads one operand tile of a K-block into shared memory.  K-major operand (its K axis is contiguous
// in memory): one box of {32 k, rows}.  MN-major operand: rows/32 boxes of {32 mn, 32 k}, each a
// 4 KiB block of 32 k-rows x 128 bytes.
__device__ __forceinline__ void load_operand(const CUtensorMap *map, char *dst, unsigned long long *bar, bool kmajor, int rows,
                                             int mn0, int k0, int batch, int plane) {
    if (kmajor) {
        tma_load_4d(dst, map, bar, k0, mn0, batch, plane);
    } else {
        for (int j = 0; j < rows / 32; ++j) tma_load_4d(dst + j * (BK * 128), map, bar, mn0 + 32 * j, k0, batch, plane);
    }
}

__device__ __forceinline__ void tile_coords(const TcParams &p, int tile, int bn, int *m0, int *n0, int *batch) {
    const int per_batch = p.tiles_m * p.tiles_n;
    *batch = tile / per_batch;
    const int r = tile - *batch * per_batch;
    *m0 = (r / p.tiles_n) * BM;  // consecutive CTAs share the A rows and take neighbouring B columns
    *n0 = (r % p.tiles_n) * bn;
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p) {
    extern __shared__ __align__(1024) char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[8], empty_bar[8], tmem_full[2], tmem_empty[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ volatile int abort_flag;

    constexpr int A_BYTES = BM * BK * 4, B_BYTES = BN * BK * 4, STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
    constexpr unsigned BUF_COLS = BN == 192 ? 256u : (unsigned)BN;  // column stride between the two TMEM buffers
    constexpr unsigned TMEM_COLS = 2 * BUF_COLS;                    // 128, 256 or 512: a power of two
    constexpr int HALF = BN / 2;                                    // columns per epilogue warp

    // dynamic shared memory is only guaranteed 16-byte aligned; swizzled tiles need 1024
    char *smem = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (p.k + BK - 1) / BK;
    const int chunks_per_tile = (num_kb + kChunkKB - 1) / kChunkKB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kEpiWarps);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------------ TMA producer
        int kbg = 0;  // K-blocks issued so far, across tiles
        for (int tile = blockIdx.x; tile < p.num_tiles && !abort_flag; tile += gridDim.x) {
            int m0, n0, batch;
            tile_coords(p, tile, BN, &m0, &n0, &batch);
            for (int kb = 0; kb < num_kb; ++kb, ++kbg) {
                const int s = kbg % p.stages;
                if (!mbar_wait(&empty_bar[s], ((kbg / p.stages) & 1) ^ 1)) {
                    flag_timeout(p, &abort_flag, 1);
                    break;
                }
                if (abort_flag) break;
                char *st = smem + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], (unsigned)STAGE_BYTES);
                load_operand(&map_a, st, &full_bar[s], p.a_kmajor, BM, m0, kb * BK, batch, 0);
                load_operand(&map_a, st + A_BYTES, &full_bar[s], p.a_kmajor, BM, m0, kb * BK, batch, 1);
                load_operand(&map_b, st + 2 * A_BYTES, &full_bar[s], p.b_kmajor, BN, n0, kb * BK, batch, 0);
                load_operand(&map_b, st + 2 * A_BYTES + B_BYTES, &full_bar[s], p.b_kmajor, BN, n0, kb * BK, batch, 1);
            }
        }
        // Do not leave the CTA with bulk copies still landing in its shared memory.
        for (int i = kbg > p.stages ? kbg - p.stages : 0; i < kbg; ++i)
            if (!mbar_wait(&full_bar[i % p.stages], (i / p.stages) & 1)) flag_timeout(p, &abort_flag, 2);
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        // instruction descriptor: D = f32, A = B = tf32, majors, N >> 3, M >> 4
        const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((p.a_kmajor ? 0u : 1u) << 15) | ((p.b_kmajor ? 0u : 1u) << 16) |
                               ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
        // K-major tile: 8-row groups 1024 B apart (stride offset), a k-step is 32 B further along the
        // swizzled row.  MN-major tile: 32-wide column blocks BK*128 B apart (leading offset), groups of
        // 4 k-rows 512 B apart (stride offset), a k-step (8 k-rows) is 1024 B further.
        const unsigned a_lbo = p.a_kmajor ? 16u : (unsigned)(BK * 128), a_step = p.a_kmajor ? 32u : 1024u;
        const unsigned b_lbo = p.b_kmajor ? 16u : (unsigned)(BK * 128), b_step = p.b_kmajor ? 32u : 1024u;
        constexpr unsigned K_SBO = 8u * BK * 4u;           // 8 rows of a K-major tile
        constexpr unsigned K_LT = BK == 32 ? 2u : 4u;      // 128-byte or 64-byte swizzle
        const unsigned a_sbo = p.a_kmajor ? K_SBO : 512u, b_sbo = p.b_kmajor ? K_SBO : 512u;
        const unsigned a_lt = p.a_kmajor ? K_LT : 1u, b_lt = p.b_kmajor ? K_LT : 1u;
        int kbg = 0, cg = 0;  // K-blocks / chunks consumed so far, across tiles
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
            for (int c = 0; c < chunks_per_tile && ok; ++c, ++cg) {
                const int buf = cg & 1;
                if (!mbar_wait(&tmem_empty[buf], ((cg >> 1) & 1) ^ 1)) {  // epilogue has drained this buffer
                    flag_timeout(p, &abort_flag, 16);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned tmem_d = tmem_base + (unsigned)buf * BUF_COLS;
                const int kb_end = min(num_kb, (c + 1) * kChunkKB);
                for (int kb = c * kChunkKB; kb < kb_end; ++kb, ++kbg) {
                    const int s = kbg % p.stages;
                    if (abort_flag || !mbar_wait(&full_bar[s], (kbg / p.stages) & 1)) {
                        if (!abort_flag) flag_timeout(p, &abort_flag, 4);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a_hi = smem_u32(smem + (size_t)s * STAGE_BYTES), a_lo = a_hi + A_BYTES;
                    const unsigned b_hi = a_hi + 2 * A_BYTES, b_lo = b_hi + B_BYTES;
#pragma unroll
                    for (int ks = 0; ks < BK / 8; ++ks) {
                        const unsigned long long da_hi = smem_desc(a_hi + ks * a_step, a_lbo, a_sbo, a_lt), da_lo = smem_desc(a_lo + ks * a_step, a_lbo, a_sbo, a_lt);
                        const unsigned long long db_hi = smem_desc(b_hi + ks * b_step, b_lbo, b_sbo, b_lt), db_lo = smem_desc(b_lo + ks * b_step, b_lbo, b_sbo, b_lt);
                        umma_tf32(tmem_d, da_lo, db_hi, idesc, (kb > c * kChunkKB || ks > 0) ? 1u : 0u);  // small terms first
                        umma_tf32(tmem_d, da_hi, db_lo, idesc, 1u);
                        umma_tf32(tmem_d, da_hi, db_hi, idesc, 1u);
                    }
                    umma_commit(&empty_bar[s]);  // arrives when the MMAs above have finished reading this stage
                }
                if (ok) umma_commit(&tmem_full[buf]);
            }
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------------ epilogue (8 warps)
        const int q = warp & 3;           // TMEM lane quarter this warp may access
        const int h = (warp - 2) >> 2;    // which half of the tile's columns
        float acc[HALF];
        int cg = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
            int m0, n0, batch;
            tile_coords(p, tile, BN, &m0, &n0, &batch);
            for (int c = 0; c < chunks_per_tile && ok; ++c, ++cg) {
                const int buf = cg & 1;
                bool got = mbar_wait(&tmem_full[buf], (cg >> 1) & 1);
                if (!got && lane == 0) flag_timeout(p, &abort_flag, 8);
                ok = __all_sync(0xffffffffu, got && !abort_flag);  // the TMEM loads below are warp-collective
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned taddr = tmem_base + (unsigned)buf * BUF_COLS + ((unsigned)(q * 32) << 16) + (unsigned)(h * HALF);
#pragma unroll
                for (int j = 0; j < HALF / 16; ++j) {
                    unsigned r[16];
                    tmem_ld16(taddr + j * 16, r);
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[j * 16 + i] = (c == 0) ? __uint_as_float(r[i]) : acc[j * 16 + i] + __uint_as_float(r[i]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty[buf]);  // this warp no longer needs the buffer
            }
            if (!ok) break;
            const int row = m0 + q * 32 + lane;
            const int col0 = n0 + h * HALF;
            if (row < p.m && col0 < p.n) {
                float *crow = p.c + (size_t)batch * p.stride_c + (size_t)row * p.ldc;
                const bool vec_ok = (p.ldc % 4 == 0) && (p.stride_c % 4 == 0) && (reinterpret_cast<uintptr_t>(p.c) % 16 == 0) &&
                                    (col0 + HALF <= p.n);
                if (vec_ok) {
#pragma unroll
                    for (int j = 0; j < HALF; j += 4)
                        *reinterpret_cast<float4 *>(crow + col0 + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < HALF; ++j)
                        if (col0 + j < p.n) crow[col0 + j] = acc[j];
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------- operand split
// src: `rows` x `cols` with row stride `ld`, `batches` of them `batch_stride` apart.
// dst: [2][batches][rows][pitch] with pitch = cols rounded up to 4; plane 0 = tf32(x) rounded to
// nearest, plane 1 = x - plane 0 (exact in fp32).  Pad columns are written as zeros.
__global__ void __launch_bounds__(256) split_tf32_kernel(const float *__restrict__ src, long long ld, long long batch_stride, int rows,
                                                         int cols, int batches, float *__restrict__ dst, int pitch, long long plane_stride) {
    const int groups = pitch >> 2;
    const long long total = (long long)batches * rows * groups;
    const bool vec_in = (ld % 4 == 0) && (batch_stride % 4 == 0) && (reinterpret_cast<uintptr_t>(src) % 16 == 0);
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(g % groups) * 4;
        const long long rb = g / groups;
        const int r = (int)(rb % rows);
        const long long b = rb / rows;
        const float *s = src + b * batch_stride + (long long)r * ld + c;
        float x[4];
        if (vec_in && c + 4 <= cols) {
            const float4 v = *reinterpret_cast<const float4 *>(s);
            x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = (c + j < cols) ? s[j] : 0.f;
        }
        float hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            unsigned hbits;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hbits) : "f"(x[j]));
            float hf = __uint_as_float(hbits);
            if (!isfinite(hf)) {  // rounding overflowed, or x itself is inf/nan: keep the truncated value, no low part
                hf = __uint_as_float(__float_as_uint(x[j]) & 0xffffe000u);
                lo[j] = isfinite(x[j]) ? x[j] - hf : 0.f;
            } else {
                lo[j] = x[j] - hf;
            }
            hi[j] = hf;
        }
        float *d = dst + (b * rows + r) * (long long)pitch + c;
        *reinterpret_cast<float4 *>(d) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<float4 *>(d + plane_stride) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
}

typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 4-D tensor map {cols, rows, batch, plane} over a split operand with a {32, box_rows, 1, 1} box.
bool encode_map(PFN_encodeTiled encode, const SplitPlanes &op, unsigned box_rows, bool kmajor, CUtensorMap *map) {
    const cuuint64_t dims[4] = {(cuuint64_t)op.cols, (cuuint64_t)op.rows, (cuuint64_t)op.batches, 2};
    const cuuint64_t row_b = (cuuint64_t)op.pitch * 4;
    const cuuint64_t strides[3] = {row_b, row_b * op.rows, row_b * op.rows * op.batches};
    // K-major: {BK k, tile rows}; MN-major: {32 mn, BK k-rows}
    const cuuint32_t box[4] = {kmajor ? (cuuint32_t)BK : 32u, kmajor ? box_rows : (cuuint32_t)BK, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapSwizzle sw = !kmajor ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : (BK == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, op.planes, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int pick_bn(const Context &ctx, long long m, long long n, long long batch) {
    const int cands[4] = {256, 192, 128, 64};
    int best = 128;
    double best_cost = 1e300;
    for (int bn : cands) {
        if (bn > 64 && n <= bn / 2) continue;  // mostly padding
        const long long tiles = ((n + bn - 1) / bn) * ((m + BM - 1) / BM) * batch;
        const long long waves = (tiles + ctx.sm_count - 1) / ctx.sm_count;
        const double cost = (double)waves * (bn + 24);  // +24: per-tile fixed cost in units of columns
        if (cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

template <int BN>
sage_status launch_tc(Context &ctx, const CUtensorMap &map_a, const CUtensorMap &map_b, TcParams p, int grid, size_t smem) {
    // per device; the limit covers dynamic + static shared memory, so ask for what is used
    static int attr_set[64] = {0};  // per BN instantiation and device
    const int dev = ctx.device();
    if (dev < 0 || dev >= 64 || attr_set[dev] != (int)smem) {
        sage_status st = ctx.check_cuda(cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                                        "gemm_tc shared memory attribute");
        if (st) return st;
        if (dev >= 0 && dev < 64) attr_set[dev] = (int)smem;
    }
    gemm_tc_kernel<BN><<<grid, kThreads, smem, ctx.stream()>>>(map_a, map_b, p);
    return ctx.check_cuda(cudaGetLastError(), "gemm_tc launch");
}
}  // namespace

bool gemm_tc_supported(const GemmArgs &g) {
    // Tiny problems are latency-bound and would be mostly TMA padding: leave them to the SIMT kernel.
    if (g.m < 64 || g.n < 32 || g.k < 32 || g.batch < 1) return false;
    if (g.m > 0x7fffffffLL || g.n > 0x7fffffffLL || g.k > 0x7fffffffLL || g.batch > 0x7fffffffLL) return false;
    const long long tiles = ((g.m + BM - 1) / BM) * ((g.n + 63) / 64) * g.batch;
    return tiles < 0x7fffffffLL;
}

sage_status split_tf32(Context &ctx, const float *src, long long ld, long long batch_stride, int rows, int cols, int batches,
                       SplitPlanes *out) {
    out->rows = rows;
    out->cols = cols;
    out->batches = batches;
    out->pitch = (cols + 3) / 4 * 4;
    const size_t plane = (size_t)batches * rows * out->pitch;
    out->block = ctx.allocator().alloc(plane * 2 * sizeof(float));
    if (!out->block) return ctx.fail(SAGE_ERR_OOM, "out of memory for the tf32 operand split");
    out->planes = reinterpret_cast<float *>(out->block->ptr);
    ctx.note_launch("split_tf32");
    if (ctx.dry()) return SAGE_OK;
    const long long total = (long long)plane / 4;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)ctx.sm_count * 16;
    if (blocks > cap) blocks = cap;
    split_tf32_kernel<<<(unsigned)blocks, 256, 0, ctx.stream()>>>(src, ld, batch_stride, rows, cols, batches, out->planes, out->pitch,
                                                                  (long long)plane);
    return ctx.check_cuda(cudaGetLastError(), "split_tf32 launch");
}

// Same split, written into memory the caller provides (`dst` must hold split_tf32_bytes(...) bytes
// and be 16-byte aligned).  Nothing is allocated; out->block stays null.
size_t split_tf32_bytes(int rows, int cols, int batches) {
    return (size_t)batches * rows * ((cols + 3) / 4 * 4) * 2 * sizeof(float);
}

sage_status split_tf32_into(Context &ctx, const float *src, long long ld, long long batch_stride, int rows, int cols, int batches,
                            float *dst, SplitPlanes *out) {
    out->block = nullptr;
    out->planes = dst;
    out->rows = rows;
    out->cols = cols;
    out->batches = batches;
    out->pitch = (cols + 3) / 4 * 4;
    const size_t plane = (size_t)batches * rows * out->pitch;
    ctx.note_launch("split_tf32");
    if (ctx.dry()) return SAGE_OK;
    const long long total = (long long)plane / 4;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)ctx.sm_count * 16;
    if (blocks > cap) blocks = cap;
    split_tf32_kernel<<<(unsigned)blocks, 256, 0, ctx.stream()>>>(src, ld, batch_stride, rows, cols, batches, dst, out->pitch, (long long)plane);
    return ctx.check_cuda(cudaGetLastError(), "split_tf32 launch");
}

sage_status gemm_tcgen05_planes(Context &ctx, const GemmArgs &g, const SplitPlanes &a, const SplitPlanes &b) {
    static PFN_encodeTiled encode = nullptr;
    if (!ctx.dry() && !encode) {
        encode = reinterpret_cast<PFN_encodeTiled>(driver_symbol("cuTensorMapEncodeTiled"));
        if (!encode) return ctx.fail(SAGE_ERR_DEVICE, "cuTensorMapEncodeTiled is not available");
    }
    const int bn = pick_bn(ctx, g.m, g.n, g.batch);
    const int stage_bytes = 2 * BM * BK * 4 + 2 * bn * BK * 4;
    int stages = (227 * 1024 - 2048) / stage_bytes;
    if (stages > 8) stages = 8;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    const bool a_kmajor = !g.ta, b_kmajor = g.tb;
    ctx.note_launch("gemm_tc_3xtf32");
    if (ctx.dry()) return SAGE_OK;
    CUtensorMap map_a, map_b;
    if (!encode_map(encode, a, a_kmajor ? BM : 32, a_kmajor, &map_a) || !encode_map(encode, b, b_kmajor ? (unsigned)bn : 32, b_kmajor, &map_b))
        return ctx.fail(SAGE_ERR_DEVICE, "cuTensorMapEncodeTiled failed");
    TcParams p;
    p.c = g.c;
    p.ldc = g.ldc;
    p.stride_c = g.stride_c;
    p.m = (int)g.m;
    p.n = (int)g.n;
    p.k = (int)g.k;
    p.stages = stages;
    p.a_kmajor = a_kmajor;
    p.b_kmajor = b_kmajor;
    p.tiles_m = (int)((g.m + BM - 1) / BM);
    p.tiles_n = (int)((g.n + bn - 1) / bn);
    p.num_tiles = (int)((long long)p.tiles_m * p.tiles_n * g.batch);
    p.status = ctx.status_word_dev;
    const int grid = p.num_tiles < ctx.sm_count ? p.num_tiles : ctx.sm_count;
    switch (bn) {
    case 256: return launch_tc<256>(ctx, map_a, map_b, p, grid, smem);
    case 192: return launch_tc<192>(ctx, map_a, map_b, p, grid, smem);
    case 128: return launch_tc<128>(ctx, map_a, map_b, p, grid, smem);
    default: return launch_tc<64>(ctx, map_a, map_b, p, grid, smem);
    }
}

void free_split(Context &ctx, SplitPlanes *s) {
    if (s->block) ctx.allocator().free(s->block);
    s->block = nullptr;
}

sage_status gemm_tcgen05(Context &ctx, const GemmArgs &g) {
    if (!gemm_tc_supported(g)) return SAGE_ERR_UNSUPPORTED;
    // A as stored: [M,K] (K-major) or, transposed, [K,M] (MN-major); B: [K,N] (MN-major) or [N,K] (K-major).
    SplitPlanes a, b;
    sage_status st = split_tf32(ctx, g.a, g.lda, g.stride_a, g.ta ? (int)g.k : (int)g.m, g.ta ? (int)g.m : (int)g.k, (int)g.batch, &a);
    if (st) return st;
    st = split_tf32(ctx, g.b, g.ldb, g.stride_b, g.tb ? (int)g.n : (int)g.k, g.tb ? (int)g.k : (int)g.n, (int)g.batch, &b);
    if (!st) st = gemm_tcgen05_planes(ctx, g, a, b);
    // Stream-ordered: the split buffers may be reused by later launches on this stream.
    free_split(ctx, &a);
    free_split(ctx, &b);
    return st;
}

}  // namespace k
}  // namespace sage
