// sage_gemm_noalloc: the 3xTF32 tensor-core GEMM for callers that must not allocate device memory.
//
// The regular entry points (sage_gemm, sage_gemm_strided_batched) take the scratch for the hi/lo
// operand split from the context's allocator, which may reach cudaMalloc when its pool has to grow.
// Some hosts cannot accept that: a process whose HBM has been carved up in advance by another
// runtime (everything left belongs to somebody else), or a latency-critical loop that must never
// run into cudaMalloc's device-wide synchronisation.  For them the scratch lives in a fixed
// array that is part of this library's device image: every GPU that loads the library holds
// kScratchBytes of it until the process exits, and this entry point never calls cudaMalloc,
// cudaFree or any allocating library routine.
//
// Limits and rules
//   * 2 * 4 bytes * (rows_a * pitch(cols_a) + rows_b * pitch(cols_b)) must fit in kScratchBytes,
//     where pitch rounds the contiguous extent up to 4 floats; larger problems get SAGE_ERR_INVALID.
//   * A long K is never cut into slices here (sage_gemm does that with allocator scratch), so for k >= 1024
//     with few output tiles this entry point is slower than sage_gemm and its sum order differs from it.
//   * The first call on a device looks up the device address of the array (cudaGetSymbolAddress,
//     with that device current).  Make that first call before any stream capture begins.
//   * All calls share the one array, and it keeps whatever the previous call left in it.  Nothing
//     has to start at zero: the split pass of a call rewrites every byte (pad columns included)
//     that the GEMM of the same call reads.  Two calls whose kernels overlap on the GPU (different
//     streams / contexts on one device) race on the array; serialise them.
#include <cuda_runtime.h>

#include <string>

#include "../../../include/sage_cuda.h"
#include "kernels.h"

namespace {
constexpr size_t kScratchBytes = 32u << 20;  // 32 MiB: e.g. a 1024^3 GEMM needs 16 MiB
static __device__ __align__(256) unsigned char g_gemm_scratch[kScratchBytes];

// In host code `g_gemm_scratch` is only a handle for the symbol, not a device address.  The address
// differs per device, so it is resolved once per device with that device current.
float *scratch_for_device(int device, cudaError_t *err) {
    static float *table[64] = {nullptr};
    *err = cudaSuccess;
    if (device >= 0 && device < 64 && table[device]) return table[device];
    int current = -1;
    *err = cudaGetDevice(&current);
    if (*err != cudaSuccess) return nullptr;
    if (current != device) {
        *err = cudaSetDevice(device);
        if (*err != cudaSuccess) return nullptr;
    }
    void *p = nullptr;
    *err = cudaGetSymbolAddress(&p, g_gemm_scratch);
    if (current != device && current >= 0) cudaSetDevice(current);
    if (*err != cudaSuccess) return nullptr;
    if (device >= 0 && device < 64) table[device] = static_cast<float *>(p);
    return static_cast<float *>(p);
}
}  // namespace

extern "C" sage_status sage_gemm_noalloc(sage_ctx *ctx, int32_t trans_a, int32_t trans_b, int64_t m, int64_t n, int64_t k,
                                         const sage_buf *a, int64_t a_off, int64_t lda, const sage_buf *b, int64_t b_off, int64_t ldb,
                                         sage_buf *c, int64_t c_off, int64_t ldc) {
    using namespace sage;
    if (!ctx || !ctx->impl || !a || !b || !c) return SAGE_ERR_INVALID;
    Context &C = *ctx->impl;
    if (C.dry()) return C.fail(SAGE_ERR_NO_DEVICE, "sage_gemm_noalloc needs a CUDA device");
    C.make_current();
    k::GemmArgs g{trans_a != 0, trans_b != 0, m, n, k, (const float *)a->ptr + a_off, lda, 0, (const float *)b->ptr + b_off, ldb, 0,
                  (float *)c->ptr + c_off, ldc, 0, 1};
    if (!k::gemm_tc_supported(g))
        return C.fail(SAGE_ERR_UNSUPPORTED,
                      "sage_gemm_noalloc: needs n >= 32, k >= 32 and m >= 64 (or m >= 16 with k >= 2048): the tensor-core path; use sage_gemm");
    const int a_rows = g.ta ? (int)k : (int)m, a_cols = g.ta ? (int)m : (int)k;
    const int b_rows = g.tb ? (int)n : (int)k, b_cols = g.tb ? (int)k : (int)n;
    const size_t a_bytes = k::split_tf32_bytes(a_rows, a_cols, 1), b_bytes = k::split_tf32_bytes(b_rows, b_cols, 1);
    const size_t a_span = (a_bytes + 255) / 256 * 256;  // keep the second operand 256-byte aligned
    if (a_span + b_bytes > kScratchBytes)
        return C.fail(SAGE_ERR_INVALID, "sage_gemm_noalloc: the operand split needs " + std::to_string(a_span + b_bytes) +
                                            " bytes of scratch but the built-in scratch holds " + std::to_string(kScratchBytes) +
                                            "; use sage_gemm for this size");
    cudaError_t err;
    float *scratch = scratch_for_device(C.device(), &err);
    if (!scratch) return C.check_cuda(err, "cudaGetSymbolAddress(gemm scratch)");
    k::SplitPlanes pa, pb;
    sage_status st = k::split_tf32_into(C, g.a, g.lda, 0, a_rows, a_cols, 1, scratch, &pa);
    if (st) return st;
    st = k::split_tf32_into(C, g.b, g.ldb, 0, b_rows, b_cols, 1, scratch + a_span / sizeof(float), &pb);
    if (st) return st;
    // One pass over K: sage_gemm may cut a long K into slices, which takes partial-product scratch from the
    // allocator and a second kernel.  Neither is reachable from here.
    return k::gemm_tcgen05_planes(C, g, pa, pb, /*no_split_k=*/true);
}
