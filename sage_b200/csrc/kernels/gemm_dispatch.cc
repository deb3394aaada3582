// Chooses the GEMM kernel: tensor-core path where the operands can go through TMA, SIMT otherwise.
#include "kernels.h"

namespace sage {
namespace k {

sage_status gemm(Context &ctx, const GemmArgs &g) {
    if (ctx.opts().gemm_backend != 1) {
        sage_status st = gemm_tcgen05(ctx, g);
        if (st != SAGE_ERR_UNSUPPORTED) return st;
    }
    return gemm_simt(ctx, g);
}

}  // namespace k
}  // namespace sage
