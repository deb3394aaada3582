#include "kernels.h"
namespace sage {
namespace k {
sage_status gemm_tcgen05(Context &, const GemmArgs &) { return SAGE_ERR_UNSUPPORTED; }
}  // namespace k
}  // namespace sage
