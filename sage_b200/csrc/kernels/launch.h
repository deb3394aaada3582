// Programmatic dependent launch for the library's static kernels.
//
// A kernel that starts with grid_dependency_sync() may be launched while the kernel before it on the
// stream is still running: its CTAs are scheduled as soon as every CTA of the predecessor has
// started (and SM resources are free), run their prologue, and block in griddepcontrol.wait until
// the predecessor has completed and its writes are visible.  That hides launch latency and the
// prologue (barrier set-up, TMEM allocation, descriptor fetch) behind the predecessor's tail.
// A kernel launched this way MUST call grid_dependency_sync() before its first global access.
#pragma once
#include <cuda_runtime.h>

#include <utility>

namespace sage {
namespace k {

__device__ __forceinline__ void grid_dependency_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// `cluster` > 1 launches thread-block clusters of that many CTAs along x (the grid must be a multiple).
template <typename... P, typename... A>
inline cudaError_t launch_dependent(bool pdl, cudaStream_t stream, int cluster, void (*kernel)(P...), dim3 grid, dim3 block, size_t smem,
                                    A &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);
}
template <typename... P, typename... A>
inline cudaError_t launch_dependent(bool pdl, cudaStream_t stream, void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, A &&...args) {
    return launch_dependent(pdl, stream, 1, kernel, grid, block, smem, std::forward<A>(args)...);
}

}  // namespace k
}  // namespace sage
