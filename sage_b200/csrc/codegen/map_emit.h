// Fused elementwise map kernels: CUDA C emitted from an expression, compiled once by NVRTC and
// cached.  Replaces compile_map + translate_id of the reference (src/ops/map.rs:369-410,
// src/ops/core.rs:113-175).
#pragma once
#include <string>
#include <unordered_map>
#include <vector>

#include "../kernels/kernels.h"

namespace sage {

struct MapOperand {
    int dtype;        // sage_dtype
    const void *ptr;  // device address with the element offset applied
    k::Dims view;     // extents (equal to the output's) + element strides (0 = broadcast)
};

// Per-operator memo of compiled kernels, the counterpart of CachedAccess
// (src/session/context.rs:146-185): signature of the access pattern -> module.
struct MapCache {
    std::unordered_map<std::string, Module *> by_signature;
    Context *owner = nullptr;
};

// What the emitter decided for one launch (exposed for tests).
struct MapPlan {
    std::string source;
    std::string signature;
    int vec = 1;
    int ndim = 1;
    long long n = 0;
    unsigned long long ext[k::kMaxDims] = {0};
    std::vector<std::vector<long long>> strides;  // per input, collapsed dims
};

// `expr` is a C expression over x0..x{n-1}; helper functions come from the prelude
// (sg_exp, sg_max, ...).  The output is contiguous with `out_ext`.
// `planes`: the kernel also writes the tf32 hi / lo split of every (f32) result, laid out like y.
sage_status map_plan(const std::string &expr, const std::vector<MapOperand> &in, int out_dtype, const void *y,
                     int out_ndim, const long long *out_ext, MapPlan *plan, bool emit_source = true, bool planes = false);

// `hi` (optional, f32 results only): hi plane of y's tf32 split, the lo plane `plane` floats further; a
// tensor-core GEMM that reads y next then needs no split pass.
sage_status map_launch(Context &ctx, const std::string &expr, const std::vector<MapOperand> &in, int out_dtype,
                       void *y, int out_ndim, const long long *out_ext, MapCache *cache, float *hi = nullptr, long long plane = 0);

}  // namespace sage
