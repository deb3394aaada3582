// Parameter updates of the optimizers (src/optim.rs:42-94 Sgd::update, :125-178 Adam::update).
//
// The reference builds, for every parameter, a handful of lazy map expressions and evaluates each of
// them (m_t, v_t, param_new: three kernels and three fresh tensors per parameter and step).  Here one
// launch updates up to kOptSlots parameters in place: each slot names a parameter, its gradient and
// the optimizer's state tensors; the chunks of all slots form one index space that a grid sized to
// the machine walks with a grid-stride loop, so a bias of one element and an embedding table of
// twenty million share a launch.  The arithmetic is the reference's, operation for operation and
// rounded after every step (no contraction into fused multiply-adds), so the result does not depend
// on how the expressions are cut into kernels.  A parameter that a GEMM reads keeps tf32 hi / lo
// planes beside it; the update writes those too, which saves the separate split pass every step.
#include <cuda.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "launch.h"
#include "gemm_tc_device.inc"  // split_tf32_value

namespace sage {
namespace k {

namespace {

constexpr int kChunk = 4096;  // elements per chunk: 256 threads x 4 quads

struct OptBatch {
    OptSlot slot[kOptSlots];
    unsigned first_chunk[kOptSlots + 1];  // prefix sums of ceil(n / kChunk)
    int count;
};

struct SgdRule {
    OptSgd k;
    __device__ __forceinline__ float operator()(float p, float g, float *, float *, bool) const {
        if (k.weight_decay != 0.f) g = __fadd_rn(g, __fmul_rn(p, k.weight_decay));  // grad + param * weight_decay
        return __fsub_rn(p, __fmul_rn(g, k.lr));                                     // param - g * lr
    }
};

struct AdamRule {
    OptAdam k;
    __device__ __forceinline__ float operator()(float p, float g, float *m, float *v, bool first) const {
        if (k.weight_decay != 0.f) g = __fadd_rn(g, __fmul_rn(p, k.weight_decay));
        if (first) {  // the first update of a parameter stores zeros (optim.rs:150,158)
            *m = 0.f;
            *v = 0.f;
        } else {
            *m = __fadd_rn(__fmul_rn(*m, k.beta1), __fmul_rn(g, k.one_minus_beta1));
            *v = __fadd_rn(__fmul_rn(*v, k.beta2), __fmul_rn(__fmul_rn(g, g), k.one_minus_beta2));
        }
        const float m_hat = __fdiv_rn(*m, k.corr1), v_hat = __fdiv_rn(*v, k.corr2);
        return __fsub_rn(p, __fdiv_rn(__fmul_rn(m_hat, k.lr), __fadd_rn(__fsqrt_rn(v_hat), k.eps)));
    }
};

template <bool STATE, class Rule>
__global__ void __launch_bounds__(256) optimizer_update_kernel(const __grid_constant__ OptBatch b, const Rule rule) {
    grid_dependency_sync();
    const unsigned total = b.first_chunk[b.count];
    for (unsigned chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
        int lo = 0, hi = b.count - 1;  // the slot whose chunk range holds `chunk`
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (b.first_chunk[mid] <= chunk) lo = mid;
            else hi = mid - 1;
        }
        const OptSlot &s = b.slot[lo];
        const long long begin = (long long)(chunk - b.first_chunk[lo]) * kChunk;
        const long long end = begin + kChunk < s.n ? begin + kChunk : s.n;
        const bool first = s.first != 0;
        if (s.vec) {
            for (long long i = begin + 4 * threadIdx.x; i + 3 < end; i += 4 * 256) {
                const float4 p = *reinterpret_cast<const float4 *>(s.p + i);
                const float4 g = *reinterpret_cast<const float4 *>(s.g + i);
                float4 m = {0.f, 0.f, 0.f, 0.f}, v = m, o;
                if (STATE && !first) {
                    m = *reinterpret_cast<const float4 *>(s.m + i);
                    v = *reinterpret_cast<const float4 *>(s.v + i);
                }
                o.x = rule(p.x, g.x, &m.x, &v.x, first);
                o.y = rule(p.y, g.y, &m.y, &v.y, first);
                o.z = rule(p.z, g.z, &m.z, &v.z, first);
                o.w = rule(p.w, g.w, &m.w, &v.w, first);
                *reinterpret_cast<float4 *>(s.p + i) = o;
                if (STATE) {
                    *reinterpret_cast<float4 *>(s.m + i) = m;
                    *reinterpret_cast<float4 *>(s.v + i) = v;
                }
                if (s.hi) {
                    float4 h, l;
                    sage_tc::split_tf32_value(o.x, &h.x, &l.x);
                    sage_tc::split_tf32_value(o.y, &h.y, &l.y);
                    sage_tc::split_tf32_value(o.z, &h.z, &l.z);
                    sage_tc::split_tf32_value(o.w, &h.w, &l.w);
                    *reinterpret_cast<float4 *>(s.hi + i) = h;
                    *reinterpret_cast<float4 *>(s.hi + s.plane + i) = l;
                }
            }
        }
        // what the quads did not cover: everything when the slot is not 16-byte aligned, else the tail
        const long long scalar_from = s.vec ? begin + (end - begin) / 4 * 4 : begin;
        for (long long i = scalar_from + threadIdx.x; i < end; i += 256) {
            float m = 0.f, v = 0.f;
            if (STATE && !first) {
                m = s.m[i];
                v = s.v[i];
            }
            const float o = rule(s.p[i], s.g[i], &m, &v, first);
            s.p[i] = o;
            if (STATE) {
                s.m[i] = m;
                s.v[i] = v;
            }
            if (s.hi) {
                float h, l;
                sage_tc::split_tf32_value(o, &h, &l);
                s.hi[i] = h;
                s.hi[s.plane + i] = l;
            }
        }
    }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <bool STATE, class Rule>
sage_status run(Context &ctx, const OptSlot *slots, int count, const Rule &rule, const char *label) {
    for (int at = 0; at < count; at += kOptSlots) {
        OptBatch b;
        b.count = count - at < kOptSlots ? count - at : kOptSlots;
        unsigned chunks = 0;
        for (int i = 0; i < b.count; ++i) {
            OptSlot s = slots[at + i];
            if (s.n < 0 || !s.p || !s.g || (STATE && (!s.m || !s.v))) return ctx.fail(SAGE_ERR_INVALID, "optimizer update: bad slot");
            s.vec = aligned16(s.p) && aligned16(s.g) && (!STATE || (aligned16(s.m) && aligned16(s.v))) &&
                    (!s.hi || (aligned16(s.hi) && s.plane % 4 == 0));
            b.slot[i] = s;
            b.first_chunk[i] = chunks;
            const long long c = (s.n + kChunk - 1) / kChunk;
            if (c + chunks > 0x7fffffffll) return ctx.fail(SAGE_ERR_INVALID, "optimizer update: too many elements in one call");
            chunks += (unsigned)c;
        }
        for (int i = b.count; i <= kOptSlots; ++i) b.first_chunk[i] = chunks;
        if (!chunks) continue;
        const unsigned resident = (unsigned)ctx.sm_count * 8u;
        const unsigned grid = chunks < resident ? chunks : resident;
        ctx.note_launch(label);
        if (ctx.dry()) continue;
        sage_status st = ctx.check_cuda(
            launch_dependent(ctx.pdl, ctx.stream(), optimizer_update_kernel<STATE, Rule>, dim3(grid), dim3(256), 0, b, rule), label);
        if (st) return st;
    }
    return SAGE_OK;
}

}  // namespace

sage_status sgd_update(Context &ctx, const OptSlot *slots, int count, const OptSgd &k) {
    return run<false>(ctx, slots, count, SgdRule{k}, "sgd_update");
}

sage_status adam_update(Context &ctx, const OptSlot *slots, int count, const OptAdam &k) {
    return run<true>(ctx, slots, count, AdamRule{k}, "adam_update");
}

}  // namespace k
}  // namespace sage
