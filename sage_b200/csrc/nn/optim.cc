// Sgd / Adam over the fused multi-parameter update kernel.  Reference: src/optim.rs.
#include "optim.h"

#include <cmath>

#include "../kernels/kernels.h"

namespace sage {
namespace nn {

namespace {

// A fresh contiguous device copy of `t` (any strides).
sage_status compact_copy(Context &C, const Tensor &t, Tensor *out) {
    sage_status st = Tensor::uninit(C, t.desc, out);
    if (st) return st;
    return k::strided_copy(C, (const uint32_t *)t.ptr(), t.dims(), (uint32_t *)out->ptr(), out->desc.shape.strides.data());
}

struct Prepared {
    std::vector<k::OptSlot> slots;
    std::vector<Tensor> keep;  // gradient tensors (or their compact copies) until the launch is enqueued
};

// Resolves every (parameter, gradient) pair to device pointers.  The parameter's buffer is updated in
// place, so it must be contiguous and owned by the variable alone; otherwise the variable first gets
// a private copy (the reference assigns a fresh tensor on every update, optim.rs:90,173, so other
// holders of the old tensor never see the new values).
sage_status prepare(const std::vector<Var> &params, const std::vector<Var> &grads, Session &s, Prepared *out) {
    Context &C = s.ctx();
    if (params.size() != grads.size()) return C.fail(SAGE_ERR_INVALID, "optimizer update: one gradient per parameter is needed");
    std::vector<Var> missing;
    for (const Var &g : grads)
        if (g.is_op() && !s.data.count(g.key())) missing.push_back(g);
    if (!missing.empty()) {  // "it is inefficient to evaluate gradients in the inside of an optimizer" (optim.rs:56-59)
        sage_status st = s.eval(missing);
        if (st) return st;
    }
    for (size_t i = 0; i < params.size(); ++i) {
        const Var &p = params[i];
        if (!p.is_data()) return C.fail(SAGE_ERR_INVALID, "param is not data tensor");  // optim.rs:52-54
        if (p.dtype() != SAGE_F32 || grads[i].dtype() != SAGE_F32) return C.fail(SAGE_ERR_INVALID, "optimizer update: parameters and gradients must be f32");
        if (grads[i].extents() != p.extents()) return C.fail(SAGE_ERR_INVALID, "optimizer update: gradient extents differ from the parameter's");
        Tensor &pt = p.origin->data;
        if (!pt.defined()) return C.fail(SAGE_ERR_INVALID, "optimizer update: the parameter holds no tensor");
        sage_status st = pt.to_device(C);
        if (st) return st;
        if (pt.data.use_count() != 1 || !pt.desc.shape.has_default_strides() || pt.desc.shape.offset != 0 || pt.data->planes_only) {
            Tensor fresh;
            st = compact_copy(C, pt, &fresh);
            if (st) return st;
            pt = fresh;
        }
        Tensor gt;
        if (grads[i].is_data()) {
            gt = grads[i].origin->data;
            if (!gt.defined()) return C.fail(SAGE_ERR_INVALID, "optimizer update: the gradient holds no tensor");
            st = gt.to_device(C);
            if (st) return st;
        } else if (!s.get(grads[i], &gt)) {
            return C.fail(SAGE_ERR_INVALID, "internal: gradient not evaluated");
        }
        if (!gt.desc.shape.has_default_strides() || gt.data->planes_only) {
            if (gt.data->planes_only) return C.fail(SAGE_ERR_INVALID, "internal: gradient exists as tf32 planes only");
            Tensor c;
            st = compact_copy(C, gt, &c);
            if (st) return st;
            gt = c;
        }
        k::OptSlot slot;
        slot.p = (float *)pt.ptr();
        slot.g = (const float *)gt.ptr();
        slot.n = p.size();
        Storage &ps = *pt.data;
        ps.split_view.reset();
        ++ps.version;  // whoever cached something derived from the old values (concatenated weights) rebuilds it
        if (ps.split && ps.split->whole) {  // a GEMM reads this parameter: refresh its planes in the same pass
            slot.hi = ps.split->planes.planes;
            slot.plane = ps.split->plane;
        } else {
            ps.split.reset();
        }
        out->slots.push_back(slot);
        out->keep.push_back(gt);
    }
    return SAGE_OK;
}

}  // namespace

sage_status Sgd::update(const std::vector<Var> &params, const std::vector<Var> &grads, Session &s) {
    Context &C = s.ctx();
    // With momentum the reference reads a buffer it has never stored (`self.b.get(grad).unwrap()` under
    // `!contains_key`, optim.rs:68-69) and panics on the first update; there is no setter for momentum
    // either (Sgd::new, :28-40), so only the plain rule is reachable.
    if (momentum != 0.f) return C.fail(SAGE_ERR_UNSUPPORTED, "Sgd: momentum is unreachable in the reference (update panics)");
    Prepared prep;
    sage_status st = prepare(params, grads, s, &prep);
    if (st) return st;
    k::OptSgd r;
    r.lr = lr;
    r.weight_decay = weight_decay;
    return k::sgd_update(C, prep.slots.data(), (int)prep.slots.size(), r);
}

sage_status Adam::init(Session &) {
    state.clear();
    t = 1.0f;
    return SAGE_OK;
}

sage_status Adam::update(const std::vector<Var> &params, const std::vector<Var> &grads, Session &s) {
    Context &C = s.ctx();
    Prepared prep;
    sage_status st = prepare(params, grads, s, &prep);
    if (st) return st;
    for (size_t i = 0; i < params.size(); ++i) {
        auto it = state.find(grads[i].key());
        k::OptSlot &slot = prep.slots[i];
        if (it == state.end()) {
            Moments mo;
            mo.grad = grads[i];
            st = Tensor::uninit(C, params[i].desc, &mo.m);
            if (st) return st;
            st = Tensor::uninit(C, params[i].desc, &mo.v);
            if (st) return st;
            it = state.emplace(grads[i].key(), mo).first;
            slot.first = 1;
        }
        slot.m = (float *)it->second.m.ptr();
        slot.v = (float *)it->second.v.ptr();
    }
    k::OptAdam r;
    r.lr = lr;
    r.beta1 = beta1;
    r.beta2 = beta2;
    r.one_minus_beta1 = 1.0f - beta1;
    r.one_minus_beta2 = 1.0f - beta2;
    r.eps = eps;
    r.weight_decay = weight_decay;
    r.corr1 = -std::pow(beta1, t) + 1.0f;  // -scalar(beta1, 1).pow(&self.t) + 1.0, optim.rs:168
    r.corr2 = -std::pow(beta2, t) + 1.0f;
    st = k::adam_update(C, prep.slots.data(), (int)prep.slots.size(), r);
    if (st) return st;
    t += 1.0f;  // optim.rs:176
    return SAGE_OK;
}

}  // namespace nn
}  // namespace sage
