// Optimizers.  Reference: src/optim.rs (trait Optimizer :8-12, Sgd :14-94, Adam :97-178).
//
// The reference's update() walks a HashMap<&Var, Var> (parameter -> gradient variable), builds lazy
// expressions per parameter and evaluates them one by one.  Here the same arithmetic runs as one
// in-place launch over all parameters (kernels/optim.cu); the optimizer's state is keyed by the
// gradient variable exactly like the reference's `m_t` / `v_t` maps.
#pragma once
#include <unordered_map>
#include <vector>

#include "../graph/graph.h"

namespace sage {
namespace nn {

struct Optimizer {
    virtual ~Optimizer() {}
    virtual sage_status init(Session &s) = 0;  // Optimizer::init, optim.rs:9
    // Optimizer::update, optim.rs:11.  params[i] must be data variables; grads[i] is d loss / d params[i],
    // normally already evaluated in the session (otherwise it is evaluated here, like the reference does).
    virtual sage_status update(const std::vector<Var> &params, const std::vector<Var> &grads, Session &s) = 0;
};

struct Sgd : Optimizer {  // optim.rs:14-94
    float lr, momentum = 0.f, dampening = 0.f, weight_decay = 0.f;
    bool nesterov = false;
    explicit Sgd(float lr_) : lr(lr_) {}
    sage_status init(Session &) override { return SAGE_OK; }
    sage_status update(const std::vector<Var> &params, const std::vector<Var> &grads, Session &s) override;
};

struct Adam : Optimizer {  // optim.rs:97-178
    float lr, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-08f, weight_decay = 0.f;
    float t = 1.0f;  // the reference keeps the step count as an f32 tensor and adds 1.0 per update
    struct Moments {
        Var grad;  // keeps the key alive
        Tensor m, v;
    };
    std::unordered_map<Origin *, Moments> state;
    explicit Adam(float lr_) : lr(lr_) {}
    sage_status init(Session &s) override;
    sage_status update(const std::vector<Var> &params, const std::vector<Var> &grads, Session &s) override;
};

}  // namespace nn
}  // namespace sage
