// The optimizer classes of the reference's src/neuralnet/train_utils.h (Optimizer :26-47, SGD
// :50-80, Adam :83-134, AdamW :137-187, Adamax :190-239, NAdam :241-291, RAdam :293-355, RMSprop
// :357-396, Adagrad :398-437, Lion :439-494) and its StepLR (:496-511) for the B200 host layers:
// the same class names, constructor arguments and defaults, public members (`params`, `lr`),
// `step()` and `zero_grad()`, so a training loop written against the reference compiles unchanged.
//
// What differs is where the work happens.  The reference walks raw host pointers, one OpenMP loop
// per parameter, with the moment vectors in std::vector<float>.  Here every parameter gets ONE fused
// kernel per step (ctb_optimizer_step: parameter, gradient and moments read once and written
// once, 12 - 28 bytes per element), the moment vectors live in device memory, and zero_grad clears
// the gradient buffers on the GPU.  The arithmetic is the reference's, expression for expression:
// the kernels are tested bit for bit against the reference's own classes.
//
// Not here: the reference's train_epoch / evaluate helpers (:513-625).  They belong to its data
// loader and its dashboard, which are not part of the operator path.
#pragma once
// Included by train_utils.h of either host layer, which defines CTB_OPT_NS (ctb_host or ctb_gen1:
// the namespace with has_grad, storage_key, optimizer_state, optimizer_step and zero_grad) first.
#ifndef CTB_OPT_NS
#error "include train_utils.h, not optimizer_classes.h"
#endif
#include <iostream>
#include <memory>
#include <unordered_map>
#include <vector>

#include "ctb_optimizer.h"
#if __has_include("module.h")
#include "module.h"

inline void set_train_mode(std::vector<Module*>& layers, bool train_mode) {
    for (Module* layer : layers) train_mode ? layer->train() : layer->eval();
}
inline void set_model_mode(Module& model, bool train_mode) { train_mode ? model.train() : model.eval(); }
#endif

class Optimizer {
public:
    std::vector<Tensor*> params;
    double lr;

    Optimizer(const std::vector<Tensor*>& p, double learning_rate) : params(p), lr(learning_rate) {}
    virtual ~Optimizer() = default;
    virtual void step() = 0;

    void zero_grad() {
        for (Tensor* p : params)
            if (p) CTB_OPT_NS::zero_grad(*p);
    }

protected:
    using Kind = ctb_opt::Kind;
    // The moment vectors of one parameter, keyed like the reference's `states` map by the address
    // of the parameter's storage; created (zero) at the parameter's first step.
    struct State {
        std::shared_ptr<float> first, second;
    };
    std::unordered_map<void*, State> states;

    static bool has_grad(const Tensor* p) { return p && CTB_OPT_NS::has_grad(*p); }
    State& state_of(Tensor& p, bool two) {
        State& s = states[CTB_OPT_NS::storage_key(p)];
        if (!s.first) s.first = CTB_OPT_NS::optimizer_state(p);
        if (two && !s.second) s.second = CTB_OPT_NS::optimizer_state(p);
        return s;
    }
    // One step of `kind` on every parameter that has a gradient; the optimizers with moment vectors
    // update Float32 parameters only, as in the reference.
    void step_all(Kind kind, int moments, const ctb_opt::Hyper& hyper, int t) {
        for (Tensor* p : params) {
            if (!has_grad(p)) continue;
            if (moments == 0) {
                CTB_OPT_NS::optimizer_step(kind, *p, nullptr, nullptr, hyper, t);
                continue;
            }
            if (p->_dtype() != DType::Float32 || !p->is_contiguous()) continue;
            State& s = state_of(*p, moments == 2);
            CTB_OPT_NS::optimizer_step(kind, *p, s.first.get(), s.second.get(), hyper, t);
        }
    }
    ctb_opt::Hyper hyper(double beta1 = 0.9, double beta2 = 0.999, double eps = 1e-8, double weight_decay = 0.0,
                                   double alpha = 0.99) const {
        ctb_opt::Hyper h;
        h.lr = lr;
        h.beta1 = beta1;
        h.beta2 = beta2;
        h.eps = eps;
        h.weight_decay = weight_decay;
        h.alpha = alpha;
        return h;
    }
};

class SGD : public Optimizer {
public:
    SGD(const std::vector<Tensor*>& p, double learning_rate) : Optimizer(p, learning_rate) {}
    void step() override { step_all(Kind::SGD, 0, hyper(), 1); }
};

class Adam : public Optimizer {
    double beta1, beta2, eps;
    int t;

public:
    Adam(const std::vector<Tensor*>& p, double learning_rate = 0.001, double b1 = 0.9, double b2 = 0.999, double epsilon = 1e-8)
        : Optimizer(p, learning_rate), beta1(b1), beta2(b2), eps(epsilon), t(0) {}
    void step() override { step_all(Kind::Adam, 2, hyper(beta1, beta2, eps), ++t); }
};

class AdamW : public Optimizer {
    double beta1, beta2, eps, weight_decay;
    int t;

public:
    AdamW(const std::vector<Tensor*>& p, double learning_rate = 0.001, double b1 = 0.9, double b2 = 0.999,
          double epsilon = 1e-8, double decay = 0.01)
        : Optimizer(p, learning_rate), beta1(b1), beta2(b2), eps(epsilon), weight_decay(decay), t(0) {}
    void step() override { step_all(Kind::AdamW, 2, hyper(beta1, beta2, eps, weight_decay), ++t); }
};

class Adamax : public Optimizer {
    double beta1, beta2, eps;
    int t;

public:
    Adamax(const std::vector<Tensor*>& p, double learning_rate = 0.002, double b1 = 0.9, double b2 = 0.999,
           double epsilon = 1e-8)
        : Optimizer(p, learning_rate), beta1(b1), beta2(b2), eps(epsilon), t(0) {}
    void step() override { step_all(Kind::Adamax, 2, hyper(beta1, beta2, eps), ++t); }
};

class NAdam : public Optimizer {
    double beta1, beta2, eps, momentum_decay;      // momentum_decay is accepted and, as in the reference, not used
    int t;

public:
    NAdam(const std::vector<Tensor*>& p, double learning_rate = 0.002, double b1 = 0.9, double b2 = 0.999,
          double epsilon = 1e-8, double momentum_decay_ = 0.004)
        : Optimizer(p, learning_rate), beta1(b1), beta2(b2), eps(epsilon), momentum_decay(momentum_decay_), t(0) {}
    void step() override { step_all(Kind::NAdam, 2, hyper(beta1, beta2, eps), ++t); }
};

class RAdam : public Optimizer {
    double beta1, beta2, eps;
    int t;

public:
    RAdam(const std::vector<Tensor*>& p, double learning_rate = 0.001, double b1 = 0.9, double b2 = 0.999,
          double epsilon = 1e-8)
        : Optimizer(p, learning_rate), beta1(b1), beta2(b2), eps(epsilon), t(0) {}
    void step() override { step_all(Kind::RAdam, 2, hyper(beta1, beta2, eps), ++t); }
};

class RMSprop : public Optimizer {
    double alpha, eps;

public:
    RMSprop(const std::vector<Tensor*>& p, double learning_rate = 0.01, double alpha_ = 0.99, double epsilon = 1e-8)
        : Optimizer(p, learning_rate), alpha(alpha_), eps(epsilon) {}
    void step() override { step_all(Kind::RMSprop, 1, hyper(0.9, 0.999, eps, 0.0, alpha), 1); }
};

class Adagrad : public Optimizer {
    double eps;

public:
    Adagrad(const std::vector<Tensor*>& p, double learning_rate = 0.01, double epsilon = 1e-10)
        : Optimizer(p, learning_rate), eps(epsilon) {}
    void step() override { step_all(Kind::Adagrad, 1, hyper(0.9, 0.999, eps), 1); }
};

class Lion : public Optimizer {
    double beta1, beta2, weight_decay;

public:
    Lion(const std::vector<Tensor*>& p, double learning_rate = 0.0001, double b1 = 0.9, double b2 = 0.99, double decay = 0.01)
        : Optimizer(p, learning_rate), beta1(b1), beta2(b2), weight_decay(decay) {}
    void step() override { step_all(Kind::Lion, 1, hyper(beta1, beta2, 1e-8, weight_decay), 1); }
};

// Multiplies the optimizer's learning rate by `gamma` every `step_size` epochs (host-side
// bookkeeping; the message is the reference's).
class StepLR {
    Optimizer& optim;
    int step_size;
    double gamma;
    int last_epoch;

public:
    StepLR(Optimizer& opt, int step, double g = 0.1) : optim(opt), step_size(step), gamma(g), last_epoch(-1) {}
    void step() {
        ++last_epoch;
        if (last_epoch > 0 && last_epoch % step_size == 0) {
            optim.lr *= gamma;
            std::cout << "--- Scheduler: LR set to " << optim.lr << " ---\n";
        }
    }
};
