// Runtime knobs of the first-generation host layer (nothing here exists in the reference).
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>
#include "ctb_optimizer.h"
#include "tensor1.h"

namespace ctb_gen1 {

// CUDA device every tensor lives on (the first generation has no device field: tensor1.h:45-74).
// Throws std::runtime_error when no CUDA device is present: there is no CPU fallback.
void set_device(int index);
int device();

// Wait for the kernels issued so far (operators wait themselves; for callers that issued C-ABI
// calls of their own on the default stream).
void sync_for_host_access();

// The reference creates a result's backward node inside each operator
// (root opsmp.cpp:178-245,292,364-391,443-468; tensor1.cpp:361,405).  The node classes belong to
// the caller's autograd.h, so the translation unit that is compiled beside it
// (autograd_glue_gen1.cpp) registers this factory: `op` is the operator's name without the
// "_mp" suffix ("add", "mult_scalar", "Relu", "sum", "permute", "reshape", ...), `inputs` its
// operands, `scalar` the scalar or dim, `dims` the permutation or the old shape.
using GradFactory = std::function<std::shared_ptr<GradFn>(const std::string& op, const std::vector<Tensor>& inputs,
                                                          double scalar, const std::vector<size_t>& dims)>;
void set_grad_factory(GradFactory f);

// The entry point behind Tensor::backward() (the reference's tensor1.cpp:471-475 calls the free
// function backward(Tensor&) of autograd.cpp).
void set_backward_entry(std::function<void(Tensor&)> f);

// ---- optimizer steps: what this layer's train_utils.h is built on -----------------------------------------
// One fused in-place update of `param` from its gradient buffer (impl->storage->grad) on the GPU,
// with the arithmetic of the reference's optimizer classes (root train_utils.h:48-540).  Nothing
// happens when the parameter has no gradient buffer.  `step` is the 1-based step count; state
// vectors: numel fp32 zeros in device memory (optimizer_state), null where the optimizer has none.
bool has_grad(const Tensor& param);
void* storage_key(const Tensor& param);
std::shared_ptr<float> optimizer_state(const Tensor& param);
void optimizer_step(ctb_opt::Kind kind, Tensor& param, float* state1, float* state2, const ctb_opt::Hyper& hyper, int step);
// Clears the gradient buffer on the GPU (Optimizer::zero_grad, root train_utils.h:37-44).
void zero_grad(Tensor& param);

}  // namespace ctb_gen1
