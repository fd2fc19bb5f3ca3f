// Runtime knobs of the first-generation host layer (nothing here exists in the reference).
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>
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

}  // namespace ctb_gen1
