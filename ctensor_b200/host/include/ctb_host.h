// Runtime knobs of the host layer (nothing here exists in the reference).
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>
#include "tensor.h"

namespace ctb_host {

// CUDA device that new tensors and operators use (default 0).  Throws std::runtime_error when
// no CUDA device is present: there is no CPU fallback.
void set_device(int index);
int device();

// Callers dereference tensor storage on the host right after an operator returns, so by
// default every operator waits for its kernel.  A caller that keeps data on the GPU across a
// chain of operators can switch this off and call sync_for_host_access() before touching
// storage (the index proxies and print_t do so themselves).
void set_sync_after_op(bool on);
void sync_for_host_access();

// Tensor storage comes from a pool of managed blocks (ctb_pool_alloc_managed): freed tensors
// keep their memory cached for the next tensor of the same size.  This gives the cached blocks
// back to the driver.
void trim_storage_pool();

// Autograd hook.  The reference attaches a GradFn node to every result whose inputs require
// grad (src/core/ops_dispatch.cpp:159-167,247-255,312-315,378-381).  Those node classes belong
// to the caller's autograd library, so it registers a factory once; `op` is the operator name
// ("add", "mul_scalar", "relu", "sum", ...), `inputs` the operands, `scalar` the scalar or dim.
using GradFactory = std::function<std::shared_ptr<GradFn>(const std::string& op, const std::vector<Tensor>& inputs,
                                                          double scalar)>;
void set_grad_factory(GradFactory f);
// For op == "permute" the factory also needs the permutation: the one of the Tensor::permute call
// that is asking for the node (valid during that factory call, per host thread).
const std::vector<size_t>& last_permutation();

// accumulate_grad of the reference's autograd (src/core/autograd.cpp:63-156) on the GPU:
// `grad_buffer` (the tensor that wraps target.impl->grad) += grad_src, with the broadcast dims of
// grad_src summed first and NaN/Inf contributions skipped.  The autograd library calls this in
// place of its host loop.
void accumulate_grad(Tensor& grad_buffer, const Tensor& grad_src);

// Hook behind Tensor::backward(); the autograd library installs its backward(root) here.
void set_backward_entry(std::function<void(Tensor&)> f);

}  // namespace ctb_host
