// Runtime knobs of the host layer (nothing here exists in the reference).
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>
#include "ctb_optimizer.h"
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

// ---- optimizer steps: what the host layer's train_utils.h is built on ----------------------------------
// One fused in-place update of `param` from its gradient buffer on the GPU, with the arithmetic of
// the reference's optimizer classes (src/neuralnet/train_utils.h:50-494), expression for expression.
// Nothing happens when the parameter has no gradient buffer (the reference's own check).
using OptimizerKind = ctb_opt::Kind;
using OptimizerHyper = ctb_opt::Hyper;
// Whether the parameter has a gradient buffer, and the address its optimizer state is filed under
// (the parameter's storage, like the reference's `states` maps).
bool has_grad(const Tensor& param);
void* storage_key(const Tensor& param);
// A per-parameter state vector (moments): numel fp32 zeros in device memory on the parameter's GPU.
std::shared_ptr<float> optimizer_state(const Tensor& param);
// `step` is the 1-based step count; state1 / state2 as the optimizer needs them (null where unused).
void optimizer_step(OptimizerKind kind, Tensor& param, float* state1, float* state2, const OptimizerHyper& hyper, int step);
// Clears the parameter's gradient buffer on the GPU (Optimizer::zero_grad, :37-46).
void zero_grad(Tensor& param);

// Hook behind Tensor::backward(); the autograd library installs its backward(root) here.
void set_backward_entry(std::function<void(Tensor&)> f);

}  // namespace ctb_host
