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

// matmul / matmul_mp reproduce the reference's scalar product bit for bit (ctb_matmul, CUDA cores).
// Switched on, Float32 products run on the tensor cores instead (ctb_matmul_tc: TF32 products, fp32
// accumulation, |error| <= 2^-9 * sum |a_ik b_kj|) — the trade the reference's own SIMD GEMMs make
// against its scalar one, at 30 times the speed.  Off by default; the environment variable
// CTB_HOST_MATMUL_TENSOR_CORES=1 switches it on without a code change.
void set_matmul_tensor_cores(bool on);

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

// ---- fused bodies for the autograd and loss libraries --------------------------------------------------
// What the reference spells as chains of operators or as host loops, as one kernel each (the C ABI's
// ctb_cross_entropy, ctb_cross_entropy_backward, ctb_div_backward, ctb_tanh_backward).  Results are
// fresh tensors; hand them to accumulate_grad as the reference's bodies do with theirs.
//   cross_entropy           Loss::CrossEntropy's value (src/neuralnet/loss.cpp:90-118): logits [B, C],
//                           labels Int32 [B] or [B, 1]; mean or sum over the rows; a label outside
//                           its row throws std::out_of_range like the reference's gather
//   cross_entropy_backward  GradCrossEntropy::backward (:319-370): (softmax - onehot) * grad_scale,
//                           grad_scale = the loss's incoming gradient (divided by B for "mean")
//   div_backward            GradDiv::backward (src/core/autograd.cpp:188-202): both gradients of a / b
//                           in the broadcast shape of the result (either pointer may be null)
//   tanh_backward           GradTanh::backward (:434-438)
Tensor cross_entropy(const Tensor& logits, const Tensor& labels, bool mean = true);
Tensor cross_entropy_backward(const Tensor& logits, const Tensor& labels, double grad_scale);
void div_backward(const Tensor& grad, const Tensor& a, const Tensor& b, Tensor* grad_a, Tensor* grad_b);
Tensor tanh_backward(const Tensor& grad, const Tensor& t);

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
