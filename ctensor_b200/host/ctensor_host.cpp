// Host layer of the B200 operator library: the reference's C++ operator API (names, shapes,
// error texts) implemented on top of the C ABI of include/ctb200.h.  No arithmetic happens
// here: shapes are inferred, the output tensor is allocated, the C entry point is called, and
// — because callers dereference storage on the CPU (src/neuralnet/loss.cpp:25,
// src/core/autograd.cpp:97-155 of the reference) — the call waits for the kernel.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "include/ctb_host.h"
#include "include/ops_dispatch.h"
#include "include/opsmp.h"
#include "../../include/ctb200.h"

namespace {

int g_device = 0;
// The CUDA device is a per-thread setting: every host thread selects g_device before its first
// operator (a process-wide flag would leave a second thread on device 0).
thread_local int t_device_selected = -1;
thread_local std::vector<size_t> t_last_permutation;
bool g_sync_after_op = true;
// matmul on the tensor cores (TF32 products): -1 = not decided yet (the environment variable
// CTB_HOST_MATMUL_TENSOR_CORES=1 switches it on for programs that cannot call the setter)
int g_matmul_tc = -1;
bool matmul_on_tensor_cores() {
    if (g_matmul_tc < 0) {
        const char* e = std::getenv("CTB_HOST_MATMUL_TENSOR_CORES");
        g_matmul_tc = (e && *e == '1') ? 1 : 0;
    }
    return g_matmul_tc == 1;
}
ctb_host::GradFactory g_grad_factory;
std::function<void(Tensor&)> g_backward;

[[noreturn]] void raise(int status) {
    const std::string msg = ctb_last_error();
    switch (status) {
    case CTB_ERR_DIM: throw std::out_of_range(msg);                 // argmax: dim out of range
    case CTB_ERR_ARG: throw std::invalid_argument(msg);
    default: throw std::runtime_error(msg);                        // what the reference throws
    }
}
inline void check(int status) { if (status != CTB_OK) raise(status); }

void ensure_device() {
    if (t_device_selected >= 0) return;
    if (ctb_device_count() <= 0)
        throw std::runtime_error("ctensor_b200: no CUDA device (this library has no CPU fallback)");
    check(ctb_set_device(g_device));
    t_device_selected = g_device;
}

// The GPU an operator on `t` runs on: the index of its Device(CUDA, i) tag
// (src/core/device.h:5-25 of the reference); tensors tagged CPU or without an index live in
// managed memory as well and use the default device.
int device_index_of(const Device& d) { return (d.is_cuda() && d.index >= 0) ? d.index : g_device; }

void use_device(int index) {
    if (t_device_selected == index) return;
    const int count = ctb_device_count();
    if (count <= 0) throw std::runtime_error("ctensor_b200: no CUDA device (this library has no CPU fallback)");
    if (index >= count) throw std::runtime_error("ctensor_b200: tensor is tagged with CUDA device " + std::to_string(index) +
                                                 " but only " + std::to_string(count) + " are visible");
    check(ctb_set_device(index));
    t_device_selected = index;
}
void use_device_of(const Tensor& t) { use_device(device_index_of(t.device())); }

// Operator results are overwritten by the kernel that produces them: their storage skips the
// zero-fill that Storage::allocate otherwise promises (the reference's calloc).
thread_local bool t_alloc_uninitialized = false;
struct UninitializedScope {
    bool prev;
    UninitializedScope() : prev(t_alloc_uninitialized) { t_alloc_uninitialized = true; }
    ~UninitializedScope() { t_alloc_uninitialized = prev; }
};
Tensor new_output(const std::vector<size_t>& shape, DType dt, const Device& dev) {
    UninitializedScope scope;
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(shape, dt, false, Device(DeviceType::CUDA, device_index_of(dev)));
    return out;
}

// Element types beyond Float32 / Int32 / Double64 are served by the reference's scalar back-end
// only (the *_mp names); its dispatcher refuses them (src/core/ops_dispatch.cpp:206-209).
thread_local bool t_scalar_back_end = false;

int dtype_code(DType dt, const char* who) {
    switch (dt) {
    case DType::Float32: return CTB_F32;
    case DType::Int32: return CTB_I32;
    case DType::Double64: return CTB_F64;
    case DType::UInt8: case DType::Int8: case DType::Int16: case DType::Int64: case DType::Bool:
        if (t_scalar_back_end) return (int)dt;              // the C ABI keeps the reference's numbering
        [[fallthrough]];
    default: throw std::runtime_error(std::string(who) + ": unsupported dtype or op not registered");
    }
}

ctb_view view_of(const Tensor& t, const char* who) {
    ctb_view v;
    std::memset(&v, 0, sizeof v);
    v.base = t.impl->data->data.get();
    v.offset = (int64_t)t.impl->offset;
    v.dtype = dtype_code(t.impl->dtype, who);
    v.ndim = (int32_t)t.impl->ndim;
    for (size_t i = 0; i < t.impl->ndim; ++i) {
        v.shape[i] = (int64_t)t.impl->shape[i];
        v.stride[i] = (int64_t)t.impl->strides[i];
    }
    return v;
}

// View for bit copies: only the element size matters to ctb_copy_strided.
ctb_view view_of_bits(const Tensor& t) {
    ctb_view v;
    std::memset(&v, 0, sizeof v);
    v.base = t.impl->data->data.get();
    v.offset = (int64_t)t.impl->offset;
    const size_t es = dtype_size(t.impl->dtype);
    v.dtype = es == 8 ? CTB_F64 : es == 4 ? CTB_F32 : es == 2 ? CTB_U16 : CTB_U8;
    v.ndim = (int32_t)t.impl->ndim;
    for (size_t i = 0; i < t.impl->ndim; ++i) {
        v.shape[i] = (int64_t)t.impl->shape[i];
        v.stride[i] = (int64_t)t.impl->strides[i];
    }
    return v;
}

// All operators of the host layer are issued on the device's default stream: waiting for that
// stream is enough (a device-wide wait would also wait for unrelated streams of the process).
void after_op() { if (g_sync_after_op) check(ctb_sync(nullptr)); }

void attach_grad(Tensor& out, const char* op, const std::vector<Tensor>& inputs, double scalar) {
    bool req = false;
    for (const Tensor& t : inputs) req = req || t.impl->requires_grad;
    if (!req) return;
    out.requires_grad_(true);
    if (g_grad_factory) out.impl->grad_fn = g_grad_factory(op, inputs, scalar);
}

std::vector<size_t> broadcast_shape(const Tensor& a, const Tensor& b) {
    const std::vector<size_t> sa = a.shape(), sb = b.shape();
    const size_t nd = std::max(sa.size(), sb.size());
    std::vector<size_t> out(nd);
    for (size_t i = 0; i < nd; ++i) {
        const size_t da = i < nd - sa.size() ? 1 : sa[i - (nd - sa.size())];
        const size_t db = i < nd - sb.size() ? 1 : sb[i - (nd - sb.size())];
        if (da != db && da != 1 && db != 1) throw std::runtime_error("Shape mismatch in binary op");
        out[i] = da == 1 ? db : da;
    }
    return out;
}

Tensor binary(int op, const char* name, const Tensor& a, const Tensor& b, bool grad) {
    if (!a.impl || !b.impl) throw std::runtime_error("binary_op: null input");
    if (a.device() != b.device()) throw std::runtime_error(std::string(name) + ": tensors must be on same device");
    use_device_of(a);
    // two one-element operands give shape {1} whatever their rank (the reference's scalar
    // short-circuit, src/core/ops_dispatch.cpp:177-203)
    std::vector<size_t> shape = (a.numel() == 1 && b.numel() == 1) ? std::vector<size_t>{1} : broadcast_shape(a, b);
    Tensor out = new_output(shape, a._dtype(), a.device());
    const ctb_view va = view_of(a, name), vb = view_of(b, name), vo = view_of(out, name);
    check(ctb_binary(op, &va, &vb, &vo, nullptr));
    after_op();
    if (grad) attach_grad(out, name, {a, b}, 0.0);
    return out;
}

Tensor unary(int op, const char* name, const Tensor& a, double scalar, bool grad) {
    if (!a.impl) throw std::runtime_error("unary_op: null input");
    use_device_of(a);
    Tensor out = new_output(a.shape(), a._dtype(), a.device());
    const ctb_view va = view_of(a, name), vo = view_of(out, name);
    check(ctb_unary(op, &va, scalar, &vo, nullptr));
    after_op();
    if (grad) attach_grad(out, name, {a}, scalar);
    return out;
}

Tensor reduce(int op, const char* name, const Tensor& a, int dim, bool grad) {
    if (!a.impl) throw std::runtime_error("reduction: null input");
    use_device_of(a);
    const int nd = (int)a.impl->ndim;
    if (dim < -1) {                 // -1 is "everything"; other negative dims wrap (src/core/opsmp.cpp:598)
        dim += nd;
        if (dim < 0) throw std::out_of_range("reduction: dim out of range");
    }
    std::vector<size_t> shape;
    if (dim >= 0 && dim < nd)
        for (int d = 0; d < nd; ++d) if (d != dim) shape.push_back(a.impl->shape[d]);
    if (shape.empty()) shape.push_back(1);
    Tensor out = new_output(shape, op == CTB_ARGMAX ? DType::Int32 : a._dtype(), a.device());
    const ctb_view va = view_of(a, name), vo = view_of(out, name);
    check(ctb_reduce(op, &va, dim, &vo, nullptr));
    after_op();
    if (grad) attach_grad(out, name, {a}, (double)dim);
    return out;
}

}  // namespace

// ---- runtime knobs ------------------------------------------------------------------------------
namespace ctb_host {
ScalarBackEndScope::ScalarBackEndScope() : prev_(t_scalar_back_end) { t_scalar_back_end = true; }
ScalarBackEndScope::~ScalarBackEndScope() { t_scalar_back_end = prev_; }

void set_device(int index) {
    if (ctb_device_count() <= index || index < 0) throw std::runtime_error("ctensor_b200: no such CUDA device");
    check(ctb_set_device(index));
    g_device = index;
    t_device_selected = index;
}
int device() { return g_device; }
void set_sync_after_op(bool on) { g_sync_after_op = on; }
void set_matmul_tensor_cores(bool on) { g_matmul_tc = on ? 1 : 0; }
void sync_for_host_access() { if (t_device_selected >= 0) check(ctb_device_sync()); }
void trim_storage_pool() { check(ctb_pool_trim(-1)); }
const std::vector<size_t>& last_permutation() { return t_last_permutation; }
void set_grad_factory(GradFactory f) { g_grad_factory = std::move(f); }
void accumulate_grad(Tensor& grad_buffer, const Tensor& grad_src) {
    if (!grad_buffer.impl) return;                      // as the reference: nothing to add to
    if (!grad_src.impl) throw std::runtime_error("accumulate_grad: null gradient");
    use_device_of(grad_buffer);
    const ctb_view vg = view_of(grad_buffer, "accumulate_grad"), vs = view_of(grad_src, "accumulate_grad");
    check(ctb_accumulate_grad(&vg, &vs, nullptr));
    after_op();
}

namespace {
// One int32 per device the kernels raise for a label outside its row (managed: the host reads it).
int32_t* bad_label_flag(int index) {
    static thread_local std::vector<std::shared_ptr<void>> flags;
    if ((int)flags.size() <= index) flags.resize(index + 1);
    if (!flags[index]) {
        void* p = nullptr;
        check(ctb_alloc_managed(&p, sizeof(int32_t), /*zero=*/1));
        flags[index] = std::shared_ptr<void>(p, [](void*) {});
    }
    return (int32_t*)flags[index].get();
}
std::vector<size_t> broadcast_of(const Tensor& a, const Tensor& b) { return broadcast_shape(a, b); }
}  // namespace

Tensor cross_entropy(const Tensor& logits, const Tensor& labels, bool mean) {
    if (!logits.impl || !labels.impl) throw std::runtime_error("cross_entropy: null input");
    use_device_of(logits);
    Tensor loss = new_output({1}, DType::Float32, logits.device());
    int32_t* bad = bad_label_flag(device_index_of(logits.device()));
    const ctb_view vx = view_of(logits, "cross_entropy"), vl = view_of(labels, "cross_entropy"), vo = view_of(loss, "cross_entropy");
    check(ctb_cross_entropy(&vx, &vl, mean ? 1 : 0, &vo, bad, nullptr));
    check(ctb_sync(nullptr));
    if (*bad) throw std::out_of_range("Gather index out of bounds");
    return loss;
}

Tensor cross_entropy_backward(const Tensor& logits, const Tensor& labels, double grad_scale) {
    if (!logits.impl || !labels.impl) throw std::runtime_error("cross_entropy_backward: null input");
    use_device_of(logits);
    Tensor grad = new_output(logits.shape(), DType::Float32, logits.device());
    const ctb_view vx = view_of(logits, "cross_entropy_backward"), vl = view_of(labels, "cross_entropy_backward"),
                   vg = view_of(grad, "cross_entropy_backward");
    check(ctb_cross_entropy_backward(&vx, &vl, grad_scale, &vg, /*accumulate=*/0, nullptr, nullptr));
    after_op();
    return grad;
}

void div_backward(const Tensor& grad, const Tensor& a, const Tensor& b, Tensor* grad_a, Tensor* grad_b) {
    if (!grad.impl || !a.impl || !b.impl) throw std::runtime_error("div_backward: null input");
    use_device_of(grad);
    const std::vector<size_t> shape = broadcast_of(a, b);
    ctb_view va_out, vb_out;
    if (grad_a) { *grad_a = new_output(shape, grad._dtype(), grad.device()); va_out = view_of(*grad_a, "div_backward"); }
    if (grad_b) { *grad_b = new_output(shape, grad._dtype(), grad.device()); vb_out = view_of(*grad_b, "div_backward"); }
    const ctb_view vg = view_of(grad, "div_backward"), va = view_of(a, "div_backward"), vb = view_of(b, "div_backward");
    check(ctb_div_backward(&vg, &va, &vb, grad_a ? &va_out : nullptr, grad_b ? &vb_out : nullptr, /*accumulate=*/0, nullptr));
    after_op();
}

Tensor tanh_backward(const Tensor& grad, const Tensor& t) {
    if (!grad.impl || !t.impl) throw std::runtime_error("tanh_backward: null input");
    use_device_of(grad);
    Tensor out = new_output(broadcast_of(grad, t), grad._dtype(), grad.device());
    const ctb_view vg = view_of(grad, "tanh_backward"), vt = view_of(t, "tanh_backward"), vo = view_of(out, "tanh_backward");
    check(ctb_tanh_backward(&vg, &vt, &vo, /*accumulate=*/0, nullptr));
    after_op();
    return out;
}

bool has_grad(const Tensor& param) {
    return param.impl && param.impl->grad && param.impl->grad->data && param.impl->grad->data->data;
}
void* storage_key(const Tensor& param) { return param.impl ? param.impl->data->data.get() : nullptr; }

std::shared_ptr<float> optimizer_state(const Tensor& param) {
    if (!param.impl) throw std::runtime_error("optimizer: null parameter");
    use_device_of(param);
    void* p = nullptr;
    check(ctb_alloc(&p, param.numel() * sizeof(float), /*zero=*/1, nullptr));
    const int index = device_index_of(param.device());
    return std::shared_ptr<float>((float*)p, [index](float* q) {
        // the block goes back to the pool of the GPU it came from; a failure here (process exit
        // after the CUDA context is gone) is not reportable from a deleter
        if (ctb_set_device(index) == CTB_OK) ctb_free(q, nullptr);
        t_device_selected = index;
    });
}

void optimizer_step(OptimizerKind kind, Tensor& param, float* state1, float* state2, const OptimizerHyper& hyper, int step) {
    if (!has_grad(param)) return;
    use_device_of(param);
    Tensor g;
    g.impl = param.impl->grad;
    const ctb_view vp = view_of(param, "optimizer"), vg = view_of(g, "optimizer");
    ctb_optimizer_hyper h;
    h.lr = hyper.lr; h.beta1 = hyper.beta1; h.beta2 = hyper.beta2; h.eps = hyper.eps;
    h.weight_decay = hyper.weight_decay; h.alpha = hyper.alpha;
    check(ctb_optimizer_step((int)kind, &vp, &vg, state1, state2, &h, step, nullptr));
    after_op();
}

void zero_grad(Tensor& param) {
    if (!has_grad(param)) return;
    Tensor g;
    g.impl = param.impl->grad;
    use_device_of(g);
    // one zero element, broadcast over the buffer by the copy kernel (bits, so any 4- or 8-byte dtype)
    static thread_local std::vector<std::shared_ptr<void>> zeros;        // per device
    const int index = device_index_of(g.device());
    if ((int)zeros.size() <= index) zeros.resize(index + 1);
    if (!zeros[index]) {
        void* z = nullptr;
        check(ctb_alloc(&z, 8, /*zero=*/1, nullptr));
        zeros[index] = std::shared_ptr<void>(z, [](void*) {});           // lives as long as the thread's context
    }
    ctb_view vg = view_of_bits(g), vz = vg;
    vz.base = zeros[index].get();
    vz.offset = 0;
    for (int d = 0; d < vz.ndim; ++d) vz.stride[d] = 0;
    check(ctb_copy_into(&vz, &vg, nullptr));
    after_op();
}

void set_backward_entry(std::function<void(Tensor&)> f) { g_backward = std::move(f); }
int last_dim_if_negative(const Tensor& t, int dim) {
    if (!t.impl) throw std::runtime_error("reduction: null input");
    return dim < 0 ? dim + (int)t.impl->ndim : dim;
}
}  // namespace ctb_host

// ---- storage: replaces Storage::allocate (src/core/tensor.cpp:18-39) --------------------------------
// Managed memory from the library's size-bucketed pool (the reference's unfinished
// CudaMemoryPool, src/core/tensor.h:253-289), resident on the GPU the Device tag names.
// Zero-filled like the reference's calloc, except for operator results (new_output).
std::shared_ptr<Storage> Storage::allocate(size_t n, DType dt, bool /*requires_grad*/, Device dev) {
    ensure_device();
    const int index = device_index_of(dev);
    auto s = std::make_shared<Storage>();
    s->size = n;
    s->device = Device(DeviceType::CUDA, index);
    void* p = nullptr;
    if (index != t_device_selected) use_device(index);     // the clearing memset runs on that device's stream
    check(ctb_pool_alloc_managed(&p, n * dtype_size(dt), t_alloc_uninitialized ? 0 : 1, index, nullptr));
    if (!t_alloc_uninitialized) check(ctb_sync(nullptr));   // the clearing is queued: the host may write right away
    s->data = std::shared_ptr<void>(p, [](void* q) { ctb_pool_free_managed(q); });
    return s;
}

// ---- Tensor members ------------------------------------------------------------------------------------
Tensor::Tensor(const std::vector<size_t>& shape_, DType dtype_, bool requires_grad_)
    : impl(std::make_shared<Tensorimpl>(shape_, dtype_, requires_grad_, Device(DeviceType::CUDA, g_device))) {}

Device Tensor::device() const { return impl ? impl->data->device : Device(DeviceType::CPU); }

// A copy whose storage lives on `target` (src/core/tensor.h: Tensor::to).  The copy kernel runs
// on the target GPU and reads the source through managed memory.
Tensor Tensor::to(Device target) {
    if (!impl || device() == target) return *this;
    if (target.is_cuda() && target.index >= ctb_device_count())
        throw std::runtime_error("Tensor::to: no such CUDA device");
    ctb_host::sync_for_host_access();          // work queued on the source's device is done
    const int index = device_index_of(target);
    use_device(index);
    Tensor out = new_output(shape(), impl->dtype, Device(DeviceType::CUDA, index));
    out.impl->requires_grad = impl->requires_grad;
    ctb_view vs = view_of_bits(*this), vo = view_of_bits(out);
    check(ctb_copy_strided(&vs, &vo, nullptr));
    check(ctb_sync(nullptr));
    out.impl->data->device = target;            // keeps a CPU tag if that is what was asked for
    return out;
}

bool Tensor::is_contiguous() const {
    if (!impl) return true;
    size_t expect = 1;
    for (size_t i = impl->ndim; i-- > 0;) {
        if (impl->shape[i] > 1) {               // size-1 dims never break contiguity
            if (impl->strides[i] != expect) return false;
            expect *= impl->shape[i];
        }
    }
    return true;
}

Tensor Tensor::clone() const {
    if (!impl) return Tensor();
    use_device_of(*this);
    Tensor out = new_output(shape(), impl->dtype, device());
    out.impl->requires_grad = impl->requires_grad;
    ctb_view vs = view_of_bits(*this), vo = view_of_bits(out);      // strided gather on the GPU, bit copy
    check(ctb_copy_strided(&vs, &vo, nullptr));
    after_op();
    return out;
}

Tensor Tensor::contiguous() const { return is_contiguous() ? *this : clone(); }

Tensor Tensor::detach() const {
    if (!impl) return Tensor();
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(impl->data, impl->offset, impl->shape, impl->strides, impl->dtype, false);
    return out;
}

Tensor Tensor::reshape(const std::vector<size_t>& new_shape) const {
    if (!impl) throw std::runtime_error("Reshape on empty tensor");
    size_t n = 1;
    for (size_t s : new_shape) n *= s;
    if (n != numel()) throw std::runtime_error("Reshape size mismatch");
    if (!is_contiguous()) return contiguous().reshape(new_shape);    // repack first, as the reference does
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(impl->data, impl->offset, DimVec(new_shape), calc_strides(DimVec(new_shape)),
                                           impl->dtype, impl->requires_grad);
    if (impl->requires_grad && g_grad_factory) out.impl->grad_fn = g_grad_factory("reshape", {*this}, 0.0);
    return out;
}

Tensor Tensor::permute(const std::vector<size_t>& dims) const {
    if (!impl) throw std::runtime_error("Permute on empty tensor");
    if (dims.size() != impl->ndim) throw std::runtime_error("Permute dim mismatch");
    DimVec shape, strides;
    for (size_t d : dims) {
        if (d >= impl->ndim) throw std::out_of_range("Permute dimension out of range");
        shape.push_back(impl->shape[d]);
        strides.push_back(impl->strides[d]);
    }
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(impl->data, impl->offset, shape, strides, impl->dtype, impl->requires_grad);
    if (impl->requires_grad && g_grad_factory) {
        t_last_permutation = dims;
        out.impl->grad_fn = g_grad_factory("permute", {*this}, 0.0);
    }
    return out;
}

Tensor& Tensor::t_() {
    if (!impl) return *this;
    if (impl->ndim != 2) throw std::runtime_error("t_() only supports 2D tensors");
    std::swap(impl->shape[0], impl->shape[1]);
    std::swap(impl->strides[0], impl->strides[1]);
    return *this;
}

Tensor Tensor::select(size_t dim, size_t index) const {
    if (!impl) throw std::runtime_error("Select on empty tensor");
    if (dim >= impl->ndim) throw std::out_of_range("Select dimension out of range");
    if (index >= impl->shape[dim]) throw std::out_of_range("Select index out of range");
    DimVec shape, strides;
    for (size_t d = 0; d < impl->ndim; ++d)
        if (d != dim) { shape.push_back(impl->shape[d]); strides.push_back(impl->strides[d]); }
    if (shape.empty()) { shape.push_back(1); strides.push_back(1); }
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(impl->data, impl->offset + index * impl->strides[dim], shape, strides,
                                           impl->dtype, impl->requires_grad);
    return out;
}

// Tensor::gather, src/core/tensor.cpp:344-428.
Tensor Tensor::gather(const Tensor& index, size_t dim) const {
    if (!impl) throw std::runtime_error("Gather on empty tensor");
    if (!index.impl) throw std::runtime_error("Gather with empty index");
    if (dim >= impl->ndim) throw std::out_of_range("Gather dimension out of range");
    if (impl->ndim != index.impl->ndim) throw std::runtime_error("Input and index must have same number of dimensions");
    const DType index_dtype = index._dtype();            // any integer dtype (src/core/tensor.cpp:352-356)
    if (index_dtype == DType::Float32 || index_dtype == DType::Double64 || index_dtype == DType::Float16)
        throw std::runtime_error("Index tensor must be integer type");
    use_device_of(*this);
    Tensor out = new_output(index.shape(), impl->dtype, device());
    out.impl->requires_grad = impl->requires_grad;
    if (out.numel() == 0) return out;
    ctb_host::ScalarBackEndScope every_dtype;           // values are moved, indices read through double: any dtype
    const ctb_view vx = view_of(*this, "gather"), vi = view_of(index, "gather"), vo = view_of(out, "gather");
    // the kernel cannot throw: it raises a flag in managed memory that is read after the wait
    // (one flag per device, allocated on first use and kept)
    static std::mutex flag_mu;
    static int32_t* flags[64] = {};
    int32_t* flag = nullptr;
    {
        std::lock_guard<std::mutex> lk(flag_mu);
        int32_t*& slot = flags[t_device_selected & 63];
        if (!slot) check(ctb_alloc_managed((void**)&slot, sizeof(int32_t), 1));
        flag = slot;
    }
    check(ctb_gather(&vx, (int)dim, &vi, &vo, flag, nullptr));
    check(ctb_sync(nullptr));
    if (*(volatile int32_t*)flag) throw std::out_of_range("Gather index out of bounds");
    if (impl->requires_grad) attach_grad(out, "gather", {*this, index}, (double)dim);
    return out;
}

Tensor Tensor::squeeze() const {
    if (!impl) throw std::runtime_error("Squeeze on empty tensor");
    std::vector<size_t> s;
    for (size_t d : impl->shape) if (d != 1) s.push_back(d);
    if (s.empty()) s.push_back(1);
    return reshape(s);
}

Tensor Tensor::unsqueeze(size_t dim) const {
    std::vector<size_t> s = shape();
    if (dim > s.size()) dim = s.size();
    s.insert(s.begin() + (long)dim, 1);
    return reshape(s);
}

Tensor Tensor::flatten() const { return reshape({numel()}); }

void Tensor::print_shape() const {
    std::cout << "(";
    const auto s = shape();
    for (size_t i = 0; i < s.size(); ++i) std::cout << s[i] << (i + 1 < s.size() ? ", " : "");
    std::cout << ")\n";
}

Tensor Tensor::argmax(int dim) const { return ::argmax(*this, dim); }

Tensor Tensor::astype(DType new_dtype) const {
    if (_dtype() == new_dtype) return *this;
    // element-by-element through double, walking storage linearly (the reference's astype,
    // src/core/tensor.cpp:293-305); host side: this is a conversion utility, not an operator
    ctb_host::sync_for_host_access();
    Tensor out(shape(), new_dtype, requires_grad());
    const size_t n = numel();
    for (size_t i = 0; i < n; ++i) out.write_scalar(i, read_scalar(i));
    return out;
}

void Tensor::to_(DType new_dtype) {
    if (impl && impl->dtype != new_dtype) *this = astype(new_dtype);
}

static Tensor filled(const std::vector<size_t>& shape, double value, DType dt, bool req) {
    Tensor t(shape, dt, req);
    if (value != 0.0) {
        const size_t n = t.numel();
        for (size_t i = 0; i < n; ++i) t.write_scalar(i, value);
    }
    return t;
}
Tensor Tensor::ones(const std::vector<size_t>& s, DType dt, bool req) { return filled(s, 1.0, dt, req); }
Tensor Tensor::zeros(const std::vector<size_t>& s, DType dt, bool req) { return Tensor(s, dt, req); }
Tensor Tensor::empty(const std::vector<size_t>& s, DType dt, bool req) { return Tensor(s, dt, req); }
Tensor Tensor::full(const std::vector<size_t>& s, double v, DType dt, bool req) { return filled(s, v, dt, req); }

Tensor Tensor::rand(const std::vector<size_t>& s, DType dt, bool req) {
    Tensor t(s, dt, req);
    const size_t n = t.numel();
    for (size_t i = 0; i < n; ++i) t.write_scalar(i, (double)std::rand() / RAND_MAX);
    return t;
}

Tensor Tensor::from_vector(const std::vector<double>& data, const std::vector<size_t>& shape, DType dt, bool req) {
    Tensor t(shape, dt, req);
    if (t.numel() != data.size()) throw std::runtime_error("from_vector size mismatch");
    for (size_t i = 0; i < data.size(); ++i) t.write_scalar(i, data[i]);
    return t;
}

Tensor Tensor::arange(double start, double end, double step, DType dt) {
    const size_t steps = (size_t)std::ceil((end - start) / step);
    Tensor t({steps}, dt);
    for (size_t i = 0; i < steps; ++i) t.write_scalar(i, start + (double)i * step);
    return t;
}

void Tensor::backward() {
    if (!impl || !impl->requires_grad) return;
    if (!g_backward) throw std::runtime_error("backward: no autograd library registered (ctb_host::set_backward_entry)");
    g_backward(*this);
}

void Tensor::zero_grad() {
    if (!impl || !impl->grad) return;
    ctb_host::sync_for_host_access();
    std::memset(impl->grad->data->data.get(), 0, numel() * dtype_bytes());
}

// ---- operators ---------------------------------------------------------------------------------------------
Tensor add(const Tensor& a, const Tensor& b) { return binary(CTB_ADD, "add", a, b, true); }
Tensor sub(const Tensor& a, const Tensor& b) { return binary(CTB_SUB, "sub", a, b, true); }
Tensor mul(const Tensor& a, const Tensor& b) { return binary(CTB_MUL, "mul", a, b, true); }
Tensor div(const Tensor& a, const Tensor& b) { return binary(CTB_DIV, "div", a, b, true); }
Tensor pow(const Tensor& a, const Tensor& b) { return binary(CTB_POW, "pow", a, b, true); }

Tensor add_scalar(const Tensor& a, double s) { return unary(CTB_ADD_S, "add_scalar", a, s, true); }
Tensor sub_scalar(const Tensor& a, double s) { return unary(CTB_SUB_S, "sub_scalar", a, s, true); }
Tensor sub_scalar_rev(double s, const Tensor& a) { return unary(CTB_RSUB_S, "sub_scalar_rev", a, s, true); }
Tensor mul_scalar(const Tensor& a, double s) { return unary(CTB_MUL_S, "mul_scalar", a, s, true); }
Tensor div_scalar(const Tensor& a, double s) { return unary(CTB_DIV_S, "div_scalar", a, s, true); }
Tensor div_scalar_rev(double s, const Tensor& a) { return unary(CTB_RDIV_S, "div_scalar_rev", a, s, true); }
Tensor pow_scalar(const Tensor& a, double s) { return unary(CTB_POW_S, "pow_scalar", a, s, true); }
Tensor pow_scalar_rev(double s, const Tensor& a) { return unary(CTB_RPOW_S, "pow_scalar_rev", a, s, true); }

Tensor lt(const Tensor& a, const Tensor& b) { return binary(CTB_LT, "lt", a, b, false); }
Tensor le(const Tensor& a, const Tensor& b) { return binary(CTB_LE, "le", a, b, false); }
Tensor gt(const Tensor& a, const Tensor& b) { return binary(CTB_GT, "gt", a, b, false); }
Tensor ge(const Tensor& a, const Tensor& b) { return binary(CTB_GE, "ge", a, b, false); }
Tensor eq(const Tensor& a, const Tensor& b) { return binary(CTB_EQ, "eq", a, b, false); }
Tensor ne(const Tensor& a, const Tensor& b) { return binary(CTB_NE, "ne", a, b, false); }
Tensor lt(const Tensor& a, double b) { return unary(CTB_LT_S, "lt", a, b, false); }
Tensor le(const Tensor& a, double b) { return unary(CTB_LE_S, "le", a, b, false); }
Tensor gt(const Tensor& a, double b) { return unary(CTB_GT_S, "gt", a, b, false); }
Tensor ge(const Tensor& a, double b) { return unary(CTB_GE_S, "ge", a, b, false); }
Tensor eq(const Tensor& a, double b) { return unary(CTB_EQ_S, "eq", a, b, false); }
Tensor ne(const Tensor& a, double b) { return unary(CTB_NE_S, "ne", a, b, false); }

Tensor abs(const Tensor& a) { return unary(CTB_ABS, "abs", a, 0.0, true); }
Tensor log(const Tensor& a) { return unary(CTB_LOG, "log", a, 0.0, true); }
Tensor ln(const Tensor& a) { return unary(CTB_LOG, "ln", a, 0.0, true); }
Tensor exp(const Tensor& a) { return unary(CTB_EXP, "exp", a, 0.0, true); }
Tensor sqrt(const Tensor& a) { return unary(CTB_SQRT, "sqrt", a, 0.0, true); }
Tensor sin(const Tensor& a) { return unary(CTB_SIN, "sin", a, 0.0, true); }
Tensor cos(const Tensor& a) { return unary(CTB_COS, "cos", a, 0.0, true); }
Tensor tan(const Tensor& a) { return unary(CTB_TAN, "tan", a, 0.0, true); }
Tensor asin(const Tensor& a) { return unary(CTB_ASIN, "asin", a, 0.0, true); }
Tensor acos(const Tensor& a) { return unary(CTB_ACOS, "acos", a, 0.0, true); }
Tensor atan(const Tensor& a) { return unary(CTB_ATAN, "atan", a, 0.0, true); }
Tensor sinh(const Tensor& a) { return unary(CTB_SINH, "sinh", a, 0.0, true); }
Tensor cosh(const Tensor& a) { return unary(CTB_COSH, "cosh", a, 0.0, true); }
Tensor softplus(const Tensor& a) { return unary(CTB_SOFTPLUS, "softplus", a, 0.0, true); }
Tensor tanh(const Tensor& a) { return unary(CTB_TANH, "tanh", a, 0.0, true); }
Tensor sigmoid(const Tensor& a) { return unary(CTB_SIGMOID, "sigmoid", a, 0.0, true); }
Tensor relu(const Tensor& a) { return unary(CTB_RELU, "relu", a, 0.0, true); }
Tensor gelu(const Tensor& a) { return unary(CTB_GELU_TANH, "gelu", a, 0.0, true); }

Tensor sum(const Tensor& a, int dim) { return reduce(CTB_SUM, "sum", a, dim, true); }
// mean = mul_scalar(sum, 1/N) in the reference (src/core/ops_dispatch.cpp:385-390).  The fused
// kernel gives the same bits in one pass; when a gradient is wanted the two operators are
// issued as the reference issues them, so the graph has the reference's two nodes.
Tensor mean(const Tensor& a, int dim) {
    if (a.impl && a.impl->requires_grad) {
        Tensor s = sum(a, dim);
        const int nd = (int)a.impl->ndim;
        const int d = dim < -1 ? dim + nd : dim;
        const double n = (d >= 0 && d < nd) ? (double)a.impl->shape[d] : (double)a.numel();
        return mul_scalar(s, 1.0 / n);
    }
    return reduce(CTB_MEAN, "mean", a, dim, false);
}
Tensor max(const Tensor& a, int dim) { return reduce(CTB_MAX, "max", a, dim, false); }
Tensor min(const Tensor& a, int dim) { return reduce(CTB_MIN, "min", a, dim, false); }
Tensor var(const Tensor& a, int dim) { return reduce(CTB_VAR, "var", a, dim, false); }

Tensor argmax(const Tensor& a, int dim) {
    if (!a.impl) throw std::runtime_error("argmax: empty tensor");
    if (dim < 0) dim += (int)a.impl->ndim;          // negative dims wrap (src/core/ops_dispatch.cpp:432)
    return reduce(CTB_ARGMAX, "argmax", a, dim, false);
}

static Tensor softmax_impl(const Tensor& a, const Tensor* mask, int causal) {
    if (!a.impl) throw std::runtime_error("softmax: null input");
    use_device_of(a);
    Tensor out = new_output(a.shape(), a._dtype(), a.device());
    const ctb_view va = view_of(a, "softmax"), vo = view_of(out, "softmax");
    ctb_view vm;
    if (mask) vm = view_of(*mask, "softmax");
    check(ctb_softmax_lastdim(&va, mask ? &vm : nullptr, causal, &vo, nullptr));
    after_op();
    return out;
}
Tensor softmax(const Tensor& a) { return softmax_impl(a, nullptr, 0); }
Tensor softmax(const Tensor& a, const Tensor& additive_mask) {
    if (!additive_mask.impl) throw std::runtime_error("softmax: null mask");
    return softmax_impl(a, &additive_mask, 0);
}
Tensor causal_softmax(const Tensor& a) { return softmax_impl(a, nullptr, 1); }

// matmul_mp, src/core/opsmp.cpp:460-482 (shape rules) — the product itself runs in ctb_matmul.
Tensor matmul(const Tensor& a, const Tensor& b) {
    if (!a.impl || !b.impl) throw std::runtime_error("matmul: null input");
    if (a.impl->ndim < 2 || b.impl->ndim < 2) throw std::runtime_error("matmul_mp requires at least 2D tensors");
    if (b.impl->shape[b.impl->ndim - 2] != a.impl->shape[a.impl->ndim - 1]) throw std::runtime_error("matmul_mp shape mismatch");
    use_device_of(a);
    std::vector<size_t> res_shape = a.shape();
    res_shape.back() = b.impl->shape[b.impl->ndim - 1];
    const bool req = a.requires_grad() || b.requires_grad();
    Tensor out = new_output(res_shape, a._dtype(), a.device());
    out.impl->requires_grad = req;
    const ctb_view va = view_of(a, "matmul"), vb = view_of(b, "matmul"), vo = view_of(out, "matmul");
    if (matmul_on_tensor_cores() && a._dtype() == DType::Float32) {
        // A wait inside the kernel that gave up is reported through a status word.  Reading it on the
        // host moves its (managed) page across PCIe and back, so it is looked at on the first call
        // and on every 64th: enough to stop a program whose products have started to fail.
        static thread_local std::vector<std::shared_ptr<void>> status;          // one int32 per device
        static thread_local unsigned calls = 0;
        const int index = device_index_of(a.device());
        if ((int)status.size() <= index) status.resize(index + 1);
        const bool look = (calls++ % 64) == 0;
        if (look && !status[index]) {
            void* p = nullptr;
            check(ctb_alloc_managed(&p, sizeof(int32_t), /*zero=*/1));
            status[index] = std::shared_ptr<void>(p, [](void*) {});
        }
        check(ctb_matmul_tc(&va, &vb, &vo, look ? (int32_t*)status[index].get() : nullptr, nullptr));
        after_op();
        if (look) {
            check(ctb_sync(nullptr));
            if (*(const int32_t*)status[index].get() != 0) throw std::runtime_error("matmul: the tensor-core kernel gave up a wait");
        }
    } else {
        check(ctb_matmul(&va, &vb, &vo, nullptr));
        after_op();
    }
    if (req) attach_grad(out, "matmul", {a, b}, 0.0);
    return out;
}

// cat_mp, src/core/opsmp.cpp:717-804.
Tensor cat(const std::vector<Tensor>& tensors, size_t dim) {
    if (tensors.empty()) throw std::runtime_error("cat_mp: empty list");
    for (const Tensor& t : tensors)
        if (!t.impl) throw std::runtime_error("cat_mp: null tensor");
    std::vector<size_t> out_shape = tensors[0].shape();
    const size_t ndim = out_shape.size();
    if (dim >= ndim) throw std::out_of_range("cat_mp: dim out of range");
    size_t dim_sum = 0;
    for (const Tensor& t : tensors) {
        if (t.impl->ndim != ndim) throw std::runtime_error("cat_mp: ndim mismatch");
        for (size_t i = 0; i < ndim; ++i)
            if (i != dim && t.impl->shape[i] != out_shape[i]) throw std::runtime_error("cat_mp: shape mismatch outside cat dim");
        dim_sum += t.impl->shape[dim];
    }
    out_shape[dim] = dim_sum;
    use_device_of(tensors[0]);
    Tensor out = new_output(out_shape, tensors[0]._dtype(), tensors[0].device());
    std::vector<ctb_view> views;
    std::vector<const ctb_view*> ptrs;
    views.reserve(tensors.size());
    for (const Tensor& t : tensors) views.push_back(view_of(t, "cat_mp"));
    for (const ctb_view& v : views) ptrs.push_back(&v);
    const ctb_view vo = view_of(out, "cat_mp");
    check(ctb_cat(ptrs.data(), (int)ptrs.size(), (int)dim, &vo, nullptr));
    after_op();
    return out;
}

// src/neuralnet/batchnorm/batchnorm.cpp:46-61 and :103-113.
void channel_moments(const Tensor& x, Tensor& mean, Tensor& var) {
    if (!x.impl) throw std::runtime_error("batchnorm: null input");
    if (x.impl->ndim < 2) throw std::runtime_error("batchnorm: input needs [batch, channels, ...]");
    use_device_of(x);
    const Tensor xc = x.is_contiguous() ? x : x.contiguous();
    mean = new_output({x.impl->shape[1]}, x._dtype(), x.device());
    var = new_output({x.impl->shape[1]}, x._dtype(), x.device());
    const ctb_view vx = view_of(xc, "batchnorm"), vm = view_of(mean, "batchnorm"), vv = view_of(var, "batchnorm");
    check(ctb_channel_moments(&vx, &vm, &vv, nullptr));
    after_op();
}

Tensor batch_norm_apply(const Tensor& x, const Tensor& mean, const Tensor& var, const Tensor& gamma,
                        const Tensor& beta, double eps) {
    if (!x.impl || !mean.impl || !var.impl) throw std::runtime_error("batchnorm: null input");
    use_device_of(x);
    const Tensor xc = x.is_contiguous() ? x : x.contiguous();
    Tensor out = new_output(x.shape(), x._dtype(), x.device());
    const ctb_view vx = view_of(xc, "batchnorm"), vm = view_of(mean, "batchnorm"), vv = view_of(var, "batchnorm"),
                   vo = view_of(out, "batchnorm");
    ctb_view vg, vb;
    if (gamma.impl) vg = view_of(gamma, "batchnorm");
    if (beta.impl) vb = view_of(beta, "batchnorm");
    check(ctb_batchnorm_apply(&vx, &vm, &vv, gamma.impl ? &vg : nullptr, beta.impl ? &vb : nullptr, eps, &vo, nullptr));
    after_op();
    return out;
}

Tensor log_softmax(const Tensor& a) {
    if (!a.impl) throw std::runtime_error("log_softmax: null input");
    use_device_of(a);
    Tensor out = new_output(a.shape(), a._dtype(), a.device());
    const ctb_view va = view_of(a, "log_softmax"), vo = view_of(out, "log_softmax");
    check(ctb_log_softmax_lastdim(&va, nullptr, &vo, nullptr));
    after_op();
    return out;
}

Tensor layer_norm(const Tensor& a, const Tensor& gamma, const Tensor& beta, double eps) {
    if (!a.impl) throw std::runtime_error("layernorm: null input");
    use_device_of(a);
    Tensor out = new_output(a.shape(), a._dtype(), a.device());
    const ctb_view va = view_of(a, "layernorm"), vo = view_of(out, "layernorm");
    ctb_view vg, vb;
    if (gamma.impl) vg = view_of(gamma, "layernorm");
    if (beta.impl) vb = view_of(beta, "layernorm");
    check(ctb_layernorm_lastdim(&va, gamma.impl ? &vg : nullptr, beta.impl ? &vb : nullptr, eps, &vo, nullptr));
    after_op();
    return out;
}
