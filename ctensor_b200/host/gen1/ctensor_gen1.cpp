// First-generation host layer: the members of tensor1.h and the `*_mp` operators of opsmp.h
// (the reference's root tensor1.cpp and opsmp.cpp) on top of the C ABI of include/ctb200.h.
// No arithmetic happens here: shapes are inferred, the output is allocated from the library's
// managed-memory pool, the C entry point is called and — because the callers dereference
// storage on the host right away (autograd.cpp:21-34, loss.cpp:23-26) — the call waits for the
// kernel.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "include/ctb_gen1.h"
#include "include/opsmp.h"
#include "../../../include/ctb200.h"

namespace {

int g_device = 0;
thread_local int t_device_selected = -1;
ctb_gen1::GradFactory g_grad_factory;
std::function<void(Tensor&)> g_backward;

[[noreturn]] void raise(int status) {
    const std::string msg = ctb_last_error();
    switch (status) {
    case CTB_ERR_DIM: throw std::out_of_range(msg);
    case CTB_ERR_ARG: throw std::invalid_argument(msg);
    default: throw std::runtime_error(msg);
    }
}
inline void check(int status) { if (status != CTB_OK) raise(status); }

void ensure_device() {
    if (t_device_selected == g_device) return;
    if (ctb_device_count() <= 0)
        throw std::runtime_error("ctensor_b200: no CUDA device (this library has no CPU fallback)");
    check(ctb_set_device(g_device));
    t_device_selected = g_device;
}

// Operators wait for their kernel: callers read results on the host straight away.
void after_op() { check(ctb_sync(nullptr)); }

// Operator results are overwritten by the kernel that produces them and skip the zero-fill.
thread_local bool t_alloc_uninitialized = false;
struct UninitializedScope {
    bool prev;
    UninitializedScope() : prev(t_alloc_uninitialized) { t_alloc_uninitialized = true; }
    ~UninitializedScope() { t_alloc_uninitialized = prev; }
};

std::shared_ptr<void> managed_block(size_t bytes, bool zero) {
    void* p = nullptr;
    check(ctb_pool_alloc_managed(&p, bytes, zero ? 1 : 0, g_device, nullptr));
    return std::shared_ptr<void>(p, [](void* q) { ctb_pool_free_managed(q); });
}

int dtype_code(DType dt) { return dt == DType::Float32 ? CTB_F32 : dt == DType::Int32 ? CTB_I32 : CTB_F64; }

ctb_view view_of(const Tensor& t) {
    ctb_view v;
    std::memset(&v, 0, sizeof v);
    if (t.impl->ndim > CTB_MAX_DIMS) throw std::length_error("tensor: more than 8 dimensions");
    v.base = t.impl->storage->data.get();
    v.offset = (int64_t)t.impl->offset;
    v.dtype = dtype_code(t.impl->dtype);
    v.ndim = (int32_t)t.impl->ndim;
    for (size_t i = 0; i < t.impl->ndim; ++i) {
        v.shape[i] = (int64_t)t.impl->shape[i];
        v.stride[i] = (int64_t)t.impl->strides[i];
    }
    return v;
}

// A fresh contiguous result: data is left for the kernel to write; a gradient buffer (zeroed) comes
// with it when the result requires grad, as in the reference (Tensor out(shape, dtype, req)).
Tensor new_output(const std::vector<size_t>& shape, DType dt, bool requires_grad) {
    UninitializedScope scope;
    return Tensor(shape, dt, requires_grad);
}

std::vector<size_t> row_major_strides(const std::vector<size_t>& shape) {
    std::vector<size_t> st(shape.size());
    size_t run = 1;
    for (size_t i = shape.size(); i-- > 0;) {
        st[i] = run;
        run *= shape[i];
    }
    return st;
}

void attach(Tensor& out, const char* op, const std::vector<Tensor>& inputs, double scalar = 0.0,
            const std::vector<size_t>& dims = {}) {
    if (out.impl->requires_grad && g_grad_factory) out.impl->grad_fn = g_grad_factory(op, inputs, scalar, dims);
}

std::vector<size_t> broadcast_shape(const Tensor& a, const Tensor& b) {
    const std::vector<size_t> sa = a.shape(), sb = b.shape();
    const size_t nd = std::max(sa.size(), sb.size());
    std::vector<size_t> out(nd);
    for (size_t i = 0; i < nd; ++i) {
        const size_t da = i < nd - sa.size() ? 1 : sa[i - (nd - sa.size())];
        const size_t db = i < nd - sb.size() ? 1 : sb[i - (nd - sb.size())];
        if (da != db && da != 1 && db != 1) throw std::runtime_error("Shape mismatch in binary op");
        out[i] = std::max(da, db);
    }
    return out;
}

Tensor binary(int op, const char* name, const Tensor& a, const Tensor& b, bool grad) {
    if (!a.impl || !b.impl) throw std::runtime_error("binary_op: null input");
    ensure_device();
    const bool req = a.requires_grad() || b.requires_grad();
    Tensor out = new_output(broadcast_shape(a, b), a._dtype(), req);
    const ctb_view va = view_of(a), vb = view_of(b), vo = view_of(out);
    check(ctb_binary(op, &va, &vb, &vo, nullptr));
    after_op();
    if (grad) attach(out, name, {a, b});
    return out;
}

Tensor unary(int op, const char* name, const Tensor& a, double scalar, bool grad) {
    if (!a.impl) throw std::runtime_error("unary_op: null input");
    ensure_device();
    Tensor out = new_output(a.shape(), a._dtype(), a.requires_grad());
    const ctb_view va = view_of(a), vo = view_of(out);
    check(ctb_unary(op, &va, scalar, &vo, nullptr));
    after_op();
    if (grad) attach(out, name, {a}, scalar);
    return out;
}

// dim < 0 counts from the end, so -1 is the LAST dim (reduction_op_impl, root opsmp.cpp:396-441).
Tensor reduce(int op, const char* name, const Tensor& t, int dim, bool grad) {
    if (!t.impl) throw std::runtime_error("reduction: null input");
    ensure_device();
    const int nd = (int)t.impl->ndim;
    const int given = dim;
    if (dim < 0) dim += nd;
    if (dim < 0 || dim >= nd) throw std::out_of_range("reduction: dim out of range");
    std::vector<size_t> shape;
    for (int d = 0; d < nd; ++d) if (d != dim) shape.push_back(t.impl->shape[d]);
    if (shape.empty()) shape.push_back(1);
    Tensor out = new_output(shape, t._dtype(), t.requires_grad());
    const ctb_view va = view_of(t), vo = view_of(out);
    check(ctb_reduce(op, &va, dim, &vo, nullptr));
    after_op();
    if (grad) attach(out, name, {t}, (double)given);    // the node keeps the dim as the caller gave it
    return out;
}

}  // namespace

// ---- runtime knobs -------------------------------------------------------------------------------
namespace ctb_gen1 {
void set_device(int index) {
    if (index < 0 || ctb_device_count() <= index) throw std::runtime_error("ctensor_b200: no such CUDA device");
    check(ctb_set_device(index));
    g_device = index;
    t_device_selected = index;
}
int device() { return g_device; }
void sync_for_host_access() { if (t_device_selected >= 0) check(ctb_device_sync()); }
void set_grad_factory(GradFactory f) { g_grad_factory = std::move(f); }
bool has_grad(const Tensor& param) { return param.impl && param.impl->storage && param.impl->storage->grad; }
void* storage_key(const Tensor& param) { return param.impl && param.impl->storage ? param.impl->storage->data.get() : nullptr; }

std::shared_ptr<float> optimizer_state(const Tensor& param) {
    if (!param.impl) throw std::runtime_error("optimizer: null parameter");
    ensure_device();
    void* p = nullptr;
    check(ctb_alloc(&p, param.numel() * sizeof(float), /*zero=*/1, nullptr));
    return std::shared_ptr<float>((float*)p, [](float* q) { ctb_free(q, nullptr); });
}

namespace {
// The gradient buffer as a view: the parameter's own geometry over impl->storage->grad.
ctb_view grad_view_of(const Tensor& param) {
    ctb_view v = view_of(param);
    v.base = param.impl->storage->grad.get();
    return v;
}
}  // namespace

void optimizer_step(ctb_opt::Kind kind, Tensor& param, float* state1, float* state2, const ctb_opt::Hyper& hyper, int step) {
    if (!has_grad(param)) return;
    ensure_device();
    const ctb_view vp = view_of(param), vg = grad_view_of(param);
    ctb_optimizer_hyper h;
    h.lr = hyper.lr; h.beta1 = hyper.beta1; h.beta2 = hyper.beta2; h.eps = hyper.eps;
    h.weight_decay = hyper.weight_decay; h.alpha = hyper.alpha;
    check(ctb_optimizer_step((int)kind, &vp, &vg, state1, state2, &h, step, nullptr));
    after_op();
}

void zero_grad(Tensor& param) {
    if (!has_grad(param)) return;
    ensure_device();
    // one zero element broadcast over the buffer by the copy kernel
    static thread_local void* zero = nullptr;
    if (!zero) check(ctb_alloc(&zero, 8, /*zero=*/1, nullptr));
    ctb_view vg = grad_view_of(param), vz = vg;
    vz.base = zero;
    vz.offset = 0;
    for (int d = 0; d < vz.ndim; ++d) vz.stride[d] = 0;
    check(ctb_copy_into(&vz, &vg, nullptr));
    after_op();
}

void set_backward_entry(std::function<void(Tensor&)> f) { g_backward = std::move(f); }
}  // namespace ctb_gen1

// ---- Storage / Tensorimpl (tensor1.cpp:12-84) -----------------------------------------------------
std::shared_ptr<Storage> Storage::allocate(size_t n, DType dt, bool requires_grad) {
    ensure_device();
    auto s = std::make_shared<Storage>();
    s->size = n;
    const size_t bytes = n * dtype_size(dt);
    s->data = managed_block(bytes, !t_alloc_uninitialized);          // zero-filled like the reference's memset
    if (requires_grad) s->grad = managed_block(bytes, true);
    if (!t_alloc_uninitialized || requires_grad) check(ctb_sync(nullptr));   // the host may write right away
    return s;
}

Tensorimpl::Tensorimpl(const std::vector<size_t>& shape_, DType dtype_, bool requires_grad_)
    : Tensorimpl(nullptr, 0, shape_, row_major_strides(shape_), dtype_, requires_grad_) {
    size_t n = 1;
    for (size_t v : shape_) n *= v;
    storage = Storage::allocate(n, dtype_, requires_grad_);
}

Tensorimpl::Tensorimpl(std::shared_ptr<Storage> storage_, size_t offset_, const std::vector<size_t>& shape_,
                       const std::vector<size_t>& strides_, DType dtype_, bool requires_grad_)
    : storage(std::move(storage_)), offset(offset_), ndim(shape_.size()), requires_grad(requires_grad_), dtype(dtype_) {
    shape = static_cast<size_t*>(std::malloc((ndim ? ndim : 1) * sizeof(size_t)));
    strides = static_cast<size_t*>(std::malloc((ndim ? ndim : 1) * sizeof(size_t)));
    if (!shape || !strides) {
        std::free(shape);
        std::free(strides);
        throw std::bad_alloc();
    }
    for (size_t i = 0; i < ndim; ++i) {
        shape[i] = shape_[i];
        strides[i] = strides_[i];
    }
}

Tensorimpl::Tensorimpl(const Tensorimpl& o)
    : Tensorimpl(o.storage, o.offset, std::vector<size_t>(o.shape, o.shape + o.ndim),
                 std::vector<size_t>(o.strides, o.strides + o.ndim), o.dtype, o.requires_grad) {
    grad_fn = o.grad_fn;
}

Tensorimpl::~Tensorimpl() {
    std::free(shape);
    std::free(strides);
}

// ---- Tensor members (tensor1.cpp:87-581) -------------------------------------------------------------
Tensor::Tensor(const std::vector<size_t>& shape_, DType dtype_, bool requires_grad_)
    : impl(std::make_shared<Tensorimpl>(shape_, dtype_, requires_grad_)) {}

size_t Tensor::numel() const {
    if (!impl) return 0;
    size_t n = 1;
    for (size_t i = 0; i < impl->ndim; ++i) n *= impl->shape[i];
    return n;
}

std::vector<size_t> Tensor::shape() const {
    return impl ? std::vector<size_t>(impl->shape, impl->shape + impl->ndim) : std::vector<size_t>{};
}

bool Tensor::is_contiguous() const {
    if (!impl) return false;
    size_t expect = 1;
    for (size_t i = impl->ndim; i-- > 0;) {
        if (impl->shape[i] != 1) {              // size-1 dims never break contiguity
            if (impl->strides[i] != expect) return false;
            expect *= impl->shape[i];
        }
    }
    return true;
}

// Strided gather on the GPU into fresh packed storage (the reference walks an odometer on the
// host, tensor1.cpp:120-158); bit copy, any dtype.
Tensor Tensor::contiguous() const {
    if (!impl) throw std::runtime_error("Empty tensor");
    if (is_contiguous()) return *this;
    ensure_device();
    Tensor out = new_output(shape(), _dtype(), impl->requires_grad);
    const ctb_view vs = view_of(*this), vo = view_of(out);
    check(ctb_copy_strided(&vs, &vo, nullptr));
    after_op();
    return out;
}

Tensor Tensor::clone() const {
    if (!impl) throw std::runtime_error("Empty tensor");
    if (!is_contiguous()) return contiguous();
    ensure_device();
    Tensor out = new_output(shape(), _dtype(), impl->requires_grad);
    const ctb_view vs = view_of(*this), vo = view_of(out);
    check(ctb_copy_strided(&vs, &vo, nullptr));
    after_op();
    return out;
}

static Tensor filled(const std::vector<size_t>& shape, double value, DType dt, bool req) {
    Tensor t(shape, dt, req);                   // zero-filled
    if (value != 0.0) {
        void* p = t.impl->storage->data.get();
        for (size_t i = 0, n = t.numel(); i < n; ++i) write_scalar_at(p, i, dt, value);
    }
    return t;
}
Tensor Tensor::ones(const std::vector<size_t>& s, DType dt, bool req) { return filled(s, 1.0, dt, req); }
Tensor Tensor::zeros(const std::vector<size_t>& s, DType dt, bool req) { return Tensor(s, dt, req); }
Tensor Tensor::full(const std::vector<size_t>& s, double v, DType dt, bool req) { return filled(s, v, dt, req); }
Tensor Tensor::empty(const std::vector<size_t>& s, DType dt, bool req) { return Tensor(s, dt, req); }

Tensor Tensor::rand(const std::vector<size_t>& s, DType dt, bool req) {
    Tensor t(s, dt, req);
    void* p = t.impl->storage->data.get();
    for (size_t i = 0, n = t.numel(); i < n; ++i) write_scalar_at(p, i, dt, (double)std::rand() / RAND_MAX);
    return t;
}

Tensor Tensor::from_vector(const std::vector<double>& data, const std::vector<size_t>& shape, DType dt, bool req) {
    Tensor t(shape, dt, req);
    if (t.numel() != data.size()) throw std::invalid_argument("from_vector: data size does not match shape");
    void* p = t.impl->storage->data.get();
    for (size_t i = 0; i < data.size(); ++i) write_scalar_at(p, i, dt, data[i]);
    return t;
}

Tensor Tensor::arange(double start, double end, double step, DType dt) {
    if (step == 0.0) throw std::invalid_argument("arange: step must be non-zero");
    const double span = (end - start) / step;
    const size_t n = span > 0 ? (size_t)std::ceil(span) : 0;
    Tensor t({n}, dt, false);
    void* p = t.impl->storage->data.get();
    for (size_t i = 0; i < n; ++i) write_scalar_at(p, i, dt, start + (double)i * step);
    return t;
}

Tensor Tensor::detach() const {
    Tensor out;
    if (impl) {
        out.impl = std::make_shared<Tensorimpl>(*impl);
        out.impl->requires_grad = false;
        out.impl->grad_fn = nullptr;
    }
    return out;
}
Tensor Tensor::detach() { return static_cast<const Tensor*>(this)->detach(); }

Tensor::Proxy Tensor::operator[](size_t i) {
    if (!impl) throw std::runtime_error("Invalid tensor");
    if (impl->ndim == 0) throw std::out_of_range("Cannot index scalar");
    if (i >= impl->shape[0]) throw std::out_of_range("Index out of bounds");
    return Proxy(impl, impl->offset + i * impl->strides[0], 1);
}
Tensor::ConstProxy Tensor::operator[](size_t i) const {
    if (!impl) throw std::runtime_error("Invalid tensor");
    if (impl->ndim == 0) throw std::out_of_range("Cannot index scalar");
    if (i >= impl->shape[0]) throw std::out_of_range("Index out of bounds");
    return ConstProxy(impl, impl->offset + i * impl->strides[0], 1);
}

// Element by element through double, walking storage linearly (tensor1.cpp:275-292): a host-side
// conversion utility, not an operator of the path.
Tensor Tensor::astype(DType new_dtype) const {
    if (!impl) throw std::runtime_error("Empty tensor");
    if (new_dtype == impl->dtype) return *this;
    Tensor out(shape(), new_dtype, impl->requires_grad);
    const size_t n = numel_();
    for (size_t i = 0; i < n; ++i)
        write_scalar_at(out.impl->storage->data.get(), i, new_dtype, read_scalar_at(impl->storage->data.get(), i, impl->dtype));
    if (impl->requires_grad && impl->storage->grad)
        for (size_t i = 0; i < n; ++i)
            write_scalar_at(out.impl->storage->grad.get(), i, new_dtype, read_scalar_at(impl->storage->grad.get(), i, impl->dtype));
    return out;
}

void Tensor::to_(DType new_dtype) {
    if (!impl) throw std::runtime_error("Empty tensor");
    if (new_dtype == impl->dtype) return;
    const size_t n = numel_();
    auto fresh = Storage::allocate(n, new_dtype, impl->requires_grad);
    for (size_t i = 0; i < n; ++i)
        write_scalar_at(fresh->data.get(), i, new_dtype, read_scalar_at(impl->storage->data.get(), i, impl->dtype));
    if (impl->requires_grad && impl->storage->grad)
        for (size_t i = 0; i < n; ++i)
            write_scalar_at(fresh->grad.get(), i, new_dtype, read_scalar_at(impl->storage->grad.get(), i, impl->dtype));
    impl->storage = fresh;
    impl->dtype = new_dtype;
}

Tensor& Tensor::t_() {
    if (!impl) throw std::runtime_error("Empty tensor");
    if (impl->ndim < 2) throw std::invalid_argument("t_: tensor must have at least 2 dimensions");
    std::swap(impl->shape[impl->ndim - 2], impl->shape[impl->ndim - 1]);
    std::swap(impl->strides[impl->ndim - 2], impl->strides[impl->ndim - 1]);
    return *this;
}

// O(1) view.  The view gets a Storage of its own that shares the data and starts without a
// gradient buffer, so that gradients accumulated into the view do not land in the source's
// (tensor1.cpp:341-358).
Tensor Tensor::permute(const std::vector<size_t>& dims) const {
    if (!impl) throw std::runtime_error("permute: tensor has no implementation");
    if (dims.size() != impl->ndim) throw std::invalid_argument("permute: dims size must match ndim.");
    std::vector<bool> seen(impl->ndim, false);
    std::vector<size_t> nsh(impl->ndim), nst(impl->ndim);
    for (size_t i = 0; i < dims.size(); ++i) {
        const size_t d = dims[i];
        if (d >= impl->ndim || seen[d]) throw std::invalid_argument("permute: invalid or duplicate dim.");
        seen[d] = true;
        nsh[i] = impl->shape[d];
        nst[i] = impl->strides[d];
    }
    auto shadow = std::make_shared<Storage>();
    shadow->data = impl->storage->data;
    shadow->size = impl->storage->size;
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(shadow, impl->offset, nsh, nst, impl->dtype, impl->requires_grad);
    attach(out, "permute", {*this}, 0.0, dims);
    return out;
}

Tensor Tensor::reshape(const std::vector<size_t>& new_shape) const {
    if (!impl) throw std::runtime_error("Empty tensor");
    size_t n = 1;
    for (size_t v : new_shape) n *= v;
    if (n != numel()) throw std::invalid_argument("reshape: number of elements mismatch");
    if (!is_contiguous()) return contiguous().reshape(new_shape);      // repack first, as the reference does
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(impl->storage, impl->offset, new_shape, row_major_strides(new_shape),
                                           impl->dtype, impl->requires_grad);
    attach(out, "reshape", {*this}, 0.0, shape());
    return out;
}

Tensor Tensor::select(size_t dim, size_t index) const {
    if (!impl) throw std::runtime_error("Empty tensor");
    if (dim >= impl->ndim) throw std::out_of_range("select: dim out of range");
    if (index >= impl->shape[dim]) throw std::out_of_range("select: index out of range");
    std::vector<size_t> nsh, nst;
    for (size_t i = 0; i < impl->ndim; ++i)
        if (i != dim) { nsh.push_back(impl->shape[i]); nst.push_back(impl->strides[i]); }
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(impl->storage, impl->offset + index * impl->strides[dim], nsh, nst,
                                           impl->dtype, impl->requires_grad);
    return out;
}

Tensor Tensor::squeeze() const {
    if (!impl) throw std::runtime_error("Empty tensor");
    std::vector<size_t> nsh, nst;
    for (size_t i = 0; i < impl->ndim; ++i)
        if (impl->shape[i] != 1) { nsh.push_back(impl->shape[i]); nst.push_back(impl->strides[i]); }
    if (nsh.empty()) { nsh.push_back(1); nst.push_back(1); }
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(impl->storage, impl->offset, nsh, nst, impl->dtype, impl->requires_grad);
    return out;
}

// The new shape gets row-major strides over the same storage (tensor1.cpp:442-453: meaningful for
// contiguous tensors, which is what the callers pass).
Tensor Tensor::unsqueeze(size_t dim) const {
    if (!impl) throw std::runtime_error("Empty tensor");
    if (dim > impl->ndim) throw std::out_of_range("unsqueeze: dim out of range");
    std::vector<size_t> nsh = shape();
    nsh.insert(nsh.begin() + (long)dim, 1);
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(impl->storage, impl->offset, nsh, row_major_strides(nsh), impl->dtype,
                                           impl->requires_grad);
    return out;
}

Tensor Tensor::flatten() const {
    if (!impl) throw std::runtime_error("Empty tensor");
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(impl->storage, impl->offset, std::vector<size_t>{numel()},
                                           std::vector<size_t>{1}, impl->dtype, impl->requires_grad);
    return out;
}

void Tensor::print_shape() const {
    std::cout << "(";
    for (size_t i = 0; impl && i < impl->ndim; ++i) std::cout << impl->shape[i] << (i + 1 < impl->ndim ? ", " : "");
    std::cout << ")\n";
}

// out[i] = input[i with coordinate `dim` replaced by index[i]] (tensor1.cpp:478-565).  The index
// tensor may hold any dtype (its values pass through double and are truncated, :548-549), e.g. the
// Float32 one-hot targets the reference's verify.cpp hands to Loss::CrossEntropy.  No backward
// node, as in the reference.
Tensor Tensor::gather(const Tensor& index, size_t dim) const {
    if (!impl || !index.impl) throw std::runtime_error("gather: input or index tensor is empty");
    if (impl->ndim != index.impl->ndim) throw std::runtime_error("gather: input and index must have same number of dimensions");
    for (size_t i = 0; i < impl->ndim; ++i)
        if (i != dim && impl->shape[i] != index.impl->shape[i]) throw std::runtime_error("gather: shape mismatch");
    ensure_device();
    Tensor out = new_output(index.shape(), _dtype(), impl->requires_grad);
    if (out.numel() == 0) return out;
    static std::mutex flag_mu;
    static int32_t* flag = nullptr;
    {
        std::lock_guard<std::mutex> lk(flag_mu);
        if (!flag) check(ctb_alloc_managed((void**)&flag, sizeof(int32_t), 1));
    }
    const ctb_view vx = view_of(*this), vi = view_of(index), vo = view_of(out);
    check(ctb_gather(&vx, (int)dim, &vi, &vo, flag, nullptr));
    after_op();
    if (*(volatile int32_t*)flag) throw std::out_of_range("gather: index out of bounds");
    return out;
}

Tensor& Tensor::requires_grad_(bool b) {
    if (!impl) throw std::runtime_error("requires_grad_: undefined tensor");
    impl->requires_grad = b;
    return *this;
}

void Tensor::backward() {
    if (!g_backward) throw std::runtime_error("backward: no autograd library registered (ctb_gen1::set_backward_entry)");
    g_backward(*this);
}

Tensor pad_to_ndim(const Tensor& t, size_t target_ndim) {
    if (!t.impl) throw std::runtime_error("pad_to_ndim: tensor undefined");
    const size_t nd = t.impl->ndim;
    if (nd == target_ndim) return t;
    if (nd > target_ndim) throw std::invalid_argument("pad_to_ndim: target_ndim smaller than tensor ndim");
    std::vector<size_t> nsh(target_ndim, 1);
    for (size_t i = 0; i < nd; ++i) nsh[target_ndim - nd + i] = t.impl->shape[i];
    Tensor packed = t.clone();                  // fresh packed storage, offset 0
    Tensor out;
    out.impl = std::make_shared<Tensorimpl>(packed.impl->storage, 0, nsh, row_major_strides(nsh), t.impl->dtype,
                                           t.impl->requires_grad);
    return out;
}

// ---- operators (root opsmp.cpp:178-483) --------------------------------------------------------------
Tensor add_mp(const Tensor& a, const Tensor& b) { return binary(CTB_ADD, "add", a, b, true); }
Tensor diff_mp(const Tensor& a, const Tensor& b) { return binary(CTB_SUB, "diff", a, b, true); }
Tensor mult_mp(const Tensor& a, const Tensor& b) { return binary(CTB_MUL, "mult", a, b, true); }
Tensor div_mp(const Tensor& a, const Tensor& b) { return binary(CTB_DIV, "div", a, b, true); }
Tensor pow_mp(const Tensor& a, const Tensor& b) { return binary(CTB_POW, "pow", a, b, true); }

Tensor add_scalar_mp(const Tensor& a, double s) { return unary(CTB_ADD_S, "add_scalar", a, s, true); }
Tensor sub_scalar_mp(const Tensor& a, double s) { return unary(CTB_SUB_S, "sub_scalar", a, s, true); }
Tensor sub_afterscalar_mp(double s, const Tensor& a) { return unary(CTB_RSUB_S, "sub_afterscalar", a, s, true); }
Tensor mult_scalar_mp(const Tensor& a, double s) { return unary(CTB_MUL_S, "mult_scalar", a, s, true); }
Tensor div_scalar_mp(const Tensor& a, double s) { return unary(CTB_DIV_S, "div_scalar", a, s, true); }
Tensor scalar_div_mp(double s, const Tensor& a) { return unary(CTB_RDIV_S, "scalar_div", a, s, true); }
Tensor pow_scalar_mp(const Tensor& a, double s) { return unary(CTB_POW_S, "pow_scalar", a, s, true); }
Tensor scalar_pow_mp(double s, const Tensor& a) { return unary(CTB_RPOW_S, "scalar_pow", a, s, true); }

Tensor abs_mp(const Tensor& a) { return unary(CTB_ABS, "abs", a, 0.0, true); }
Tensor ln_mp(const Tensor& a) { return unary(CTB_LOG, "ln", a, 0.0, true); }
Tensor exp_mp(const Tensor& a) { return unary(CTB_EXP, "exp", a, 0.0, true); }
Tensor sqrt_mp(const Tensor& a) { return unary(CTB_SQRT, "sqrt", a, 0.0, true); }
Tensor sin_mp(const Tensor& a) { return unary(CTB_SIN, "sin", a, 0.0, true); }
Tensor asin_mp(const Tensor& a) { return unary(CTB_ASIN, "asin", a, 0.0, true); }
Tensor cos_mp(const Tensor& a) { return unary(CTB_COS, "cos", a, 0.0, true); }
Tensor acos_mp(const Tensor& a) { return unary(CTB_ACOS, "acos", a, 0.0, true); }
Tensor tan_mp(const Tensor& a) { return unary(CTB_TAN, "tan", a, 0.0, true); }
Tensor atan_mp(const Tensor& a) { return unary(CTB_ATAN, "atan", a, 0.0, true); }
Tensor tanh_mp(const Tensor& a) { return unary(CTB_TANH, "tanh", a, 0.0, true); }
Tensor sinh_mp(const Tensor& a) { return unary(CTB_SINH, "sinh", a, 0.0, true); }
Tensor cosh_mp(const Tensor& a) { return unary(CTB_COSH, "cosh", a, 0.0, true); }
Tensor sigmoid_mp(const Tensor& a) { return unary(CTB_SIGMOID, "sigmoid", a, 0.0, true); }
Tensor Relu_mp(const Tensor& a) { return unary(CTB_RELU, "Relu", a, 0.0, true); }
Tensor softplus_mp(const Tensor& a) { return unary(CTB_SOFTPLUS, "softplus", a, 0.0, true); }

Tensor sum_mp(const Tensor& t, int dim) { return reduce(CTB_SUM, "sum", t, dim, true); }
Tensor max_mp(const Tensor& t, int dim) { return reduce(CTB_MAX, "max", t, dim, false); }
Tensor min_mp(const Tensor& t, int dim) { return reduce(CTB_MIN, "min", t, dim, false); }

// sum_mp followed by mult_scalar_mp(1 / extent), two operators and two nodes (root opsmp.cpp:464-468)
Tensor mean_mp(const Tensor& t, int dim) {
    Tensor s = sum_mp(t, dim);
    const int nd = (int)t.impl->ndim;
    const double count = (double)t.impl->shape[dim < 0 ? dim + nd : dim];
    return mult_scalar_mp(s, 1.0 / count);
}

Tensor lt_mp(const Tensor& a, double b) { return unary(CTB_LT_S, "lt", a, b, false); }
Tensor le_mp(const Tensor& a, double b) { return unary(CTB_LE_S, "le", a, b, false); }
Tensor gt_mp(const Tensor& a, double b) { return unary(CTB_GT_S, "gt", a, b, false); }
Tensor ge_mp(const Tensor& a, double b) { return unary(CTB_GE_S, "ge", a, b, false); }
Tensor eq_mp(const Tensor& a, double b) { return unary(CTB_EQ_S, "eq", a, b, false); }
Tensor neq_mp(const Tensor& a, double b) { return unary(CTB_NE_S, "ne", a, b, false); }
Tensor lt_mp(const Tensor& a, const Tensor& b) { return binary(CTB_LT, "lt", a, b, false); }
Tensor le_mp(const Tensor& a, const Tensor& b) { return binary(CTB_LE, "le", a, b, false); }
Tensor gt_mp(const Tensor& a, const Tensor& b) { return binary(CTB_GT, "gt", a, b, false); }
Tensor ge_mp(const Tensor& a, const Tensor& b) { return binary(CTB_GE, "ge", a, b, false); }
Tensor eq_mp(const Tensor& a, const Tensor& b) { return binary(CTB_EQ, "eq", a, b, false); }
Tensor ne_mp(const Tensor& a, const Tensor& b) { return binary(CTB_NE, "ne", a, b, false); }

// Shape rules of matmul_mp (root opsmp.cpp:247-292): the result has A's shape with the last
// extent replaced; batch extents must match or be 1.  The C ABI takes one batch dim: leading
// dims are merged when the operand is contiguous across them, else the operand is packed.
Tensor matmul_mp(const Tensor& A, const Tensor& B) {
    if (!A.impl || !B.impl) throw std::runtime_error("matmul: null input");
    if (A.impl->ndim < 2 || B.impl->ndim < 2) throw std::runtime_error("matmul_mp requires at least 2D tensors");
    const size_t K = A.impl->shape[A.impl->ndim - 1];
    if (B.impl->shape[B.impl->ndim - 2] != K) throw std::runtime_error("matmul_mp shape mismatch");
    size_t batch_a = 1, batch_b = 1;
    for (size_t i = 0; i + 2 < A.impl->ndim; ++i) batch_a *= A.impl->shape[i];
    for (size_t i = 0; i + 2 < B.impl->ndim; ++i) batch_b *= B.impl->shape[i];
    if (batch_a != batch_b && batch_a != 1 && batch_b != 1) throw std::runtime_error("matmul_mp: batch dimensions not broadcastable");
    ensure_device();
    std::vector<size_t> res_shape = A.shape();
    res_shape.back() = B.impl->shape[B.impl->ndim - 1];
    const bool req = A.requires_grad() || B.requires_grad();
    Tensor C = new_output(res_shape, A._dtype(), req);
    // views with at most one batch dim
    auto as3d = [](const Tensor& t, size_t batch, Tensor& keep) {
        const size_t nd = t.impl->ndim;
        if (nd <= 3) return view_of(t);
        keep = t.is_contiguous() ? t : t.contiguous();
        ctb_view v = view_of(keep);
        const int64_t m = v.shape[nd - 2], n = v.shape[nd - 1];
        v.ndim = 3;
        v.shape[0] = (int64_t)batch; v.shape[1] = m; v.shape[2] = n;
        v.stride[0] = m * n; v.stride[1] = n; v.stride[2] = 1;
        return v;
    };
    Tensor keep_a, keep_b, keep_c;
    const ctb_view va = as3d(A, batch_a, keep_a), vb = as3d(B, batch_b, keep_b), vc = as3d(C, std::max(batch_a, batch_b), keep_c);
    check(ctb_matmul(&va, &vb, &vc, nullptr));
    after_op();
    attach(C, "matmul", {A, B});
    return C;
}

// Concatenation along `dim` (root opsmp.cpp:487-553); no backward node, as in the reference.
Tensor cat_mp(const std::vector<Tensor>& tensors, size_t dim) {
    if (tensors.empty()) throw std::runtime_error("cat_mp: empty list");
    for (const Tensor& t : tensors)
        if (!t.impl) throw std::runtime_error("cat_mp: null tensor");
    std::vector<size_t> out_shape = tensors[0].shape();
    if (dim >= out_shape.size()) throw std::out_of_range("cat_mp: dim out of range");
    size_t dim_sum = 0;
    for (const Tensor& t : tensors) {
        if (t.impl->ndim != out_shape.size()) throw std::runtime_error("cat_mp: dim mismatch");
        dim_sum += t.impl->shape[dim];
    }
    out_shape[dim] = dim_sum;
    ensure_device();
    Tensor out = new_output(out_shape, tensors[0]._dtype(), false);
    std::vector<ctb_view> views;
    views.reserve(tensors.size());
    for (const Tensor& t : tensors) views.push_back(view_of(t));
    std::vector<const ctb_view*> ptrs;
    for (const ctb_view& v : views) ptrs.push_back(&v);
    const ctb_view vo = view_of(out);
    check(ctb_cat(ptrs.data(), (int)ptrs.size(), (int)dim, &vo, nullptr));
    after_op();
    return out;
}
