// Host-side Tensor types of the B200 operator library.
//
// Source-compatible with what callers of the reference use from src/core/tensor.h:23-607
// (and, for the field names, tensor1.h:45-189): DType, dtype_size, read/write_scalar_at,
// Storage{data,size,device}, Tensorimpl{data,grad,offset,ndim,shape,strides,requires_grad,
// dtype,grad_fn}, and the Tensor handle with its factories, view operations and index proxies.
// Callers poke `impl->data->data.get()` directly (e.g. src/neuralnet/loss.cpp:25,
// src/core/autograd.cpp:97-98), so storage is CUDA *managed* memory: kernels read it from HBM,
// the host can dereference it, and every operator synchronises before it returns.
//
// Differences on purpose: shapes/strides live in a fixed-capacity array (8 dims, the C ABI's
// limit) instead of a small-vector with heap fallback; reference counting uses
// std::shared_ptr; the unfinished CUDA pool of the reference is replaced by ctb_host.h.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <iostream>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "device.h"

enum class DType { Float32, Int32, Double64, UInt8, UInt16, UInt32, UInt64, Int8, Int16, Int64, Bool, Float16 };

inline size_t dtype_size(DType dt) {
    switch (dt) {
    case DType::Double64: case DType::UInt64: case DType::Int64: return 8;
    case DType::Float32: case DType::Int32: case DType::UInt32: return 4;
    case DType::UInt16: case DType::Int16: case DType::Float16: return 2;
    default: return 1;
    }
}

// Element access through double, the reference's conversion rule (tensor.h:54-86): stores
// are static_cast from double, i.e. truncation for the integer types.
inline double read_scalar_at(const void* p, size_t i, DType dt) {
    switch (dt) {
    case DType::Float32:  return static_cast<const float*>(p)[i];
    case DType::Int32:    return static_cast<const int32_t*>(p)[i];
    case DType::Double64: return static_cast<const double*>(p)[i];
    case DType::UInt8:    return static_cast<const uint8_t*>(p)[i];
    case DType::UInt16:   return static_cast<const uint16_t*>(p)[i];
    case DType::UInt32:   return static_cast<const uint32_t*>(p)[i];
    case DType::UInt64:   return static_cast<double>(static_cast<const uint64_t*>(p)[i]);
    case DType::Int8:     return static_cast<const int8_t*>(p)[i];
    case DType::Int16:    return static_cast<const int16_t*>(p)[i];
    case DType::Int64:    return static_cast<double>(static_cast<const int64_t*>(p)[i]);
    case DType::Bool:     return static_cast<const bool*>(p)[i] ? 1.0 : 0.0;
    default:              return 0.0;
    }
}
inline void write_scalar_at(void* p, size_t i, DType dt, double v) {
    switch (dt) {
    case DType::Float32:  static_cast<float*>(p)[i] = static_cast<float>(v); break;
    case DType::Int32:    static_cast<int32_t*>(p)[i] = static_cast<int32_t>(v); break;
    case DType::Double64: static_cast<double*>(p)[i] = v; break;
    case DType::UInt8:    static_cast<uint8_t*>(p)[i] = static_cast<uint8_t>(v); break;
    case DType::Int8:     static_cast<int8_t*>(p)[i] = static_cast<int8_t>(v); break;
    case DType::Int16:    static_cast<int16_t*>(p)[i] = static_cast<int16_t>(v); break;
    case DType::Int64:    static_cast<int64_t*>(p)[i] = static_cast<int64_t>(v); break;
    case DType::Bool:     static_cast<bool*>(p)[i] = (v != 0.0); break;
    default: break;
    }
}

struct GradFn;   // autograd node, defined by the caller's autograd library

// Fixed-capacity dimension list with the vector-like surface callers use
// (operator[], size(), begin/end, push_back, data(), to_vector()).
class DimVec {
public:
    static constexpr size_t kMax = 8;
    DimVec() = default;
    DimVec(const std::vector<size_t>& v) { assign(v.begin(), v.end()); }
    DimVec(std::initializer_list<size_t> v) { assign(v.begin(), v.end()); }
    size_t& operator[](size_t i) { return v_[i]; }
    const size_t& operator[](size_t i) const { return v_[i]; }
    size_t size() const { return n_; }
    bool empty() const { return n_ == 0; }
    size_t* data() { return v_; }
    const size_t* data() const { return v_; }
    size_t* begin() { return v_; }
    size_t* end() { return v_ + n_; }
    const size_t* begin() const { return v_; }
    const size_t* end() const { return v_ + n_; }
    void push_back(size_t x) {
        if (n_ == kMax) throw std::length_error("tensor: more than 8 dimensions");
        v_[n_++] = x;
    }
    std::vector<size_t> to_vector() const { return std::vector<size_t>(v_, v_ + n_); }

private:
    template <typename It> void assign(It b, It e) {
        n_ = 0;
        for (; b != e; ++b) push_back(*b);
    }
    size_t n_ = 0;
    size_t v_[kMax] = {};
};
template <typename T, size_t N> using SmallVector = DimVec;   // spelled SmallVector<size_t,5> by callers

inline DimVec calc_strides(const DimVec& shape) {
    DimVec st(shape);
    size_t run = 1;
    for (size_t i = shape.size(); i-- > 0;) {
        st[i] = run;
        run *= shape[i];
    }
    return st;
}

// Raw buffer on a device.  `data` frees itself through its deleter.
struct Storage {
    std::shared_ptr<void> data;
    size_t size = 0;            // elements
    Device device;
    static std::shared_ptr<Storage> allocate(size_t n, DType dt, bool requires_grad = false,
                                             Device dev = Device(DeviceType::CPU));
};

struct Tensorimpl;
// Handle type used for impl and grad.  get()/operator->/bool as the reference's intrusive_ptr.
template <typename T> using intrusive_ptr = std::shared_ptr<T>;

struct Tensorimpl {
    std::shared_ptr<Storage> data;
    intrusive_ptr<Tensorimpl> grad;
    size_t offset = 0;
    size_t ndim = 0;
    DimVec shape;
    DimVec strides;
    bool requires_grad = false;
    DType dtype = DType::Float32;
    std::shared_ptr<GradFn> grad_fn;

    Tensorimpl(const std::vector<size_t>& shape_, DType dtype_, bool requires_grad_, Device dev_)
        : ndim(shape_.size()), shape(shape_), strides(calc_strides(DimVec(shape_))),
          requires_grad(requires_grad_), dtype(dtype_) {
        size_t n = 1;
        for (size_t s : shape_) n *= s;
        data = Storage::allocate(n, dtype_, requires_grad_, dev_);
    }
    Tensorimpl(std::shared_ptr<Storage> storage_, size_t offset_, const DimVec& shape_, const DimVec& strides_,
               DType dtype_, bool requires_grad_)
        : data(std::move(storage_)), offset(offset_), ndim(shape_.size()), shape(shape_), strides(strides_),
          requires_grad(requires_grad_), dtype(dtype_) {}
    virtual ~Tensorimpl() = default;
};

struct Tensor {
    intrusive_ptr<Tensorimpl> impl;
    std::shared_ptr<GradFn> grad_fn;

    Tensor() = default;
    Tensor(const std::vector<size_t>& shape_, DType dtype_ = DType::Float32, bool requires_grad_ = false);
    Tensor(const size_t* shape_ptr, size_t ndim, DType dtype, bool requires_grad)
        : Tensor(std::vector<size_t>(shape_ptr, shape_ptr + ndim), dtype, requires_grad) {}

    Device device() const;
    Tensor to(Device target_device);

    size_t numel() const {
        if (!impl) return 0;
        size_t n = 1;
        for (size_t s : impl->shape) n *= s;
        return n;
    }
    size_t numel_() const { return numel(); }
    std::vector<size_t> shape() const { return impl ? impl->shape.to_vector() : std::vector<size_t>{}; }
    DType _dtype() const { need(); return impl->dtype; }
    size_t dtype_bytes() const { need(); return dtype_size(impl->dtype); }
    bool requires_grad() const { need(); return impl->requires_grad; }

    bool is_contiguous() const;
    Tensor contiguous() const;

    // idx is a raw storage index (offset and strides are NOT applied — as in the reference).
    double read_scalar(size_t idx) const { need(); return read_scalar_at(impl->data->data.get(), idx, impl->dtype); }
    void write_scalar(size_t idx, double v) { need(); write_scalar_at(impl->data->data.get(), idx, impl->dtype, v); }

    static Tensor ones(const std::vector<size_t>& shape_, DType dt = DType::Float32, bool requires_grad_ = false);
    static Tensor zeros(const std::vector<size_t>& shape_, DType dt = DType::Float32, bool requires_grad_ = false);
    static Tensor full(const std::vector<size_t>& shape_, double value, DType dt = DType::Float32, bool requires_grad_ = false);
    static Tensor rand(const std::vector<size_t>& shape_, DType dt = DType::Float32, bool requires_grad_ = false);
    static Tensor empty(const std::vector<size_t>& shape_, DType dt = DType::Float32, bool requires_grad_ = false);
    static Tensor from_vector(const std::vector<double>& data, const std::vector<size_t>& shape,
                              DType dtype = DType::Float32, bool requires_grad = false);
    static Tensor arange(double start, double end, double step, DType dtype);

    Tensor clone() const;
    Tensor detach() const;
    Tensor& requires_grad_(bool b) { if (impl) impl->requires_grad = b; return *this; }

    // t[i][j] = v / double(t[i][j]) element access; assigning at a shallower depth fills.
    template <bool Writable> struct ProxyBase {
        intrusive_ptr<Tensorimpl> impl;
        size_t offset, depth;
        ProxyBase(intrusive_ptr<Tensorimpl> p, size_t off, size_t dp) : impl(std::move(p)), offset(off), depth(dp) {}
        ProxyBase operator[](size_t i) const {
            if (!impl) throw std::runtime_error("Invalid tensor");
            if (depth >= impl->ndim) throw std::out_of_range("Too many indices");
            if (i >= impl->shape[depth]) throw std::out_of_range("Index out of bounds");
            return ProxyBase(impl, offset + i * impl->strides[depth], depth + 1);
        }
        operator double() const;
        template <bool W = Writable, typename = std::enable_if_t<W>> ProxyBase& operator=(double v);
        template <bool W = Writable, typename T, typename = std::enable_if_t<W && std::is_arithmetic<T>::value>>
        ProxyBase& operator=(T v) { return operator=(static_cast<double>(v)); }
    };
    using Proxy = ProxyBase<true>;
    using ConstProxy = ProxyBase<false>;
    Proxy operator[](size_t i);
    ConstProxy operator[](size_t i) const;

    Tensor astype(DType new_dtype) const;
    void to_(DType new_dtype);
    Tensor& t_();
    Tensor permute(const std::vector<size_t>& dims) const;
    Tensor reshape(const std::vector<size_t>& new_shape) const;
    Tensor select(size_t dim, size_t index) const;
    Tensor gather(const Tensor& index, size_t dim = 0) const;
    Tensor squeeze() const;
    Tensor unsqueeze(size_t dim) const;
    Tensor flatten() const;
    void print_shape() const;
    Tensor argmax(int dim = -1) const;

    template <typename T> T item() const {
        if (!impl) throw std::runtime_error("item() on empty tensor");
        if (numel() != 1) throw std::runtime_error("item() only for 1-element tensors");
        return static_cast<T>(read_scalar_at(impl->data->data.get(), impl->offset, impl->dtype));
    }

    void backward();
    Tensor grad() const {
        Tensor g;
        if (impl && impl->grad) g.impl = impl->grad;
        return g;
    }
    void zero_grad();

private:
    void need() const { if (!impl) throw std::runtime_error("Tensor is empty"); }
};

namespace ctb_host { void sync_for_host_access(); }

template <bool W> Tensor::ProxyBase<W>::operator double() const {
    if (!impl) throw std::runtime_error("Invalid tensor");
    if (depth != impl->ndim) throw std::out_of_range("Not at leaf index");
    ctb_host::sync_for_host_access();
    return read_scalar_at(impl->data->data.get(), offset, impl->dtype);
}

template <bool W> template <bool W2, typename> Tensor::ProxyBase<W>& Tensor::ProxyBase<W>::operator=(double v) {
    if (!impl) throw std::runtime_error("Invalid tensor");
    ctb_host::sync_for_host_access();
    // fill every element of the sub-tensor below this proxy (one element at leaf depth)
    const size_t nd = impl->ndim;
    size_t count = 1;
    for (size_t d = depth; d < nd; ++d) count *= impl->shape[d];
    void* base = impl->data->data.get();
    for (size_t k = 0; k < count; ++k) {
        size_t t = k, off = offset;
        for (size_t d = nd; d-- > depth;) {
            off += (t % impl->shape[d]) * impl->strides[d];
            t /= impl->shape[d];
        }
        write_scalar_at(base, off, impl->dtype, v);
    }
    return *this;
}

inline Tensor::Proxy Tensor::operator[](size_t i) {
    if (!impl) throw std::runtime_error("Invalid tensor");
    if (impl->ndim == 0) throw std::out_of_range("Cannot index scalar");
    if (i >= impl->shape[0]) throw std::out_of_range("Index out of bounds");
    return Proxy(impl, impl->offset + i * impl->strides[0], 1);
}
inline Tensor::ConstProxy Tensor::operator[](size_t i) const {
    if (!impl) throw std::runtime_error("Invalid tensor");
    if (impl->ndim == 0) throw std::out_of_range("Cannot index scalar");
    if (i >= impl->shape[0]) throw std::out_of_range("Index out of bounds");
    return ConstProxy(impl, impl->offset + i * impl->strides[0], 1);
}

inline void print_t(const Tensor& t) {
    ctb_host::sync_for_host_access();
    const size_t n = t.numel_();
    std::cout << "[";
    for (size_t i = 0; i < n; ++i) std::cout << read_scalar_at(t.impl->data->data.get(), i, t.impl->dtype) << (i + 1 < n ? ", " : "");
    std::cout << "]\n";
}

inline const char* dtype_to_str(DType dt) {
    switch (dt) {
    case DType::Float32: return "float32";
    case DType::Double64: return "double64";
    case DType::Int32: return "int32";
    case DType::Int64: return "int64";
    default: return "unknown";
    }
}
