// First-generation tensor types of the reference (root tensor1.h:12-189), laid out exactly as
// its callers dereference them — autograd.cpp:21-34,54-55,85-86,157-158, loss.cpp:23-26,50-56 and
// layer.cpp reach straight into impl->storage->data / impl->storage->grad and the raw
// impl->shape / impl->strides arrays — over the B200 operator library.
//
//   Storage    { data, grad, size }                       tensor1.h:45-52
//   Tensorimpl { storage, offset, ndim, size_t* shape, size_t* strides, requires_grad, dtype,
//                grad_fn }                                tensor1.h:55-74
//   Tensor     { impl, grad_fn } + members                tensor1.h:77-189, tensor1.cpp:87-581
//
// What differs from the reference's file, on purpose:
//  * `data` and `grad` are CUDA managed memory from the library's pool (the host may
//    dereference them, kernels read them from HBM); every operator waits for its kernel.
//  * Tensorimpl copies deeply (the reference copies the raw shape/strides pointers in
//    Tensor::detach, tensor1.cpp:262-270,569-576, and frees them twice).
//  * Integer stores from the host helpers round like the reference (std::lrint, tensor1.h:36);
//    results of GPU operators on Int32 tensors truncate as the second generation does.
// Members are implemented in libctensor_gen1.so (ctensor_b200/host/gen1/ctensor_gen1.cpp).
#pragma once
#include <cmath>
#include <cstddef>
#include <iostream>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

enum class DType { Float32, Int32, Double64 };

inline size_t dtype_size(DType dt) {
    return dt == DType::Double64 ? sizeof(double) : dt == DType::Int32 ? sizeof(int) : sizeof(float);
}

inline double read_scalar_at(const void* data, size_t idx, DType dt) {
    if (dt == DType::Float32) return static_cast<const float*>(data)[idx];
    if (dt == DType::Int32) return static_cast<const int*>(data)[idx];
    return static_cast<const double*>(data)[idx];
}

inline void write_scalar_at(void* data, size_t idx, DType dt, double val) {
    if (dt == DType::Float32) static_cast<float*>(data)[idx] = static_cast<float>(val);
    else if (dt == DType::Int32) static_cast<int*>(data)[idx] = static_cast<int>(std::lrint(val));
    else static_cast<double*>(data)[idx] = val;
}

struct GradFn;   // the autograd node type of the caller's autograd.h

struct Storage {
    std::shared_ptr<void> data;
    std::shared_ptr<void> grad;
    size_t size = 0;                      // elements
    static std::shared_ptr<Storage> allocate(size_t n, DType dt, bool requires_grad = false);
};

struct Tensorimpl {
    std::shared_ptr<Storage> storage;
    size_t offset = 0;
    size_t ndim = 0;
    size_t* shape = nullptr;
    size_t* strides = nullptr;
    bool requires_grad = false;
    DType dtype = DType::Float32;
    std::shared_ptr<GradFn> grad_fn;

    Tensorimpl(const std::vector<size_t>& shape_, DType dtype_ = DType::Float32, bool requires_grad_ = false);
    Tensorimpl(std::shared_ptr<Storage> storage_, size_t offset_, const std::vector<size_t>& shape_,
               const std::vector<size_t>& strides_, DType dtype_, bool requires_grad_);
    Tensorimpl(const Tensorimpl& other);
    Tensorimpl& operator=(const Tensorimpl&) = delete;
    ~Tensorimpl();
};

struct Tensor {
    std::shared_ptr<Tensorimpl> impl;

    Tensor() = default;
    Tensor(const std::vector<size_t>& shape_, DType dtype_ = DType::Float32, bool requires_grad_ = false);
    Tensor(const size_t* shape_ptr, size_t ndim, DType dtype, bool requires_grad)
        : Tensor(std::vector<size_t>(shape_ptr, shape_ptr + ndim), dtype, requires_grad) {}

    size_t numel() const;
    size_t numel_() const { return numel(); }
    std::vector<size_t> shape() const;
    DType _dtype() const { need(); return impl->dtype; }
    size_t dtype_bytes() const { need(); return dtype_size(impl->dtype); }
    bool requires_grad() const { need(); return impl->requires_grad; }

    // raw storage index: offset and strides are not applied (as in the reference)
    double read_scalar(size_t idx) const { need(); return read_scalar_at(impl->storage->data.get(), idx, impl->dtype); }
    void write_scalar(size_t idx, double val) { need(); write_scalar_at(impl->storage->data.get(), idx, impl->dtype, val); }

    bool is_contiguous() const;
    Tensor contiguous() const;

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
    Tensor detach();

    template <bool Writable> struct ProxyBase {
        std::shared_ptr<Tensorimpl> impl;
        size_t offset, depth;
        ProxyBase(std::shared_ptr<Tensorimpl> impl_, size_t off, size_t dp = 0) : impl(std::move(impl_)), offset(off), depth(dp) {}
        ProxyBase operator[](size_t i) const {
            if (!impl) throw std::runtime_error("Invalid tensor");
            if (depth >= impl->ndim) throw std::out_of_range("Too many indices");
            if (i >= impl->shape[depth]) throw std::out_of_range("Index out of bounds");
            return ProxyBase(impl, offset + i * impl->strides[depth], depth + 1);
        }
        operator double() const {
            if (!impl) throw std::runtime_error("Invalid tensor");
            if (depth != impl->ndim) throw std::out_of_range("Not at leaf index");
            return read_scalar_at(impl->storage->data.get(), offset, impl->dtype);
        }
        template <bool W = Writable, typename = std::enable_if_t<W>> ProxyBase& operator=(double val) {
            if (!impl) throw std::runtime_error("Invalid tensor");
            if (depth != impl->ndim) throw std::out_of_range("Not at leaf index");
            write_scalar_at(impl->storage->data.get(), offset, impl->dtype, val);
            return *this;
        }
        template <bool W = Writable, typename T, typename = std::enable_if_t<W>> ProxyBase& operator=(T val) {
            return operator=(static_cast<double>(val));
        }
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
    Tensor squeeze() const;
    Tensor unsqueeze(size_t dim) const;
    Tensor flatten() const;
    void print_shape() const;
    Tensor gather(const Tensor& index, size_t dim = 1) const;

    // image I/O belongs to the caller's data.cpp (the reference's tensorio); declared so that
    // code which uses it still compiles, defined only if that file is linked
    static Tensor from_image(const std::string& path, DType dt = DType::Float32);
    void save_image(const std::string& path) const;

    std::shared_ptr<GradFn> grad_fn;
    Tensor& requires_grad_(bool b);
    void backward();

private:
    void need() const { if (!impl) throw std::runtime_error("Tensor is empty"); }
};

// ---- small host helpers of the reference's header that callers and tests use ------------------------
// Storage index of `padded_idx` (an index of the left-padded, broadcast shape) inside `orig`.
inline size_t linear_index_from_padded(const Tensor& orig, const std::vector<size_t>& padded_idx) {
    if (!orig.impl) throw std::runtime_error("linear_index_from_padded: orig undefined");
    if (padded_idx.size() < orig.impl->ndim) throw std::invalid_argument("linear_index_from_padded: padded_idx smaller than orig.ndim");
    const size_t pad = padded_idx.size() - orig.impl->ndim;
    size_t off = orig.impl->offset;
    for (size_t i = 0; i < orig.impl->ndim; ++i)
        if (orig.impl->shape[i] != 1) off += padded_idx[pad + i] * orig.impl->strides[i];
    return off;
}

// `t` with size-1 dims added on the left up to `target_ndim` (a packed copy, like the reference's).
Tensor pad_to_ndim(const Tensor& t, size_t target_ndim);

inline void print_t(const Tensor& t) {
    const size_t n = t.numel_();
    std::cout << "[";
    for (size_t i = 0; i < n; ++i) std::cout << read_scalar_at(t.impl->storage->data.get(), i, t.impl->dtype) << (i + 1 != n ? ", " : "");
    std::cout << "]\n";
}

inline void print_(const Tensor& t, const std::string& name = "Tensor") {
    std::cout << name << " shape: [";
    for (size_t i = 0; i < t.impl->ndim; ++i) std::cout << t.impl->shape[i] << (i + 1 < t.impl->ndim ? ", " : "");
    std::cout << "]\n" << name << " values: ";
    for (size_t i = 0, n = t.numel(); i < n; ++i) std::cout << t.read_scalar(i) << " ";
    std::cout << "\n\n";
}
