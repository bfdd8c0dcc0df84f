// Thin host-side tensor for the attention hot path: the subset of
// vesper::Tensor (include/vesper/core/tensor.h:26-223 of the reference) that
// the attention operators, the KV cache and their tests use -- a shape /
// element-stride / element-offset view over shared storage, with the same
// accessor names.  Device, DType, Slice and Stream mirror
// include/vesper/core/{device,dtype,slice,stream}.h.
//
// What the reference cannot express and this layer adds: bf16/fp16 storage on
// CUDA and a device ordinal (Device::CUDA tensors live on the CUDA device that
// is current when they are created).
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <stdexcept>
#include <variant>
#include <vector>

namespace vesper {

enum class Device { CPU, CUDA, HIP };

enum class DType { Float32, Float64, Float16, BFloat16, Int32, Int64 };

inline size_t GetDTypeSize(DType dtype) {
    switch (dtype) {
        case DType::Float32: return 4;
        case DType::Float64: return 8;
        case DType::Float16: return 2;
        case DType::BFloat16: return 2;
        case DType::Int32: return 4;
        case DType::Int64: return 8;
    }
    throw std::runtime_error("Unknown DType");
}

// Python-style slice start:stop:step (include/vesper/core/slice.h:11-22)
struct Slice {
    std::optional<int64_t> start, stop, step;
    Slice() {}
    Slice(int64_t stop_) : start(0), stop(stop_), step(1) {}
    Slice(int64_t start_, int64_t stop_, int64_t step_ = 1) : start(start_), stop(stop_), step(step_) {}
};
using IndexSelector = std::variant<int64_t, Slice>;

// Current stream of the calling thread (include/vesper/core/stream.h:10-51).
// The default is the legacy stream 0, as in the reference.
class Stream {
public:
    explicit Stream(Device device);                 // creates a new CUDA stream
    ~Stream();
    Stream(const Stream&) = delete;
    Stream& operator=(const Stream&) = delete;
    void synchronize() const;
    void* raw_handle() const { return handle_; }
    Device device() const { return device_; }
    static Stream& default_stream(Device device);
    static void set_current(const Stream& stream);
    static Stream& current(Device device);

private:
    Stream(Device device, void* handle, bool own) : device_(device), handle_(handle), own_(own) {}
    Device device_;
    void* handle_ = nullptr;
    bool own_ = true;
};

// Reference-counted buffer; CUDA buffers come from a small caching allocator
// (power-of-two bins, as src/core/allocator.cpp:171-221 does).
class Storage {
public:
    Storage(size_t bytes, Device device);
    ~Storage();
    Storage(const Storage&) = delete;
    void* data() const { return data_; }
    size_t size_bytes() const { return bytes_; }
    Device device() const { return device_; }
    int device_index() const { return ordinal_; }

private:
    void* data_ = nullptr;
    size_t bytes_ = 0, alloc_bytes_ = 0;
    Device device_;
    int ordinal_ = 0;
};

class Tensor {
public:
    Tensor() = default;
    Tensor(std::shared_ptr<Storage> storage, std::vector<int64_t> shape, std::vector<int64_t> strides,
           size_t offset, DType dtype)
        : storage_(std::move(storage)), shape_(std::move(shape)), strides_(std::move(strides)),
          offset_(offset), dtype_(dtype) {}

    const std::vector<int64_t>& shape() const { return shape_; }
    const std::vector<int64_t>& strides() const { return strides_; }
    int64_t ndim() const { return static_cast<int64_t>(shape_.size()); }
    DType dtype() const { return dtype_; }
    Device device() const { return storage_->device(); }
    int device_index() const { return storage_->device_index(); }
    size_t offset() const { return offset_; }
    size_t numel() const;
    bool is_contiguous() const;
    bool defined() const { return storage_ != nullptr; }
    bool requires_grad() const { return false; }     // inference path: no autograd in this layer

    template <typename T> T* data_ptr() {
        return reinterpret_cast<T*>(static_cast<char*>(storage_->data()) + offset_ * GetDTypeSize(dtype_));
    }
    template <typename T> const T* data_ptr() const {
        return reinterpret_cast<const T*>(static_cast<const char*>(storage_->data()) + offset_ * GetDTypeSize(dtype_));
    }

    // host <-> tensor (the tensor must be contiguous); synchronous
    void copy_from_host(const void* host_ptr);
    void copy_to_host(void* host_ptr) const;
    // same-shape copy; on CUDA the destination may be a strided [B,H,S,D] view
    void copy_from(const Tensor& other);

    Tensor transpose(int64_t dim0, int64_t dim1) const;
    Tensor view(const std::vector<int64_t>& new_shape) const;       // contiguous tensors only
    Tensor reshape(const std::vector<int64_t>& new_shape) const;    // copies when not contiguous
    Tensor contiguous() const;
    Tensor index(const std::vector<IndexSelector>& selectors) const;
    Tensor narrow(int64_t dim, int64_t start, int64_t length) const;
    // Splits the last dimension (which must have stride 1) into [outer, inner] without a copy, whatever the other
    // strides are: how q / k / v heads are seen inside a slice of the fused projection's output.
    Tensor unflatten_last(int64_t outer, int64_t inner) const;
    Tensor to(Device device) const;
    Tensor clone() const { return contiguous_copy(); }
    void zero_();

private:
    Tensor contiguous_copy() const;
    std::shared_ptr<Storage> storage_;
    std::vector<int64_t> shape_, strides_;
    size_t offset_ = 0;
    DType dtype_ = DType::Float32;
};

// include/vesper/core/factories.h:8-14
Tensor empty(const std::vector<int64_t>& shape, DType dtype, Device device, bool requires_grad = false);
Tensor zeros(const std::vector<int64_t>& shape, DType dtype, Device device, bool requires_grad = false);

// Host-side 16-bit conversions.  BFloat16 rounds to nearest even like
// include/vesper/core/half.h:162-173; Float16 rounds to nearest even too (the
// reference truncates, half.h:56, which does not match what the GPU does).
uint16_t float_to_bf16(float f);
float bf16_to_float(uint16_t h);
uint16_t float_to_fp16(float f);
float fp16_to_float(uint16_t h);

}  // namespace vesper
