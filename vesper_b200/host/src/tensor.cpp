// Host tensor, storage, stream and allocator for the attention path.
// CUDA runtime use is confined to this file (allocation, memcpy, memset,
// streams); all compute goes through the C ABI of libvesper_b200.
#include <vesper/core/tensor.h>

#include <cuda_runtime.h>
#include <vesper_b200.h>

#include <cstring>
#include <map>
#include <mutex>
#include <string>

namespace vesper {

namespace {

void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// Caching allocator: freed blocks are kept per (device, rounded size) and
// handed out again; nothing is returned to the driver before process exit
// (src/core/allocator.cpp:205-221 has the same policy).
class CachingAllocator {
public:
    static CachingAllocator& get() { static CachingAllocator* a = new CachingAllocator(); return *a; }
    static size_t round(size_t n) {
        size_t r = 512;
        while (r < n) r <<= 1;
        return r;
    }
    void* alloc(size_t rounded, int dev) {
        {
            std::lock_guard<std::mutex> lock(mu_);
            auto& bin = free_[{dev, rounded}];
            if (!bin.empty()) { void* p = bin.back(); bin.pop_back(); return p; }
        }
        void* p = nullptr;
        cuda_check(cudaMalloc(&p, rounded), "cudaMalloc");
        return p;
    }
    void release(void* p, size_t rounded, int dev) {
        std::lock_guard<std::mutex> lock(mu_);
        free_[{dev, rounded}].push_back(p);
    }

private:
    std::mutex mu_;
    std::map<std::pair<int, size_t>, std::vector<void*>> free_;
};

thread_local Stream* t_current = nullptr;

std::vector<int64_t> contiguous_strides(const std::vector<int64_t>& shape) {
    std::vector<int64_t> st(shape.size(), 1);
    for (int i = static_cast<int>(shape.size()) - 2; i >= 0; --i) st[i] = st[i + 1] * shape[i + 1];
    return st;
}

int dtype_code(DType d) {
    switch (d) {
        case DType::Float32: return VB200_F32;
        case DType::BFloat16: return VB200_BF16;
        case DType::Float16: return VB200_F16;
        default: throw std::runtime_error("dtype not supported by the CUDA attention backend");
    }
}

}  // namespace

// ---- Stream ----
Stream::Stream(Device device) : device_(device) {
    if (device == Device::CUDA) {
        cudaStream_t s;
        cuda_check(cudaStreamCreate(&s), "cudaStreamCreate");
        handle_ = s;
    }
}
Stream::~Stream() {
    if (own_ && handle_) cudaStreamDestroy(static_cast<cudaStream_t>(handle_));
    if (t_current == this) t_current = nullptr;
}
void Stream::synchronize() const {
    if (device_ == Device::CUDA) cuda_check(cudaStreamSynchronize(static_cast<cudaStream_t>(handle_)), "cudaStreamSynchronize");
}
Stream& Stream::default_stream(Device device) {
    static Stream cuda_default(Device::CUDA, nullptr, false);   // legacy stream 0 (src/core/stream.cpp:104-111)
    static Stream cpu_default(Device::CPU, nullptr, false);
    return device == Device::CUDA ? cuda_default : cpu_default;
}
void Stream::set_current(const Stream& stream) { t_current = const_cast<Stream*>(&stream); }
Stream& Stream::current(Device device) {
    if (device == Device::CUDA && t_current && t_current->device() == Device::CUDA) return *t_current;
    return default_stream(device);
}

// ---- Storage ----
Storage::Storage(size_t bytes, Device device) : bytes_(bytes), device_(device) {
    if (device == Device::HIP) throw std::runtime_error("HIP backend not enabled");
    if (device == Device::CUDA) {
        cuda_check(cudaGetDevice(&ordinal_), "cudaGetDevice");
        alloc_bytes_ = CachingAllocator::round(bytes ? bytes : 1);
        data_ = CachingAllocator::get().alloc(alloc_bytes_, ordinal_);
    } else {
        data_ = ::operator new(bytes ? bytes : 1);
    }
}
Storage::~Storage() {
    if (device_ == Device::CUDA) CachingAllocator::get().release(data_, alloc_bytes_, ordinal_);
    else ::operator delete(data_);
}

// ---- Tensor ----
size_t Tensor::numel() const {
    size_t n = 1;
    for (auto s : shape_) n *= static_cast<size_t>(s);
    return n;
}

bool Tensor::is_contiguous() const {
    int64_t expect = 1;
    for (int i = static_cast<int>(shape_.size()) - 1; i >= 0; --i) {
        if (shape_[i] != 1 && strides_[i] != expect) return false;
        expect *= shape_[i];
    }
    return true;
}

void Tensor::copy_from_host(const void* host_ptr) {
    if (!is_contiguous()) throw std::runtime_error("copy_from_host: tensor must be contiguous");
    size_t bytes = numel() * GetDTypeSize(dtype_);
    if (device() == Device::CUDA) cuda_check(cudaMemcpy(data_ptr<char>(), host_ptr, bytes, cudaMemcpyHostToDevice), "cudaMemcpy H2D");
    else std::memcpy(data_ptr<char>(), host_ptr, bytes);
}

void Tensor::copy_to_host(void* host_ptr) const {
    if (!is_contiguous()) { contiguous().copy_to_host(host_ptr); return; }
    size_t bytes = numel() * GetDTypeSize(dtype_);
    if (device() == Device::CUDA) {
        cuda_check(cudaStreamSynchronize(static_cast<cudaStream_t>(Stream::current(Device::CUDA).raw_handle())), "sync");
        cuda_check(cudaMemcpy(host_ptr, data_ptr<char>(), bytes, cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
    } else {
        std::memcpy(host_ptr, data_ptr<char>(), bytes);
    }
}

Tensor Tensor::transpose(int64_t d0, int64_t d1) const {
    if (d0 < 0) d0 += ndim();
    if (d1 < 0) d1 += ndim();
    Tensor t = *this;
    std::swap(t.shape_[d0], t.shape_[d1]);
    std::swap(t.strides_[d0], t.strides_[d1]);
    return t;
}

Tensor Tensor::view(const std::vector<int64_t>& new_shape) const {
    if (!is_contiguous()) throw std::runtime_error("view: tensor must be contiguous");
    size_t n = 1;
    for (auto s : new_shape) n *= static_cast<size_t>(s);
    if (n != numel()) throw std::runtime_error("view: shape is invalid for input size");
    return Tensor(storage_, new_shape, contiguous_strides(new_shape), offset_, dtype_);
}

Tensor Tensor::reshape(const std::vector<int64_t>& new_shape) const {
    return (is_contiguous() ? *this : contiguous()).view(new_shape);
}

Tensor Tensor::index(const std::vector<IndexSelector>& selectors) const {
    if (static_cast<int64_t>(selectors.size()) > ndim()) throw std::runtime_error("index: too many indices");
    std::vector<int64_t> shape, strides;
    size_t off = offset_;
    for (int64_t d = 0; d < ndim(); ++d) {
        if (d >= static_cast<int64_t>(selectors.size())) { shape.push_back(shape_[d]); strides.push_back(strides_[d]); continue; }
        const IndexSelector& sel = selectors[d];
        if (std::holds_alternative<int64_t>(sel)) {
            int64_t i = std::get<int64_t>(sel);
            if (i < 0) i += shape_[d];
            if (i < 0 || i >= shape_[d]) throw std::runtime_error("index: out of range");
            off += static_cast<size_t>(i * strides_[d]);
        } else {
            const Slice& s = std::get<Slice>(sel);
            int64_t step = s.step.value_or(1);
            if (step <= 0) throw std::runtime_error("index: slice step must be positive");
            int64_t start = s.start.value_or(0), stop = s.stop.value_or(shape_[d]);
            if (start < 0) start += shape_[d];
            if (stop < 0) stop += shape_[d];
            start = std::max<int64_t>(0, std::min(start, shape_[d]));
            stop = std::max<int64_t>(start, std::min(stop, shape_[d]));
            off += static_cast<size_t>(start * strides_[d]);
            shape.push_back((stop - start + step - 1) / step);
            strides.push_back(strides_[d] * step);
        }
    }
    return Tensor(storage_, shape, strides, off, dtype_);
}

Tensor Tensor::unflatten_last(int64_t outer, int64_t inner) const {
    if (ndim() < 1 || strides_.back() != 1 || shape_.back() != outer * inner)
        throw std::runtime_error("unflatten_last: the last dimension must be contiguous and equal outer * inner");
    std::vector<int64_t> shape(shape_.begin(), shape_.end() - 1), strides(strides_.begin(), strides_.end() - 1);
    shape.push_back(outer); shape.push_back(inner);
    strides.push_back(inner); strides.push_back(1);
    return Tensor(storage_, shape, strides, offset_, dtype_);
}

Tensor Tensor::narrow(int64_t dim, int64_t start, int64_t length) const {
    if (dim < 0) dim += ndim();
    std::vector<IndexSelector> sel(static_cast<size_t>(dim) + 1, Slice());
    sel[dim] = Slice(start, start + length);
    return index(sel);
}

namespace {
// generic strided element copy on the host
void host_strided_copy(const Tensor& src, Tensor& dst) {
    size_t esz = GetDTypeSize(src.dtype());
    size_t n = src.numel();
    std::vector<int64_t> idx(src.ndim(), 0);
    const char* sp = src.data_ptr<char>();
    char* dp = dst.data_ptr<char>();
    for (size_t i = 0; i < n; ++i) {
        int64_t so = 0, dofs = 0;
        for (int64_t d = 0; d < src.ndim(); ++d) { so += idx[d] * src.strides()[d]; dofs += idx[d] * dst.strides()[d]; }
        std::memcpy(dp + dofs * esz, sp + so * esz, esz);
        for (int64_t d = src.ndim() - 1; d >= 0; --d) { if (++idx[d] < src.shape()[d]) break; idx[d] = 0; }
    }
}

// [.., S, D] views with D contiguous, padded to 4-D: pointer + (B,H,S) strides
bool as_view4(const Tensor& t, vb200_tensor4* v, int64_t dims[4]) {
    if (t.ndim() < 1 || t.ndim() > 4 || t.strides().back() != 1) return false;
    int64_t sh[4] = {1, 1, 1, 1}, st[4] = {0, 0, 0, 1};
    int pad = 4 - static_cast<int>(t.ndim());
    for (int i = 0; i < t.ndim(); ++i) { sh[pad + i] = t.shape()[i]; st[pad + i] = t.strides()[i]; }
    for (int i = 0; i < 4; ++i) dims[i] = sh[i];
    v->ptr = const_cast<char*>(t.data_ptr<char>());
    v->stride_b = st[0]; v->stride_h = st[1]; v->stride_s = st[2];
    return true;
}
}  // namespace

void Tensor::copy_from(const Tensor& other) {
    if (other.shape() != shape_) throw std::runtime_error("copy_from: shape mismatch");
    if (other.dtype() != dtype_) throw std::runtime_error("copy_from: dtype mismatch");
    if (device() == Device::CPU && other.device() == Device::CPU) { host_strided_copy(other, *this); return; }
    if (device() != other.device()) {
        Tensor src = other.is_contiguous() ? other : other.contiguous();
        if (!is_contiguous()) throw std::runtime_error("copy_from: cross-device copy needs a contiguous destination");
        size_t bytes = numel() * GetDTypeSize(dtype_);
        cuda_check(cudaMemcpy(data_ptr<char>(), src.data_ptr<char>(), bytes,
                              device() == Device::CUDA ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost), "cudaMemcpy");
        return;
    }
    // device -> device
    cudaStream_t s = static_cast<cudaStream_t>(Stream::current(Device::CUDA).raw_handle());
    if (is_contiguous() && other.is_contiguous()) {
        cuda_check(cudaMemcpyAsync(data_ptr<char>(), other.data_ptr<char>(), numel() * GetDTypeSize(dtype_), cudaMemcpyDeviceToDevice, s), "cudaMemcpyAsync");
        return;
    }
    // strided views with a contiguous last dimension: the append kernel is a strided row copy
    vb200_tensor4 sv, dv;
    int64_t sd[4], dd[4];
    if (!as_view4(other, &sv, sd) || !as_view4(*this, &dv, dd) || sd[3] % 8 != 0)
        throw std::runtime_error("copy_from: this strided device copy is not provided by the attention backend");
    int rc = vb200_kv_append(-1, s, dtype_code(dtype_), static_cast<int>(sd[0]), static_cast<int>(sd[1]), static_cast<int>(sd[2]),
                             static_cast<int>(sd[3]), 0, &sv, &sv, &dv, &dv, static_cast<int>(sd[2]), nullptr);
    if (rc != VB200_OK) throw std::runtime_error(std::string("copy_from: ") + vb200_strerror(rc) + ": " + vb200_last_error_detail());
}

Tensor Tensor::contiguous_copy() const {
    Tensor out = empty(shape_, dtype_, device());
    out.copy_from(*this);
    return out;
}

Tensor Tensor::contiguous() const { return is_contiguous() ? *this : contiguous_copy(); }

Tensor Tensor::to(Device dev) const {
    if (dev == device()) return *this;
    Tensor out = empty(shape_, dtype_, dev);
    out.copy_from(*this);
    return out;
}

void Tensor::zero_() {
    if (!is_contiguous()) throw std::runtime_error("zero_: tensor must be contiguous");
    size_t bytes = numel() * GetDTypeSize(dtype_);
    if (device() == Device::CUDA)
        cuda_check(cudaMemsetAsync(data_ptr<char>(), 0, bytes, static_cast<cudaStream_t>(Stream::current(Device::CUDA).raw_handle())), "cudaMemsetAsync");
    else
        std::memset(data_ptr<char>(), 0, bytes);
}

Tensor empty(const std::vector<int64_t>& shape, DType dtype, Device device, bool) {
    size_t n = 1;
    for (auto s : shape) {
        if (s < 0) throw std::runtime_error("empty: negative dimension");
        n *= static_cast<size_t>(s);
    }
    auto st = std::make_shared<Storage>(n * GetDTypeSize(dtype), device);
    return Tensor(st, shape, contiguous_strides(shape), 0, dtype);
}

Tensor zeros(const std::vector<int64_t>& shape, DType dtype, Device device, bool) {
    Tensor t = empty(shape, dtype, device);
    t.zero_();
    return t;
}

// ---- 16-bit conversions ----
uint16_t float_to_bf16(float f) {
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    bits += 0x7FFFu + ((bits >> 16) & 1u);
    return static_cast<uint16_t>(bits >> 16);
}
float bf16_to_float(uint16_t h) {
    uint32_t bits = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
uint16_t float_to_fp16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    int32_t exp = static_cast<int32_t>((x >> 23) & 0xFF) - 127 + 15;
    uint32_t man = x & 0x7FFFFFu;
    if (((x >> 23) & 0xFF) == 0xFF) return static_cast<uint16_t>(sign | 0x7C00u | (man ? 0x200u : 0));
    if (exp >= 31) return static_cast<uint16_t>(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return static_cast<uint16_t>(sign);
        man |= 0x800000u;
        uint32_t shift = static_cast<uint32_t>(14 - exp);
        uint32_t half = man >> shift, rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) ++half;
        return static_cast<uint16_t>(sign | half);
    }
    uint32_t half = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
}
float fp16_to_float(uint16_t h) {
    uint32_t sign = (static_cast<uint32_t>(h) & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { ++e; man <<= 1; } while (!(man & 0x400u));
            bits = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

}  // namespace vesper
