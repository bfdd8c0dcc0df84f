// nn::Linear / FusedQKVLinear / RMSNorm / SwiGLUMLP: thin owners of device weights in front of the C ABI
// of vesper_b200_block.h.
#include <vesper/nn/linear.h>

#include <vesper_b200.h>
#include <vesper_b200_block.h>

#include <stdexcept>
#include <string>

namespace vesper::nn {

namespace {

void check(int rc, const char* who) {
    if (rc != VB200_OK)
        throw std::runtime_error(std::string(who) + ": " + vb200_strerror(rc) + ": " + vb200_last_error_detail());
}
void* current_stream() { return Stream::current(Device::CUDA).raw_handle(); }

Tensor bf16_from_host(const float* src, const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    std::vector<uint16_t> tmp(static_cast<size_t>(n));
    for (int64_t i = 0; i < n; ++i) tmp[static_cast<size_t>(i)] = float_to_bf16(src[i]);
    Tensor t = empty(shape, DType::BFloat16, Device::CUDA);
    t.copy_from_host(tmp.data());
    return t;
}

// rows of the flattened [..., last] view and the output shape with a new last dimension
int64_t leading_rows(const Tensor& t, int64_t last, const char* who) {
    if (t.ndim() < 1 || t.shape().back() != last)
        throw std::runtime_error(std::string(who) + ": last dimension must be " + std::to_string(last));
    return static_cast<int64_t>(t.numel()) / last;
}
std::vector<int64_t> with_last(const Tensor& t, int64_t last) {
    std::vector<int64_t> s = t.shape();
    s.back() = last;
    return s;
}
void require(const Tensor& t, DType dt, const char* who) {
    if (t.device() != Device::CUDA) throw std::runtime_error(std::string(who) + ": this library is the CUDA backend; CPU tensors are not handled here");
    if (t.dtype() != dt) throw std::runtime_error(std::string(who) + ": unexpected dtype");
}

Tensor weight_from_host(const float* src, const std::vector<int64_t>& shape, DType dt) {
    if (dt == DType::BFloat16) return bf16_from_host(src, shape);
    Tensor t = empty(shape, DType::Float32, Device::CUDA);
    t.copy_from_host(src);
    return t;
}

Tensor run_linear(const Tensor& input, const Tensor& weight, const Tensor& bias, int64_t in_f, int64_t out_f, int epilogue, const char* who) {
    require(input, weight.dtype(), who);
    const int64_t M = leading_rows(input, in_f, who);
    Tensor x = input.is_contiguous() ? input : input.contiguous();
    const int64_t out_cols = epilogue == VB200_EPI_SWIGLU ? out_f / 2 : out_f;
    Tensor out = empty(with_last(input, out_cols), weight.dtype(), Device::CUDA);
    if (weight.dtype() == DType::Float32) {
        if (epilogue != VB200_EPI_BF16) throw std::runtime_error(std::string(who) + ": the Float32 path has no fused epilogue");
        check(vb200_linear_f32(x.device_index(), current_stream(), x.data_ptr<float>(), in_f, weight.data_ptr<float>(), in_f,
                               bias.defined() ? bias.data_ptr<float>() : nullptr, out.data_ptr<float>(), out_cols, static_cast<int>(M),
                               static_cast<int>(out_f), static_cast<int>(in_f)), who);
        return out;
    }
    check(vb200_linear_bias(x.device_index(), current_stream(), x.data_ptr<char>(), in_f, weight.data_ptr<char>(), in_f,
                            bias.defined() ? bias.data_ptr<float>() : nullptr, out.data_ptr<char>(), out_cols, static_cast<int>(M),
                            static_cast<int>(out_f), static_cast<int>(in_f), epilogue, 0), who);
    return out;
}

void require_dtype(DType dt, const char* who) {
    if (dt != DType::BFloat16 && dt != DType::Float32) throw std::runtime_error(std::string(who) + ": dtype must be BFloat16 or Float32");
}

}  // namespace

Linear::Linear(int64_t in_features, int64_t out_features, bool use_bias, Device device, DType dtype)
    : in_features_(in_features), out_features_(out_features), use_bias_(use_bias), dtype_(dtype) {
    if (device != Device::CUDA) throw std::runtime_error("Linear: this library is the CUDA backend");
    require_dtype(dtype, "Linear");
    weight = zeros({out_features, in_features}, dtype, Device::CUDA);
    if (use_bias) bias = zeros({out_features}, DType::Float32, Device::CUDA);
}
void Linear::load_weight(const float* host_weight, const float* host_bias) {
    weight = weight_from_host(host_weight, {out_features_, in_features_}, dtype_);
    if (use_bias_ && host_bias) bias.copy_from_host(host_bias);
}
Tensor Linear::forward(const Tensor& input) { return run_linear(input, weight, bias, in_features_, out_features_, VB200_EPI_BF16, "Linear"); }

FusedQKVLinear::FusedQKVLinear(int64_t in_features, int64_t q_features, int64_t kv_features, bool use_bias, Device device, DType dtype)
    : in_features_(in_features), q_features_(q_features), kv_features_(kv_features), use_bias_(use_bias), dtype_(dtype) {
    if (device != Device::CUDA) throw std::runtime_error("FusedQKVLinear: this library is the CUDA backend");
    require_dtype(dtype, "FusedQKVLinear");
    weight = zeros({q_features + 2 * kv_features, in_features}, dtype, Device::CUDA);
    if (use_bias) bias = zeros({q_features + 2 * kv_features}, DType::Float32, Device::CUDA);
}
void FusedQKVLinear::load_weight(const float* host_weight, const float* host_bias) {
    weight = weight_from_host(host_weight, {q_features_ + 2 * kv_features_, in_features_}, dtype_);
    if (use_bias_ && host_bias) bias.copy_from_host(host_bias);
}
Tensor FusedQKVLinear::forward(const Tensor& input) {
    return run_linear(input, weight, bias, in_features_, q_features_ + 2 * kv_features_, VB200_EPI_BF16, "FusedQKVLinear");
}
std::tuple<Tensor, Tensor, Tensor> FusedQKVLinear::forward_split(const Tensor& input) {
    Tensor qkv = forward(input);
    const int64_t last = qkv.ndim() - 1;
    return {qkv.narrow(last, 0, q_features_), qkv.narrow(last, q_features_, kv_features_),
            qkv.narrow(last, q_features_ + kv_features_, kv_features_)};
}

RMSNorm::RMSNorm(std::vector<int64_t> shape, float eps_, bool affine) : normalized_shape(std::move(shape)), eps(eps_), elementwise_affine(affine) {
    if (normalized_shape.size() != 1) throw std::runtime_error("RMSNorm: one normalized dimension is supported");
    std::vector<float> ones(static_cast<size_t>(normalized_shape[0]), 1.0f);
    weight = empty({normalized_shape[0]}, DType::Float32, Device::CUDA);
    weight.copy_from_host(ones.data());
}
void RMSNorm::load_weight(const float* host_weight) { weight.copy_from_host(host_weight); }
Tensor RMSNorm::forward(const Tensor& input) {
    require(input, DType::Float32, "RMSNorm");
    const int64_t dim = normalized_shape[0];
    const int64_t M = leading_rows(input, dim, "RMSNorm");
    Tensor x = input.is_contiguous() ? input : input.contiguous();
    Tensor out = empty(input.shape(), DType::BFloat16, Device::CUDA);
    check(vb200_rms_norm(x.device_index(), current_stream(), x.data_ptr<float>(), weight.data_ptr<float>(), out.data_ptr<char>(),
                         static_cast<int>(M), static_cast<int>(dim), eps), "RMSNorm");
    return out;
}

SwiGLUMLP::SwiGLUMLP(int64_t d_model, int64_t hidden_dim, bool bias) : d_model_(d_model), hidden_dim_(hidden_dim) {
    if (d_model <= 0 || hidden_dim <= 0) throw std::invalid_argument("SwiGLUMLP: d_model and hidden_dim must be positive");
    if (bias) throw std::runtime_error("SwiGLUMLP: bias is not built on this path");
    w13_ = zeros({2 * hidden_dim, d_model}, DType::BFloat16, Device::CUDA);
    w2_ = zeros({d_model, hidden_dim}, DType::BFloat16, Device::CUDA);
}
int64_t SwiGLUMLP::compute_hidden_dim(int64_t d_model, int64_t multiple_of) {
    int64_t hidden = (8 * d_model) / 3;                     // src/nn/swiglu.cpp:50-61
    if (multiple_of > 1) hidden = ((hidden + multiple_of - 1) / multiple_of) * multiple_of;
    return hidden;
}
void SwiGLUMLP::load_weights(const float* gate, const float* up, const float* down) {
    Tensor g = bf16_from_host(gate, {hidden_dim_, d_model_}), u = bf16_from_host(up, {hidden_dim_, d_model_});
    check(vb200_interleave_rows(g.device_index(), current_stream(), g.data_ptr<char>(), u.data_ptr<char>(), w13_.data_ptr<char>(), hidden_dim_, d_model_),
          "SwiGLUMLP::load_weights");
    Stream::current(Device::CUDA).synchronize();
    w2_ = bf16_from_host(down, {d_model_, hidden_dim_});
}
Tensor SwiGLUMLP::forward(const Tensor& x) {
    Tensor hidden = run_linear(x, w13_, Tensor(), d_model_, 2 * hidden_dim_, VB200_EPI_SWIGLU, "SwiGLUMLP");
    return run_linear(hidden, w2_, Tensor(), hidden_dim_, d_model_, VB200_EPI_BF16, "SwiGLUMLP");
}

}  // namespace vesper::nn
