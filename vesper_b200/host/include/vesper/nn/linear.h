// nn::Linear, nn::FusedQKVLinear, nn::RMSNorm and nn::SwiGLUMLP of the reference
// (include/vesper/nn/linear.h:10-46, include/vesper/nn/normalization.h:20-29, include/vesper/nn/swiglu.h:27-57)
// on the B200 operators.  Same constructor arguments and forward() shapes; what differs is the number
// format: weights are BFloat16 on CUDA by default (norm weights and biases Float32), Linear and SwiGLUMLP take
// and return BFloat16 activations, RMSNorm takes the Float32 residual stream and returns BFloat16.  Linear and
// FusedQKVLinear also come in Float32 (trailing constructor argument): the reference's own number format, for
// parity at 1e-4.  Weights start at zero (norm weights at one); load_weight() takes host Float32 values in the
// reference's layouts.
#pragma once
#include <vesper/core/tensor.h>

#include <tuple>
#include <vector>

namespace vesper::nn {

class Linear {
public:
    Linear(int64_t in_features, int64_t out_features, bool use_bias = true, Device device = Device::CUDA,
           DType dtype = DType::BFloat16);
    // input [..., in_features] -> [..., out_features], both of the module's dtype: matmul(input, weight^T) (+ bias)
    Tensor forward(const Tensor& input);
    Tensor operator()(const Tensor& input) { return forward(input); }
    void load_weight(const float* host_weight, const float* host_bias = nullptr);   // [out, in], [out]
    DType dtype() const { return dtype_; }

    Tensor weight;   // [out_features, in_features] BFloat16 (or Float32)
    Tensor bias;     // [out_features] Float32 (undefined without bias)
private:
    int64_t in_features_, out_features_;
    bool use_bias_;
    DType dtype_;
};

class FusedQKVLinear {
public:
    FusedQKVLinear(int64_t in_features, int64_t q_features, int64_t kv_features, bool use_bias = false, Device device = Device::CUDA,
                   DType dtype = DType::BFloat16);
    Tensor forward(const Tensor& input);                                            // [..., q + 2 kv]
    // q, k, v as VIEWS of the fused output (no copies; the attention kernels honour the strides)
    std::tuple<Tensor, Tensor, Tensor> forward_split(const Tensor& input);
    void load_weight(const float* host_weight, const float* host_bias = nullptr);

    Tensor weight;
    Tensor bias;
private:
    int64_t in_features_, q_features_, kv_features_;
    bool use_bias_;
    DType dtype_;
};

class RMSNorm {
public:
    RMSNorm(std::vector<int64_t> normalized_shape, float eps = 1e-5f, bool elementwise_affine = true);
    Tensor forward(const Tensor& input);            // Float32 [..., dim] -> BFloat16 [..., dim]
    void load_weight(const float* host_weight);

    std::vector<int64_t> normalized_shape;
    float eps;
    bool elementwise_affine;
    Tensor weight;   // [dim] Float32
};

class SwiGLUMLP {
public:
    SwiGLUMLP(int64_t d_model, int64_t hidden_dim, bool bias = false);
    // down_proj(silu(gate_proj(x)) * up_proj(x)), x BFloat16 [..., d_model] -> BFloat16 [..., d_model];
    // gate and up run as ONE GEMM over row-interleaved weights with the SiLU product in its epilogue
    Tensor forward(const Tensor& x);
    void load_weights(const float* gate, const float* up, const float* down);       // [hidden, d], [hidden, d], [d, hidden]
    static int64_t compute_hidden_dim(int64_t d_model, int64_t multiple_of = 256);
    int64_t d_model() const { return d_model_; }
    int64_t hidden_dim() const { return hidden_dim_; }

private:
    int64_t d_model_, hidden_dim_;
    Tensor w13_;     // [2 * hidden, d_model] BFloat16, row 2j = gate_j, row 2j + 1 = up_j
    Tensor w2_;      // [d_model, hidden] BFloat16
};

}  // namespace vesper::nn
