// nn::functional attention helpers with the reference's names and semantics
// (include/vesper/nn/functional.h:132-154, src/nn/functional.cpp:370-494).
#pragma once
#include <vesper/core/tensor.h>

namespace vesper::nn::functional {

// softmax(Q K^T / sqrt(D) [+ causal mask]) V for [B,H,T,D] queries and [B,Hkv,L,D] keys/values
// on Device::CUDA.  The reference routes on the query length (flash op at >= 512, five generic
// ops below); here every case is one fused call.  Causal with T != L is bottom-right aligned.
// dropout_p must be 0 (inference path).
Tensor scaled_dot_product_attention(const Tensor& query, const Tensor& key, const Tensor& value,
                                    bool is_causal = false, double dropout_p = 0.0);

// Angle table [seq_len, head_dim/2], a[m,i] = (start_pos+m) * theta^(-2i/head_dim), built on the
// host in fp32 exactly as the reference does and moved to `device`.
Tensor compute_rope_frequencies(int seq_len, int head_dim, int start_pos = 0, float theta = 10000.0f,
                                Device device = Device::CPU);

// Rotation of adjacent pairs (x[2i], x[2i+1]) of x [B,H,S,D] (Float32, CUDA) by freqs [S, D/2].
Tensor apply_rotary_emb(const Tensor& x, const Tensor& freqs);

}  // namespace vesper::nn::functional
