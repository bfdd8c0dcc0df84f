// ops::flash_attention on the B200 backend.  Same signature and error
// behaviour as include/vesper/ops/flash_attention.h:34-41 of the reference;
// the CUDA dispatch function keeps the reference's name and parameters
// (src/ops/flash_attention.cpp:28-32) and forwards to vb200_prefill_fwd.
#pragma once
#include <vesper/core/tensor.h>
#include <tuple>
#include <utility>

namespace vesper::ops {

// q, k, v: [Batch, Heads, SeqLen, HeadDim] on Device::CUDA, same shape and dtype
// (Float32, BFloat16 or Float16).  Throws std::runtime_error on invalid input.
// dropout_p is validated and otherwise ignored, as the reference's CUDA path does.
Tensor flash_attention(const Tensor& q, const Tensor& k, const Tensor& v, float scale,
                       bool is_causal = true, float dropout_p = 0.0f, bool training = false);

// Extension: also returns the log-sum-exp [B, H, N] (fp32) the reference keeps private.
// K/V may carry fewer heads than Q (grouped queries) here.
std::pair<Tensor, Tensor> flash_attention_with_lse(const Tensor& q, const Tensor& k, const Tensor& v,
                                                   float scale, bool is_causal = true);

void flash_attention_cuda_dispatch(const Tensor& q, const Tensor& k, const Tensor& v,
                                   Tensor& output, Tensor& lse, float scale, bool is_causal,
                                   float dropout_p, bool training, Tensor* dropout_mask_out);

// Backward for training (include/vesper/ops/flash_attention.h:61-70 of the reference): gradients of
// q, k, v from the saved output and log-sum-exp.  Float32, contiguous inputs are made as the reference does
// (src/ops/flash_attention.cpp:373-378); dropout is not part of the CUDA path (dropout_p must be 0).
std::tuple<Tensor, Tensor, Tensor> flash_attention_backward(const Tensor& grad_output, const Tensor& q, const Tensor& k,
                                                            const Tensor& v, const Tensor& output, const Tensor& lse,
                                                            float scale, bool is_causal = true, float dropout_p = 0.0f,
                                                            const Tensor& dropout_mask = Tensor());
void flash_attention_backward_cuda_dispatch(const Tensor& grad_output, const Tensor& q, const Tensor& k, const Tensor& v,
                                            const Tensor& output, const Tensor& lse, Tensor& grad_q, Tensor& grad_k,
                                            Tensor& grad_v, float scale, bool is_causal, float dropout_p,
                                            const Tensor* dropout_mask);

}  // namespace vesper::ops
