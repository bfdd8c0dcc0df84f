// nn::GroupedQueryAttention of the reference (include/vesper/nn/gqa_attention.h:27-101,
// src/nn/gqa_attention.cpp:26-159) on the B200 attention path: fused QKV projection, then ONE backend call for
// RoPE of q and k, the cache append and grouped-query attention (kv_head = q_head / num_rep inside the kernels:
// no repeat_kv, none of the reference's transposes and .contiguous() copies -- q, k, v are strided views of the
// fused projection's output and the kernel writes the head-merged layout), then the output projection.
//
// Same constructor arguments, validation and forward overloads as the reference.  forward(x) is causal.  Dropout
// is training-only in the reference and this layer is the inference path: a non-zero value is accepted and never
// applied.  The trailing dtype argument (not in the reference, whose modules are Float32) selects the number
// format of weights and activations: Float32 reproduces the reference at 1e-4, BFloat16 is the serving format.
// With a cache, pass a KVCache of the same dtype sized with num_kv_heads (src/models/transformer.cpp:194-200).
// Unlike the reference's cached path, which reads the strided cache views as if they were contiguous
// (src/ops/attention_ops.cpp:34-52) and so returns wrong values when num_rep > 1 and the cache is not full, the
// cached forward here equals the uncached one.
#pragma once
#include <vesper/core/tensor.h>
#include <vesper/nn/linear.h>
#include <vesper/nn/transformer.h>

namespace vesper::nn {

class GroupedQueryAttention {
public:
    GroupedQueryAttention(int64_t embed_dim, int64_t num_heads, int64_t num_kv_heads, int64_t max_seq_len = 4096,
                          float rope_base = 10000.0f, float dropout = 0.0f, bool bias = false, DType dtype = DType::BFloat16);

    Tensor forward(const Tensor& x);                       // [Batch, SeqLen, EmbedDim] -> same; causal
    Tensor forward(const Tensor& x, bool causal);
    Tensor forward(const Tensor& x, KVCache* cache, int64_t start_pos = 0);

    int64_t embed_dim() const { return embed_dim_; }
    int64_t num_heads() const { return num_heads_; }
    int64_t num_kv_heads() const { return num_kv_heads_; }
    int64_t head_dim() const { return head_dim_; }
    int64_t num_rep() const { return num_rep_; }
    float kv_cache_ratio() const { return static_cast<float>(num_kv_heads_) / num_heads_; }

    // parameters, named as the reference registers them ("wqkv", "wo")
    FusedQKVLinear& wqkv() { return wqkv_; }
    Linear& wo() { return wo_; }

private:
    Tensor run(const Tensor& x, KVCache* cache, int64_t start_pos, bool causal_when_uncached);
    int64_t embed_dim_, num_heads_, num_kv_heads_, head_dim_, num_rep_;
    float dropout_, rope_base_;
    int64_t max_seq_len_;
    FusedQKVLinear wqkv_;
    Linear wo_;
};

}  // namespace vesper::nn
