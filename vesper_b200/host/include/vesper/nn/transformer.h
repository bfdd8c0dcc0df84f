// nn::KVCache and the fused attention core used by MultiHeadAttention /
// GroupedQueryAttention forward(x, cache, start_pos)
// (include/vesper/nn/transformer.h:21-56, src/nn/transformer.cpp:32-93,166-216).
#pragma once
#include <vesper/core/tensor.h>
#include <vesper/nn/linear.h>
#include <utility>

namespace vesper::nn {

class KVCache {
public:
    // dtype: the reference stores Float32 only (src/nn/transformer.cpp:40-41); BFloat16 /
    // Float16 caches are what the B200 kernels are built for.
    KVCache(int batch_size, int num_heads, int max_seq_len, int head_dim, Device device,
            DType dtype = DType::Float32);

    // Writes new_k/new_v [Batch, Heads, SeqLen, HeadDim] at rows start_pos.. and returns views
    // [:, :, 0:current_len, :] of the two caches (strides keep max_seq_len * head_dim).
    std::pair<Tensor, Tensor> update(const Tensor& new_k, const Tensor& new_v, int start_pos);

    void reset();                                   // zero both caches, length 0
    int current_seq_len() const { return current_len_; }
    int get_max_seq_len() const { return max_seq_len_; }

    // Needed by the fused attention call (the reference keeps these private).
    Tensor& k() { return k_cache_; }
    Tensor& v() { return v_cache_; }
    void set_current_len(int n) { current_len_ = n; }

private:
    Tensor k_cache_, v_cache_;
    int max_seq_len_;
    int current_len_ = 0;
};

// Steps 3-6 of GroupedQueryAttention::forward(x, cache, start_pos)
// (src/nn/gqa_attention.cpp:124-149) and of MultiHeadAttention::forward
// (src/nn/transformer.cpp:184-204) as ONE backend call: RoPE of q and k at start_pos,
// append of rotated k and raw v to the cache, grouped-query attention over the cached
// context with causal = (T > 1).  q: [B,Hq,T,D]; k, v: [B,Hkv,T,D]; returns [B,Hq,T,D].
// cache == nullptr: attention over the T new tokens only (the uncached forward).
// out_view (optional): where the result goes -- a [B,Hq,T,D] view with any batch / head / row strides, e.g. the
// transposed view of a [B,T,Hq,D] buffer, so that the heads come out already merged.
Tensor fused_attention(const Tensor& q, const Tensor& k, const Tensor& v, KVCache* cache, int64_t start_pos,
                       bool use_rope = true, float rope_base = 10000.0f, bool causal_when_uncached = true,
                       Tensor* out_view = nullptr);

// nn::MultiHeadAttention (include/vesper/nn/transformer.h:41-56, src/nn/transformer.cpp:97-216): c_attn =
// Linear(C, 3C) with bias, three slices of its output as q, k, v, optional RoPE with theta fixed at 10000,
// attention, c_proj = Linear(C, C) with bias.  forward(x) is NON-causal, as in the reference (:108-110);
// forward(x, cache, start_pos) masks causally when more than one token comes in.  Dropout is training-only in the
// reference and this layer is the inference path: a non-zero dropout is accepted and never applied.
// The trailing dtype argument (not in the reference, whose modules are Float32) selects the number format of the
// weights and activations: Float32 reproduces the reference at 1e-4, BFloat16 is the serving format.
class MultiHeadAttention {
public:
    MultiHeadAttention(int embed_dim, int num_heads, float dropout = 0.0, bool use_rope = true, DType dtype = DType::Float32);
    Tensor forward(const Tensor& x);
    Tensor forward(const Tensor& x, bool causal);
    Tensor forward(const Tensor& x, KVCache* cache, int start_pos = 0);

    Linear c_attn;
    Linear c_proj;
    int n_head;
    int n_embd;
    float dropout_;
    bool use_rope_;
};

}  // namespace vesper::nn
