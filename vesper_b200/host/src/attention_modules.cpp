// nn::GroupedQueryAttention and nn::MultiHeadAttention: the reference's module surface
// (src/nn/gqa_attention.cpp:26-159, src/nn/transformer.cpp:97-216) composed from this layer's projections and
// the fused attention call.
#include <vesper/nn/gqa_attention.h>

#include <stdexcept>
#include <string>

namespace vesper::nn {

namespace {

// x [B,T,C] -> fused projection [B,T,(Hq+2Hkv)*D]; q, k, v as [B,H,T,D] views of it (strides only), attention
// written straight into a [B,T,Hq*D] buffer through its [B,Hq,T,D] view; returns that buffer.
Tensor attend(const Tensor& qkv, int64_t Hq, int64_t Hkv, int64_t D, KVCache* cache, int64_t start_pos, bool use_rope,
              float rope_base, bool causal_when_uncached) {
    const int64_t B = qkv.shape()[0], T = qkv.shape()[1];
    auto heads = [&](int64_t first_col, int64_t H) {
        return qkv.narrow(2, first_col, H * D).unflatten_last(H, D).transpose(1, 2);      // [B,T,H,D] memory as [B,H,T,D]
    };
    Tensor q = heads(0, Hq), k = heads(Hq * D, Hkv), v = heads((Hq + Hkv) * D, Hkv);
    Tensor merged = empty({B, T, Hq * D}, qkv.dtype(), Device::CUDA);
    Tensor out_view = merged.view({B, T, Hq, D}).transpose(1, 2);
    fused_attention(q, k, v, cache, start_pos, use_rope, rope_base, causal_when_uncached, &out_view);
    return merged;
}

void require_input(const Tensor& x, int64_t C, DType dt, const char* who) {
    if (x.ndim() != 3 || x.shape()[2] != C)
        throw std::runtime_error(std::string(who) + ": input must be [Batch, SeqLen, " + std::to_string(C) + "]");
    if (x.dtype() != dt) throw std::runtime_error(std::string(who) + ": input dtype differs from the module's");
}

}  // namespace

GroupedQueryAttention::GroupedQueryAttention(int64_t embed_dim, int64_t num_heads, int64_t num_kv_heads, int64_t max_seq_len,
                                             float rope_base, float dropout, bool bias, DType dtype)
    : embed_dim_(embed_dim), num_heads_(num_heads), num_kv_heads_(num_kv_heads),
      head_dim_(num_heads > 0 ? embed_dim / num_heads : 0), num_rep_(num_kv_heads > 0 ? num_heads / num_kv_heads : 0),
      dropout_(dropout), rope_base_(rope_base), max_seq_len_(max_seq_len),
      wqkv_(embed_dim, num_heads * head_dim_, num_kv_heads * head_dim_, bias, Device::CUDA, dtype),
      wo_(num_heads * head_dim_, embed_dim, bias, Device::CUDA, dtype) {
    // src/nn/gqa_attention.cpp:47-56
    if (num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        throw std::invalid_argument("GroupedQueryAttention: num_heads (" + std::to_string(num_heads) +
                                    ") must be divisible by num_kv_heads (" + std::to_string(num_kv_heads) + ")");
    if (num_heads <= 0 || embed_dim % num_heads != 0)
        throw std::invalid_argument("GroupedQueryAttention: embed_dim (" + std::to_string(embed_dim) +
                                    ") must be divisible by num_heads (" + std::to_string(num_heads) + ")");
}

Tensor GroupedQueryAttention::forward(const Tensor& x) { return forward(x, true); }          // src/nn/gqa_attention.cpp:63-65

Tensor GroupedQueryAttention::forward(const Tensor& x, bool causal) { return run(x, nullptr, 0, causal); }

Tensor GroupedQueryAttention::forward(const Tensor& x, KVCache* cache, int64_t start_pos) {
    // without a cache the reference still masks by (T > 1): src/nn/gqa_attention.cpp:143-149
    return run(x, cache, start_pos, x.ndim() == 3 && x.shape()[1] > 1);
}

Tensor GroupedQueryAttention::run(const Tensor& x, KVCache* cache, int64_t start_pos, bool causal_when_uncached) {
    require_input(x, embed_dim_, wqkv_.weight.dtype(), "GroupedQueryAttention");
    Tensor qkv = wqkv_.forward(x);
    Tensor merged = attend(qkv, num_heads_, num_kv_heads_, head_dim_, cache, start_pos, true, rope_base_, causal_when_uncached);
    return wo_.forward(merged);
}

MultiHeadAttention::MultiHeadAttention(int embed_dim, int num_heads, float dropout, bool use_rope, DType dtype)
    : c_attn(embed_dim, 3 * embed_dim, true, Device::CUDA, dtype), c_proj(embed_dim, embed_dim, true, Device::CUDA, dtype),
      n_head(num_heads), n_embd(embed_dim), dropout_(dropout), use_rope_(use_rope) {
    if (num_heads <= 0 || embed_dim % num_heads != 0) throw std::invalid_argument("MultiHeadAttention: embed_dim must be divisible by num_heads");
}

Tensor MultiHeadAttention::forward(const Tensor& x) { return forward(x, false); }           // src/nn/transformer.cpp:108-110

Tensor MultiHeadAttention::forward(const Tensor& x, bool causal) {
    require_input(x, n_embd, c_attn.dtype(), "MultiHeadAttention");
    Tensor qkv = c_attn(x);                                                                  // [B, T, 3C]: q | k | v
    Tensor merged = attend(qkv, n_head, n_head, n_embd / n_head, nullptr, 0, use_rope_, 10000.0f, causal);
    return c_proj(merged);
}

Tensor MultiHeadAttention::forward(const Tensor& x, KVCache* cache, int start_pos) {
    require_input(x, n_embd, c_attn.dtype(), "MultiHeadAttention");
    Tensor qkv = c_attn(x);
    Tensor merged = attend(qkv, n_head, n_head, n_embd / n_head, cache, start_pos, use_rope_, 10000.0f, x.shape()[1] > 1);
    return c_proj(merged);
}

}  // namespace vesper::nn
