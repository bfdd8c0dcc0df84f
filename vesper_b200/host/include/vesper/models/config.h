// models::TransformerConfig -- the fields of the reference's configuration
// (include/vesper/models/config.h:22-99) that the Llama-style inference path reads.
#pragma once
#include <cstdint>

namespace vesper::models {

struct TransformerConfig {
    int64_t vocab_size = 32000;
    int64_t dim = 4096;
    int64_t n_layers = 32;
    int64_t n_heads = 32;
    int64_t n_kv_heads = -1;        // -1 = same as n_heads
    int64_t max_seq_len = 4096;
    int64_t ffn_hidden_dim = 0;     // 0 = 8/3 * dim rounded up to ffn_multiple_of
    int64_t ffn_multiple_of = 256;
    float norm_eps = 1e-5f;
    bool use_rms_norm = true;       // only the RMSNorm / RoPE / SwiGLU family is built here
    float rope_base = 10000.0f;
    bool tie_word_embeddings = false;
    bool use_bias = false;

    int64_t head_dim() const { return dim / n_heads; }
    int64_t kv_heads() const { return n_kv_heads > 0 ? n_kv_heads : n_heads; }
    bool uses_gqa() const { return kv_heads() < n_heads; }
    bool uses_rope() const { return rope_base > 0; }
    // SwiGLUMLP::compute_hidden_dim (src/nn/swiglu.cpp:50-61)
    int64_t hidden_dim() const {
        if (ffn_hidden_dim > 0) return ffn_hidden_dim;
        int64_t h = (8 * dim) / 3;
        if (ffn_multiple_of > 1) h = ((h + ffn_multiple_of - 1) / ffn_multiple_of) * ffn_multiple_of;
        return h;
    }
};

}  // namespace vesper::models
