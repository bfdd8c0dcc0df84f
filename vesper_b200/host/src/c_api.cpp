// extern "C" facade over models::TransformerLM and generation::Generator for harnesses that
// cannot include C++ headers (the Python tests and the benchmark bind it with ctypes).  Host
// arrays in, host arrays out; errors come back as -1 with the text in vbh_last_error().
#include <vesper/generation/generator.h>
#include <vesper/models/transformer.h>
#include <vesper/nn/gqa_attention.h>

#include <cstring>
#include <string>

using vesper::Device;
using vesper::DType;
using vesper::Tensor;
using vesper::models::TransformerConfig;
using vesper::models::TransformerLM;

namespace {
thread_local std::string g_err;
Tensor ids_to_device(const int32_t* ids, int64_t B, int64_t T) {
    Tensor t = vesper::empty({B, T}, DType::Int32, Device::CUDA);
    t.copy_from_host(ids);
    return t;
}
// host fp32 <-> device tensor of the module's dtype
Tensor act_to_device(const float* x, const std::vector<int64_t>& shape, DType dt) {
    Tensor t = vesper::empty(shape, dt, Device::CUDA);
    if (dt == DType::Float32) { t.copy_from_host(x); return t; }
    std::vector<uint16_t> h(t.numel());
    for (size_t i = 0; i < h.size(); ++i) h[i] = vesper::float_to_bf16(x[i]);
    t.copy_from_host(h.data());
    return t;
}
void act_to_host(const Tensor& y, float* out) {
    Tensor c = y.is_contiguous() ? y : y.contiguous();
    if (c.dtype() == DType::Float32) { c.copy_to_host(out); return; }
    std::vector<uint16_t> h(c.numel());
    c.copy_to_host(h.data());
    for (size_t i = 0; i < h.size(); ++i) out[i] = vesper::bf16_to_float(h[i]);
}
struct AttnModule {
    std::unique_ptr<vesper::nn::GroupedQueryAttention> gqa;
    std::unique_ptr<vesper::nn::MultiHeadAttention> mha;
    DType dt;
};
}  // namespace

extern "C" {

// ---- nn::GroupedQueryAttention / nn::MultiHeadAttention / nn::KVCache ----
// kind 0: GroupedQueryAttention(embed_dim, num_heads, num_kv_heads, max_seq_len, rope_base, 0, bias);
// kind 1: MultiHeadAttention(embed_dim, num_heads, 0, use_rope).  dtype 0 = Float32, 1 = BFloat16.
void* vbh_attn_new(int kind, int64_t embed_dim, int64_t num_heads, int64_t num_kv_heads, int64_t max_seq_len, float rope_base,
                   int bias, int use_rope, int dtype) {
    try {
        auto m = std::make_unique<AttnModule>();
        m->dt = dtype == 0 ? DType::Float32 : DType::BFloat16;
        if (kind == 0) m->gqa = std::make_unique<vesper::nn::GroupedQueryAttention>(embed_dim, num_heads, num_kv_heads, max_seq_len, rope_base, 0.0f, bias != 0, m->dt);
        else m->mha = std::make_unique<vesper::nn::MultiHeadAttention>(static_cast<int>(embed_dim), static_cast<int>(num_heads), 0.0f, use_rope != 0, m->dt);
        return m.release();
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void vbh_attn_free(void* m) { delete static_cast<AttnModule*>(m); }
// host fp32 weights in the reference's layouts: input projection [out, in] (+ bias [out], nullable), output projection
int vbh_attn_load(void* h, const float* w_in, const float* b_in, const float* w_out, const float* b_out) {
    try {
        auto* m = static_cast<AttnModule*>(h);
        if (m->gqa) { m->gqa->wqkv().load_weight(w_in, b_in); m->gqa->wo().load_weight(w_out, b_out); }
        else { m->mha->c_attn.load_weight(w_in, b_in); m->mha->c_proj.load_weight(w_out, b_out); }
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
void* vbh_kvcache_new(int64_t B, int64_t H, int64_t max_seq_len, int64_t D, int dtype) {
    try {
        return new vesper::nn::KVCache(static_cast<int>(B), static_cast<int>(H), static_cast<int>(max_seq_len), static_cast<int>(D), Device::CUDA,
                                       dtype == 0 ? DType::Float32 : DType::BFloat16);
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void vbh_kvcache_free(void* c) { delete static_cast<vesper::nn::KVCache*>(c); }
int vbh_kvcache_len(void* c) { return static_cast<vesper::nn::KVCache*>(c)->current_seq_len(); }
// mode 0: forward(x); 1: forward(x, causal); 2: forward(x, cache, start_pos).  x, y: host fp32 [B, T, embed_dim].
int vbh_attn_forward(void* h, const float* x_host, int64_t B, int64_t T, int64_t C, int mode, int causal, void* cache, int64_t start_pos,
                     float* y_host) {
    try {
        auto* m = static_cast<AttnModule*>(h);
        Tensor x = act_to_device(x_host, {B, T, C}, m->dt);
        auto* kc = static_cast<vesper::nn::KVCache*>(cache);
        Tensor y;
        if (m->gqa) y = mode == 0 ? m->gqa->forward(x) : mode == 1 ? m->gqa->forward(x, causal != 0) : m->gqa->forward(x, kc, start_pos);
        else y = mode == 0 ? m->mha->forward(x) : mode == 1 ? m->mha->forward(x, causal != 0) : m->mha->forward(x, kc, static_cast<int>(start_pos));
        act_to_host(y, y_host);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

const char* vbh_last_error() { return g_err.c_str(); }

void* vbh_model_new(int64_t vocab, int64_t dim, int64_t n_layers, int64_t n_heads, int64_t n_kv_heads,
                    int64_t ffn_hidden, int64_t max_seq_len, float norm_eps, float rope_base) {
    try {
        TransformerConfig c;
        c.vocab_size = vocab; c.dim = dim; c.n_layers = n_layers; c.n_heads = n_heads; c.n_kv_heads = n_kv_heads;
        c.ffn_hidden_dim = ffn_hidden; c.max_seq_len = max_seq_len; c.norm_eps = norm_eps; c.rope_base = rope_base;
        return new TransformerLM(c);
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void vbh_model_free(void* m) { delete static_cast<TransformerLM*>(m); }

int vbh_model_set_param(void* m, const char* name, const float* data, int64_t numel) {
    try { static_cast<TransformerLM*>(m)->load_parameter(name, data, numel); return 0; }
    catch (const std::exception& e) { g_err = e.what(); return -1; }
}
int vbh_model_init_cache(void* m, int64_t B) {
    try { static_cast<TransformerLM*>(m)->init_cache(B, Device::CUDA); return 0; }
    catch (const std::exception& e) { g_err = e.what(); return -1; }
}
// logits_host: [B, T, vocab] fp32, or [B, 1, vocab] when last_only
int vbh_model_forward_with_cache(void* m, const int32_t* ids_host, int64_t B, int64_t T, int64_t start_pos,
                                 int last_only, float* logits_host) {
    try {
        Tensor y = static_cast<TransformerLM*>(m)->forward_with_cache(ids_to_device(ids_host, B, T), start_pos, last_only != 0);
        y.copy_to_host(logits_host);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
// out_host: [B, P + max_new] int32; returns the number of columns written.  timings (nullable):
// {prefill_ms, decode_ms, decode_steps, graph_replay}.
int64_t vbh_generate_greedy(void* m, const int32_t* prompt_host, int64_t B, int64_t P, int64_t max_new,
                            const int64_t* stop_ids, int64_t n_stop, int64_t min_new, int use_graph,
                            int32_t* out_host, double* timings) {
    try {
        vesper::generation::Generator gen(static_cast<TransformerLM*>(m));
        gen.set_use_graph(use_graph != 0);
        vesper::generation::SamplingParams sp;
        sp.do_sample = false;
        sp.max_new_tokens = max_new;
        sp.min_new_tokens = min_new;
        for (int64_t i = 0; i < n_stop; ++i) sp.stop_token_ids.push_back(stop_ids[i]);
        Tensor r = gen.generate(ids_to_device(prompt_host, B, P), sp);
        r.copy_to_host(out_host);
        if (timings) {
            const auto& t = gen.last_timings();
            timings[0] = t.prefill_ms; timings[1] = t.decode_ms;
            timings[2] = static_cast<double>(t.decode_steps); timings[3] = t.graph_replay ? 1.0 : 0.0;
        }
        return r.shape()[1];
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

}  // extern "C"
