// extern "C" facade over models::TransformerLM and generation::Generator for harnesses that
// cannot include C++ headers (the Python tests and the benchmark bind it with ctypes).  Host
// arrays in, host arrays out; errors come back as -1 with the text in vbh_last_error().
#include <vesper/generation/generator.h>
#include <vesper/models/transformer.h>

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
}  // namespace

extern "C" {

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
