// extern "C" shim over the UNMODIFIED reference CPU implementation -- TEST
// INFRASTRUCTURE ONLY.  Compiled by oracle/Makefile together with the
// reference's own sources (read where they lie, never copied) into
// oracle/_ref/libvesper_ref.so.  It is used to (1) generate the golden vectors
// under tests/golden, (2) validate the plain-C restatement in
// vesper_attn_oracle.c, and (3) serve as the timed CPU baseline.
//
// Each entry point takes raw host fp32 buffers, wraps them in reference
// Tensors and calls the reference's public functions:
//   ops::flash_attention_cpu_dispatch          include/vesper/ops/flash_attention.h:88-92
//   nn::functional::scaled_dot_product_attention  include/vesper/nn/functional.h:132-136
//   nn::functional::compute_rope_frequencies / apply_rotary_emb  :148-154
//   ops::repeat_kv                             include/vesper/ops/attention_ops.h:21
//   nn::KVCache                                include/vesper/nn/transformer.h:21-39
//   nn::GroupedQueryAttention / MultiHeadAttention forward
#include <vesper/core/tensor.h>
#include <vesper/core/factories.h>
#include <vesper/core/slice.h>
#include <vesper/ops/flash_attention.h>
#include <vesper/ops/attention_ops.h>
#include <vesper/ops/random.h>
#include <vesper/nn/functional.h>
#include <vesper/nn/transformer.h>
#include <vesper/nn/gqa_attention.h>
#include <vesper/autograd/guard.h>
#include <vesper/ops/gemm.h>
#include <vesper/ops/normalization.h>
#include <vesper/ops/elementwise.h>
#include <vesper/ops/embedding.h>
#include <vesper/ops/sampling_ops.h>
#include <vesper/models/transformer.h>
#include <vesper/generation/generator.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

using vesper::Tensor;
using vesper::DType;
using vesper::Device;

namespace {

Tensor from_host(const float* p, std::vector<int64_t> shape) {
    Tensor t = vesper::empty(shape, DType::Float32, Device::CPU);
    t.copy_from_host(p);
    return t;
}

void to_host(const Tensor& t, float* p) {
    Tensor c = t.is_contiguous() ? t : t.contiguous();
    c.copy_to_host(p);
}

thread_local std::string g_err;

}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// vesper::randn after ops::manual_seed(seed): std::mt19937 + normal_distribution<float>
// (src/ops/random.cpp:54-95).
int ref_randn(uint64_t seed, int64_t n, float* out) {
    try {
        vesper::ops::manual_seed(seed);
        Tensor t = vesper::randn({n}, DType::Float32, Device::CPU);
        to_host(t, out);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// Several randn calls in sequence after one manual_seed (q, then k, then v).
int ref_randn_seq(uint64_t seed, int count, const int64_t* sizes, float** outs) {
    try {
        vesper::ops::manual_seed(seed);
        for (int i = 0; i < count; ++i) {
            Tensor t = vesper::randn({sizes[i]}, DType::Float32, Device::CPU);
            to_host(t, outs[i]);
        }
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

int ref_flash_attention(const float* q, const float* k, const float* v, float* o, float* lse,
                        int64_t B, int64_t H, int64_t N, int64_t D, float scale, int causal) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor tq = from_host(q, {B, H, N, D}), tk = from_host(k, {B, H, N, D}), tv = from_host(v, {B, H, N, D});
        Tensor to = vesper::empty({B, H, N, D}, DType::Float32, Device::CPU);
        Tensor tl = vesper::empty({B, H, N}, DType::Float32, Device::CPU);
        vesper::ops::flash_attention_cpu_dispatch(tq, tk, tv, to, tl, scale, causal != 0, 0.0f, false, nullptr);
        to_host(to, o);
        if (lse) to_host(tl, lse);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// Public op (router included): ops::flash_attention(q,k,v,scale,causal).
int ref_flash_attention_op(const float* q, const float* k, const float* v, float* o,
                           int64_t B, int64_t H, int64_t N, int64_t D, float scale, int causal) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor tq = from_host(q, {B, H, N, D}), tk = from_host(k, {B, H, N, D}), tv = from_host(v, {B, H, N, D});
        Tensor to = vesper::ops::flash_attention(tq, tk, tv, scale, causal != 0);
        to_host(to, o);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

int ref_sdpa(const float* q, const float* k, const float* v, float* out,
             int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t D, int causal) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor tq = from_host(q, {B, H, Tq, D}), tk = from_host(k, {B, H, Tk, D}), tv = from_host(v, {B, H, Tk, D});
        Tensor to = vesper::nn::functional::scaled_dot_product_attention(tq, tk, tv, causal != 0, 0.0);
        to_host(to, out);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

int ref_rope_frequencies(int T, int D, int start_pos, float theta, float* freqs) {
    try {
        Tensor f = vesper::nn::functional::compute_rope_frequencies(T, D, start_pos, theta, Device::CPU);
        to_host(f, freqs);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

int ref_apply_rope(const float* x, float* out, int64_t B, int64_t H, int64_t S, int64_t D,
                   int start_pos, float theta) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor tx = from_host(x, {B, H, S, D});
        Tensor f = vesper::nn::functional::compute_rope_frequencies((int)S, (int)D, start_pos, theta, Device::CPU);
        Tensor r = vesper::nn::functional::apply_rotary_emb(tx, f);
        to_host(r, out);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

int ref_repeat_kv(const float* in, float* out, int64_t B, int64_t KVH, int64_t S, int64_t D, int64_t n_rep) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor ti = from_host(in, {B, KVH, S, D});
        Tensor r = vesper::ops::repeat_kv(ti, n_rep);
        to_host(r, out);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// ---- nn::KVCache as an opaque handle ----
void* ref_kvcache_new(int B, int H, int cap, int D) {
    try { return new vesper::nn::KVCache(B, H, cap, D, Device::CPU); }
    catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void ref_kvcache_free(void* h) { delete static_cast<vesper::nn::KVCache*>(h); }
int ref_kvcache_len(void* h) { return static_cast<vesper::nn::KVCache*>(h)->current_seq_len(); }
int ref_kvcache_reset(void* h) {
    try { static_cast<vesper::nn::KVCache*>(h)->reset(); return 0; }
    catch (const std::exception& e) { g_err = e.what(); return -1; }
}
// update(new_k,new_v,start_pos); k_out/v_out (nullable) receive the returned
// views [:,:,0:len,:] made contiguous: [B,H,len,D].
int ref_kvcache_update(void* h, const float* new_k, const float* new_v,
                       int64_t B, int64_t H, int64_t T, int64_t D, int start_pos,
                       float* k_out, float* v_out) {
    try {
        vesper::autograd::NoGradGuard ng;
        auto* c = static_cast<vesper::nn::KVCache*>(h);
        Tensor tk = from_host(new_k, {B, H, T, D}), tv = from_host(new_v, {B, H, T, D});
        auto kv = c->update(tk, tv, start_pos);
        if (k_out) to_host(kv.first, k_out);
        if (v_out) to_host(kv.second, v_out);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// The attention core of GroupedQueryAttention::forward(x, cache, start_pos)
// (src/nn/gqa_attention.cpp:111-159, steps 2-6) composed from the reference's
// own ops, with .contiguous() on the cache views before ops::repeat_kv (the
// reference dispatcher ignores the views' strides).  T>1 requires start_pos==0
// here (the reference cannot express anything else).
int ref_gqa_attention_cached(void* cache, const float* q, const float* k_new, const float* v_new,
                             float* out, int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t D,
                             int start_pos, float theta, int use_rope) {
    try {
        vesper::autograd::NoGradGuard ng;
        namespace F = vesper::nn::functional;
        auto* c = static_cast<vesper::nn::KVCache*>(cache);
        Tensor tq = from_host(q, {B, Hq, T, D}), tk = from_host(k_new, {B, Hkv, T, D}), tv = from_host(v_new, {B, Hkv, T, D});
        if (use_rope) {
            Tensor f = F::compute_rope_frequencies((int)T, (int)D, start_pos, theta, Device::CPU);
            tq = F::apply_rotary_emb(tq, f);
            tk = F::apply_rotary_emb(tk, f);
        }
        auto kv = c->update(tk, tv, start_pos);
        Tensor k = kv.first.contiguous(), v = kv.second.contiguous();
        int64_t n_rep = Hq / Hkv;
        k = vesper::ops::repeat_kv(k, n_rep);
        v = vesper::ops::repeat_kv(v, n_rep);
        Tensor o = F::scaled_dot_product_attention(tq, k, v, T > 1, 0.0);
        to_host(o, out);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// ---- module level: GroupedQueryAttention with caller-supplied weights ----
// wqkv: [(Hq+2Hkv)*D, C] row-major (Linear weight layout [out,in]), wo: [C, Hq*D].
void* ref_gqa_new(int64_t C, int64_t Hq, int64_t Hkv, int64_t max_seq, float theta,
                  const float* wqkv, const float* wo) {
    try {
        auto* m = new vesper::nn::GroupedQueryAttention(C, Hq, Hkv, max_seq, theta, 0.0f, false);
        m->eval();
        auto params = m->named_parameters_ptrs();
        for (auto& kv : params) {
            if (kv.first.find("wqkv") != std::string::npos && kv.first.find("weight") != std::string::npos)
                kv.second->copy_from_host(wqkv);
            else if (kv.first.find("wo") != std::string::npos && kv.first.find("weight") != std::string::npos)
                kv.second->copy_from_host(wo);
        }
        return m;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void ref_gqa_free(void* m) { delete static_cast<vesper::nn::GroupedQueryAttention*>(m); }
// forward(x, causal) -- the uncached path, numerically right for any n_rep.
int ref_gqa_forward(void* m, const float* x, float* y, int64_t B, int64_t T, int64_t C, int causal) {
    try {
        vesper::autograd::NoGradGuard ng;
        auto* g = static_cast<vesper::nn::GroupedQueryAttention*>(m);
        Tensor tx = from_host(x, {B, T, C});
        Tensor ty = g->forward(tx, causal != 0);
        to_host(ty, y);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
// forward(x, cache, start_pos) exactly as the reference runs it (including its
// strided repeat_kv defect when n_rep>1).
int ref_gqa_forward_cached(void* m, void* cache, const float* x, float* y,
                           int64_t B, int64_t T, int64_t C, int64_t start_pos) {
    try {
        vesper::autograd::NoGradGuard ng;
        auto* g = static_cast<vesper::nn::GroupedQueryAttention*>(m);
        Tensor tx = from_host(x, {B, T, C});
        Tensor ty = g->forward(tx, static_cast<vesper::nn::KVCache*>(cache), start_pos);
        to_host(ty, y);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// ---- module level: MultiHeadAttention (src/nn/transformer.cpp:97-216) with caller-supplied weights ----
// c_attn: weight [3C, C] + bias [3C]; c_proj: weight [C, C] + bias [C].
void* ref_mha_new(int C, int H, int use_rope, const float* w_attn, const float* b_attn, const float* w_proj, const float* b_proj) {
    try {
        auto* m = new vesper::nn::MultiHeadAttention(C, H, 0.0f, use_rope != 0);
        m->eval();
        m->c_attn.weight.copy_from_host(w_attn);
        m->c_attn.bias.copy_from_host(b_attn);
        m->c_proj.weight.copy_from_host(w_proj);
        m->c_proj.bias.copy_from_host(b_proj);
        return m;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void ref_mha_free(void* m) { delete static_cast<vesper::nn::MultiHeadAttention*>(m); }
// mode 0: forward(x) (non-causal by default, :108-110); 1: forward(x, causal); 2: forward(x, cache, start_pos)
int ref_mha_forward(void* m, const float* x, float* y, int64_t B, int64_t T, int64_t C, int mode, int causal, void* cache, int start_pos) {
    try {
        vesper::autograd::NoGradGuard ng;
        auto* g = static_cast<vesper::nn::MultiHeadAttention*>(m);
        Tensor tx = from_host(x, {B, T, C});
        Tensor ty = mode == 0 ? g->forward(tx) : mode == 1 ? g->forward(tx, causal != 0)
                                                           : g->forward(tx, static_cast<vesper::nn::KVCache*>(cache), start_pos);
        to_host(ty, y);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// ops::flash_attention_backward (src/ops/flash_attention.cpp:165-215 -> CPU backward :366-482)
int ref_flash_attention_backward(const float* d_out, const float* q, const float* k, const float* v,
                                 const float* out, const float* lse, float* dq, float* dk, float* dv,
                                 int64_t B, int64_t H, int64_t N, int64_t D, float scale, int causal) {
    try {
        vesper::autograd::NoGradGuard ng;
        std::vector<int64_t> sh = {B, H, N, D};
        auto g = vesper::ops::flash_attention_backward(from_host(d_out, sh), from_host(q, sh), from_host(k, sh), from_host(v, sh),
                                                       from_host(out, sh), from_host(lse, {B, H, N}), scale, causal != 0, 0.0f, Tensor());
        to_host(std::get<0>(g), dq);
        to_host(std::get<1>(g), dk);
        to_host(std::get<2>(g), dv);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// ---- decoder-block operators --------------------------------------------------------------
// y[M,N] = x[M,K] w[N,K]^T exactly as nn::Linear::forward does it: matmul(x, weight.transpose(0,1))
// (src/nn/linear.cpp:41-48).
int ref_linear(const float* x, const float* w, float* y, int64_t M, int64_t N, int64_t K) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor tx = from_host(x, {M, K}), tw = from_host(w, {N, K});
        Tensor ty = vesper::ops::matmul(tx, tw.transpose(0, 1));
        to_host(ty, y);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
int ref_rms_norm(const float* x, const float* w, float* y, int64_t M, int64_t dim, float eps) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor ty = vesper::ops::rms_norm(from_host(x, {M, dim}), {dim}, from_host(w, {dim}), eps);
        to_host(ty, y);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
int ref_silu_mul(const float* gate, const float* up, float* y, int64_t n) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor ty = vesper::ops::silu_mul(from_host(gate, {n}), from_host(up, {n}));
        to_host(ty, y);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
int ref_embedding(const int32_t* ids, const float* table, float* y, int64_t M, int64_t vocab, int64_t dim) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor ti = vesper::empty({M}, DType::Int32, Device::CPU);
        std::memcpy(ti.data_ptr<int32_t>(), ids, sizeof(int32_t) * M);
        Tensor ty = vesper::ops::embedding(ti, from_host(table, {vocab, dim}));
        to_host(ty, y);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
int ref_argmax(const float* logits, int32_t* out, int64_t B, int64_t vocab) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor t = vesper::ops::argmax(from_host(logits, {B, vocab}), -1);
        std::memcpy(out, t.data_ptr<int32_t>(), sizeof(int32_t) * B);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

// ---- model level: models::TransformerLM with caller-supplied weights ----------------------
void* ref_model_new(int64_t vocab, int64_t dim, int64_t n_layers, int64_t n_heads, int64_t n_kv_heads,
                    int64_t ffn_hidden, int64_t max_seq_len, float norm_eps, float rope_base) {
    try {
        vesper::models::TransformerConfig c;
        c.vocab_size = vocab; c.dim = dim; c.n_layers = n_layers; c.n_heads = n_heads; c.n_kv_heads = n_kv_heads;
        c.ffn_hidden_dim = ffn_hidden; c.max_seq_len = max_seq_len; c.norm_eps = norm_eps; c.use_rms_norm = true;
        c.rope_base = rope_base; c.use_bias = false; c.tie_word_embeddings = false; c.dropout = 0.0f;
        auto* m = new vesper::models::TransformerLM(c);
        m->eval();
        return m;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void ref_model_free(void* m) { delete static_cast<vesper::models::TransformerLM*>(m); }
// Parameter names, one per line as "name d0 d1 ...", into buf; returns the length needed.
int64_t ref_model_param_names(void* m, char* buf, int64_t buflen) {
    std::string out;
    for (auto& kv : static_cast<vesper::models::TransformerLM*>(m)->named_parameters_ptrs()) {
        out += kv.first;
        for (auto d : kv.second->shape()) out += " " + std::to_string(d);
        out += "\n";
    }
    if (buf && buflen > 0) {
        const int64_t n = std::min<int64_t>(buflen - 1, static_cast<int64_t>(out.size()));
        std::memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    return static_cast<int64_t>(out.size()) + 1;
}
int ref_model_set_param(void* m, const char* name, const float* data, int64_t numel) {
    try {
        auto params = static_cast<vesper::models::TransformerLM*>(m)->named_parameters_ptrs();
        auto it = params.find(name);
        if (it == params.end()) { g_err = std::string("no parameter ") + name; return -1; }
        if (it->second->numel() != numel) { g_err = std::string("size mismatch for ") + name; return -1; }
        it->second->copy_from_host(data);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
static Tensor ids_tensor(const int32_t* ids, int64_t B, int64_t T) {
    Tensor t = vesper::empty({B, T}, DType::Int32, Device::CPU);
    std::memcpy(t.data_ptr<int32_t>(), ids, sizeof(int32_t) * B * T);
    return t;
}
// TransformerLM::forward (uncached, causal): logits [B,T,vocab]  (src/models/transformer.cpp:97-150)
int ref_model_forward(void* m, const int32_t* ids, int64_t B, int64_t T, float* logits) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor y = static_cast<vesper::models::TransformerLM*>(m)->forward(ids_tensor(ids, B, T));
        to_host(y, logits);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
int ref_model_init_cache(void* m, int64_t B) {
    try { static_cast<vesper::models::TransformerLM*>(m)->init_cache(B, Device::CPU); return 0; }
    catch (const std::exception& e) { g_err = e.what(); return -1; }
}
// TransformerLM::forward_with_cache (src/models/transformer.cpp:152-188): logits [B,T,vocab]
int ref_model_forward_with_cache(void* m, const int32_t* ids, int64_t B, int64_t T, int64_t start_pos, float* logits) {
    try {
        vesper::autograd::NoGradGuard ng;
        Tensor y = static_cast<vesper::models::TransformerLM*>(m)->forward_with_cache(ids_tensor(ids, B, T), start_pos);
        to_host(y, logits);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}
// generation::Generator::generate with greedy sampling (src/generation/generator.cpp:36-142):
// out [B, P + max_new] int32; returns the number of columns written or -1.
int64_t ref_generate_greedy(void* m, const int32_t* prompt, int64_t B, int64_t P, int64_t max_new,
                            const int64_t* stop_ids, int64_t n_stop, int64_t min_new, int32_t* out) {
    try {
        vesper::autograd::NoGradGuard ng;
        vesper::generation::Generator gen(static_cast<vesper::models::TransformerLM*>(m));
        vesper::generation::SamplingParams sp;
        sp.do_sample = false; sp.max_new_tokens = max_new; sp.min_new_tokens = min_new;
        for (int64_t i = 0; i < n_stop; ++i) sp.stop_token_ids.push_back(stop_ids[i]);
        Tensor r = gen.generate(ids_tensor(prompt, B, P), sp);
        Tensor rc = r.is_contiguous() ? r : r.contiguous();
        const int64_t cols = rc.shape()[1];
        if (rc.dtype() == DType::Int32) {
            std::memcpy(out, rc.data_ptr<int32_t>(), sizeof(int32_t) * B * cols);
        } else if (rc.dtype() == DType::Int64) {
            const int64_t* p = rc.data_ptr<int64_t>();
            for (int64_t i = 0; i < B * cols; ++i) out[i] = static_cast<int32_t>(p[i]);
        } else { g_err = "generate returned an unexpected dtype"; return -1; }
        return cols;
    } catch (const std::exception& e) { g_err = e.what(); return -1; }
}

}  // extern "C"
