// models::TransformerLM on the B200 operators: every step of the decoder is one C-ABI call of
// libvesper_b200 (vesper_b200.h for attention, vesper_b200_block.h for the rest).  Nothing here
// computes on the host.
#include <vesper/models/transformer.h>

#include <vesper_b200.h>
#include <vesper_b200_block.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>

namespace vesper::models {

namespace {

void check(int rc, const char* who) {
    if (rc != VB200_OK)
        throw std::runtime_error(std::string(who) + ": " + vb200_strerror(rc) + ": " + vb200_last_error_detail());
}
void* current_stream() { return Stream::current(Device::CUDA).raw_handle(); }

Tensor bf16_from_host(const float* src, const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    std::vector<uint16_t> tmp(static_cast<size_t>(n));
    for (int64_t i = 0; i < n; ++i) tmp[static_cast<size_t>(i)] = float_to_bf16(src[i]);
    Tensor t = empty(shape, DType::BFloat16, Device::CUDA);
    t.copy_from_host(tmp.data());
    return t;
}

}  // namespace

struct TransformerLM::Layer {
    Tensor attn_norm, ffn_norm;        // [dim] fp32
    Tensor wqkv;                       // [(Hq + 2 Hkv) * D, dim] bf16
    Tensor wo;                         // [dim, Hq * D] bf16
    Tensor w13;                        // [2 * hidden, dim] bf16, row 2j = gate_j, row 2j+1 = up_j
    Tensor w2;                         // [dim, hidden] bf16
    Tensor gate_tmp, up_tmp;           // held until both halves of w13 have been loaded
};

// Activations, sized for the largest (rows, batch) seen so far; allocated outside any graph capture.
struct TransformerLM::Buffers {
    int64_t rows = 0, batch = 0;
    Tensor h;          // [rows, dim] fp32 residual stream
    Tensor xn;         // [rows, dim] bf16: the residual stream times the weight of the norm that comes next (its 1/rms is applied by the consuming GEMM)
    Tensor inv;        // [rows] fp32: 1/rms of the residual rows (prompt passes; decode steps compute it inside the GEMM)
    Tensor qkv;        // [rows, (Hq + 2 Hkv) * D] bf16
    Tensor attn;       // [rows, Hq * D] bf16, heads merged
    Tensor act;        // [rows, hidden] bf16
    Tensor logits;     // [logit_rows, vocab] fp32
    Tensor attn_ws;    // attention workspace (angle table / split-KV partials)
    int64_t logit_rows = 0;
};

TransformerLM::TransformerLM(const TransformerConfig& config) : config_(config) {
    if (!config.use_rms_norm || !config.uses_rope() || config.use_bias || config.tie_word_embeddings)
        throw std::runtime_error("TransformerLM: this backend builds the RMSNorm + RoPE + SwiGLU family without bias or tied embeddings");
    if (config.dim % config.n_heads != 0) throw std::runtime_error("TransformerLM: dim must be divisible by n_heads");
    if (config.n_heads % config.kv_heads() != 0)
        throw std::invalid_argument("GroupedQueryAttention: num_heads must be divisible by num_kv_heads");
    if (config.head_dim() != 128 && config.head_dim() != 64)
        throw std::runtime_error("TransformerLM: head_dim must be 64 or 128 for the 16-bit attention kernels");
    if (config.dim % 8 != 0 || config.hidden_dim() % 8 != 0) throw std::runtime_error("TransformerLM: dim and ffn hidden size must be multiples of 8");
    vb200_rope_inv_freq(config.rope_base, static_cast<int>(config.head_dim()), inv_freq_);
    const int64_t dim = config.dim, hid = config.hidden_dim();
    const int64_t qkv_n = (config.n_heads + 2 * config.kv_heads()) * config.head_dim();
    tok_emb_ = zeros({config.vocab_size, dim}, DType::BFloat16, Device::CUDA);
    lm_head_ = zeros({config.vocab_size, dim}, DType::BFloat16, Device::CUDA);
    std::vector<float> ones(static_cast<size_t>(dim), 1.0f);
    final_norm_ = empty({dim}, DType::Float32, Device::CUDA);
    final_norm_.copy_from_host(ones.data());
    for (int64_t l = 0; l < config.n_layers; ++l) {
        auto L = std::make_unique<Layer>();
        L->attn_norm = empty({dim}, DType::Float32, Device::CUDA);
        L->attn_norm.copy_from_host(ones.data());
        L->ffn_norm = empty({dim}, DType::Float32, Device::CUDA);
        L->ffn_norm.copy_from_host(ones.data());
        L->wqkv = zeros({qkv_n, dim}, DType::BFloat16, Device::CUDA);
        L->wo = zeros({dim, config.n_heads * config.head_dim()}, DType::BFloat16, Device::CUDA);
        L->w13 = zeros({2 * hid, dim}, DType::BFloat16, Device::CUDA);
        L->w2 = zeros({dim, hid}, DType::BFloat16, Device::CUDA);
        layers_.push_back(std::move(L));
    }
    buf_ = std::make_unique<Buffers>();
}

TransformerLM::~TransformerLM() = default;

std::map<std::string, std::vector<int64_t>> TransformerLM::parameter_shapes() const {
    const int64_t dim = config_.dim, hid = config_.hidden_dim();
    const int64_t qkv_n = (config_.n_heads + 2 * config_.kv_heads()) * config_.head_dim();
    std::map<std::string, std::vector<int64_t>> m;
    m["tok_embeddings.weight"] = {config_.vocab_size, dim};
    m["norm.weight"] = {dim};
    m["output.weight"] = {config_.vocab_size, dim};
    for (int64_t l = 0; l < config_.n_layers; ++l) {
        const std::string p = "layers." + std::to_string(l) + ".";
        m[p + "attention_norm.weight"] = {dim};
        m[p + "attention.wqkv.weight"] = {qkv_n, dim};
        m[p + "attention.wo.weight"] = {dim, config_.n_heads * config_.head_dim()};
        m[p + "ffn_norm.weight"] = {dim};
        m[p + "feed_forward.gate_proj.weight"] = {hid, dim};
        m[p + "feed_forward.up_proj.weight"] = {hid, dim};
        m[p + "feed_forward.down_proj.weight"] = {dim, hid};
    }
    return m;
}

int64_t TransformerLM::num_parameters() const {
    int64_t n = 0;
    for (auto& kv : parameter_shapes()) {
        int64_t c = 1;
        for (auto d : kv.second) c *= d;
        n += c;
    }
    return n;
}

void TransformerLM::load_parameter(const std::string& name, const float* host_values, int64_t numel) {
    auto shapes = parameter_shapes();
    auto it = shapes.find(name);
    if (it == shapes.end()) throw std::runtime_error("TransformerLM::load_parameter: no parameter named " + name);
    int64_t want = 1;
    for (auto d : it->second) want *= d;
    if (want != numel) throw std::runtime_error("TransformerLM::load_parameter: size mismatch for " + name);
    auto load_f32 = [&](Tensor& dst) { dst.copy_from_host(host_values); };
    if (name == "tok_embeddings.weight") { tok_emb_ = bf16_from_host(host_values, it->second); return; }
    if (name == "output.weight") { lm_head_ = bf16_from_host(host_values, it->second); return; }
    if (name == "norm.weight") { load_f32(final_norm_); return; }
    // layers.N.<rest>
    const size_t dot = name.find('.', 7);
    const int64_t l = std::stoll(name.substr(7, dot - 7));
    const std::string rest = name.substr(dot + 1);
    Layer& L = *layers_.at(static_cast<size_t>(l));
    if (rest == "attention_norm.weight") load_f32(L.attn_norm);
    else if (rest == "ffn_norm.weight") load_f32(L.ffn_norm);
    else if (rest == "attention.wqkv.weight") L.wqkv = bf16_from_host(host_values, it->second);
    else if (rest == "attention.wo.weight") L.wo = bf16_from_host(host_values, it->second);
    else if (rest == "feed_forward.down_proj.weight") L.w2 = bf16_from_host(host_values, it->second);
    else {
        if (rest == "feed_forward.gate_proj.weight") L.gate_tmp = bf16_from_host(host_values, it->second);
        else L.up_tmp = bf16_from_host(host_values, it->second);
        if (L.gate_tmp.defined() && L.up_tmp.defined()) {
            check(vb200_interleave_rows(L.w13.device_index(), current_stream(), L.gate_tmp.data_ptr<char>(), L.up_tmp.data_ptr<char>(),
                                        L.w13.data_ptr<char>(), config_.hidden_dim(), config_.dim),
                  "TransformerLM::load_parameter");
            Stream::current(Device::CUDA).synchronize();
            L.gate_tmp = Tensor();
            L.up_tmp = Tensor();
        }
    }
}

void TransformerLM::init_cache(int64_t batch_size, Device device) {
    if (device != Device::CUDA) throw std::runtime_error("TransformerLM::init_cache: this library is the CUDA backend");
    kv_caches_.clear();
    for (int64_t i = 0; i < config_.n_layers; ++i)
        kv_caches_.push_back(std::make_unique<nn::KVCache>(static_cast<int>(batch_size), static_cast<int>(config_.kv_heads()),
                                                           static_cast<int>(config_.max_seq_len), static_cast<int>(config_.head_dim()),
                                                           device, DType::BFloat16));
}

void TransformerLM::clear_cache() { kv_caches_.clear(); }

void TransformerLM::ensure_buffers(int64_t rows, int64_t batch) {
    Buffers& b = *buf_;
    if (rows <= b.rows && batch <= b.batch) return;
    rows = std::max(rows, b.rows);
    batch = std::max(batch, b.batch);
    const int64_t dim = config_.dim, hid = config_.hidden_dim(), D = config_.head_dim();
    const int64_t qkv_n = (config_.n_heads + 2 * config_.kv_heads()) * D;
    b.h = empty({rows, dim}, DType::Float32, Device::CUDA);
    b.xn = empty({rows, dim}, DType::BFloat16, Device::CUDA);
    b.inv = empty({rows}, DType::Float32, Device::CUDA);
    b.qkv = empty({rows, qkv_n}, DType::BFloat16, Device::CUDA);
    b.attn = empty({rows, config_.n_heads * D}, DType::BFloat16, Device::CUDA);
    b.act = empty({rows, hid}, DType::BFloat16, Device::CUDA);
    // attention workspace: the larger of the prompt pass's angle table and the split-KV partials of the
    // most demanding decode step the cache capacity allows
    vb200_prefill_args pa{};
    pa.struct_size = sizeof(pa);
    pa.dtype = VB200_BF16;
    pa.B = static_cast<int>(batch); pa.Hq = static_cast<int>(config_.n_heads); pa.Hkv = static_cast<int>(config_.kv_heads());
    pa.T = static_cast<int>(std::max<int64_t>(1, rows / std::max<int64_t>(1, batch))); pa.D = static_cast<int>(D);
    vb200_rope rope{1, inv_freq_};
    pa.rope = rope;
    size_t ws = vb200_prefill_workspace_bytes(&pa);
    vb200_decode_args da{};
    da.struct_size = sizeof(da);
    da.dtype = VB200_BF16;
    da.B = static_cast<int>(batch); da.Hq = pa.Hq; da.Hkv = pa.Hkv; da.D = pa.D;
    da.cache_cap = static_cast<int>(config_.max_seq_len);
    // the split plan is not monotone in the step's max_len (a shorter context can take more, smaller splits),
    // and steps run both with a common length and with the device length array: size for the worst of them
    ws = std::max(ws, vb200_decode_workspace_bytes_max(&da));
    b.attn_ws = empty({static_cast<int64_t>((ws + 255) / 256 * 64)}, DType::Float32, Device::CUDA);
    b.rows = rows;
    b.batch = batch;
}

void TransformerLM::run_blocks(int64_t B, int64_t T, int64_t start_pos, bool device_positions, int* lens_dev, int64_t max_len) {
    Buffers& b = *buf_;
    void* s = current_stream();
    const int dev = b.h.device_index();
    const int M = static_cast<int>(B * T);
    const int dim = static_cast<int>(config_.dim), hid = static_cast<int>(config_.hidden_dim());
    const int D = static_cast<int>(config_.head_dim()), Hq = static_cast<int>(config_.n_heads), Hkv = static_cast<int>(config_.kv_heads());
    const int qkv_n = (Hq + 2 * Hkv) * D;
    const float scale = 1.0f / std::sqrt(static_cast<float>(D));
    uint16_t* qkv = b.qkv.data_ptr<uint16_t>();
    // RMSNorm is deferred: b.xn holds bf16(h * g) of the norm that comes next, and the GEMM that consumes it scales
    // its output rows by 1/rms(h) -- computed inside the weight-streaming kernel for up to 64 rows, from b.inv
    // (one small kernel per norm) for prompt passes.  No stand-alone norm kernel runs in a decode step.
    auto consume = [&](const void* x, const Tensor& w, void* out, int64_t ldo, int N, int epilogue, const char* who) {
        vb200_linear_args a{};
        a.struct_size = sizeof(a);
        a.device = dev; a.stream = s;
        a.x = x; a.ldx = dim; a.w = w.data_ptr<char>(); a.ldw = dim; a.out = out; a.ldo = ldo;
        a.M = M; a.N = N; a.K = dim; a.epilogue = epilogue;
        if (M <= 64) { a.rms_rows = b.h.data_ptr<float>(); a.rms_dim = dim; a.rms_ld = dim; a.rms_eps = config_.norm_eps; }
        else {
            check(vb200_row_inv_rms(dev, s, b.h.data_ptr<float>(), dim, b.inv.data_ptr<float>(), M, dim, config_.norm_eps), "row_inv_rms");
            a.row_scale = b.inv.data_ptr<float>();
        }
        check(vb200_linear_ex(&a), who);
    };
    auto produce = [&](const void* x, int K, const Tensor& w, const float* next_norm, const char* who) {
        vb200_linear_args a{};
        a.struct_size = sizeof(a);
        a.device = dev; a.stream = s;
        a.x = x; a.ldx = K; a.w = w.data_ptr<char>(); a.ldw = K; a.out = b.h.data_ptr<float>(); a.ldo = dim;
        a.M = M; a.N = dim; a.K = K; a.epilogue = VB200_EPI_ADD_F32;
        a.scaled_copy = b.xn.data_ptr<char>(); a.copy_scale = next_norm;
        check(vb200_linear_ex(&a), who);
    };
    // [B,T,H,D] memory seen as [B,H,T,D]: strides (batch, head, row) in elements
    const vb200_tensor4 qv{qkv, static_cast<int64_t>(T) * qkv_n, D, qkv_n};
    const vb200_tensor4 kv{qkv + Hq * D, static_cast<int64_t>(T) * qkv_n, D, qkv_n};
    const vb200_tensor4 vv{qkv + (Hq + Hkv) * D, static_cast<int64_t>(T) * qkv_n, D, qkv_n};
    const vb200_tensor4 ov{b.attn.data_ptr<uint16_t>(), static_cast<int64_t>(T) * Hq * D, D, static_cast<int64_t>(Hq) * D};
    for (size_t l = 0; l < layers_.size(); ++l) {
        Layer& L = *layers_[l];
        nn::KVCache& cache = *kv_caches_[l];
        // on entry b.xn = bf16(h * attention_norm_l): written by the embedding call (l = 0) or by the previous
        // block's down projection
        consume(b.xn.data_ptr<char>(), L.wqkv, qkv, qkv_n, qkv_n, VB200_EPI_BF16, "linear(wqkv)");
        const vb200_tensor4 kc{cache.k().data_ptr<char>(), cache.k().strides()[0], cache.k().strides()[1], cache.k().strides()[2]};
        const vb200_tensor4 vc{cache.v().data_ptr<char>(), cache.v().strides()[0], cache.v().strides()[1], cache.v().strides()[2]};
        if (T == 1) {                        // one new token per sequence: the split-KV decode path (tuned for head_dim 128)
            vb200_decode_args d{};
            d.struct_size = sizeof(d);
            d.device = dev; d.stream = s; d.dtype = VB200_BF16;
            d.B = static_cast<int>(B); d.Hq = Hq; d.Hkv = Hkv; d.D = D; d.scale = scale;
            d.q = qv; d.k_new = kv; d.v_new = vv; d.o = ov;
            d.rope = {1, inv_freq_};
            d.k_cache = kc; d.v_cache = vc; d.cache_cap = cache.get_max_seq_len();
            d.append_enabled = 1;
            if (device_positions) {
                d.seq_lens = lens_dev;
                d.advance_lens = (l + 1 == layers_.size()) ? 1 : 0;      // every layer appends at the same row; the last one advances
                d.max_len = static_cast<int>(max_len);
            } else {
                d.uniform_len = static_cast<int>(start_pos);
                d.max_len = static_cast<int>(start_pos) + 1;
            }
            d.workspace = b.attn_ws.data_ptr<char>();
            d.workspace_bytes = b.attn_ws.numel() * 4;
            check(vb200_decode_fwd(&d), "attention(decode)");
        } else {
            if (device_positions) throw std::runtime_error("TransformerLM: device-side positions need one token per sequence");
            vb200_prefill_args a{};
            a.struct_size = sizeof(a);
            a.device = dev; a.stream = s; a.dtype = VB200_BF16;
            a.B = static_cast<int>(B); a.Hq = Hq; a.Hkv = Hkv; a.T = static_cast<int>(T); a.D = D;
            a.start_pos = static_cast<int>(start_pos);
            a.causal = T > 1 ? 1 : 0;                                     // src/nn/gqa_attention.cpp:146
            a.scale = scale;
            a.q = qv; a.k = kv; a.v = vv; a.o = ov;
            a.rope = {1, inv_freq_};
            a.k_cache = kc; a.v_cache = vc; a.cache_cap = cache.get_max_seq_len();
            a.workspace = b.attn_ws.data_ptr<char>();
            a.workspace_bytes = b.attn_ws.numel() * 4;
            check(vb200_prefill_fwd(&a), "attention(prefill)");
        }
        if (!device_positions) cache.set_current_len(std::max(cache.current_seq_len(), static_cast<int>(start_pos + T)));
        produce(b.attn.data_ptr<char>(), Hq * D, L.wo, L.ffn_norm.data_ptr<float>(), "linear(wo) + residual");
        consume(b.xn.data_ptr<char>(), L.w13, b.act.data_ptr<char>(), hid, 2 * hid, VB200_EPI_SWIGLU, "linear(gate,up)");
        const float* next_norm = (l + 1 < layers_.size()) ? layers_[l + 1]->attn_norm.data_ptr<float>() : final_norm_.data_ptr<float>();
        produce(b.act.data_ptr<char>(), hid, L.w2, next_norm, "linear(down) + residual");
    }
}

Tensor TransformerLM::forward_with_cache(const Tensor& tokens, int64_t start_pos, bool last_only) {
    if (kv_caches_.empty()) throw std::runtime_error("KV cache not initialized. Call init_cache first.");
    if (tokens.ndim() != 2) throw std::runtime_error("TransformerLM::forward_with_cache: tokens must be [Batch, NewTokens]");
    if (tokens.dtype() != DType::Int32 && tokens.dtype() != DType::Int64)
        throw std::runtime_error("TransformerLM::forward_with_cache: tokens must be Int32 or Int64");
    const int64_t B = tokens.shape()[0], T = tokens.shape()[1];
    if (start_pos < 0 || start_pos + T > config_.max_seq_len)
        throw std::runtime_error("Sequence length " + std::to_string(start_pos + T) + " exceeds maximum " + std::to_string(config_.max_seq_len));
    ensure_buffers(B * T, B);
    Buffers& b = *buf_;
    void* s = current_stream();
    const int dev = b.h.device_index();
    const int dim = static_cast<int>(config_.dim), vocab = static_cast<int>(config_.vocab_size);
    Tensor ids = tokens.is_contiguous() ? tokens : tokens.contiguous();
    if (ids.device() != Device::CUDA) ids = ids.to(Device::CUDA);
    const float* first_norm = layers_.empty() ? final_norm_.data_ptr<float>() : layers_[0]->attn_norm.data_ptr<float>();
    check(vb200_embedding_scaled(dev, s, ids.data_ptr<char>(), ids.dtype() == DType::Int64 ? 1 : 0, tok_emb_.data_ptr<char>(), b.h.data_ptr<float>(),
                                 static_cast<int>(B * T), dim, vocab, first_norm, b.xn.data_ptr<char>()), "embedding");
    run_blocks(B, T, start_pos, false, nullptr, 0);          // leaves bf16(h * final_norm) in b.xn
    const int64_t out_rows = last_only ? B : B * T;
    if (b.logit_rows < out_rows) {
        b.logits = empty({out_rows, config_.vocab_size}, DType::Float32, Device::CUDA);
        b.logit_rows = out_rows;
    }
    // last_only: row b of the GEMM input is the last new token of sequence b (row stride T * dim)
    {
        const int64_t row_ld = last_only ? T * static_cast<int64_t>(dim) : dim;
        const int64_t first = last_only ? (T - 1) * static_cast<int64_t>(dim) : 0;
        vb200_linear_args a{};
        a.struct_size = sizeof(a);
        a.device = dev; a.stream = s;
        a.x = b.xn.data_ptr<uint16_t>() + first; a.ldx = row_ld;
        a.w = lm_head_.data_ptr<char>(); a.ldw = dim; a.out = b.logits.data_ptr<float>(); a.ldo = vocab;
        a.M = static_cast<int>(out_rows); a.N = vocab; a.K = dim; a.epilogue = VB200_EPI_F32;
        // the final norm's 1/rms of the same rows of the residual stream
        if (out_rows <= 64) { a.rms_rows = b.h.data_ptr<float>() + first; a.rms_ld = row_ld; a.rms_dim = dim; a.rms_eps = config_.norm_eps; }
        else {
            check(vb200_row_inv_rms(dev, s, b.h.data_ptr<float>() + first, row_ld, b.inv.data_ptr<float>(), static_cast<int>(out_rows), dim, config_.norm_eps), "row_inv_rms");
            a.row_scale = b.inv.data_ptr<float>();
        }
        check(vb200_linear_ex(&a), "linear(output)");
    }
    Tensor out = b.logits.narrow(0, 0, out_rows).view({B, last_only ? 1 : T, config_.vocab_size});
    return out;
}

void TransformerLM::pick_from_last_logits(DecodeState& st) {
    Buffers& b = *buf_;
    const int64_t B = st.ids.shape()[0];
    vb200_greedy_args g{};
    g.struct_size = sizeof(g);
    g.device = b.h.device_index();
    g.stream = current_stream();
    g.logits = b.logits.data_ptr<float>();
    g.ld_logits = config_.vocab_size;
    g.B = static_cast<int>(B);
    g.vocab = static_cast<int>(config_.vocab_size);
    g.out_ids = st.ids.data_ptr<int32_t>();
    g.history = st.history.data_ptr<int32_t>();
    g.history_ld = st.history.strides()[0];
    g.pos_dev = st.lens.data_ptr<int32_t>();
    g.pos_base = static_cast<int>(st.prompt_len);
    if (st.stop_ids.defined() && st.stop_ids.numel() > 0) {
        g.stop_ids = st.stop_ids.data_ptr<int32_t>();
        g.n_stop = static_cast<int>(st.stop_ids.numel());
    }
    g.min_new_tokens = static_cast<int>(st.min_new_tokens);
    g.done = st.done.data_ptr<int32_t>();
    check(vb200_greedy_step(&g), "greedy_step");
}

void TransformerLM::decode_step(DecodeState& st) {
    if (kv_caches_.empty()) throw std::runtime_error("KV cache not initialized. Call init_cache first.");
    const int64_t B = st.ids.shape()[0];
    ensure_buffers(B, B);
    Buffers& b = *buf_;
    if (b.logit_rows < B) {
        b.logits = empty({B, config_.vocab_size}, DType::Float32, Device::CUDA);
        b.logit_rows = B;
    }
    void* s = current_stream();
    const int dev = b.h.device_index();
    const int dim = static_cast<int>(config_.dim), vocab = static_cast<int>(config_.vocab_size);
    const float* first_norm = layers_.empty() ? final_norm_.data_ptr<float>() : layers_[0]->attn_norm.data_ptr<float>();
    check(vb200_embedding_scaled(dev, s, st.ids.data_ptr<char>(), 0, tok_emb_.data_ptr<char>(), b.h.data_ptr<float>(), static_cast<int>(B), dim, vocab,
                                 first_norm, b.xn.data_ptr<char>()), "embedding");
    run_blocks(B, 1, 0, true, st.lens.data_ptr<int32_t>(), st.max_len);      // leaves bf16(h * final_norm) in b.xn
    {
        vb200_linear_args a{};
        a.struct_size = sizeof(a);
        a.device = dev; a.stream = s;
        a.x = b.xn.data_ptr<char>(); a.ldx = dim; a.w = lm_head_.data_ptr<char>(); a.ldw = dim; a.out = b.logits.data_ptr<float>(); a.ldo = vocab;
        a.M = static_cast<int>(B); a.N = vocab; a.K = dim; a.epilogue = VB200_EPI_F32;
        if (B <= 64) { a.rms_rows = b.h.data_ptr<float>(); a.rms_ld = dim; a.rms_dim = dim; a.rms_eps = config_.norm_eps; }
        else {
            check(vb200_row_inv_rms(dev, s, b.h.data_ptr<float>(), dim, b.inv.data_ptr<float>(), static_cast<int>(B), dim, config_.norm_eps), "row_inv_rms");
            a.row_scale = b.inv.data_ptr<float>();
        }
        check(vb200_linear_ex(&a), "linear(output)");
    }
    pick_from_last_logits(st);
}

}  // namespace vesper::models
