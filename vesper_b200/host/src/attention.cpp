// Host-side attention operators with Vesper's names, forwarding to the C ABI
// of libvesper_b200.  Validation messages follow the reference front-ends so
// callers see the same std::runtime_error texts.
#include <vesper/nn/functional.h>
#include <vesper/nn/transformer.h>
#include <vesper/ops/attention_ops.h>
#include <vesper/ops/flash_attention.h>

#include <vesper_b200.h>

#include <cmath>
#include <string>

namespace vesper {

namespace {

vb200_tensor4 view4(const Tensor& t) {
    return {const_cast<char*>(t.data_ptr<char>()), t.strides()[0], t.strides()[1], t.strides()[2]};
}

int dtype_of(const Tensor& t, const char* who) {
    switch (t.dtype()) {
        case DType::Float32: return VB200_F32;
        case DType::BFloat16: return VB200_BF16;
        case DType::Float16: return VB200_F16;
        default: throw std::runtime_error(std::string(who) + ": dtype must be Float32, BFloat16 or Float16");
    }
}

void check(int rc, const char* who) {
    if (rc != VB200_OK)
        throw std::runtime_error(std::string(who) + ": " + vb200_strerror(rc) + ": " + vb200_last_error_detail());
}

void require_cuda(const Tensor& t, const char* who) {
    if (t.device() == Device::HIP) throw std::runtime_error(std::string(who) + ": HIP backend not enabled");
    if (t.device() != Device::CUDA)
        throw std::runtime_error(std::string(who) + ": this library is the CUDA backend; CPU tensors are not handled here");
}

void* current_stream() { return Stream::current(Device::CUDA).raw_handle(); }

// workspace from the caching allocator, kept alive by the returned tensor
Tensor workspace(size_t bytes) {
    return empty({static_cast<int64_t>((bytes + 255) / 256 * 64)}, DType::Float32, Device::CUDA);
}

}  // namespace

namespace ops {

void flash_attention_cuda_dispatch(const Tensor& q, const Tensor& k, const Tensor& v,
                                   Tensor& output, Tensor& lse, float scale, bool is_causal,
                                   float /*dropout_p*/, bool /*training*/, Tensor* /*dropout_mask_out*/) {
    vb200_prefill_args a{};
    a.struct_size = sizeof(a);
    a.device = q.device_index();
    a.stream = current_stream();
    a.dtype = dtype_of(q, "flash_attention");
    a.B = static_cast<int>(q.shape()[0]); a.Hq = static_cast<int>(q.shape()[1]); a.Hkv = static_cast<int>(k.shape()[1]);
    a.T = static_cast<int>(q.shape()[2]); a.D = static_cast<int>(q.shape()[3]);
    a.causal = is_causal ? 1 : 0;
    a.scale = scale;
    a.q = view4(q); a.k = view4(k); a.v = view4(v); a.o = view4(output);
    a.lse = lse.defined() ? lse.data_ptr<float>() : nullptr;
    check(vb200_prefill_fwd(&a), "flash_attention");
}

std::pair<Tensor, Tensor> flash_attention_with_lse(const Tensor& q, const Tensor& k, const Tensor& v,
                                                   float scale, bool is_causal) {
    if (q.ndim() != 4 || k.ndim() != 4 || v.ndim() != 4)
        throw std::runtime_error("flash_attention: inputs must be 4D [B, H, N, D]");
    if (k.shape() != v.shape() || q.shape()[0] != k.shape()[0] || q.shape()[2] != k.shape()[2] || q.shape()[3] != k.shape()[3])
        throw std::runtime_error("flash_attention: Q, K, V must have same shape");
    if (q.dtype() != k.dtype() || k.dtype() != v.dtype())
        throw std::runtime_error("flash_attention: Q, K, V must have same dtype");
    require_cuda(q, "flash_attention");
    Tensor out = empty(q.shape(), q.dtype(), Device::CUDA);
    Tensor lse = empty({q.shape()[0], q.shape()[1], q.shape()[2]}, DType::Float32, Device::CUDA);
    flash_attention_cuda_dispatch(q, k, v, out, lse, scale, is_causal, 0.0f, false, nullptr);
    return {out, lse};
}

Tensor flash_attention(const Tensor& q, const Tensor& k, const Tensor& v, float scale,
                       bool is_causal, float dropout_p, bool /*training*/) {
    // src/ops/flash_attention.cpp:45-59
    if (q.ndim() != 4 || k.ndim() != 4 || v.ndim() != 4)
        throw std::runtime_error("flash_attention: inputs must be 4D [B, H, N, D]");
    if (q.shape() != k.shape() || k.shape() != v.shape())
        throw std::runtime_error("flash_attention: Q, K, V must have same shape");
    if (q.dtype() != k.dtype() || k.dtype() != v.dtype())
        throw std::runtime_error("flash_attention: Q, K, V must have same dtype");
    if (dropout_p < 0.0f || dropout_p >= 1.0f)
        throw std::runtime_error("flash_attention: dropout_p must be in [0, 1)");
    return flash_attention_with_lse(q, k, v, scale, is_causal).first;
}

void flash_attention_backward_cuda_dispatch(const Tensor& grad_output, const Tensor& q, const Tensor& k, const Tensor& v,
                                            const Tensor& output, const Tensor& lse, Tensor& grad_q, Tensor& grad_k,
                                            Tensor& grad_v, float scale, bool is_causal, float dropout_p,
                                            const Tensor* /*dropout_mask*/) {
    if (dropout_p > 0.0f) throw std::runtime_error("flash_attention_backward: dropout is not part of the CUDA path");
    if (q.dtype() != DType::Float32) throw std::runtime_error("flash_attention_backward: Float32 only");
    // contiguous copies where needed, as src/ops/flash_attention.cpp:373-378
    Tensor dO = grad_output.contiguous(), qc = q.contiguous(), kc = k.contiguous(), vc = v.contiguous(), oc = output.contiguous(),
           lc = lse.contiguous();
    vb200_attention_bwd_args a{};
    a.struct_size = sizeof(a);
    a.device = q.device_index();
    a.stream = current_stream();
    a.dtype = VB200_F32;
    a.B = static_cast<int>(q.shape()[0]); a.H = static_cast<int>(q.shape()[1]); a.N = static_cast<int>(q.shape()[2]); a.D = static_cast<int>(q.shape()[3]);
    a.causal = is_causal ? 1 : 0;
    a.scale = scale;
    a.d_out = dO.data_ptr<char>(); a.q = qc.data_ptr<char>(); a.k = kc.data_ptr<char>(); a.v = vc.data_ptr<char>(); a.out = oc.data_ptr<char>();
    a.lse = lc.data_ptr<float>();
    a.dq = grad_q.data_ptr<char>(); a.dk = grad_k.data_ptr<char>(); a.dv = grad_v.data_ptr<char>();
    Tensor ws = workspace(vb200_attention_bwd_workspace_bytes(&a));
    a.workspace = ws.data_ptr<char>();
    a.workspace_bytes = ws.numel() * 4;
    check(vb200_attention_bwd(&a), "flash_attention_backward");
}

std::tuple<Tensor, Tensor, Tensor> flash_attention_backward(const Tensor& grad_output, const Tensor& q, const Tensor& k,
                                                            const Tensor& v, const Tensor& output, const Tensor& lse,
                                                            float scale, bool is_causal, float dropout_p,
                                                            const Tensor& dropout_mask) {
    if (q.ndim() != 4 || q.shape() != k.shape() || k.shape() != v.shape() || grad_output.shape() != q.shape() || output.shape() != q.shape())
        throw std::runtime_error("flash_attention_backward: grad_output, Q, K, V, output must have the same 4D shape");
    require_cuda(q, "flash_attention_backward");
    Tensor gq = empty(q.shape(), q.dtype(), Device::CUDA), gk = empty(q.shape(), q.dtype(), Device::CUDA), gv = empty(q.shape(), q.dtype(), Device::CUDA);
    flash_attention_backward_cuda_dispatch(grad_output, q, k, v, output, lse, gq, gk, gv, scale, is_causal, dropout_p,
                                           dropout_mask.defined() ? &dropout_mask : nullptr);
    return {gq, gk, gv};
}

void repeat_kv_cuda_dispatch(const Tensor& input, Tensor& output, int64_t n_rep) {
    vb200_tensor4 in = view4(input);
    check(vb200_repeat_kv(input.device_index(), current_stream(), dtype_of(input, "repeat_kv"), &in, output.data_ptr<char>(),
                          static_cast<int>(input.shape()[0]), static_cast<int>(input.shape()[1]),
                          static_cast<int>(input.shape()[2]), static_cast<int>(input.shape()[3]), static_cast<int>(n_rep)),
          "repeat_kv");
}

Tensor repeat_kv(const Tensor& x, int64_t n_rep) {
    if (n_rep == 1) return x;                              // src/ops/attention_ops.cpp:93-95
    if (x.ndim() != 4) throw std::runtime_error("repeat_kv: input must be 4D [B, KV_H, S, D]");
    if (n_rep < 1) throw std::runtime_error("repeat_kv: n_rep must be >= 1");
    require_cuda(x, "repeat_kv");
    Tensor out = empty({x.shape()[0], x.shape()[1] * n_rep, x.shape()[2], x.shape()[3]}, x.dtype(), Device::CUDA);
    repeat_kv_cuda_dispatch(x, out, n_rep);
    return out;
}

}  // namespace ops

namespace nn {

KVCache::KVCache(int batch_size, int num_heads, int max_seq_len, int head_dim, Device device, DType dtype)
    : max_seq_len_(max_seq_len) {
    std::vector<int64_t> shape = {batch_size, num_heads, max_seq_len, head_dim};
    k_cache_ = zeros(shape, dtype, device);
    v_cache_ = zeros(shape, dtype, device);
}

void KVCache::reset() {
    current_len_ = 0;
    k_cache_.zero_();
    v_cache_.zero_();
}

std::pair<Tensor, Tensor> KVCache::update(const Tensor& new_k, const Tensor& new_v, int start_pos) {
    if (new_k.ndim() != 4 || new_k.shape() != new_v.shape()) throw std::runtime_error("KVCache::update: new_k/new_v must be 4D with equal shapes");
    const int T = static_cast<int>(new_k.shape()[2]);
    if (start_pos < 0 || start_pos + T > max_seq_len_) throw std::runtime_error("KVCache::update: position range exceeds max_seq_len");
    std::vector<IndexSelector> rows = {Slice(), Slice(), Slice(start_pos, start_pos + T), Slice()};
    if (k_cache_.device() == Device::CUDA) {
        require_cuda(new_k, "KVCache::update");
        vb200_tensor4 k = view4(new_k), v = view4(new_v), kc = view4(k_cache_), vc = view4(v_cache_);
        check(vb200_kv_append(k_cache_.device_index(), current_stream(), dtype_of(k_cache_, "KVCache::update"),
                              static_cast<int>(new_k.shape()[0]), static_cast<int>(new_k.shape()[1]), T,
                              static_cast<int>(new_k.shape()[3]), start_pos, &k, &v, &kc, &vc, max_seq_len_, nullptr),
              "KVCache::update");
    } else {
        Tensor ks = k_cache_.index(rows), vs = v_cache_.index(rows);
        ks.copy_from(new_k);
        vs.copy_from(new_v);
    }
    current_len_ = std::max(current_len_, start_pos + T);
    std::vector<IndexSelector> active = {Slice(), Slice(), Slice(0, current_len_), Slice()};
    return {k_cache_.index(active), v_cache_.index(active)};
}

Tensor fused_attention(const Tensor& q, const Tensor& k, const Tensor& v, KVCache* cache, int64_t start_pos,
                       bool use_rope, float rope_base, bool causal_when_uncached, Tensor* out_view) {
    if (q.ndim() != 4 || k.ndim() != 4 || v.ndim() != 4) throw std::runtime_error("attention: q, k, v must be 4D [B, H, T, D]");
    if (k.shape() != v.shape()) throw std::runtime_error("attention: k and v must have the same shape");
    const int B = static_cast<int>(q.shape()[0]), Hq = static_cast<int>(q.shape()[1]), T = static_cast<int>(q.shape()[2]),
              D = static_cast<int>(q.shape()[3]), Hkv = static_cast<int>(k.shape()[1]);
    if (Hq % Hkv != 0) throw std::invalid_argument("GroupedQueryAttention: num_heads must be divisible by num_kv_heads");
    require_cuda(q, "attention");
    float inv_freq[64];
    if (use_rope) {
        if (D > 128) throw std::runtime_error("attention: head_dim > 128 is not supported");
        vb200_rope_inv_freq(rope_base, D, inv_freq);
    }
    const float scale = 1.0f / std::sqrt(static_cast<float>(D));
    if (out_view && (out_view->shape() != q.shape() || out_view->dtype() != q.dtype() || out_view->strides()[3] != 1))
        throw std::runtime_error("attention: the output view must have q's shape and dtype with contiguous head_dim");
    if (cache && cache->k().dtype() != q.dtype()) throw std::runtime_error("attention: the KV cache must have the dtype of q, k, v");
    Tensor out = out_view ? *out_view : empty(q.shape(), q.dtype(), Device::CUDA);
    // one new token per sequence: the split-KV decode path, whatever the dtype, head_dim and group size
    const bool fast_decode = cache && T == 1 && D % 8 == 0;
    if (fast_decode) {
        vb200_decode_args d{};
        d.struct_size = sizeof(d);
        d.device = q.device_index();
        d.stream = current_stream();
        d.dtype = dtype_of(q, "attention");
        d.B = B; d.Hq = Hq; d.Hkv = Hkv; d.D = D; d.scale = scale;
        d.q = view4(q); d.k_new = view4(k); d.v_new = view4(v); d.o = view4(out);
        d.rope = {use_rope ? 1 : 0, inv_freq};
        d.k_cache = view4(cache->k()); d.v_cache = view4(cache->v());
        d.cache_cap = cache->get_max_seq_len();
        d.uniform_len = static_cast<int>(start_pos);           // one length for the whole batch, as in the reference
        d.max_len = static_cast<int>(start_pos) + 1;
        d.append_enabled = 1;
        Tensor ws = workspace(vb200_decode_workspace_bytes(&d));
        d.workspace = ws.data_ptr<char>();
        d.workspace_bytes = ws.numel() * 4;
        check(vb200_decode_fwd(&d), "attention");
        cache->set_current_len(std::max(cache->current_seq_len(), static_cast<int>(start_pos) + 1));
        return out;
    }
    vb200_prefill_args a{};
    a.struct_size = sizeof(a);
    a.device = q.device_index();
    a.stream = current_stream();
    a.dtype = dtype_of(q, "attention");
    a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.T = T; a.D = D;
    a.start_pos = cache ? static_cast<int>(start_pos) : 0;
    a.causal = cache ? (T > 1 ? 1 : 0) : (causal_when_uncached ? 1 : 0);      // src/nn/gqa_attention.cpp:146
    a.scale = scale;
    a.q = view4(q); a.k = view4(k); a.v = view4(v); a.o = view4(out);
    a.rope = {use_rope ? 1 : 0, inv_freq};
    if (cache) {
        a.k_cache = view4(cache->k()); a.v_cache = view4(cache->v());
        a.cache_cap = cache->get_max_seq_len();
    }
    Tensor ws = workspace(vb200_prefill_workspace_bytes(&a));
    a.workspace = ws.data_ptr<char>();
    a.workspace_bytes = ws.numel() * 4;
    check(vb200_prefill_fwd(&a), "attention");
    if (cache) cache->set_current_len(std::max(cache->current_seq_len(), static_cast<int>(start_pos) + T));
    return out;
}

namespace functional {

Tensor scaled_dot_product_attention(const Tensor& query, const Tensor& key, const Tensor& value,
                                    bool is_causal, double dropout_p) {
    if (query.ndim() != 4 || key.ndim() != 4 || value.ndim() != 4)
        throw std::runtime_error("scaled_dot_product_attention: inputs must be 4D [B, H, S, D]");
    if (dropout_p > 0.0) throw std::runtime_error("scaled_dot_product_attention: dropout is not part of the inference path");
    require_cuda(query, "scaled_dot_product_attention");
    const int64_t T = query.shape()[2], L = key.shape()[2], D = query.shape()[3];
    const float scale = 1.0f / std::sqrt(static_cast<float>(D));
    if (T == L) return ops::flash_attention_with_lse(query, key, value, scale, is_causal).first;
    if (T > L) throw std::runtime_error("scaled_dot_product_attention: more queries than keys");
    // T queries against L > T keys (src/nn/functional.cpp:399-421; the decode shape is T = 1): key and value
    // already hold every row attended to, so they are passed as a read-only cache -- nothing is written.
    Tensor out = empty(query.shape(), query.dtype(), Device::CUDA);
    const int B = static_cast<int>(query.shape()[0]), Hq = static_cast<int>(query.shape()[1]), Hkv = static_cast<int>(key.shape()[1]);
    if (Hq % Hkv != 0) throw std::runtime_error("scaled_dot_product_attention: query heads must be a multiple of key heads");
    if (T == 1 && D % 8 == 0) {                                  // (with one query row the causal flag changes nothing)
        // one query row per head: the split-KV kernel, no append, no rotation
        vb200_decode_args d{};
        d.struct_size = sizeof(d);
        d.device = query.device_index();
        d.stream = current_stream();
        d.dtype = dtype_of(query, "scaled_dot_product_attention");
        d.B = B; d.Hq = Hq; d.Hkv = Hkv; d.D = static_cast<int>(D); d.scale = scale;
        d.q = view4(query); d.o = view4(out);
        d.k_cache = view4(key); d.v_cache = view4(value);
        d.cache_cap = static_cast<int>(L);
        d.uniform_len = static_cast<int>(L);
        d.max_len = static_cast<int>(L);
        Tensor ws = workspace(vb200_decode_workspace_bytes(&d));
        d.workspace = ws.data_ptr<char>();
        d.workspace_bytes = ws.numel() * 4;
        check(vb200_decode_fwd(&d), "scaled_dot_product_attention");
        return out;
    }
    vb200_prefill_args a{};
    a.struct_size = sizeof(a);
    a.device = query.device_index();
    a.stream = current_stream();
    a.dtype = dtype_of(query, "scaled_dot_product_attention");
    a.B = B; a.Hq = Hq; a.Hkv = Hkv;
    a.T = static_cast<int>(T); a.D = static_cast<int>(D);
    a.start_pos = static_cast<int>(L - T);
    a.causal = is_causal ? 1 : 0;
    a.scale = scale;
    a.q = view4(query); a.o = view4(out);
    a.k_cache = view4(key); a.v_cache = view4(value);
    a.cache_cap = static_cast<int>(L);
    a.cache_read_only = 1;
    check(vb200_prefill_fwd(&a), "scaled_dot_product_attention");
    return out;
}

Tensor compute_rope_frequencies(int seq_len, int head_dim, int start_pos, float theta, Device device) {
    const int half = head_dim / 2;
    std::vector<float> f(static_cast<size_t>(seq_len) * half);
    for (int m = 0; m < seq_len; ++m) {
        int pos = start_pos + m;
        for (int i = 0; i < half; ++i) {
            float freq = std::pow(theta, -2.0f * i / head_dim);     // src/nn/functional.cpp:433
            f[static_cast<size_t>(m) * half + i] = pos * freq;
        }
    }
    Tensor t = empty({seq_len, half}, DType::Float32, Device::CPU);
    t.copy_from_host(f.data());
    return t.to(device);
}

Tensor apply_rotary_emb(const Tensor& x, const Tensor& freqs) {
    if (x.ndim() != 4) throw std::runtime_error("apply_rotary_emb: x must be 4D [B, H, S, D]");
    if (x.dtype() != DType::Float32) throw std::runtime_error("apply_rotary_emb: Float32 only (use the fused attention call for 16-bit types)");
    require_cuda(x, "apply_rotary_emb");
    const int S = static_cast<int>(x.shape()[2]), D = static_cast<int>(x.shape()[3]);
    if (freqs.ndim() != 2 || freqs.shape()[0] != S || freqs.shape()[1] != D / 2)
        throw std::runtime_error("apply_rotary_emb: freqs must be [S, D/2]");
    // cos/sin on the host with std::cos/std::sin, as src/ops/elementwise.cpp:1038-1044 does
    std::vector<float> a(static_cast<size_t>(S) * (D / 2)), c(a.size()), s(a.size());
    freqs.to(Device::CPU).copy_to_host(a.data());
    for (size_t i = 0; i < a.size(); ++i) { c[i] = std::cos(a[i]); s[i] = std::sin(a[i]); }
    Tensor ct = empty({S, D / 2}, DType::Float32, Device::CUDA), st = empty({S, D / 2}, DType::Float32, Device::CUDA);
    ct.copy_from_host(c.data());
    st.copy_from_host(s.data());
    Tensor out = x.clone();
    check(vb200_apply_rope(x.device_index(), current_stream(), out.data_ptr<float>(), ct.data_ptr<float>(), st.data_ptr<float>(),
                           static_cast<int>(x.shape()[0]), static_cast<int>(x.shape()[1]), S, D),
          "apply_rotary_emb");
    Stream::current(Device::CUDA).synchronize();      // the host tables above go out of scope
    return out;
}

}  // namespace functional
}  // namespace nn
}  // namespace vesper
