// C++ tests of the host layer (Vesper's names over the B200 C ABI), written in the
// style of the reference's own assert-style executables:
//   flash op on the GPU vs the CPU implementation   tests/test_flash_attention.cpp:195-284, 547-576
//   KV cache literal values and views               tests/test_kv_cache.cpp:8-58
//   cached == uncached forward                      tests/test_kv_cache_chapter33.cpp:66-188
//   RoPE angle table / 90 degree rotation           tests/test_rope.cpp:11-73
//   repeat_kv index pattern                         tests/test_gqa_chapter33.cpp:76-118
//   flash backward: finite, non-zero, vs CPU        tests/test_flash_attention.cpp:292-339
//   model forward_with_cache / greedy generation    src/models/transformer.cpp:152-206, src/generation/generator.cpp:36-142
// The CPU side is the oracle (oracle/vesper_attn_oracle.c, pinned to the reference).
#include <vesper/core/factories.h>
#include <vesper/nn/functional.h>
#include <vesper/nn/transformer.h>
#include <vesper/ops/attention_ops.h>
#include <vesper/ops/flash_attention.h>
#include <vesper/generation/generator.h>
#include <vesper/models/transformer.h>
#include <vesper/nn/linear.h>
#include "../../oracle/vesper_block_oracle.h"

#include "../../oracle/vesper_attn_oracle.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

using namespace vesper;

#define CHECK(cond)                                                                       \
    do { if (!(cond)) { std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); std::exit(1); } } while (0)

static std::vector<float> randn(size_t n, unsigned seed, float scale = 1.0f) {
    std::mt19937 g(seed);
    std::normal_distribution<float> d(0.f, 1.f);
    std::vector<float> v(n);
    for (auto& x : v) x = scale * d(g);
    return v;
}

static Tensor to_cuda(const std::vector<float>& h, std::vector<int64_t> shape, DType dt = DType::Float32) {
    Tensor t = empty(shape, dt, Device::CUDA);
    if (dt == DType::Float32) { t.copy_from_host(h.data()); return t; }
    std::vector<uint16_t> b(h.size());
    for (size_t i = 0; i < h.size(); ++i) b[i] = dt == DType::BFloat16 ? float_to_bf16(h[i]) : float_to_fp16(h[i]);
    t.copy_from_host(b.data());
    return t;
}

static std::vector<float> to_host(const Tensor& t) {
    std::vector<float> out(t.numel());
    if (t.dtype() == DType::Float32) { t.copy_to_host(out.data()); return out; }
    std::vector<uint16_t> b(t.numel());
    t.copy_to_host(b.data());
    for (size_t i = 0; i < b.size(); ++i) out[i] = t.dtype() == DType::BFloat16 ? bf16_to_float(b[i]) : fp16_to_float(b[i]);
    return out;
}

static std::vector<float> round_like(const std::vector<float>& h, DType dt) {
    std::vector<float> r(h);
    if (dt == DType::BFloat16) for (auto& x : r) x = bf16_to_float(float_to_bf16(x));
    if (dt == DType::Float16) for (auto& x : r) x = fp16_to_float(float_to_fp16(x));
    return r;
}

static bool allclose(const std::vector<float>& a, const std::vector<float>& b, float rtol, float atol, float* worst = nullptr) {
    float w = 0.f;
    bool ok = a.size() == b.size();
    for (size_t i = 0; ok && i < a.size(); ++i) {
        float d = std::fabs(a[i] - b[i]);
        w = std::max(w, d);
        if (!(d <= atol + rtol * std::fabs(b[i]))) ok = false;
    }
    if (worst) *worst = w;
    return ok;
}

// GPU flash op vs the CPU implementation, the reference's tolerances (rtol 1e-2, atol 1e-3).
static void test_flash_vs_cpu(int B, int H, int N, int D, bool causal, DType dt, float rtol, float atol) {
    size_t n = static_cast<size_t>(B) * H * N * D;
    auto q = round_like(randn(n, 1, 0.5f), dt), k = round_like(randn(n, 2, 0.5f), dt), v = round_like(randn(n, 3, 0.5f), dt);
    float scale = 1.0f / std::sqrt(static_cast<float>(D));
    std::vector<float> o_cpu(n), lse_cpu(static_cast<size_t>(B) * H * N);
    vo_flash_attention_fwd(q.data(), k.data(), v.data(), o_cpu.data(), lse_cpu.data(), B, H, N, D, scale, causal);
    Tensor out = ops::flash_attention(to_cuda(q, {B, H, N, D}, dt), to_cuda(k, {B, H, N, D}, dt), to_cuda(v, {B, H, N, D}, dt), scale, causal);
    CHECK(out.shape() == (std::vector<int64_t>{B, H, N, D}));
    CHECK(out.dtype() == dt);
    float worst = 0.f;
    bool ok = allclose(to_host(out), o_cpu, rtol, atol, &worst);
    std::printf("  flash B%d H%d N%d D%d %s dtype %d: max diff %.3g\n", B, H, N, D, causal ? "causal" : "full", static_cast<int>(dt), worst);
    CHECK(ok);
    auto [o2, lse] = ops::flash_attention_with_lse(to_cuda(q, {B, H, N, D}, dt), to_cuda(k, {B, H, N, D}, dt), to_cuda(v, {B, H, N, D}, dt), scale, causal);
    CHECK(allclose(to_host(lse), lse_cpu, 0.f, 1e-3f, &worst));
}

static void test_flash_large_is_finite() {      // tests/test_flash_attention.cpp:248-284
    int B = 1, H = 8, N = 1024, D = 64;
    size_t n = static_cast<size_t>(B) * H * N * D;
    Tensor out = ops::flash_attention(to_cuda(randn(n, 4), {B, H, N, D}), to_cuda(randn(n, 5), {B, H, N, D}), to_cuda(randn(n, 6), {B, H, N, D}), 0.125f, true);
    for (float x : to_host(out)) CHECK(std::isfinite(x));
}

static void test_flash_errors() {               // src/ops/flash_attention.cpp:45-59
    Tensor a = zeros({1, 2, 8, 64}, DType::Float32, Device::CUDA), b = zeros({1, 2, 9, 64}, DType::Float32, Device::CUDA);
    auto throws = [](auto fn, const char* needle) {
        try { fn(); } catch (const std::runtime_error& e) { return std::string(e.what()).find(needle) != std::string::npos; }
        return false;
    };
    CHECK(throws([&] { ops::flash_attention(a, b, b, 1.f); }, "Q, K, V must have same shape"));
    CHECK(throws([&] { ops::flash_attention(a.index({int64_t(0)}), a.index({int64_t(0)}), a.index({int64_t(0)}), 1.f); }, "inputs must be 4D"));
    CHECK(throws([&] { ops::flash_attention(a, a, a, 1.f, true, 1.5f); }, "dropout_p must be in [0, 1)"));
    Tensor h = zeros({1, 2, 8, 64}, DType::BFloat16, Device::CUDA);
    CHECK(throws([&] { ops::flash_attention(a, h, h, 1.f); }, "same dtype"));
}

static void test_kv_cache_basic() {             // tests/test_kv_cache.cpp:8-58
    nn::KVCache cache(1, 2, 8, 8, Device::CUDA);
    CHECK(cache.current_seq_len() == 0 && cache.get_max_seq_len() == 8);
    std::vector<float> k1(1 * 2 * 3 * 8), v1(k1.size());
    for (size_t i = 0; i < k1.size(); ++i) { k1[i] = 1.0f + i; v1[i] = -1.0f - i; }
    auto [kv, vv] = cache.update(to_cuda(k1, {1, 2, 3, 8}), to_cuda(v1, {1, 2, 3, 8}), 0);
    CHECK(cache.current_seq_len() == 3);
    CHECK(kv.shape() == (std::vector<int64_t>{1, 2, 3, 8}) && kv.strides()[1] == 8 * 8);     // a view: strides keep max_seq_len * D
    CHECK(to_host(kv) == k1 && to_host(vv) == v1);
    std::vector<float> k2(1 * 2 * 1 * 8, 7.f), v2(k2.size(), 9.f);
    auto [kv2, vv2] = cache.update(to_cuda(k2, {1, 2, 1, 8}), to_cuda(v2, {1, 2, 1, 8}), 3);
    CHECK(cache.current_seq_len() == 4 && kv2.shape()[2] == 4);
    auto hk = to_host(kv2);
    CHECK(hk[0] == 1.0f && hk[3 * 8] == 7.f && hk[4 * 8] == k1[3 * 8]);      // head 0 rows 0,3; head 1 row 0
    auto all = to_host(cache.k());
    for (size_t r = 4; r < 8; ++r) CHECK(all[r * 8] == 0.f);                    // rows past the length stay zero
    cache.reset();
    CHECK(cache.current_seq_len() == 0);
    for (float x : to_host(cache.k())) CHECK(x == 0.f);
}

// Token-by-token cached attention reproduces the full causal pass (the property
// tests/test_kv_cache_chapter33.cpp:66-188 asserts at 1e-4 for MHA; here also for grouped heads).
static void test_cached_equals_uncached(int Hq, int Hkv, DType dt, float tol) {
    int B = 2, T = 40, D = 128, cap = 64;
    auto q = round_like(randn(static_cast<size_t>(B) * Hq * T * D, 11, 0.5f), dt);
    auto k = round_like(randn(static_cast<size_t>(B) * Hkv * T * D, 12, 0.5f), dt);
    auto v = round_like(randn(static_cast<size_t>(B) * Hkv * T * D, 13, 0.5f), dt);
    Tensor tq = to_cuda(q, {B, Hq, T, D}, dt), tk = to_cuda(k, {B, Hkv, T, D}, dt), tv = to_cuda(v, {B, Hkv, T, D}, dt);
    Tensor full = nn::fused_attention(tq, tk, tv, nullptr, 0, true, 10000.0f, true);
    // oracle for the full pass
    std::vector<float> kc(static_cast<size_t>(B) * Hkv * cap * D, 0.f), vc(kc.size(), 0.f), o_cpu(q.size());
    int64_t cur = 0;
    vo_gqa_attention_cached(q.data(), k.data(), v.data(), kc.data(), vc.data(), o_cpu.data(), nullptr, B, Hq, Hkv, T, D, cap, 0, 10000.0f, 1, &cur);
    float worst = 0.f;
    CHECK(allclose(to_host(full), o_cpu, 0.f, tol, &worst));
    std::printf("  uncached vs oracle Hq%d Hkv%d dtype %d: max diff %.3g\n", Hq, Hkv, static_cast<int>(dt), worst);
    // prefill 16 tokens, then decode one by one
    nn::KVCache cache(B, Hkv, cap, D, Device::CUDA, dt);
    int P = 16;
    Tensor o_pre = nn::fused_attention(tq.narrow(2, 0, P), tk.narrow(2, 0, P), tv.narrow(2, 0, P), &cache, 0);
    CHECK(cache.current_seq_len() == P);
    auto hf = to_host(full);
    auto cmp_rows = [&](const Tensor& part, int t0, int nt) {
        auto hp = to_host(part);
        for (int b = 0; b < B; ++b) for (int h = 0; h < Hq; ++h) for (int t = 0; t < nt; ++t) for (int d = 0; d < D; ++d) {
            float a = hp[((static_cast<size_t>(b) * Hq + h) * nt + t) * D + d];
            float e = hf[((static_cast<size_t>(b) * Hq + h) * T + t0 + t) * D + d];
            CHECK(std::fabs(a - e) <= tol);
        }
    };
    cmp_rows(o_pre, 0, P);
    for (int t = P; t < T; ++t) {
        Tensor o1 = nn::fused_attention(tq.narrow(2, t, 1), tk.narrow(2, t, 1), tv.narrow(2, t, 1), &cache, t);
        cmp_rows(o1, t, 1);
    }
    CHECK(cache.current_seq_len() == T);
}

static void test_rope_table_and_rotation() {    // tests/test_rope.cpp:11-73
    Tensor f = nn::functional::compute_rope_frequencies(4, 8, 0, 10000.0f, Device::CPU);
    std::vector<float> h(16);
    f.copy_to_host(h.data());
    CHECK(h[0] == 0.f && std::fabs(h[4] - 1.0f) < 1e-7f && std::fabs(h[3 * 4 + 1] - 3.0f * std::pow(10000.0f, -0.25f)) < 1e-6f);
    std::vector<float> ref(16);
    vo_rope_frequencies(4, 8, 0, 10000.0f, ref.data());
    CHECK(h == ref);
    // rotation vs the oracle (bit-identical tables, fp32 products rounded separately)
    int B = 1, H = 2, S = 5, D = 64;
    auto x = randn(static_cast<size_t>(B) * H * S * D, 21);
    Tensor fr = nn::functional::compute_rope_frequencies(S, D, 1000, 10000.0f, Device::CUDA);
    Tensor y = nn::functional::apply_rotary_emb(to_cuda(x, {B, H, S, D}), fr);
    std::vector<float> fh(static_cast<size_t>(S) * D / 2), y_cpu(x.size());
    vo_rope_frequencies(S, D, 1000, 10000.0f, fh.data());
    vo_apply_rotary_emb(x.data(), fh.data(), y_cpu.data(), B, H, S, D);
    CHECK(to_host(y) == y_cpu);
}

static void test_repeat_kv_pattern() {          // tests/test_gqa_chapter33.cpp:76-118
    int B = 2, KVH = 2, S = 3, D = 8, n_rep = 3;
    std::vector<float> x(static_cast<size_t>(B) * KVH * S * D);
    for (size_t i = 0; i < x.size(); ++i) x[i] = static_cast<float>(i);
    Tensor y = ops::repeat_kv(to_cuda(x, {B, KVH, S, D}), n_rep);
    CHECK(y.shape() == (std::vector<int64_t>{B, KVH * n_rep, S, D}));
    std::vector<float> y_cpu(x.size() * n_rep);
    vo_repeat_kv(x.data(), y_cpu.data(), B, KVH, S, D, n_rep);
    CHECK(to_host(y) == y_cpu);
    // on a strided cache view too (where the reference's dispatcher goes wrong)
    nn::KVCache cache(B, KVH, 6, D, Device::CUDA);
    auto views = cache.update(to_cuda(x, {B, KVH, S, D}), to_cuda(x, {B, KVH, S, D}), 0);
    CHECK(!views.first.is_contiguous());
    CHECK(to_host(ops::repeat_kv(views.first, n_rep)) == y_cpu);
    CHECK(ops::repeat_kv(views.first, 1).data_ptr<float>() == views.first.data_ptr<float>());   // n_rep 1: input returned
}

static void test_sdpa_routes() {                // src/nn/functional.cpp:370-422
    int B = 1, H = 2, D = 64;
    for (int S : {37, 512}) {                    // below and at the reference's flash threshold
        size_t n = static_cast<size_t>(B) * H * S * D;
        auto q = randn(n, 31, 0.5f), k = randn(n, 32, 0.5f), v = randn(n, 33, 0.5f);
        std::vector<float> o_cpu(n);
        CHECK(vo_sdpa(q.data(), k.data(), v.data(), o_cpu.data(), B, H, S, S, D, 1) == 0);
        Tensor o = nn::functional::scaled_dot_product_attention(to_cuda(q, {B, H, S, D}), to_cuda(k, {B, H, S, D}), to_cuda(v, {B, H, S, D}), true);
        CHECK(allclose(to_host(o), o_cpu, 1e-3f, 1e-4f));
    }
    // the decode shape: one query row against L cached keys, non-causal (src/nn/functional.cpp:399-421); key and
    // value are inputs and must come back untouched.  fp32 / head_dim 64 takes the read-only-cache prefill route,
    // bf16 / head_dim 128 the split-KV decode kernel.
    struct Case { int L, D; DType dt; float atol; };
    for (const Case& c : {Case{37, 64, DType::Float32, 1e-4f}, Case{300, 128, DType::BFloat16, 1e-2f}, Case{300, 128, DType::Float16, 2e-3f}}) {
        const int Bq = 2, Hh = 4;
        size_t nq = static_cast<size_t>(Bq) * Hh * c.D, nk = nq * c.L;
        auto q = round_like(randn(nq, 34, 0.5f), c.dt), k = round_like(randn(nk, 35, 0.5f), c.dt), v = round_like(randn(nk, 36, 0.5f), c.dt);
        std::vector<float> o_cpu(nq);
        vo_sdpa_standard(q.data(), k.data(), v.data(), o_cpu.data(), nullptr, Bq, Hh, 1, c.L, c.D, 0);
        Tensor tk = to_cuda(k, {Bq, Hh, c.L, c.D}, c.dt), tv = to_cuda(v, {Bq, Hh, c.L, c.D}, c.dt);
        Tensor o = nn::functional::scaled_dot_product_attention(to_cuda(q, {Bq, Hh, 1, c.D}, c.dt), tk, tv, false);
        CHECK(o.shape() == (std::vector<int64_t>{Bq, Hh, 1, c.D}));
        CHECK(allclose(to_host(o), o_cpu, 0.f, c.atol));
        CHECK(to_host(tk) == k && to_host(tv) == v);
    }
}

static void test_flash_backward() {             // tests/test_flash_attention.cpp:292-339: d(sum(out)) exists, finite, non-zero
    int B = 1, H = 2, N = 16, D = 32;
    size_t n = static_cast<size_t>(B) * H * N * D;
    float scale = 1.0f / std::sqrt(static_cast<float>(D));
    auto q = randn(n, 41), k = randn(n, 42), v = randn(n, 43);
    std::vector<float> ones(n, 1.0f), o(n), lse(static_cast<size_t>(B) * H * N), dq(n), dk(n), dv(n);
    vo_flash_attention_fwd(q.data(), k.data(), v.data(), o.data(), lse.data(), B, H, N, D, scale, 1);
    vo_flash_attention_bwd(ones.data(), q.data(), k.data(), v.data(), o.data(), lse.data(), dq.data(), dk.data(), dv.data(), B, H, N, D, scale, 1);
    Tensor tq = to_cuda(q, {B, H, N, D}), tk = to_cuda(k, {B, H, N, D}), tv = to_cuda(v, {B, H, N, D});
    auto fwd = ops::flash_attention_with_lse(tq, tk, tv, scale, true);
    auto g = ops::flash_attention_backward(to_cuda(ones, {B, H, N, D}), tq, tk, tv, fwd.first, fwd.second, scale, true);
    auto gq = to_host(std::get<0>(g)), gk = to_host(std::get<1>(g)), gv = to_host(std::get<2>(g));
    CHECK(std::get<0>(g).shape() == tq.shape());
    bool nonzero = false;
    for (float x : gq) { CHECK(std::isfinite(x)); nonzero = nonzero || x != 0.f; }
    CHECK(nonzero);
    CHECK(allclose(gq, dq, 1e-3f, 1e-4f) && allclose(gk, dk, 1e-3f, 1e-4f) && allclose(gv, dv, 1e-3f, 1e-4f));
}

static void test_modules() {                    // nn::Linear (bias), FusedQKVLinear views, RMSNorm, SwiGLUMLP vs the CPU oracle
    const int M = 6, in_f = 256, out_f = 384, hid = 320;
    auto x = round_like(randn(static_cast<size_t>(M) * in_f, 51), DType::BFloat16);
    auto w = round_like(randn(static_cast<size_t>(out_f) * in_f, 52, 0.06f), DType::BFloat16);
    auto b = randn(out_f, 53);
    std::vector<float> y(static_cast<size_t>(M) * out_f);
    vo_linear(x.data(), w.data(), y.data(), M, out_f, in_f);
    for (int m = 0; m < M; ++m) for (int n = 0; n < out_f; ++n) y[static_cast<size_t>(m) * out_f + n] += b[n];
    nn::Linear lin(in_f, out_f, true);
    lin.load_weight(w.data(), b.data());
    Tensor tx = to_cuda(x, {2, 3, in_f}, DType::BFloat16);
    Tensor ty = lin.forward(tx);
    CHECK(ty.shape() == (std::vector<int64_t>{2, 3, out_f}));
    CHECK(allclose(to_host(ty), y, 1.0f / 128, 2e-3f));
    nn::FusedQKVLinear qkv(in_f, 256, 64, false);
    qkv.load_weight(w.data());                                   // 256 + 2 * 64 = 384 rows
    auto parts = qkv.forward_split(tx);
    CHECK(std::get<0>(parts).shape().back() == 256 && std::get<1>(parts).shape().back() == 64 && std::get<2>(parts).shape().back() == 64);
    CHECK(std::get<1>(parts).strides()[1] == 384);               // views of the fused output, not copies
    auto h = randn(static_cast<size_t>(M) * in_f, 54, 3.0f);
    auto g = randn(in_f, 55, 0.1f);
    for (auto& v : g) v += 1.0f;
    std::vector<float> hn(h.size());
    vo_rms_norm(h.data(), g.data(), hn.data(), M, in_f, 1e-6f);
    nn::RMSNorm norm({in_f}, 1e-6f);
    norm.load_weight(g.data());
    CHECK(allclose(to_host(norm.forward(to_cuda(h, {M, in_f}))), hn, 1.0f / 128, 1e-5f));
    auto wg = round_like(randn(static_cast<size_t>(hid) * in_f, 56, 0.06f), DType::BFloat16), wu = round_like(randn(static_cast<size_t>(hid) * in_f, 57, 0.06f), DType::BFloat16);
    auto wd = round_like(randn(static_cast<size_t>(in_f) * hid, 58, 0.06f), DType::BFloat16);
    std::vector<float> a(static_cast<size_t>(M) * hid), u(a.size()), act(a.size()), out(static_cast<size_t>(M) * in_f);
    vo_linear(x.data(), wg.data(), a.data(), M, hid, in_f);
    vo_linear(x.data(), wu.data(), u.data(), M, hid, in_f);
    vo_silu_mul(a.data(), u.data(), act.data(), static_cast<int64_t>(act.size()));
    vo_linear(act.data(), wd.data(), out.data(), M, in_f, hid);
    nn::SwiGLUMLP mlp(in_f, hid);
    mlp.load_weights(wg.data(), wu.data(), wd.data());
    CHECK(allclose(to_host(mlp.forward(tx)), out, 2.0f / 128, 3e-3f));
    CHECK(nn::SwiGLUMLP::compute_hidden_dim(2048) == 5632);      // src/nn/swiglu.cpp:50-61
}

static void test_model_generate() {             // cached decode == full forward; greedy loop shape and determinism
    models::TransformerConfig c;
    c.vocab_size = 128; c.dim = 256; c.n_layers = 2; c.n_heads = 2; c.n_kv_heads = 1; c.ffn_hidden_dim = 320; c.max_seq_len = 32;
    c.norm_eps = 1e-6f;
    models::TransformerLM m(c);
    unsigned seed = 100;
    for (auto& kv : m.parameter_shapes()) {
        size_t n = 1;
        for (auto d : kv.second) n *= static_cast<size_t>(d);
        auto w = kv.second.size() == 1 ? std::vector<float>(n, 1.0f) : randn(n, seed++, 0.06f);
        m.load_parameter(kv.first, w.data(), static_cast<int64_t>(n));
    }
    bool threw = false;
    Tensor ids = empty({2, 10}, DType::Int32, Device::CPU);
    for (int i = 0; i < 20; ++i) ids.data_ptr<int32_t>()[i] = (7 * i + 3) % 128;
    try { m.forward_with_cache(ids, 0); } catch (const std::runtime_error& e) { threw = std::string(e.what()).find("KV cache not initialized") != std::string::npos; }
    CHECK(threw);
    m.init_cache(2, Device::CUDA);
    CHECK(m.has_cache());
    auto full = to_host(m.forward_with_cache(ids, 0));                       // [2, 10, 128]
    m.init_cache(2, Device::CUDA);
    Tensor head = empty({2, 9}, DType::Int32, Device::CPU), last = empty({2, 1}, DType::Int32, Device::CPU);
    for (int b = 0; b < 2; ++b) {
        for (int t = 0; t < 9; ++t) head.data_ptr<int32_t>()[b * 9 + t] = ids.data_ptr<int32_t>()[b * 10 + t];
        last.data_ptr<int32_t>()[b] = ids.data_ptr<int32_t>()[b * 10 + 9];
    }
    m.forward_with_cache(head, 0);
    auto step = to_host(m.forward_with_cache(last, 9));                      // [2, 1, 128]
    float scale = 0.f;
    for (float x : full) scale = std::max(scale, std::fabs(x));
    for (int b = 0; b < 2; ++b)
        for (int vv = 0; vv < 128; ++vv) CHECK(std::fabs(step[b * 128 + vv] - full[(b * 10 + 9) * 128 + vv]) <= 2e-2f * scale);
    generation::Generator gen(&m);
    generation::SamplingParams sp;
    sp.do_sample = false; sp.max_new_tokens = 8;
    Tensor a = gen.generate(ids, sp), b2 = gen.generate(ids, sp);
    CHECK(a.shape()[0] == 2 && a.shape()[1] == 18 && a.dtype() == DType::Int32);
    CHECK(gen.last_timings().graph_replay && gen.last_timings().decode_steps == 7);
    for (int i = 0; i < 36; ++i) CHECK(a.data_ptr<int32_t>()[i] == b2.data_ptr<int32_t>()[i]);      // deterministic
    for (int b = 0; b < 2; ++b) for (int t = 0; t < 10; ++t) CHECK(a.data_ptr<int32_t>()[b * 18 + t] == ids.data_ptr<int32_t>()[b * 10 + t]);
    sp.do_sample = true;
    threw = false;
    try { gen.generate(ids, sp); } catch (const std::runtime_error&) { threw = true; }
    CHECK(threw);
    CHECK(!m.has_cache());                                                    // generate() clears the cache (generator.cpp:133)
}

int main() {
    std::printf("flash attention: GPU vs CPU\n");
    test_flash_vs_cpu(2, 4, 64, 64, false, DType::Float32, 1e-2f, 1e-3f);
    test_flash_vs_cpu(2, 8, 128, 64, true, DType::Float32, 1e-2f, 1e-3f);
    test_flash_vs_cpu(4, 2, 32, 128, true, DType::Float32, 1e-2f, 1e-3f);
    test_flash_vs_cpu(2, 4, 300, 128, true, DType::BFloat16, 0.f, 1e-2f);
    test_flash_vs_cpu(1, 2, 200, 64, false, DType::Float16, 0.f, 2e-3f);
    test_flash_large_is_finite();
    test_flash_errors();
    std::printf("kv cache\n");
    test_kv_cache_basic();
    test_cached_equals_uncached(4, 4, DType::Float32, 1e-4f);
    test_cached_equals_uncached(8, 2, DType::Float32, 1e-4f);
    test_cached_equals_uncached(8, 2, DType::BFloat16, 1e-2f);
    std::printf("rope / repeat_kv / sdpa\n");
    test_rope_table_and_rotation();
    test_repeat_kv_pattern();
    test_sdpa_routes();
    std::printf("flash backward / model / generator\n");
    test_flash_backward();
    test_modules();
    test_model_generate();
    std::printf("All B200 host-layer tests passed\n");
    return 0;
}
