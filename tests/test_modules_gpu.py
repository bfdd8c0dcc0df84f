"""nn::GroupedQueryAttention and nn::MultiHeadAttention of the host layer (the reference's module surface:
include/vesper/nn/gqa_attention.h:27-101, include/vesper/nn/transformer.h:41-56) on the GPU, against fixtures the
UNMODIFIED reference modules produced (tests/golden/make_golden.py) and against the oracle composition.

Float32 modules must reproduce the reference at 1e-4; BFloat16 modules (the serving format) within 2e-2 of it on
these O(1) outputs (weights, activations and the attention probabilities are rounded to bf16 between operators);
cached forward == uncached forward through the classes, which the reference's own GQA path does not achieve when
num_rep > 1 (it reads the strided cache views as if contiguous, src/ops/attention_ops.cpp:34-52).
"""
import numpy as np
import pytest

from helpers import bf16_round, golden, maxabs

pytestmark = pytest.mark.gpu


def gqa_from_fixture(dtype):
    from vesper_b200.model import AttentionModule
    g = golden("gqa_module_forward")
    Cdim, Hq, Hkv, T = (int(v) for v in g["dims"])
    m = AttentionModule("gqa", Cdim, Hq, Hkv, max_seq_len=64, rope_base=10000.0, dtype=dtype)
    m.load(g["wqkv"], g["wo"])
    return m, g, (Cdim, Hq, Hkv, T)


def test_gqa_module_fp32_matches_the_reference_module(lib, cuda):
    """GroupedQueryAttention::forward(x) and forward(x, causal=true) (src/nn/gqa_attention.cpp:63-109), Float32:
    the reference-made fixture at 1e-4."""
    m, g, _ = gqa_from_fixture("f32")
    assert maxabs(m.forward(g["x"], True), g["y"]) <= 1e-4
    assert maxabs(m.forward(g["x"]), g["y"]) <= 1e-4            # forward(x) is causal


def oracle_attention_module(oracle, x, w_in, b_in, w_out, b_out, Hq, Hkv, kc, vc, start, cur):
    """The module composed from the oracle's operators on bf16-rounded activations: input projection (+ bias) ->
    [B,H,T,D] -> RoPE + cache + grouped attention (src/nn/gqa_attention.cpp:111-159) -> merge heads -> output projection."""
    B, T, C_ = x.shape
    D = C_ // Hq
    qkv = oracle.linear(x.reshape(-1, C_), w_in)
    if b_in is not None:
        qkv = qkv + b_in
    qkv = bf16_round(qkv).reshape(B, T, Hq + 2 * Hkv, D)
    q = np.ascontiguousarray(qkv[:, :, :Hq].transpose(0, 2, 1, 3))
    k = np.ascontiguousarray(qkv[:, :, Hq:Hq + Hkv].transpose(0, 2, 1, 3))
    v = np.ascontiguousarray(qkv[:, :, Hq + Hkv:].transpose(0, 2, 1, 3))
    o, _, cur = oracle.gqa_attention_cached(q, k, v, kc, vc, start, cur)
    merged = bf16_round(o.transpose(0, 2, 1, 3).reshape(-1, C_))
    y = oracle.linear(merged, w_out)
    if b_out is not None:
        y = y + b_out
    return y.reshape(B, T, C_), cur


def test_gqa_module_bf16_and_cached_equals_uncached(lib, cuda, oracle):
    """The serving format through the GQA class at head_dim 128 with two query heads per KV head: uncached causal
    forward against the oracle composition, then the same sequence as a prompt pass and two single-token steps through
    forward(x, cache, start_pos) -- which must agree with the uncached result (the reference's own cached GQA path does
    not when the cache is not full)."""
    from vesper_b200.model import AttentionModule, KVCache
    Cdim, Hq, Hkv, T, B = 512, 4, 2, 70, 2
    D = Cdim // Hq
    rng = np.random.default_rng(33)
    wqkv = bf16_round((0.05 * rng.standard_normal(((Hq + 2 * Hkv) * D, Cdim))).astype(np.float32))
    wo = bf16_round((0.05 * rng.standard_normal((Cdim, Cdim))).astype(np.float32))
    x = bf16_round(rng.standard_normal((B, T, Cdim)).astype(np.float32))
    m = AttentionModule("gqa", Cdim, Hq, Hkv, max_seq_len=128, rope_base=10000.0, dtype="bf16")
    m.load(wqkv, wo)
    y = m.forward(x, True)
    kc, vc = np.zeros((B, Hkv, 128, D), np.float32), np.zeros((B, Hkv, 128, D), np.float32)
    want, _ = oracle_attention_module(oracle, x, wqkv, None, wo, None, Hq, Hkv, kc, vc, 0, 0)
    assert maxabs(y, want) <= 2e-2
    cache = KVCache(B, Hkv, 128, D, "bf16")
    y0 = m.forward_cached(cache, x[:, :T - 2], 0)
    y1 = m.forward_cached(cache, x[:, T - 2:T - 1], T - 2)
    y2 = m.forward_cached(cache, x[:, T - 1:T], T - 1)
    assert len(cache) == T
    got = np.concatenate([y0, y1, y2], axis=1)
    assert maxabs(got, y) <= 1e-2                                # same kernels; the bf16 cache rounds the rotated K once more
    assert maxabs(got, want) <= 2e-2


def test_gqa_module_fp32_cached_equals_uncached(lib, cuda):
    from vesper_b200.model import KVCache
    m, g, (Cdim, Hq, Hkv, T) = gqa_from_fixture("f32")
    cache = KVCache(g["x"].shape[0], Hkv, 64, Cdim // Hq, "f32")
    parts = [m.forward_cached(cache, g["x"][:, :5], 0)]
    for t in range(5, T):
        parts.append(m.forward_cached(cache, g["x"][:, t:t + 1], t))
    assert maxabs(np.concatenate(parts, axis=1), g["y"]) <= 1e-4


def test_gqa_module_constructor_validation(lib, cuda):
    from vesper_b200.model import AttentionModule
    with pytest.raises(RuntimeError, match="must be divisible by num_kv_heads"):
        AttentionModule("gqa", 64, 4, 3)
    with pytest.raises(RuntimeError, match="must be divisible by num_heads"):
        AttentionModule("gqa", 66, 4, 2)


@pytest.mark.parametrize("tag", ["rope", "norope"])
def test_mha_module_fp32_matches_the_reference_module(lib, cuda, tag):
    """MultiHeadAttention (src/nn/transformer.cpp:97-216) with c_attn = Linear(C, 3C) + bias: forward(x) is
    non-causal, forward(x, true) causal, forward(x, cache, pos) a prompt pass and two steps; with and without RoPE."""
    from vesper_b200.model import AttentionModule, KVCache
    g = golden("mha_module_" + tag)
    Cm, Hm, Tm, use_rope = (int(v) for v in g["dims"])
    m = AttentionModule("mha", Cm, Hm, use_rope=bool(use_rope), dtype="f32")
    m.load(g["w_attn"], g["w_proj"], g["b_attn"], g["b_proj"])
    x = g["x"]
    assert maxabs(m.forward(x[:, :Tm]), g["y_default"]) <= 1e-4
    assert maxabs(m.forward(x[:, :Tm], True), g["y_causal"]) <= 1e-4
    assert maxabs(g["y_default"], g["y_causal"]) > 1e-2           # the two really differ: forward(x) must not mask
    cache = KVCache(x.shape[0], Hm, 16, Cm // Hm, "f32")
    assert maxabs(m.forward_cached(cache, x[:, :Tm], 0), g["y_cached_prefill"]) <= 1e-4
    assert maxabs(m.forward_cached(cache, x[:, Tm:Tm + 1], Tm), g["y_cached_step1"]) <= 1e-4
    assert maxabs(m.forward_cached(cache, x[:, Tm + 1:Tm + 2], Tm + 1), g["y_cached_step2"]) <= 1e-4


def test_mha_module_bf16_head_dim_128(lib, cuda, oracle):
    """The serving format through the MHA class at head_dim 128 (tensor-core prefill, split-KV decode): against the
    oracle composition Linear + bias -> RoPE -> cache -> attention -> Linear + bias on the same bf16-rounded values."""
    from vesper_b200.model import AttentionModule, KVCache
    Cm, Hm, T, B = 256, 2, 40, 2
    D = Cm // Hm
    rng = np.random.default_rng(31)
    w_attn = bf16_round((0.06 * rng.standard_normal((3 * Cm, Cm))).astype(np.float32))
    b_attn = (0.1 * rng.standard_normal(3 * Cm)).astype(np.float32)
    w_proj = bf16_round((0.06 * rng.standard_normal((Cm, Cm))).astype(np.float32))
    b_proj = (0.1 * rng.standard_normal(Cm)).astype(np.float32)
    x = bf16_round(rng.standard_normal((B, T + 1, Cm)).astype(np.float32))
    m = AttentionModule("mha", Cm, Hm, use_rope=True, dtype="bf16")
    m.load(w_attn, w_proj, b_attn, b_proj)
    cache = KVCache(B, Hm, 64, D, "bf16")
    y0 = m.forward_cached(cache, x[:, :T], 0)
    y1 = m.forward_cached(cache, x[:, T:], T)

    def want(xs, start, kc, vc, cur):
        return oracle_attention_module(oracle, xs, w_attn, b_attn, w_proj, b_proj, Hm, Hm, kc, vc, start, cur)

    kc, vc = np.zeros((B, Hm, 64, D), np.float32), np.zeros((B, Hm, 64, D), np.float32)
    w0, cur = want(x[:, :T], 0, kc, vc, 0)
    w1, cur = want(x[:, T:], T, kc, vc, cur)
    assert cur == T + 1 == len(cache)
    assert maxabs(y0, w0) <= 2e-2 and maxabs(y1, w1) <= 2e-2
