"""The plain-C oracle against the golden vectors the UNMODIFIED reference produced
(tests/golden/make_golden.py), and against the compiled reference where present."""
import numpy as np
import pytest

from helpers import golden, maxabs

FLASH_CASES = [
    "c1_flash_fp32", "flash_b2h4n64d64_noncausal", "flash_b2h8n128d64_causal", "flash_b4h2n32d128_causal",
    "flash_b1h2n50d64_causal", "flash_b1h2n33d128_noncausal", "flash_b1h1n1d64_causal", "flash_b1h2n130d128_causal",
]


@pytest.mark.parametrize("name", FLASH_CASES)
def test_flash_matches_reference_bits(oracle, name):
    g = golden(name)
    causal = bool(g["causal"]) if "causal" in g else True
    o, lse = oracle.flash_attention(g["q"], g["k"], g["v"], float(g["scale"]), causal)
    # same operation order as src/ops/flash_attention.cpp:218-364 -> identical fp32 results
    assert maxabs(o, g["o"]) <= 1e-6
    assert maxabs(lse, g["lse"]) <= 1e-6
    assert np.array_equal(o, g["o"]) and np.array_equal(lse, g["lse"])


def test_config1_smoke_values(oracle):
    g = golden("c1_flash_fp32")
    assert abs(float(g["q"].flat[0]) - 2.21221) < 1e-5      # libstdc++ stream after manual_seed(0)
    assert abs(float(g["o"][0, 0, 0, 0]) - 0.714812) < 1e-6  # causal row 0 = v[0]
    o_std = oracle.sdpa(g["q"], g["k"], g["v"], True)        # standard path (S < 512)
    assert np.array_equal(o_std, g["o_sdpa"])
    assert maxabs(o_std, g["o"]) < 2e-6


def test_router_takes_flash_at_512(oracle):
    g = golden("sdpa_router_s512")
    assert np.array_equal(oracle.sdpa(g["q"], g["k"], g["v"], True), g["o"])


def test_standard_path_decode_shape(oracle):
    g = golden("sdpa_decode_t1_l37")
    assert np.array_equal(oracle.sdpa(g["q"], g["k"], g["v"], False), g["o"])


@pytest.mark.parametrize("name", ["rope_s8d64_pos0", "rope_s5d128_pos1000", "rope_s3d128_pos131000", "rope_s4d32_theta500k"])
def test_rope(oracle, name):
    g = golden(name)
    S, D = g["x"].shape[2], g["x"].shape[3]
    f = oracle.rope_frequencies(S, D, int(g["start_pos"]), float(g["theta"]))
    assert np.array_equal(f, g["freqs"])
    assert np.array_equal(oracle.apply_rope(g["x"], int(g["start_pos"]), float(g["theta"])), g["y"])


def test_rope_known_answers(oracle):
    # tests/test_rope.py-style analytic checks (tests/test_rope.cpp:11-73): theta table and a 90 degree turn
    f = oracle.rope_frequencies(4, 8, 0, 10000.0)
    assert f[0].tolist() == [0.0] * 4 and abs(f[1, 0] - 1.0) < 1e-7 and abs(f[3, 1] - 3 * 10000.0 ** (-0.25)) < 1e-6
    x = np.zeros((1, 1, 1, 2), np.float32)
    x[..., 0] = 1.0
    import ctypes as C
    y = np.empty_like(x)
    ang = np.array([[np.pi / 2]], np.float32)
    oracle.lib.vo_apply_rotary_emb(x.ctypes.data_as(C.POINTER(C.c_float)), ang.ctypes.data_as(C.POINTER(C.c_float)),
                                   y.ctypes.data_as(C.POINTER(C.c_float)), 1, 1, 1, 2)
    assert abs(y[0, 0, 0, 0]) < 1e-6 and abs(y[0, 0, 0, 1] - 1.0) < 1e-6


def test_repeat_kv(oracle):
    g = golden("repeat_kv_n3")
    assert np.array_equal(oracle.repeat_kv(g["x"], int(g["n_rep"])), g["y"])


def test_kvcache_update(oracle):
    g = golden("kvcache_update")
    kc = np.zeros((2, 2, 8, 4), np.float32)
    vc = np.zeros_like(kc)
    cur = 0
    for i in range(3):
        cur = oracle.kv_cache_update(kc, vc, g[f"new_k{i}"], g[f"new_v{i}"], int(g[f"start{i}"]), cur)
        assert np.array_equal(kc[:, :, :cur], g[f"k_view{i}"]) and np.array_equal(vc[:, :, :cur], g[f"v_view{i}"])
    assert cur == 5 and not kc[:, :, cur:].any()      # rows past current_len stay zero


@pytest.mark.parametrize("name", ["gqa_cached_b2hq4hkv2d32", "gqa_cached_b1hq8hkv2d128", "mha_cached_b2h2d64"])
def test_gqa_attention_with_cache(oracle, name):
    g = golden(name)
    B, Hq, Hkv, D, cap, T0, nsteps = (int(x) for x in g["dims"])
    kc = np.zeros((B, Hkv, cap, D), np.float32)
    vc = np.zeros_like(kc)
    cur, pos = 0, 0
    for i in range(nsteps + 1):
        T = T0 if i == 0 else 1
        o, lse, cur = oracle.gqa_attention_cached(g[f"q{i}"], g[f"k{i}"], g[f"v{i}"], kc, vc, pos, cur)
        assert np.array_equal(o, g[f"o{i}"]), f"step {i}"
        pos += T
    assert cur == T0 + nsteps


def test_cached_decode_equals_uncached_row(oracle):
    """Property the reference's cache tests assert (tests/test_kv_cache_chapter33.cpp:66-188):
    token-by-token cached attention reproduces the causal full-sequence result."""
    rng = np.random.default_rng(3)
    B, Hq, Hkv, D, S = 1, 4, 2, 32, 12
    q = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    kc = np.zeros((B, Hkv, 16, D), np.float32); vc = np.zeros_like(kc)
    full, _, _ = oracle.gqa_attention_cached(q, k, v, kc.copy(), vc.copy(), 0, 0)
    cur = 0
    for t in range(S):
        o, _, cur = oracle.gqa_attention_cached(q[:, :, t:t + 1], k[:, :, t:t + 1], v[:, :, t:t + 1], kc, vc, t, cur)
        assert maxabs(o[:, :, 0], full[:, :, t]) < 1e-5


def test_lse_combine_matches_full_softmax(oracle):
    rng = np.random.default_rng(5)
    H, L, D, R = 3, 96, 16, 4
    q = rng.standard_normal((1, H, 1, D), dtype=np.float32)
    k = rng.standard_normal((1, H, L, D), dtype=np.float32)
    v = rng.standard_normal((1, H, L, D), dtype=np.float32)
    full, sc = oracle.sdpa_standard(q, k, v, False, want_scores=True)
    ms, ls, os_ = [], [], []
    for r in range(R):
        sl = slice(r * L // R, (r + 1) * L // R)
        o_r, s_r = oracle.sdpa_standard(q, k[:, :, sl], v[:, :, sl], False, want_scores=True)
        m = s_r.max(-1)[0, :, 0]
        ms.append(m); ls.append(np.exp(s_r[0, :, 0] - m[:, None]).sum(-1)); os_.append(o_r[0, :, 0])
    out, lse = oracle.lse_combine(np.stack(ms), np.stack(ls), np.stack(os_))
    assert maxabs(out, full[0, :, 0]) < 1e-5
    ref_lse = np.log(np.exp(sc[0, :, 0].astype(np.float64)).sum(-1))
    assert maxabs(lse, ref_lse) < 1e-5


def test_oracle_equals_compiled_reference(oracle, ref):
    """Where the reference tree was compiled (oracle/_ref) the restatement is checked live as well."""
    q, k, v = ref.randn_seq(11, [(1, 2, 70, 64)] * 3)
    ro, rl = ref.flash_attention(q, k, v, 0.125, True)
    oo, ol = oracle.flash_attention(q, k, v, 0.125, True)
    assert np.array_equal(ro, oo) and np.array_equal(rl, ol)
    assert np.array_equal(ref.apply_rope(q, 77, 10000.0), oracle.apply_rope(q, 77, 10000.0))


def test_reference_gqa_cache_defect_is_real(ref, oracle):
    """The reference's own cached GQA forward differs from its uncached forward when
    n_rep > 1 and cap != len (strided repeat_kv, src/ops/attention_ops.cpp:34-52);
    the oracle composition does not."""
    g = golden("gqa_module_forward")
    Cdim, Hq, Hkv, T = (int(x) for x in g["dims"])
    m = ref.gqa(Cdim, Hq, Hkv, 64, 10000.0, g["wqkv"], g["wo"])
    y_uncached = m.forward(g["x"], True)
    assert np.array_equal(y_uncached, g["y"])
    cache = ref.kvcache(2, Hkv, 32, Cdim // Hq)
    y_cached = m.forward_cached(cache, g["x"], 0)
    assert maxabs(y_cached, y_uncached) > 1e-2
