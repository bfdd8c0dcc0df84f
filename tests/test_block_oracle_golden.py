"""The CPU oracle for the decoder-block operators and its model composition, pinned to outputs of
the UNMODIFIED reference (tests/golden/block_ops.npz, model_*.npz, made by tests/golden/make_golden.py)
and, where the compiled reference is present, to the reference itself."""
import numpy as np
import pytest

from helpers import OracleDecoder, golden, model_weights
from vesper_b200.model import param_shapes

MODELS = ["model_gqa_d128", "model_gqa_d64", "model_mha_d128"]


def test_block_ops_bit_exact_against_reference_fixture(oracle):
    g = golden("block_ops")
    assert np.array_equal(oracle.linear(g["x"], g["w"]), g["y_linear"])                 # same summation order
    assert np.array_equal(oracle.rms_norm(g["x"], g["g"], float(g["eps"])), g["y_rms"])
    assert np.array_equal(oracle.silu_mul(g["gate"], g["up"]), g["y_silu_mul"])
    assert np.array_equal(oracle.embedding(g["ids"], g["w"]), g["y_embedding"])
    assert np.array_equal(oracle.argmax(g["logits"]), g["y_argmax"]) and g["y_argmax"][2] == 10


def test_block_ops_bit_exact_against_live_reference(oracle, ref):
    rng = np.random.default_rng(99)
    x = rng.standard_normal((7, 130)).astype(np.float32)
    w = rng.standard_normal((33, 130)).astype(np.float32)
    assert np.array_equal(oracle.linear(x, w), ref.linear(x, w))
    gw = rng.standard_normal(130).astype(np.float32)
    assert np.array_equal(oracle.rms_norm(x, gw, 1e-5), ref.rms_norm(x, gw, 1e-5))
    assert np.array_equal(oracle.silu_mul(x, x[::-1].copy()), ref.silu_mul(x, x[::-1].copy()))
    lg = rng.standard_normal((3, 999)).astype(np.float32)
    assert np.array_equal(oracle.argmax(lg), ref.argmax(lg))


def test_embedding_rejects_out_of_range_ids(oracle):
    with pytest.raises(IndexError):
        oracle.embedding(np.array([0, 5], np.int32), np.zeros((5, 8), np.float32))


def test_check_stop_tokens(oracle):
    tok = np.array([3, 9, 4, 9], np.int32)
    assert list(oracle.check_stop_tokens(tok, [9, 4], 0, 1)) == [0, 1, 1, 1]
    assert list(oracle.check_stop_tokens(tok, [9, 4], 5, 4)) == [0, 0, 0, 0]      # below min_new_tokens nothing stops


def _decoder(oracle, g):
    vocab, dim, n_layers, Hq, Hkv, ffn, max_seq, seed = [int(v) for v in g["cfg"]]
    w = model_weights(param_shapes(vocab, dim, n_layers, Hq, Hkv, ffn), seed, std=0.06)
    return OracleDecoder(oracle, w, n_layers=n_layers, n_heads=Hq, n_kv_heads=Hkv, max_seq_len=max_seq)


@pytest.mark.parametrize("name", MODELS)
def test_model_composition_matches_reference_forward(oracle, name):
    """Prompt pass of the oracle composition (RoPE + cache + GQA attention) vs TransformerLM::forward
    of the reference; the two use different attention code paths, hence 1e-4 and not bit equality."""
    g = golden(name)
    d = _decoder(oracle, g)
    B, T = g["ids"].shape
    d.init_cache(B)
    got = d.forward_with_cache(g["ids"], 0)
    assert np.abs(got - g["logits"]).max() <= 1e-4 * max(1.0, np.abs(g["logits"]).max())
    # token by token through the cache gives the same logits as the full pass
    d.init_cache(B)
    d.forward_with_cache(g["ids"][:, : T - 3], 0)
    for t in range(T - 3, T):
        step = d.forward_with_cache(g["ids"][:, t:t + 1], t)[:, 0]
        assert np.abs(step - g["logits"][:, t]).max() <= 1e-4 * max(1.0, np.abs(g["logits"]).max())


def test_greedy_generation_matches_reference_generator(oracle):
    g = golden("model_mha_d128")
    d = _decoder(oracle, g)
    toks, _ = d.generate_greedy(g["ids"], 10)
    assert np.array_equal(toks, g["greedy"])
    # the reference's own cached path (usable because Hkv == Hq) agrees with its uncached forward
    assert np.abs(g["logits_cached_prefill"] - g["logits"]).max() <= 1e-4 * np.abs(g["logits"]).max()


def test_flash_backward_bit_exact_against_reference_fixture(oracle):
    """vo_flash_attention_bwd vs ops::flash_attention_backward of the reference (same loop order)."""
    g = golden("flash_backward")
    for tag in "abc":
        dq, dk, dv = oracle.flash_attention_bwd(g[f"{tag}_do"], g[f"{tag}_q"], g[f"{tag}_k"], g[f"{tag}_v"], g[f"{tag}_o"], g[f"{tag}_lse"],
                                                float(g[f"{tag}_scale"]), bool(g[f"{tag}_causal"]))
        assert np.array_equal(dq, g[f"{tag}_dq"]) and np.array_equal(dk, g[f"{tag}_dk"]) and np.array_equal(dv, g[f"{tag}_dv"])
    # numerical gradient of sum(out) w.r.t. a few q entries (tests/test_flash_attention.cpp:341-420)
    q, k, v = g["b_q"].copy(), g["b_k"], g["b_v"]
    sc = float(g["b_scale"])
    o, lse = oracle.flash_attention(q, k, v, sc, True)
    dq, _, _ = oracle.flash_attention_bwd(np.ones_like(o), q, k, v, o, lse, sc, True)
    for idx in [(0, 0, 0, 0), (0, 0, 3, 5), (0, 0, 7, 15)]:
        eps = 1e-3
        qp, qm = q.copy(), q.copy()
        qp[idx] += eps
        qm[idx] -= eps
        num = (oracle.flash_attention(qp, k, v, sc, True)[0].sum(dtype=np.float64) - oracle.flash_attention(qm, k, v, sc, True)[0].sum(dtype=np.float64)) / (2 * eps)
        assert abs(num - dq[idx]) <= 5e-2 * max(1.0, abs(num))
