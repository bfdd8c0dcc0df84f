"""Generate the golden vectors under tests/golden from the UNMODIFIED reference.

Run where the reference tree is mounted:

    make -C oracle ref            # builds oracle/_ref/libvesper_ref.so from the reference sources
    python tests/golden/make_golden.py

Every .npz holds the inputs and the outputs the reference's own CPU code
produced for them (through oracle/ref_shim.cpp).  The reference entry point
behind each file is named in CASES below.  The files are what pins the plain-C
oracle (tests/test_oracle_golden.py) on machines without the reference tree.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle.binding import Ref  # noqa: E402


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


def main():
    r = Ref()

    # -- config 1: ops::manual_seed(0); randn q,k,v; flash_attention_cpu_dispatch
    #    (src/ops/flash_attention.cpp:218-364), B=1 H=8 S=256 D=64 causal, scale 1/8.
    q, k, v = r.randn_seq(0, [(1, 8, 256, 64)] * 3)
    o, lse = r.flash_attention(q, k, v, 0.125, True)
    o_sdpa = r.sdpa(q, k, v, True)   # standard path (S<512), src/nn/functional.cpp:399-421
    save("c1_flash_fp32", q=q, k=k, v=v, o=o, lse=lse, o_sdpa=o_sdpa, scale=np.float32(0.125))

    # -- the shapes tests/test_flash_attention.cpp uses (:110-179, :195-284), plus ragged N
    rng = np.random.default_rng(1234)
    for name, (B, H, N, D), causal in [
        ("flash_b2h4n64d64_noncausal", (2, 4, 64, 64), False),
        ("flash_b2h8n128d64_causal", (2, 8, 128, 64), True),
        ("flash_b4h2n32d128_causal", (4, 2, 32, 128), True),
        ("flash_b1h2n50d64_causal", (1, 2, 50, 64), True),
        ("flash_b1h2n33d128_noncausal", (1, 2, 33, 128), False),
        ("flash_b1h1n1d64_causal", (1, 1, 1, 64), True),
        ("flash_b1h2n130d128_causal", (1, 2, 130, 128), True),
    ]:
        q, k, v = (rng.standard_normal((B, H, N, D), dtype=np.float32) for _ in range(3))
        scale = np.float32(1.0 / np.sqrt(D))
        o, lse = r.flash_attention(q, k, v, float(scale), causal)
        save(name, q=q, k=k, v=v, o=o, lse=lse, scale=scale, causal=np.int32(causal))

    # -- the router at S>=512: functional::scaled_dot_product_attention -> flash
    #    (src/nn/functional.cpp:385-395), one head S=512 D=64.
    q, k, v = (rng.standard_normal((1, 1, 512, 64), dtype=np.float32) for _ in range(3))
    save("sdpa_router_s512", q=q, k=k, v=v, o=r.sdpa(q, k, v, True))

    # -- standard path with q_len != kv_len (decode shape), non-causal
    q = rng.standard_normal((2, 4, 1, 64), dtype=np.float32)
    k, v = (rng.standard_normal((2, 4, 37, 64), dtype=np.float32) for _ in range(2))
    save("sdpa_decode_t1_l37", q=q, k=k, v=v, o=r.sdpa(q, k, v, False))

    # -- RoPE: compute_rope_frequencies + apply_rotary_emb (src/nn/functional.cpp:424-494)
    for name, (B, H, S, D), sp, theta in [
        ("rope_s8d64_pos0", (1, 2, 8, 64), 0, 10000.0),
        ("rope_s5d128_pos1000", (2, 2, 5, 128), 1000, 10000.0),
        ("rope_s3d128_pos131000", (1, 1, 3, 128), 131000, 10000.0),
        ("rope_s4d32_theta500k", (1, 1, 4, 32), 7, 500000.0),
    ]:
        x = rng.standard_normal((B, H, S, D), dtype=np.float32)
        save(name, x=x, freqs=r.rope_frequencies(S, D, sp, theta), y=r.apply_rope(x, sp, theta),
             start_pos=np.int32(sp), theta=np.float32(theta))

    # -- ops::repeat_kv (src/ops/attention_ops.cpp:92-130) on contiguous input
    x = rng.standard_normal((2, 2, 5, 16), dtype=np.float32)
    save("repeat_kv_n3", x=x, y=r.repeat_kv(x, 3), n_rep=np.int32(3))

    # -- nn::KVCache::update (src/nn/transformer.cpp:56-93): prefill 3 rows, then 2 appends
    c = r.kvcache(2, 2, 8, 4)
    steps = {}
    pos = 0
    for i, T in enumerate([3, 1, 1]):
        nk, nv = (rng.standard_normal((2, 2, T, 4), dtype=np.float32) for _ in range(2))
        ko, vo = c.update(nk, nv, pos)
        steps.update({f"new_k{i}": nk, f"new_v{i}": nv, f"k_view{i}": ko, f"v_view{i}": vo,
                      f"start{i}": np.int32(pos)})
        pos += T
    save("kvcache_update", **steps)

    # -- GQA attention core with cache (src/nn/gqa_attention.cpp:111-159 composed from
    #    reference ops with contiguous cache views): prefill T=8 at pos 0, then 4 decode steps.
    for name, (B, Hq, Hkv, D, cap, T0, nsteps) in [
        ("gqa_cached_b2hq4hkv2d32", (2, 4, 2, 32, 64, 8, 4)),
        ("gqa_cached_b1hq8hkv2d128", (1, 8, 2, 128, 160, 70, 3)),
        ("mha_cached_b2h2d64", (2, 2, 2, 64, 32, 5, 3)),
    ]:
        c = r.kvcache(B, Hkv, cap, D)
        out = {"dims": np.array([B, Hq, Hkv, D, cap, T0, nsteps], np.int32)}
        pos = 0
        for i in range(nsteps + 1):
            T = T0 if i == 0 else 1
            qq = rng.standard_normal((B, Hq, T, D), dtype=np.float32)
            kk = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
            vv = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
            out.update({f"q{i}": qq, f"k{i}": kk, f"v{i}": vv,
                        f"o{i}": r.gqa_attention_cached(c, qq, kk, vv, pos, 10000.0, True)})
            pos += T
        save(name, **out)

    # -- module level: GroupedQueryAttention::forward(x, causal) (uncached; right for any
    #    n_rep) with caller-set weights.  C=64, Hq=4, Hkv=2, D=16, T=12.
    Cdim, Hq, Hkv, T = 64, 4, 2, 12
    D = Cdim // Hq
    wqkv = (0.1 * rng.standard_normal(((Hq + 2 * Hkv) * D, Cdim))).astype(np.float32)
    wo = (0.1 * rng.standard_normal((Cdim, Hq * D))).astype(np.float32)
    x = rng.standard_normal((2, T, Cdim), dtype=np.float32)
    g = r.gqa(Cdim, Hq, Hkv, 64, 10000.0, wqkv, wo)
    save("gqa_module_forward", wqkv=wqkv, wo=wo, x=x, y=g.forward(x, True),
         dims=np.array([Cdim, Hq, Hkv, T], np.int32))

    # -- module level: MultiHeadAttention (src/nn/transformer.cpp:97-216), c_attn = Linear(C, 3C) and c_proj with BIAS:
    #    forward(x) (non-causal, :108-110), forward(x, causal=True), and forward(x, cache, pos) as a prompt pass of
    #    T=9 then two single-token steps (Hkv == Hq: the reference's cached path is right); with and without RoPE.
    Cm, Hm, Tm = 64, 4, 9
    for tag, use_rope in (("rope", True), ("norope", False)):
        rngm = np.random.default_rng(900 + int(use_rope))
        w_attn = (0.1 * rngm.standard_normal((3 * Cm, Cm))).astype(np.float32)
        b_attn = (0.1 * rngm.standard_normal(3 * Cm)).astype(np.float32)
        w_proj = (0.1 * rngm.standard_normal((Cm, Cm))).astype(np.float32)
        b_proj = (0.1 * rngm.standard_normal(Cm)).astype(np.float32)
        x = rngm.standard_normal((2, Tm + 2, Cm), dtype=np.float32)
        m = r.mha(Cm, Hm, use_rope, w_attn, b_attn, w_proj, b_proj)
        c = r.kvcache(2, Hm, 16, Cm // Hm)
        save("mha_module_" + tag, w_attn=w_attn, b_attn=b_attn, w_proj=w_proj, b_proj=b_proj, x=x,
             y_default=m.forward(x[:, :Tm]), y_causal=m.forward(x[:, :Tm], True),
             y_cached_prefill=m.forward_cached(c, x[:, :Tm], 0), y_cached_step1=m.forward_cached(c, x[:, Tm:Tm + 1], Tm),
             y_cached_step2=m.forward_cached(c, x[:, Tm + 1:Tm + 2], Tm + 1), dims=np.array([Cm, Hm, Tm, int(use_rope)], np.int32))

    # -- ops::flash_attention_backward (src/ops/flash_attention.cpp:165-215, CPU form :366-482), the shapes of
    #    tests/test_flash_attention.cpp:295,345 plus a ragged one, causal and not
    bw = {}
    for tag, (B, H, N, D, causal) in {"a": (1, 2, 16, 32, True), "b": (1, 1, 8, 16, True), "c": (1, 2, 45, 64, False)}.items():
        rng2 = np.random.default_rng(700 + N)
        q, k, v, do = [rng2.standard_normal((B, H, N, D)).astype(np.float32) for _ in range(4)]
        sc = np.float32(1.0 / np.sqrt(D))
        o, lse = r.flash_attention(q, k, v, float(sc), causal)
        dq, dk, dv = r.flash_attention_bwd(do, q, k, v, o, lse, float(sc), causal)
        bw.update({f"{tag}_q": q, f"{tag}_k": k, f"{tag}_v": v, f"{tag}_do": do, f"{tag}_o": o, f"{tag}_lse": lse,
                   f"{tag}_dq": dq, f"{tag}_dk": dk, f"{tag}_dv": dv, f"{tag}_scale": sc, f"{tag}_causal": np.int32(causal)})
    save("flash_backward", **bw)
    block_and_model_fixtures(r)


MODEL_CASES = {
    # name: (vocab, dim, n_layers, n_heads, n_kv_heads, ffn_hidden, max_seq_len, weight seed, B, T)
    "model_gqa_d128": (384, 256, 2, 2, 1, 320, 48, 21, 2, 20),     # grouped-query, head_dim 128
    "model_gqa_d64": (384, 256, 1, 4, 2, 320, 48, 22, 2, 20),      # grouped-query, head_dim 64
    "model_mha_d128": (384, 256, 2, 2, 2, 320, 48, 23, 2, 12),     # Hkv == Hq: the reference's cached path and Generator are usable
}


def block_and_model_fixtures(r):
    """Decoder-block operators and models::TransformerLM through the reference's own classes."""
    sys.path.insert(0, os.path.join(HERE, ".."))
    from helpers import bf16_round, model_weights
    from vesper_b200.model import param_shapes
    rng = np.random.default_rng(4321)
    # -- nn::Linear::forward = matmul(x, W^T) (src/nn/linear.cpp:41-48; src/ops/cpu/gemm_cpu.cpp:12-48)
    x = bf16_round(rng.standard_normal((9, 200)).astype(np.float32))
    w = bf16_round((rng.standard_normal((70, 200)) / 14.0).astype(np.float32))
    g = (1.0 + 0.1 * rng.standard_normal(200)).astype(np.float32)
    gate = rng.standard_normal((9, 70)).astype(np.float32) * 3.0
    up = rng.standard_normal((9, 70)).astype(np.float32)
    ids = rng.integers(0, 70, size=(11,)).astype(np.int32)
    logits = rng.standard_normal((5, 333)).astype(np.float32)
    logits[2, 10] = logits[2, 300] = 8.0            # a tie: the first index wins (src/ops/sampling_ops.cpp:28-33)
    save("block_ops", x=x, w=w, y_linear=r.linear(x, w), g=g, y_rms=r.rms_norm(x, g, 1e-6), eps=np.float32(1e-6),
         gate=gate, up=up, y_silu_mul=r.silu_mul(gate, up), ids=ids, y_embedding=r.embedding(ids, w),
         logits=logits, y_argmax=r.argmax(logits))
    # -- models::TransformerLM::forward (uncached, causal; src/models/transformer.cpp:97-150) on seeded weights
    #    (tests/helpers.py: model_weights(param_shapes, seed, std=0.06)); for the MHA case also
    #    forward_with_cache (:152-188) and generation::Generator::generate greedy (src/generation/generator.cpp:36-142).
    for name, (vocab, dim, n_layers, Hq, Hkv, ffn, max_seq, seed, B, T) in MODEL_CASES.items():
        shapes = param_shapes(vocab, dim, n_layers, Hq, Hkv, ffn)
        wts = model_weights(shapes, seed, std=0.06)
        m = r.model(vocab, dim, n_layers, Hq, Hkv, ffn, max_seq)
        assert {k: tuple(v) for k, v in m.param_shapes().items()} == shapes
        for k, v in wts.items():
            m.set_param(k, v)
        tok = np.random.default_rng(seed + 100).integers(0, vocab, size=(B, T)).astype(np.int32)
        out = dict(cfg=np.array([vocab, dim, n_layers, Hq, Hkv, ffn, max_seq, seed], np.int64), ids=tok, logits=m.forward(tok))
        if Hkv == Hq:
            m.init_cache(B)
            out["logits_cached_prefill"] = m.forward_with_cache(tok, 0)
            out["logits_cached_step"] = m.forward_with_cache(tok[:, :1], T)
            out["greedy"] = m.generate_greedy(tok, 10)
        save(name, **out)


if __name__ == "__main__":
    main()
