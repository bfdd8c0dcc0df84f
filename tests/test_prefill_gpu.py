"""Parity of the CUDA prefill / flash-attention path (through the C ABI) with the CPU oracle.

Gates: fp32 path within 1e-4 of the oracle (the reference's own CPU-vs-GPU
tolerance is rtol 1e-2 / atol 1e-3, tests/test_flash_attention.cpp:217,243);
bf16 max-abs <= 1e-2, fp16 <= 2e-3, LSE <= 1e-3, all against the fp32 oracle on
the same (rounded) input values.
"""
import ctypes as C

import numpy as np
import pytest

from helpers import bf16_round, fp16_round, from_torch, golden, maxabs, to_torch

pytestmark = pytest.mark.gpu

FLASH_CASES = [
    "c1_flash_fp32", "flash_b2h4n64d64_noncausal", "flash_b2h8n128d64_causal", "flash_b4h2n32d128_causal",
    "flash_b1h2n50d64_causal", "flash_b1h2n33d128_noncausal", "flash_b1h1n1d64_causal", "flash_b1h2n130d128_causal",
]


def run_flash(capi, cuda, q, k, v, dtype, scale, causal):
    import torch
    tq, tk, tv = (to_torch(x, dtype, cuda) for x in (q, k, v))
    o = torch.empty_like(tq)
    lse = torch.empty(tq.shape[:3], dtype=torch.float32, device=cuda)
    capi.prefill(tq, tk, tv, o, lse, scale=scale, causal=causal)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    return from_torch(o), from_torch(lse)


@pytest.mark.parametrize("name", FLASH_CASES)
def test_fp32_flash_matches_reference_golden(lib, cuda, name):
    import torch
    from vesper_b200 import capi
    g = golden(name)
    causal = bool(g["causal"]) if "causal" in g else True
    o, lse = run_flash(capi, cuda, g["q"], g["k"], g["v"], torch.float32, float(g["scale"]), causal)
    assert maxabs(o, g["o"]) <= 1e-4
    assert maxabs(lse, g["lse"]) <= 1e-4


def test_fp32_strided_views(lib, cuda):
    """q/k/v given as [B,T,H,D] storage viewed as [B,H,T,D] (the layout the QKV
    projection produces, src/nn/gqa_attention.cpp:120-122) must need no copy."""
    import torch
    from vesper_b200 import capi
    from oracle.binding import Oracle
    rng = np.random.default_rng(7)
    B, H, T, D = 2, 3, 70, 64
    q, k, v = (rng.standard_normal((B, T, H, D), dtype=np.float32) for _ in range(3))
    tq, tk, tv = (to_torch(x, torch.float32, cuda).transpose(1, 2) for x in (q, k, v))
    o = torch.empty(B, T, H, D, device=cuda).transpose(1, 2)
    capi.prefill(tq, tk, tv, o, None, scale=0.125, causal=True)
    torch.cuda.synchronize()
    want, _ = Oracle().flash_attention(q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3), 0.125, True)
    assert maxabs(from_torch(o), want) <= 1e-4


SHAPES_16BIT = [
    # B, Hq, Hkv, S, D, causal
    (1, 2, 2, 128, 128, True),
    (1, 2, 1, 256, 128, True),
    (2, 4, 2, 300, 128, True),
    (1, 1, 1, 1, 128, True),
    (1, 2, 2, 257, 128, False),
    (1, 4, 1, 640, 128, True),
    (2, 2, 2, 200, 64, True),
    (1, 2, 1, 384, 64, False),
]


@pytest.mark.parametrize("shape", SHAPES_16BIT)
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_16bit_flash_matches_oracle(lib, cuda, oracle, shape, dt):
    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, S, D, causal = shape
    rng = np.random.default_rng(100 + S + D)
    rnd = bf16_round if dt == "bf16" else fp16_round
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    q = rnd(0.5 * rng.standard_normal((B, Hq, S, D), dtype=np.float32))
    k = rnd(0.5 * rng.standard_normal((B, Hkv, S, D), dtype=np.float32))
    v = rnd(0.5 * rng.standard_normal((B, Hkv, S, D), dtype=np.float32))
    scale = float(1.0 / np.sqrt(D))
    o, lse = run_flash(capi, cuda, q, k, v, tdt, scale, causal)
    want_o, want_lse = oracle.flash_attention(q, oracle.repeat_kv(k, Hq // Hkv), oracle.repeat_kv(v, Hq // Hkv), scale, causal)
    tol = 1e-2 if dt == "bf16" else 2e-3
    assert np.isfinite(o).all()
    assert maxabs(o, want_o) <= tol
    assert maxabs(lse, want_lse) <= 1e-3


@pytest.mark.parametrize("dt", ["bf16", "fp32"])
def test_rope_append_prefill_then_chunk(lib, cuda, oracle, dt):
    """RoPE(Q,K) + KV append + causal attention in one call, at start_pos 0 and
    then a second chunk at start_pos > 0 (bottom-right aligned mask)."""
    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, D, cap = 2, 8, 2, 128, 512
    T0, T1 = 200, 72
    rng = np.random.default_rng(21)
    rnd = bf16_round if dt == "bf16" else (lambda x: np.asarray(x, np.float32))
    tdt = torch.bfloat16 if dt == "bf16" else torch.float32
    tol = 1e-2 if dt == "bf16" else 2e-4
    kc = torch.zeros(B, Hkv, cap, D, dtype=tdt, device=cuda)
    vc = torch.zeros_like(kc)
    okc = np.zeros((B, Hkv, cap, D), np.float32)
    ovc = np.zeros_like(okc)
    cur, pos = 0, 0
    scale = float(1.0 / np.sqrt(D))
    for T in (T0, T1):
        q = rnd(0.5 * rng.standard_normal((B, Hq, T, D), dtype=np.float32))
        k = rnd(0.5 * rng.standard_normal((B, Hkv, T, D), dtype=np.float32))
        v = rnd(0.5 * rng.standard_normal((B, Hkv, T, D), dtype=np.float32))
        tq, tk, tv = (to_torch(x, tdt, cuda) for x in (q, k, v))
        o = torch.empty_like(tq)
        lse = torch.empty(B, Hq, T, dtype=torch.float32, device=cuda)
        capi.prefill(tq, tk, tv, o, lse, scale=scale, causal=True, start_pos=pos, theta=10000.0, k_cache=kc, v_cache=vc)
        torch.cuda.synchronize()
        capi.check_kernel_status(0)
        want_o, want_lse, cur = oracle.gqa_attention_cached(q, k, v, okc, ovc, pos, cur)
        assert maxabs(from_torch(o), want_o) <= tol, f"chunk at {pos}"
        assert maxabs(from_torch(lse), want_lse) <= 1e-3
        pos += T
    # cache contents: rotated K within one rounding of the oracle's fp32 K, V exact, tail untouched
    gk, gv = from_torch(kc), from_torch(vc)
    rel = 2.0 ** -8 if dt == "bf16" else 1e-6
    assert np.all(np.abs(gk[:, :, :cur] - okc[:, :, :cur]) <= rel * np.abs(okc[:, :, :cur]) + 1e-6)
    assert np.array_equal(gv[:, :, :cur], ovc[:, :, :cur])
    assert not gk[:, :, cur:].any() and not gv[:, :, cur:].any()


def test_config2_full_size_every_slice_against_the_oracle(lib, cuda, oracle):
    """GQA causal prefill at the benchmark size: B=4, Hq=32, Hkv=8, S=2048, D=128, bf16,
    RoPE theta 1e4, append into an empty cache of capacity 4096.  Size-independent
    checks on everything, and oracle parity on ALL 128 (batch, head) slices (the oracle
    calls run on the host cores in parallel): O <= 1e-2, LSE <= 1e-3, rotated K in the
    cache within one bf16 rounding (2^-8 relative)."""
    import os
    from concurrent.futures import ThreadPoolExecutor

    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, S, D, cap = 4, 32, 8, 2048, 128, 4096
    g = torch.Generator(device="cpu").manual_seed(1)
    q = (0.5 * torch.randn(B, Hq, S, D, generator=g)).to(torch.bfloat16)
    k = (0.5 * torch.randn(B, Hkv, S, D, generator=g)).to(torch.bfloat16)
    v = (0.5 * torch.randn(B, Hkv, S, D, generator=g)).to(torch.bfloat16)
    tq, tk, tv = q.to(cuda), k.to(cuda), v.to(cuda)
    kc = torch.zeros(B, Hkv, cap, D, dtype=torch.bfloat16, device=cuda)
    vc = torch.zeros_like(kc)
    o = torch.empty_like(tq)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=cuda)
    scale = float(1.0 / np.sqrt(D))
    capi.prefill(tq, tk, tv, o, lse, scale=scale, causal=True, theta=10000.0, k_cache=kc, v_cache=vc)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    # causal row 0 attends to key 0 only: O[.,h,0,:] == V[., h/4, 0, :] and LSE == scale * q0.k0 (position 0: no rotation)
    assert torch.equal(o[:, :, 0, :], tv[:, :, 0, :].repeat_interleave(Hq // Hkv, dim=1))
    s00 = scale * (tq[:, :, 0, :].float() * tk[:, :, 0, :].float().repeat_interleave(Hq // Hkv, dim=1)).sum(-1)
    assert (lse[:, :, 0] - s00).abs().max().item() <= 1e-3
    # V appended bit-exactly, rows past S untouched, K row 0 unrotated
    assert torch.equal(vc[:, :, :S], tv) and not vc[:, :, S:].any() and not kc[:, :, S:].any()
    assert torch.equal(kc[:, :, 0], tk[:, :, 0])
    # oracle parity, every (batch, head)
    qf, kf, vf = q.float().numpy(), k.float().numpy(), v.float().numpy()
    go, glse, gk = from_torch(o), from_torch(lse), from_torch(kc[:, :, :S])
    n_rep = Hq // Hkv

    def one(bh):
        b, h = divmod(bh, Hq)
        hk = h // n_rep
        okc = np.zeros((1, 1, S, D), np.float32)
        ovc = np.zeros_like(okc)
        want_o, want_lse, _ = oracle.gqa_attention_cached(qf[b:b + 1, h:h + 1], kf[b:b + 1, hk:hk + 1], vf[b:b + 1, hk:hk + 1], okc, ovc, 0, 0)
        k_ok = True
        if h % n_rep == 0:
            k_ok = bool(np.all(np.abs(gk[b, hk] - okc[0, 0]) <= 2.0 ** -8 * np.abs(okc[0, 0]) + 1e-6))
        return maxabs(go[b, h], want_o[0, 0]), maxabs(glse[b, h], want_lse[0, 0]), k_ok

    with ThreadPoolExecutor(max_workers=max(1, min(32, os.cpu_count() or 1))) as ex:
        res = list(ex.map(one, range(B * Hq)))
    worst_o = max(r[0] for r in res)
    worst_l = max(r[1] for r in res)
    bad = [divmod(i, Hq) for i, r in enumerate(res) if r[0] > 1e-2 or r[1] > 1e-3 or not r[2]]
    assert not bad, f"(batch, head) slices outside the gates: {bad[:8]} (worst O {worst_o:.3e}, LSE {worst_l:.3e})"


def test_sdpa_decode_shape_reads_a_cache_it_does_not_write(lib, cuda):
    """scaled_dot_product_attention's T < L shape (src/nn/functional.cpp:399-421): one query row against 37
    keys, non-causal, fp32, head_dim 64 -- the reference-made fixture -- through cache_read_only, which must
    leave key and value untouched; then 3 query rows against 40 keys, bottom-right causal, bf16."""
    import torch
    from vesper_b200 import capi
    from oracle.binding import Oracle
    g = golden("sdpa_decode_t1_l37")
    tq, tk, tv = (to_torch(g[n], torch.float32, cuda) for n in ("q", "k", "v"))
    k0, v0 = tk.clone(), tv.clone()
    o = torch.empty_like(tq)
    L = tk.shape[2]
    capi.prefill(tq, None, None, o, None, scale=float(1.0 / np.sqrt(64)), causal=False, start_pos=L - 1,
                 k_cache=tk, v_cache=tv, cache_read_only=True)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    assert maxabs(from_torch(o), g["o"]) <= 1e-4
    assert torch.equal(tk, k0) and torch.equal(tv, v0)
    # 16-bit, several query rows, bottom-right aligned mask, GQA
    rng = np.random.default_rng(5)
    B, Hq, Hkv, T, L, D = 2, 4, 2, 3, 40, 128
    q = bf16_round(0.5 * rng.standard_normal((B, Hq, T, D), dtype=np.float32))
    k = bf16_round(0.5 * rng.standard_normal((B, Hkv, L, D), dtype=np.float32))
    v = bf16_round(0.5 * rng.standard_normal((B, Hkv, L, D), dtype=np.float32))
    tq, tk, tv = (to_torch(x, torch.bfloat16, cuda) for x in (q, k, v))
    k0, v0 = tk.clone(), tv.clone()
    o = torch.empty_like(tq)
    capi.prefill(tq, None, None, o, None, scale=float(1.0 / np.sqrt(D)), causal=True, start_pos=L - T,
                 k_cache=tk, v_cache=tv, cache_read_only=True)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    orc = Oracle()
    # the same through the oracle: append the last T rows (already in place) onto a cache holding the first L - T
    okc, ovc = k.copy(), v.copy()
    want, _, _ = orc.gqa_attention_cached(q, k[:, :, L - T:], v[:, :, L - T:], okc, ovc, L - T, L - T, use_rope=False)
    assert maxabs(from_torch(o), want) <= 1e-2
    assert torch.equal(tk, k0) and torch.equal(tv, v0)


def test_argument_errors_are_status_codes(lib, cuda):
    import torch
    from vesper_b200 import capi
    q = torch.zeros(1, 3, 16, 128, dtype=torch.bfloat16, device=cuda)
    k = torch.zeros(1, 2, 16, 128, dtype=torch.bfloat16, device=cuda)
    o = torch.empty_like(q)
    with pytest.raises(capi.Vb200Error) as e:          # Hq % Hkv != 0
        capi.prefill(q, k, k, o, None, scale=1.0)
    assert e.value.status == -1
    q2 = torch.zeros(1, 2, 16, 96, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(capi.Vb200Error) as e:          # head_dim without a tensor-core kernel
        capi.prefill(q2, q2, q2, torch.empty_like(q2), None, scale=1.0)
    assert e.value.status == -2
    base = torch.zeros(2 * 16 * 128 + 4, dtype=torch.bfloat16, device=cuda)
    q3 = base[4:].view(1, 2, 16, 128)                  # 8-byte aligned only
    with pytest.raises(capi.Vb200Error) as e:
        capi.prefill(q3, k, k, torch.empty_like(q3), None, scale=1.0)
    assert e.value.status == -3
    a = capi.prefill_args(q[:, :2], k, k, o[:, :2], None, scale=1.0, theta=10000.0)
    assert lib.vb200_prefill_workspace_bytes(C.byref(a)) > 0
    assert lib.vb200_prefill_fwd(C.byref(a)) == -4     # rope needs a workspace
    a.struct_size = 8
    assert lib.vb200_prefill_fwd(C.byref(a)) == -1
    torch.cuda.synchronize()
    capi.check_kernel_status(0)


def test_prefill_chunk_at_far_position(lib, cuda, oracle):
    """A prompt chunk appended behind 20000 cached keys: RoPE angles ~2e4 rad (where the fp32
    angle pos*f of the reference is itself coarse, so every row must use the exact table) and a
    bottom-right aligned causal mask over 158 key blocks."""
    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, D, P, T = 1, 2, 1, 128, 20000, 200
    cap = P + 256
    rng = np.random.default_rng(77)
    okc = np.zeros((B, Hkv, cap, D), np.float32)
    ovc = np.zeros_like(okc)
    okc[:, :, :P] = bf16_round(rng.standard_normal((B, Hkv, P, D), dtype=np.float32))
    ovc[:, :, :P] = bf16_round(rng.standard_normal((B, Hkv, P, D), dtype=np.float32))
    kc, vc = to_torch(okc, torch.bfloat16, cuda), to_torch(ovc, torch.bfloat16, cuda)
    q = bf16_round(rng.standard_normal((B, Hq, T, D), dtype=np.float32))
    k = bf16_round(rng.standard_normal((B, Hkv, T, D), dtype=np.float32))
    v = bf16_round(rng.standard_normal((B, Hkv, T, D), dtype=np.float32))
    tq, tk, tv = (to_torch(x, torch.bfloat16, cuda) for x in (q, k, v))
    o = torch.empty_like(tq)
    lse = torch.empty(B, Hq, T, dtype=torch.float32, device=cuda)
    scale = float(1.0 / np.sqrt(D))
    capi.prefill(tq, tk, tv, o, lse, scale=scale, causal=True, start_pos=P, theta=10000.0, k_cache=kc, v_cache=vc)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    want_o, want_lse, cur = oracle.gqa_attention_cached(q, k, v, okc, ovc, P, P)
    assert cur == P + T
    assert maxabs(from_torch(o), want_o) <= 1e-2
    assert maxabs(from_torch(lse), want_lse) <= 2e-3     # scores of |s| ~ 10 with K rounded to bf16 in the cache
    gk = from_torch(kc)
    assert np.all(np.abs(gk[:, :, P:P + T] - okc[:, :, P:P + T]) <= 2.0 ** -8 * np.abs(okc[:, :, P:P + T]) + 1e-6)


def test_output_rows_aligned_to_16_but_not_32_bytes(cuda, oracle):
    """O with a row stride of 136 elements (272 bytes): every other row starts 16 bytes off a 32-byte
    boundary, which the 32-byte stores of the epilogue must not be used for."""
    import torch
    from vesper_b200 import capi
    B, H, S, D = 1, 2, 200, 128
    rng = np.random.default_rng(9)
    q, k, v = [bf16_round(0.5 * rng.standard_normal((B, H, S, D)).astype(np.float32)) for _ in range(3)]
    scale = float(1.0 / np.sqrt(D))
    want, want_lse = oracle.flash_attention(q, k, v, scale, True)
    buf = torch.zeros(B, H, S, 136, dtype=torch.bfloat16, device=cuda)
    o = buf[..., :D]
    lse = torch.empty(B, H, S, dtype=torch.float32, device=cuda)
    capi.prefill(to_torch(q, torch.bfloat16, cuda), to_torch(k, torch.bfloat16, cuda), to_torch(v, torch.bfloat16, cuda), o, lse, scale=scale, causal=True)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    assert maxabs(from_torch(o), want) <= 1e-2 and maxabs(from_torch(lse), want_lse) <= 1e-3
    assert bool((buf[..., D:] == 0).all())
