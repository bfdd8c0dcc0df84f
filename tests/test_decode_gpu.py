"""Parity of the split-KV decode path (through the C ABI) with the CPU oracle.

Decode oracle: the reference's standard attention path applied per sequence on
contiguous fp32 copies of the cache (src/nn/functional.cpp:399-421), RoPE and
cache update as in src/nn/gqa_attention.cpp:124-137.  Gates: bf16 max-abs <= 1e-2,
fp16 <= 2e-3, LSE <= 1e-3.
"""
import numpy as np
import pytest

from helpers import bf16_round, fp16_round, from_torch, maxabs, to_torch

pytestmark = pytest.mark.gpu


def make_cache(rng, B, Hkv, cap, D, lens, rnd):
    k = np.zeros((B, Hkv, cap, D), np.float32)
    v = np.zeros_like(k)
    for b, L in enumerate(lens):
        k[b, :, :L] = rnd(rng.standard_normal((Hkv, L, D), dtype=np.float32))
        v[b, :, :L] = rnd(rng.standard_normal((Hkv, L, D), dtype=np.float32))
    return k, v


@pytest.mark.parametrize("n_rep", [1, 2, 4, 8])
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
def test_decode_uniform_no_append(lib, cuda, oracle, n_rep, dt):
    import torch
    from vesper_b200 import capi
    B, Hkv, D, L, cap = 2, 2, 128, 300, 320
    Hq = Hkv * n_rep
    rnd = bf16_round if dt == "bf16" else fp16_round
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    rng = np.random.default_rng(40 + n_rep)
    k, v = make_cache(rng, B, Hkv, cap, D, [L] * B, rnd)
    q = rnd(rng.standard_normal((B, Hq, 1, D), dtype=np.float32))
    tq, tk, tv = to_torch(q, tdt, cuda), to_torch(k, tdt, cuda), to_torch(v, tdt, cuda)
    o = torch.empty_like(tq)
    lse = torch.empty(B, Hq, dtype=torch.float32, device=cuda)
    scale = float(1.0 / np.sqrt(D))
    capi.decode(tq, o, tk, tv, scale=scale, lse=lse, uniform_len=L, max_len=L)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    want_o, want_lse = oracle.decode_ragged(q[:, :, 0], k, v, [L] * B)
    assert maxabs(from_torch(o)[:, :, 0], want_o) <= (1e-2 if dt == "bf16" else 2e-3)
    assert maxabs(from_torch(lse), want_lse) <= 1e-3


@pytest.mark.parametrize("num_splits", [0, 1, 3, 11])
def test_decode_ragged_rope_append_steps(lib, cuda, oracle, num_splits):
    """Ragged lengths (incl. 1 and tile multiples), RoPE at position len, append, attend; three
    consecutive steps with the kernel advancing seq_lens on the device."""
    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, D, cap = 5, 8, 2, 128, 800
    lens = [1, 63, 64, 700, 512]
    rng = np.random.default_rng(50)
    k, v = make_cache(rng, B, Hkv, cap, D, lens, bf16_round)
    tk, tv = to_torch(k, torch.bfloat16, cuda), to_torch(v, torch.bfloat16, cuda)
    seq = torch.tensor(lens, dtype=torch.int32, device=cuda)
    scale = float(1.0 / np.sqrt(D))
    cur = list(lens)
    for step in range(3):
        q = bf16_round(rng.standard_normal((B, Hq, 1, D), dtype=np.float32))
        kn = bf16_round(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32))
        vn = bf16_round(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32))
        tq, tkn, tvn = (to_torch(x, torch.bfloat16, cuda) for x in (q, kn, vn))
        o = torch.empty_like(tq)
        lse = torch.empty(B, Hq, dtype=torch.float32, device=cuda)
        capi.decode(tq, o, tk, tv, scale=scale, k_new=tkn, v_new=tvn, lse=lse, theta=10000.0, seq_lens=seq,
                    advance_lens=True, max_len=max(cur) + 1, num_splits=num_splits)
        torch.cuda.synchronize()
        capi.check_kernel_status(0)
        for b in range(B):
            kc1, vc1 = k[b:b + 1].copy(), v[b:b + 1].copy()
            want_o, want_lse, n = oracle.gqa_attention_cached(q[b:b + 1], kn[b:b + 1], vn[b:b + 1], kc1, vc1, cur[b], cur[b])
            k[b], v[b] = kc1[0], vc1[0]
            assert n == cur[b] + 1
            assert maxabs(from_torch(o)[b], want_o[0]) <= 1e-2, f"step {step} seq {b}"
            assert maxabs(from_torch(lse)[b], want_lse[0, :, 0]) <= 1e-3
            cur[b] += 1
        assert seq.tolist() == cur
        # the oracle cache keeps fp32 rotated K; the device cache holds its bf16 rounding: carry the device values on
        k = from_torch(tk); v = from_torch(tv)
    # appended rows: V exact, K within one bf16 rounding; nothing written past the new length
    gk, gv = from_torch(tk), from_torch(tv)
    for b in range(B):
        assert not gk[b, :, cur[b]:].any() and not gv[b, :, cur[b]:].any()


@pytest.mark.parametrize("num_splits", [0, 11, 15])
@pytest.mark.parametrize("n_rep", [1, 4])
def test_decode_ragged_no_advance_cluster_merge(lib, cuda, oracle, num_splits, n_rep):
    """Ragged lengths with one-tile splits and no length advance: the splits of a (sequence, kv head) run as one
    thread-block cluster (sizes above 8 included) that merges its own partials; short sequences leave most members
    of their cluster without keys.  RoPE at position len, append, attend."""
    import torch
    from vesper_b200 import capi
    B, Hkv, D, cap = 5, 2, 128, 800
    Hq = Hkv * n_rep
    lens = [1, 63, 64, 700, 512]
    rng = np.random.default_rng(57 + n_rep)
    k, v = make_cache(rng, B, Hkv, cap, D, lens, bf16_round)
    tk, tv = to_torch(k, torch.bfloat16, cuda), to_torch(v, torch.bfloat16, cuda)
    seq = torch.tensor(lens, dtype=torch.int32, device=cuda)
    scale = float(1.0 / np.sqrt(D))
    q = bf16_round(rng.standard_normal((B, Hq, 1, D), dtype=np.float32))
    kn = bf16_round(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32))
    vn = bf16_round(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32))
    tq, tkn, tvn = (to_torch(x, torch.bfloat16, cuda) for x in (q, kn, vn))
    o = torch.empty_like(tq)
    lse = torch.empty(B, Hq, dtype=torch.float32, device=cuda)
    capi.decode(tq, o, tk, tv, scale=scale, k_new=tkn, v_new=tvn, lse=lse, theta=10000.0, seq_lens=seq,
                advance_lens=False, max_len=max(lens) + 1, num_splits=num_splits)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    assert seq.tolist() == lens                                   # not advanced
    for b in range(B):
        kc1, vc1 = k[b:b + 1].copy(), v[b:b + 1].copy()
        want_o, want_lse, n = oracle.gqa_attention_cached(q[b:b + 1], kn[b:b + 1], vn[b:b + 1], kc1, vc1, lens[b], lens[b])
        assert n == lens[b] + 1
        assert maxabs(from_torch(o)[b], want_o[0]) <= 1e-2, f"seq {b}"
        assert maxabs(from_torch(lse)[b], want_lse[0, :, 0]) <= 1e-3, f"seq {b}"
    # the new rows were appended at position len of each sequence, nothing beyond
    gk, gv = from_torch(tk), from_torch(tv)
    for b in range(B):
        assert np.array_equal(gv[b, :, lens[b]], vn[b, :, 0])
        assert not gk[b, :, lens[b] + 1:].any() and not gv[b, :, lens[b] + 1:].any()


def test_decode_sharded_partials_combine(lib, cuda, oracle):
    """Sequence-sharded form on one GPU: R shards of the KV sequence each emit (O/l, m, l);
    vb200_lse_combine merges them to the unsharded result (the algebra of
    src/ops/flash_attention.cpp:309-345 across shards)."""
    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, D, L, R = 1, 16, 2, 128, 4096, 4
    rng = np.random.default_rng(60)
    k, v = make_cache(rng, B, Hkv, L, D, [L], bf16_round)
    q = bf16_round(rng.standard_normal((B, Hq, 1, D), dtype=np.float32))
    scale = float(1.0 / np.sqrt(D))
    # q is rotated at the absolute position L (no new token appended): oracle applies the same
    q_rot = oracle.apply_rope(q, L, 10000.0)
    want_o, want_lse = oracle.decode_ragged(q_rot[:, :, 0], k, v, [L])
    tq = to_torch(q, torch.bfloat16, cuda)
    partials = torch.empty(R, B * Hq, D + 2, dtype=torch.float32, device=cuda)
    qpos = torch.tensor([L], dtype=torch.int32, device=cuda)
    per = L // R
    for r in range(R):
        tk = to_torch(k[:, :, r * per:(r + 1) * per], torch.bfloat16, cuda)
        tv = to_torch(v[:, :, r * per:(r + 1) * per], torch.bfloat16, cuda)
        capi.decode(tq, None, tk, tv, scale=scale, theta=10000.0, uniform_len=per, max_len=per,
                    pos_offset=r * per, q_positions=qpos, partial_out=partials[r])
    out = torch.empty(B * Hq, D, dtype=torch.bfloat16, device=cuda)
    lse = torch.empty(B * Hq, dtype=torch.float32, device=cuda)
    capi.lse_combine(partials, out, lse)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    # q was rotated in bf16 storage by neither side: both rotate the same bf16 values in fp32
    assert maxabs(from_torch(out), want_o[0]) <= 1e-2
    assert maxabs(from_torch(lse), want_lse[0]) <= 1e-3


def test_config3_full_size_steps_0_1_255(lib, cuda, oracle):
    """Batched GQA decode at the benchmark size: B=32, Hq=32, Hkv=8, D=128, ragged lengths
    U[1024, 8192]; 256 consecutive steps with RoPE + append, the kernel advancing the length
    array on the device.  Oracle parity on steps 0, 1 and 255 for 4 sequences x all heads."""
    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, D, steps = 32, 32, 8, 128, 256
    rs = np.random.RandomState(2)
    lens = rs.randint(1024, 8193, size=B).astype(np.int32)
    cap = 8192 + steps
    g = torch.Generator(device="cuda").manual_seed(3)
    tk = torch.randn(B, Hkv, cap, D, generator=g, device=cuda, dtype=torch.float32).to(torch.bfloat16)
    tv = torch.randn(B, Hkv, cap, D, generator=g, device=cuda, dtype=torch.float32).to(torch.bfloat16)
    for b in range(B):
        tk[b, :, lens[b]:] = 0
        tv[b, :, lens[b]:] = 0
    seq = torch.from_numpy(lens).to(cuda)
    o = torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=cuda)
    lse = torch.empty(B, Hq, dtype=torch.float32, device=cuda)
    scale = float(1.0 / np.sqrt(D))
    check = [0, 7, int(np.argmin(lens)), int(np.argmax(lens))]
    ws = None
    max_len = int(lens.max()) + steps
    for step in range(steps):
        gs = torch.Generator(device="cuda").manual_seed(4 + step)
        tq = torch.randn(B, Hq, 1, D, generator=gs, device=cuda).to(torch.bfloat16)
        tkn = torch.randn(B, Hkv, 1, D, generator=gs, device=cuda).to(torch.bfloat16)
        tvn = torch.randn(B, Hkv, 1, D, generator=gs, device=cuda).to(torch.bfloat16)
        checked = step in (0, 1, steps - 1)
        if checked:
            before = {b: (from_torch(tk[b:b + 1]), from_torch(tv[b:b + 1])) for b in check}
        ws = capi.decode(tq, o, tk, tv, scale=scale, k_new=tkn, v_new=tvn, lse=lse, theta=10000.0, seq_lens=seq,
                         advance_lens=True, max_len=max_len, workspace=ws)
        if not checked:
            continue
        torch.cuda.synchronize()
        capi.check_kernel_status(0)
        assert torch.isfinite(o.float()).all()
        assert seq.tolist() == (lens + step + 1).tolist()
        for b in check:
            kc1, vc1 = before[b]
            L = int(lens[b]) + step
            want_o, want_lse, n = oracle.gqa_attention_cached(from_torch(tq[b:b + 1]), from_torch(tkn[b:b + 1]), from_torch(tvn[b:b + 1]),
                                                              kc1, vc1, L, L)
            assert n == L + 1
            assert maxabs(from_torch(o[b]), want_o[0]) <= 1e-2, f"step {step} sequence {b}"
            assert maxabs(from_torch(lse[b]), want_lse[0, :, 0]) <= 1e-3, f"step {step} sequence {b}"
            assert torch.equal(tv[b, :, L], tvn[b, :, 0])
            gk = from_torch(tk[b, :, L])
            assert np.all(np.abs(gk - kc1[0, :, L]) <= 2.0 ** -8 * np.abs(kc1[0, :, L]) + 1e-6)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    # nothing was written past the final lengths
    for b in check:
        assert not tk[b, :, int(lens[b]) + steps:].any() and not tv[b, :, int(lens[b]) + steps:].any()


def test_config4_full_context_131072_keys_against_the_oracle(lib, cuda, oracle):
    """Long-context decode at the benchmark size on one GPU: B=1, Hq=64, Hkv=8, D=128, 131072 cached keys,
    the query rotated at position 131072.  Checked against the oracle's attention over all 131072 keys
    for all 64 heads (src/nn/functional.cpp:399-421 on contiguous fp32 copies; RoPE src/nn/functional.cpp:424-494):
    once as a single call, once as 8 sequence shards whose (O/l, m, l) records vb200_lse_combine merges
    (the algebra of src/ops/flash_attention.cpp:309-345)."""
    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, D, L, R = 1, 64, 8, 128, 131072, 8
    g = torch.Generator(device="cuda").manual_seed(5)
    tk = torch.randn(B, Hkv, L, D, generator=g, device=cuda, dtype=torch.float32).to(torch.bfloat16)
    tv = torch.randn(B, Hkv, L, D, generator=g, device=cuda, dtype=torch.float32).to(torch.bfloat16)
    tq = torch.randn(B, Hq, 1, D, generator=torch.Generator(device="cuda").manual_seed(6), device=cuda).to(torch.bfloat16)
    scale = float(1.0 / np.sqrt(D))
    qpos = torch.tensor([L], dtype=torch.int32, device=cuda)
    # one call over the whole context
    o1 = torch.empty_like(tq)
    lse1 = torch.empty(B, Hq, dtype=torch.float32, device=cuda)
    capi.decode(tq, o1, tk, tv, scale=scale, lse=lse1, theta=10000.0, uniform_len=L, max_len=L, q_positions=qpos)
    # eight contiguous shards, then the LSE merge
    partials = torch.empty(R, B * Hq, D + 2, dtype=torch.float32, device=cuda)
    per = L // R
    for r in range(R):
        capi.decode(tq, None, tk[:, :, r * per:(r + 1) * per], tv[:, :, r * per:(r + 1) * per], scale=scale, theta=10000.0,
                    uniform_len=per, max_len=per, pos_offset=r * per, q_positions=qpos, partial_out=partials[r])
    o8 = torch.empty(B * Hq, D, dtype=torch.bfloat16, device=cuda)
    lse8 = torch.empty(B * Hq, dtype=torch.float32, device=cuda)
    capi.lse_combine(partials, o8, lse8)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    q_rot = oracle.apply_rope(from_torch(tq), L, 10000.0)
    want_o, want_lse = oracle.decode_ragged(q_rot[:, :, 0], from_torch(tk), from_torch(tv), [L])
    assert maxabs(from_torch(o1)[:, :, 0], want_o) <= 1e-2
    assert maxabs(from_torch(lse1), want_lse) <= 1e-3
    assert maxabs(from_torch(o8), want_o[0]) <= 1e-2
    assert maxabs(from_torch(lse8), want_lse[0]) <= 1e-3


def test_decode_full_sequence_is_reported_not_overrun(lib, cuda, oracle):
    """A sequence whose length already equals the cache capacity cannot take its new token: the kernel must
    not write, not advance that length, attend to the keys it has, and leave VB200_ERR_CACHE_OVERFLOW in the
    status word; its neighbours step normally.  (The reference throws from KVCache::update,
    src/nn/transformer.cpp:62-66.)  Also a length that exceeds the planned max_len."""
    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, D, cap = 3, 8, 2, 128, 256
    for lens, max_len in (([cap, 100, 255], 0), ([200, 100, 64], 128)):
        rng = np.random.default_rng(90 + max_len)
        k, v = make_cache(rng, B, Hkv, cap, D, lens, bf16_round)
        tk, tv = to_torch(k, torch.bfloat16, cuda), to_torch(v, torch.bfloat16, cuda)
        seq = torch.tensor(lens, dtype=torch.int32, device=cuda)
        q = bf16_round(rng.standard_normal((B, Hq, 1, D), dtype=np.float32))
        kn = bf16_round(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32))
        vn = bf16_round(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32))
        tq, tkn, tvn = (to_torch(x, torch.bfloat16, cuda) for x in (q, kn, vn))
        o = torch.empty_like(tq)
        capi.decode(tq, o, tk, tv, scale=float(1.0 / np.sqrt(D)), k_new=tkn, v_new=tvn, theta=10000.0, seq_lens=seq,
                    advance_lens=True, max_len=max_len)
        torch.cuda.synchronize()
        with pytest.raises(capi.Vb200Error) as e:
            capi.check_kernel_status(0)
        assert e.value.status == -8 and "sequence 0" in str(e.value)
        capi.check_kernel_status(0)                                  # the word was cleared
        assert seq.tolist() == [lens[0], lens[1] + 1, lens[2] + 1]
        gk, gv = from_torch(tk), from_torch(tv)
        assert np.array_equal(gk[0], k[0]) and np.array_equal(gv[0], v[0])          # sequence 0: cache untouched
        assert torch.isfinite(o.float()).all()
        for b in (1, 2):
            kc1, vc1 = k[b:b + 1].copy(), v[b:b + 1].copy()
            want_o, _, _ = oracle.gqa_attention_cached(q[b:b + 1], kn[b:b + 1], vn[b:b + 1], kc1, vc1, lens[b], lens[b])
            assert maxabs(from_torch(o)[b], want_o[0]) <= 1e-2


@pytest.mark.parametrize("case", [
    # dtype, B, Hq, Hkv, D, lens, cache row stride (elements; 0 = D)
    ("fp32", 2, 4, 4, 64, [37, 300], 0),          # the reference's own cache format and a small head (tests/test_kv_cache_chapter33.cpp:66-188)
    ("fp32", 2, 6, 2, 64, [1, 129], 0),           # three query heads per KV head
    ("fp32", 1, 8, 2, 128, [700], 0),
    ("bf16", 2, 8, 2, 64, [63, 512], 0),
    ("fp16", 1, 4, 4, 32, [100], 0),
    ("bf16", 2, 8, 2, 128, [200, 90], 160),       # head_dim 128 but strided cache rows: not the tuned kernels' layout
    ("bf16", 1, 12, 2, 128, [333], 0),            # six query heads per KV head
])
def test_decode_generic_shapes_rope_append_two_steps(lib, cuda, oracle, case):
    """Split-KV decode for the shapes outside the two tuned kernels (fp32 caches, head_dim != 128, other group sizes,
    strided cache rows): ragged lengths, RoPE at position len, append, attend, two steps with the length array advanced
    on the device.  fp32 within 1e-4 of the oracle, 16-bit within the usual gates."""
    import torch
    from vesper_b200 import capi
    dt, B, Hq, Hkv, D, lens, row_stride = case
    rnd = {"fp32": (lambda x: np.asarray(x, np.float32)), "bf16": bf16_round, "fp16": fp16_round}[dt]
    tdt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[dt]
    tol, lse_tol = {"fp32": (1e-4, 1e-4), "bf16": (1e-2, 1e-3), "fp16": (2e-3, 1e-3)}[dt]
    cap = max(lens) + 8
    rng = np.random.default_rng(80 + D + Hq)
    k, v = make_cache(rng, B, Hkv, cap, D, lens, rnd)
    if row_stride:
        bk = torch.zeros(B, Hkv, cap, row_stride, dtype=tdt, device=cuda)
        bv = torch.zeros_like(bk)
        tk, tv = bk[..., :D], bv[..., :D]
        tk.copy_(to_torch(k, tdt, cuda)); tv.copy_(to_torch(v, tdt, cuda))
    else:
        tk, tv = to_torch(k, tdt, cuda), to_torch(v, tdt, cuda)
    seq = torch.tensor(lens, dtype=torch.int32, device=cuda)
    scale = float(1.0 / np.sqrt(D))
    cur = list(lens)
    for step in range(2):
        q = rnd(rng.standard_normal((B, Hq, 1, D), dtype=np.float32))
        kn = rnd(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32))
        vn = rnd(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32))
        tq, tkn, tvn = (to_torch(x, tdt, cuda) for x in (q, kn, vn))
        o = torch.empty_like(tq)
        lse = torch.empty(B, Hq, dtype=torch.float32, device=cuda)
        capi.decode(tq, o, tk, tv, scale=scale, k_new=tkn, v_new=tvn, lse=lse, theta=10000.0, seq_lens=seq,
                    advance_lens=True, max_len=max(cur) + 1, num_splits=(0 if step == 0 else 3))
        torch.cuda.synchronize()
        capi.check_kernel_status(0)
        for b in range(B):
            kc1, vc1 = k[b:b + 1].copy(), v[b:b + 1].copy()
            want_o, want_lse, n = oracle.gqa_attention_cached(q[b:b + 1], kn[b:b + 1], vn[b:b + 1], kc1, vc1, cur[b], cur[b])
            assert n == cur[b] + 1
            assert maxabs(from_torch(o)[b], want_o[0]) <= tol, f"step {step} seq {b}"
            assert maxabs(from_torch(lse)[b], want_lse[0, :, 0]) <= lse_tol, f"step {step} seq {b}"
            cur[b] += 1
        assert seq.tolist() == cur
        k, v = from_torch(tk), from_torch(tv)          # carry the device cache (rounded rotated K) forward
    for b in range(B):
        assert not k[b, :, cur[b]:].any() and not v[b, :, cur[b]:].any()
    if row_stride:
        assert not bool(bk[..., D:].any()) and not bool(bv[..., D:].any())
