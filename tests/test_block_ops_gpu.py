"""Decoder-block operators (include/vesper_b200_block.h) on the GPU against the CPU oracle.

Protocol as for attention: inputs are generated in fp32, rounded to bf16 (RNE); the GPU gets the
bf16 bits, the oracle the same values widened to fp32 and computes in fp32.  Tolerances: a bf16
output carries one rounding (2^-9 relative) on top of fp32 accumulation-order noise, so
|gpu - oracle| <= 2^-8 * |oracle| + small absolute term; fp32 outputs are compared at 1e-3 of the
row scale (K-long dot products summed in a different order).
"""
import numpy as np
import pytest

from helpers import bf16_round, from_torch, to_torch

pytestmark = pytest.mark.gpu


def _linear_case(cuda, oracle, M, N, K, epilogue, seed, splits=0, ld_pad=0):
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(seed)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = bf16_round((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32))
    xb = torch.zeros(M, K + ld_pad, dtype=torch.bfloat16, device=cuda)
    xb[:, :K] = to_torch(x, torch.bfloat16, cuda)
    wb = to_torch(w, torch.bfloat16, cuda)
    want = oracle.linear(x, w)
    if epilogue == capi.EPI_BF16:
        out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=cuda)
    elif epilogue == capi.EPI_SWIGLU:
        out = torch.full((M, N // 2), 7.0, dtype=torch.bfloat16, device=cuda)
        want = oracle.silu_mul(want[:, 0::2].copy(), want[:, 1::2].copy())
    else:
        h0 = rng.standard_normal((M, N)).astype(np.float32)
        out = to_torch(h0, torch.float32, cuda)
        if epilogue == capi.EPI_ADD_F32:
            want = h0 + want
    capi.linear(xb[:, :K], wb, out, epilogue=epilogue, splits=splits)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    got = from_torch(out)
    if epilogue in (capi.EPI_BF16, capi.EPI_SWIGLU):
        tol = 2.0 ** -8 * np.abs(want) + 2e-3
    else:
        tol = 1e-3 * (1.0 + np.abs(want))
    err = np.abs(got - want)
    assert np.all(err <= tol), (M, N, K, epilogue, float(err.max()), float((err - tol).max()))


@pytest.mark.parametrize("M", [1, 8, 16, 17, 32, 40, 64])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_linear_skinny(cuda, oracle, M, epilogue):
    # 304 = partial last 128-row tile; 456 = K tail that is not a multiple of 64
    _linear_case(cuda, oracle, M, 304, 456, epilogue, seed=10 + M)


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8])
def test_linear_skinny_split_k(cuda, oracle, splits):
    _linear_case(cuda, oracle, 8, 512, 2048, 0, seed=3, splits=splits)
    _linear_case(cuda, oracle, 8, 512, 2048, 2, seed=4, splits=splits)


def test_linear_skinny_is_deterministic(cuda):
    import torch
    from vesper_b200 import capi
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(8, 2048, generator=g).to(cuda, torch.bfloat16)
    w = (torch.randn(1024, 2048, generator=g) / 45.0).to(cuda, torch.bfloat16)
    outs = []
    for _ in range(3):
        o = torch.empty(8, 1024, dtype=torch.float32, device=cuda)
        capi.linear(x, w, o, epilogue=capi.EPI_F32)
        outs.append(o)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("shape", [(65, 256, 64), (128, 256, 128), (200, 528, 456), (384, 1024, 2048), (1000, 304, 192)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_linear_wide(cuda, oracle, shape, epilogue):
    M, N, K = shape
    _linear_case(cuda, oracle, M, N, K, epilogue, seed=M + N + K)


def test_linear_strided_activations(cuda, oracle):
    _linear_case(cuda, oracle, 8, 256, 512, 0, seed=5, ld_pad=64)
    _linear_case(cuda, oracle, 256, 256, 512, 0, seed=6, ld_pad=64)


def test_linear_model_shapes(cuda, oracle):
    """The projections of the 2048-wide Llama-style block: QKV (3072), W13 interleaved (11264), W2 (K=5632)."""
    for (M, N, K, epi) in [(8, 3072, 2048, 0), (8, 2048, 5632, 2), (8, 11264, 2048, 3), (192, 3072, 2048, 0), (192, 2048, 5632, 2)]:
        _linear_case(cuda, oracle, M, N, K, epi, seed=N)


def test_linear_rejects_bad_arguments(cuda, lib):
    import torch
    from vesper_b200 import capi
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device=cuda)
    w = torch.zeros(16, 64, dtype=torch.bfloat16, device=cuda)
    o = torch.zeros(8, 16, dtype=torch.bfloat16, device=cuda)
    s = capi._stream_ptr(None)
    assert lib.vb200_linear(0, s, None, 64, capi._ptr(w), 64, capi._ptr(o), 16, 8, 16, 64, 0, 0) == -1
    assert lib.vb200_linear(0, s, capi._ptr(x), 64, capi._ptr(w), 64, capi._ptr(o), 16, 8, 16, 60, 0, 0) == -3   # K % 8
    assert lib.vb200_linear(0, s, capi._ptr(x), 64, capi._ptr(w), 64, capi._ptr(o), 16, 8, 16, 64, 9, 0) == -1   # epilogue
    assert lib.vb200_linear(0, s, capi._ptr(x), 64, capi._ptr(w), 64, capi._ptr(o), 4, 8, 16, 64, 0, 0) == -1    # ldo < N


def test_interleave_rows(cuda):
    import torch
    from vesper_b200 import capi
    a = torch.randn(40, 64, device=cuda).to(torch.bfloat16)
    b = torch.randn(40, 64, device=cuda).to(torch.bfloat16)
    out = torch.empty(80, 64, dtype=torch.bfloat16, device=cuda)
    capi.interleave_rows(a, b, out)
    torch.cuda.synchronize()
    assert torch.equal(out[0::2], a) and torch.equal(out[1::2], b)


@pytest.mark.parametrize("M,dim", [(1, 64), (8, 2048), (300, 2048), (5, 8192), (3, 100)])
def test_rms_norm(cuda, oracle, M, dim):
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(dim + M)
    x = (3.0 * rng.standard_normal((M, dim))).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    out = torch.empty(M, dim, dtype=torch.bfloat16, device=cuda)
    capi.rms_norm(to_torch(x, torch.float32, cuda), to_torch(g, torch.float32, cuda), out, 1e-6)
    torch.cuda.synchronize()
    want = oracle.rms_norm(x, g, 1e-6)
    err = np.abs(from_torch(out) - want)
    assert np.all(err <= 2.0 ** -8 * np.abs(want) + 1e-6), float(err.max())


def test_silu_mul(cuda, oracle):
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(1)
    gate = bf16_round(4.0 * rng.standard_normal(8 * 5632).astype(np.float32))
    up = bf16_round(rng.standard_normal(8 * 5632).astype(np.float32))
    out = torch.empty(8 * 5632, dtype=torch.bfloat16, device=cuda)
    capi.silu_mul(to_torch(gate, torch.bfloat16, cuda), to_torch(up, torch.bfloat16, cuda), out)
    torch.cuda.synchronize()
    want = oracle.silu_mul(gate, up)
    err = np.abs(from_torch(out) - want)
    assert np.all(err <= 2.0 ** -8 * np.abs(want) + 1e-6), float(err.max())


@pytest.mark.parametrize("ids_dtype", ["int32", "int64"])
def test_embedding(cuda, oracle, ids_dtype):
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(2)
    table = bf16_round(rng.standard_normal((1000, 256)).astype(np.float32))
    ids = rng.integers(0, 1000, size=(37,)).astype(np.int32)
    out = torch.empty(37, 256, dtype=torch.float32, device=cuda)
    tid = torch.from_numpy(ids.astype(ids_dtype)).to(cuda)
    capi.embedding(tid, to_torch(table, torch.bfloat16, cuda), out)
    torch.cuda.synchronize()
    assert np.array_equal(from_torch(out), oracle.embedding(ids, table))        # a gather: bit-exact


def test_embedding_out_of_range_id_sets_status(cuda):
    import torch
    from vesper_b200 import capi
    table = torch.ones(10, 64, dtype=torch.bfloat16, device=cuda)
    out = torch.full((2, 64), 5.0, dtype=torch.float32, device=cuda)
    capi.embedding(torch.tensor([3, 10], dtype=torch.int32, device=cuda), table, out)
    torch.cuda.synchronize()
    with pytest.raises(capi.Vb200Error):
        capi.check_kernel_status(0)
    capi.check_kernel_status(0)                       # reading clears the word
    assert torch.all(out[0] == 1.0) and torch.all(out[1] == 0.0)


def test_greedy_step_matches_reference_argmax_and_stop_rule(cuda, oracle):
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(3)
    B, V = 8, 32000
    logits = rng.standard_normal((B, V)).astype(np.float32)
    logits[1, 17] = logits[1, 31999] = 9.0         # tie: the first index wins
    logits[2, 0] = 11.0
    logits[3, V - 1] = 12.0
    want = oracle.argmax(logits)
    lg = to_torch(logits, torch.float32, cuda)
    out = torch.empty(B, dtype=torch.int32, device=cuda)
    hist = torch.full((B, 6), -1, dtype=torch.int32, device=cuda)
    done = torch.zeros(B, dtype=torch.int32, device=cuda)
    stop = torch.tensor([int(want[2]), int(want[5])], dtype=torch.int32, device=cuda)
    capi.greedy_step(lg, out, history=hist, step=4, stop_ids=stop, min_new_tokens=5, done=done)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want) and want[1] == 17
    assert np.array_equal(hist[:, 4].cpu().numpy(), want) and int((hist[:, :4] == -1).all())
    want_done = oracle.check_stop_tokens(want, [int(want[2]), int(want[5])], 5, 5)
    assert np.array_equal(done.cpu().numpy(), want_done) and want_done.sum() == 2
    # below min_new_tokens nothing stops; device-side positions pick the history column
    done.zero_()
    pos = torch.tensor([2, 3, 2, 3, 2, 3, 2, 3], dtype=torch.int32, device=cuda)
    capi.greedy_step(lg, out, history=hist, stop_ids=stop, min_new_tokens=5, done=done, pos_dev=pos, pos_base=2)
    torch.cuda.synchronize()
    assert int(done.sum()) == 0
    assert np.array_equal(hist[0::2, 2].cpu().numpy(), want[0::2]) and np.array_equal(hist[1::2, 3].cpu().numpy(), want[1::2])


@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (8, 2048, 2048), (8, 2048, 5632), (16, 384, 456), (40, 2048, 512), (200, 512, 256)])
def test_linear_add_rmsnorm(cuda, oracle, M, N, K):
    """h += x W^T and the next RMSNorm in one call, behind both GEMM kernels."""
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(M + N + K)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = bf16_round((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32))
    h0 = rng.standard_normal((M, N)).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(N)).astype(np.float32)
    h = to_torch(h0, torch.float32, cuda)
    xn = torch.full((M, N), 9.0, dtype=torch.bfloat16, device=cuda)
    for rep in range(2):
        capi.linear_add_rmsnorm(to_torch(x, torch.bfloat16, cuda), to_torch(w, torch.bfloat16, cuda), h, to_torch(g, torch.float32, cuda), 1e-6, xn)
        torch.cuda.synchronize()
        capi.check_kernel_status(0)
        want_h = h0 + (rep + 1) * oracle.linear(x, w)
        got_h = from_torch(h)
        assert np.all(np.abs(got_h - want_h) <= 1e-3 * (1.0 + np.abs(want_h)))
        want_n = oracle.rms_norm(got_h, g, 1e-6)            # the norm of the rows the GPU actually holds
        err = np.abs(from_torch(xn) - want_n)
        assert np.all(err <= 2.0 ** -8 * np.abs(want_n) + 1e-5), (rep, float(err.max()))


def test_embedding_rmsnorm(cuda, oracle):
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(12)
    table = bf16_round(rng.standard_normal((500, 2048)).astype(np.float32))
    g = (1.0 + 0.1 * rng.standard_normal(2048)).astype(np.float32)
    ids = rng.integers(0, 500, size=(9,)).astype(np.int32)
    out = torch.empty(9, 2048, dtype=torch.float32, device=cuda)
    xn = torch.empty(9, 2048, dtype=torch.bfloat16, device=cuda)
    capi.embedding_rmsnorm(torch.from_numpy(ids).to(cuda), to_torch(table, torch.bfloat16, cuda), out, to_torch(g, torch.float32, cuda), 1e-6, xn)
    torch.cuda.synchronize()
    want = oracle.embedding(ids, table)
    assert np.array_equal(from_torch(out), want)
    wn = oracle.rms_norm(want, g, 1e-6)
    assert np.all(np.abs(from_torch(xn) - wn) <= 2.0 ** -8 * np.abs(wn) + 1e-6)


@pytest.mark.parametrize("M", [8, 200])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_linear_with_bias(cuda, oracle, M, epilogue):
    """nn::Linear with bias (src/nn/linear.cpp:44-46): y = x W^T + b before the epilogue's own step."""
    import torch
    from vesper_b200 import capi
    N, K = 384, 256
    rng = np.random.default_rng(77 + M + epilogue)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = bf16_round((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32))
    b = rng.standard_normal(N).astype(np.float32)
    want = oracle.linear(x, w) + b[None, :]
    if epilogue == capi.EPI_BF16:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=cuda)
    elif epilogue == capi.EPI_SWIGLU:
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=cuda)
        want = oracle.silu_mul(want[:, 0::2].copy(), want[:, 1::2].copy())
    else:
        h0 = rng.standard_normal((M, N)).astype(np.float32)
        out = to_torch(h0, torch.float32, cuda)
        if epilogue == capi.EPI_ADD_F32:
            want = h0 + want
    capi.linear(to_torch(x, torch.bfloat16, cuda), to_torch(w, torch.bfloat16, cuda), out, epilogue=epilogue, bias=to_torch(b, torch.float32, cuda))
    torch.cuda.synchronize()
    tol = 2.0 ** -8 * np.abs(want) + 2e-3 if epilogue in (capi.EPI_BF16, capi.EPI_SWIGLU) else 1e-3 * (1.0 + np.abs(want))
    assert np.all(np.abs(from_torch(out) - want) <= tol)


@pytest.mark.parametrize("M", [8, 40, 200])
def test_deferred_rms_norm_chain(cuda, oracle, M):
    """rmsnorm(h) * g @ W^T through the deferred form: a += GEMM that also emits bf16(h * g) (producer), then a GEMM
    whose output rows are scaled by 1/rms(h) -- inside the weight-streaming kernel (M <= 64) or from
    vb200_row_inv_rms (tiled kernel) -- must equal the oracle's linear(rms_norm(h, g), W)."""
    import torch
    from vesper_b200 import capi
    dim, N2, K1 = 512, 384, 256
    rng = np.random.default_rng(300 + M)
    x = bf16_round(rng.standard_normal((M, K1)).astype(np.float32))
    w1 = bf16_round((rng.standard_normal((dim, K1)) / np.sqrt(K1)).astype(np.float32))
    w2 = bf16_round((rng.standard_normal((N2, dim)) / np.sqrt(dim)).astype(np.float32))
    g = (1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    h0 = rng.standard_normal((M, dim)).astype(np.float32)
    h = to_torch(h0, torch.float32, cuda)
    hg = torch.empty(M, dim, dtype=torch.bfloat16, device=cuda)
    tg = to_torch(g, torch.float32, cuda)
    capi.linear_ex(to_torch(x, torch.bfloat16, cuda), to_torch(w1, torch.bfloat16, cuda), h, epilogue=capi.EPI_ADD_F32, scaled_copy=hg, copy_scale=tg)
    y = torch.empty(M, N2, dtype=torch.float32, device=cuda)
    if M <= 64:
        capi.linear_ex(hg, to_torch(w2, torch.bfloat16, cuda), y, epilogue=capi.EPI_F32, rms_rows=h, rms_eps=1e-6)
    else:
        inv = torch.empty(M, dtype=torch.float32, device=cuda)
        capi.row_inv_rms(h, inv, 1e-6)
        capi.linear_ex(hg, to_torch(w2, torch.bfloat16, cuda), y, epilogue=capi.EPI_F32, row_scale=inv)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    h_new = from_torch(h)
    assert np.all(np.abs(h_new - (h0 + oracle.linear(x, w1))) <= 1e-3 * (1.0 + np.abs(h0)))
    assert np.all(np.abs(from_torch(hg) - h_new * g[None, :]) <= 2.0 ** -8 * np.abs(h_new * g[None, :]) + 1e-6)
    want = oracle.linear(oracle.rms_norm(h_new, g, 1e-6), w2)
    # one bf16 rounding of the activations on the GPU side (2^-9 relative per element, averaged over the dot product)
    assert np.abs(from_torch(y) - want).max() <= 1e-2 * max(1.0, np.abs(want).max())


def test_embedding_scaled_and_row_inv_rms(cuda, oracle):
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(13)
    table = bf16_round(rng.standard_normal((300, 1024)).astype(np.float32))
    g = (1.0 + 0.1 * rng.standard_normal(1024)).astype(np.float32)
    ids = rng.integers(0, 300, size=(5,)).astype(np.int32)
    out = torch.empty(5, 1024, dtype=torch.float32, device=cuda)
    sc = torch.empty(5, 1024, dtype=torch.bfloat16, device=cuda)
    capi.embedding_scaled(torch.from_numpy(ids).to(cuda), to_torch(table, torch.bfloat16, cuda), out, to_torch(g, torch.float32, cuda), sc)
    inv = torch.empty(5, dtype=torch.float32, device=cuda)
    capi.row_inv_rms(out, inv, 1e-6)
    torch.cuda.synchronize()
    e = oracle.embedding(ids, table)
    assert np.array_equal(from_torch(out), e)
    assert np.all(np.abs(from_torch(sc) - e * g[None, :]) <= 2.0 ** -8 * np.abs(e * g[None, :]) + 1e-6)
    want_inv = 1.0 / np.sqrt((e.astype(np.float64) ** 2).mean(axis=1) + 1e-6)
    assert np.abs(from_torch(inv) - want_inv).max() <= 1e-5 * want_inv.max()
