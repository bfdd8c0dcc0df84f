"""vb200_attention_bwd (fp32 flash-attention backward) against the CPU oracle, which is pinned bit for bit
to the reference's flash_attention_backward (tests/test_oracle_golden.py).  Tolerance: fp32 sums in a
different order, 2e-4 of the largest gradient magnitude."""
import numpy as np
import pytest

from helpers import from_torch, to_torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(1, 2, 16, 32), (1, 1, 8, 16), (2, 3, 100, 64), (1, 2, 257, 128), (1, 4, 64, 40)])
@pytest.mark.parametrize("causal", [True, False])
def test_backward_matches_oracle(cuda, oracle, shape, causal):
    import torch
    from vesper_b200 import capi
    B, H, N, D = shape
    rng = np.random.default_rng(N * D + int(causal))
    q, k, v, do = [rng.standard_normal(shape).astype(np.float32) for _ in range(4)]
    scale = float(1.0 / np.sqrt(D))
    out, lse = oracle.flash_attention(q, k, v, scale, causal)
    want = oracle.flash_attention_bwd(do, q, k, v, out, lse, scale, causal)
    t = [to_torch(x, torch.float32, cuda) for x in (do, q, k, v, out, lse)]
    got = capi.attention_bwd(*t, scale=scale, causal=causal)
    torch.cuda.synchronize()
    for name, g, w in zip(("dq", "dk", "dv"), got, want):
        err = np.abs(from_torch(g) - w).max()
        assert err <= 2e-4 * max(1.0, np.abs(w).max()), (name, float(err))


def test_backward_uses_the_forward_kernels_output(cuda, oracle):
    """Forward on the GPU (fp32 path, O and LSE), backward on the GPU, both against the oracle chain."""
    import torch
    from vesper_b200 import capi
    B, H, N, D = 1, 8, 256, 64
    rng = np.random.default_rng(0)
    q, k, v = [rng.standard_normal((B, H, N, D)).astype(np.float32) for _ in range(3)]
    do = np.ones((B, H, N, D), np.float32)                      # d(sum(out)) as in tests/test_flash_attention.cpp:305-307
    scale = float(1.0 / np.sqrt(D))
    tq, tk, tv = [to_torch(x, torch.float32, cuda) for x in (q, k, v)]
    o = torch.empty_like(tq)
    lse = torch.empty(B, H, N, dtype=torch.float32, device=cuda)
    capi.prefill(tq, tk, tv, o, lse, scale=scale, causal=True)
    dq, dk, dv = capi.attention_bwd(to_torch(do, torch.float32, cuda), tq, tk, tv, o, lse, scale=scale, causal=True)
    torch.cuda.synchronize()
    out, l = oracle.flash_attention(q, k, v, scale, True)
    want = oracle.flash_attention_bwd(do, q, k, v, out, l, scale, True)
    for g, w in zip((dq, dk, dv), want):
        assert np.isfinite(from_torch(g)).all() and np.abs(from_torch(g)).max() > 0
        assert np.abs(from_torch(g) - w).max() <= 5e-4 * max(1.0, np.abs(w).max())


def test_backward_argument_errors(cuda, lib):
    import ctypes as C
    import torch
    from vesper_b200 import capi
    a = capi.AttnBwdArgs()
    assert lib.vb200_attention_bwd(C.byref(a)) == -1                # struct_size
    x = torch.zeros(1, 1, 8, 16, device=cuda)
    with pytest.raises(capi.Vb200Error, match="fp32 only"):
        capi.attention_bwd(x.bfloat16(), x.bfloat16(), x.bfloat16(), x.bfloat16(), x.bfloat16(), torch.zeros(1, 1, 8, device=cuda), scale=1.0)
