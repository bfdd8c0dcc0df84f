"""vb200_decode_fwd_static is compared with vb200_decode_fwd (bit-equal), whose kernels the
decode tests check against the CPU oracle; one oracle comparison is repeated here.

The entry point is the decode step for callers that cannot allocate device memory
(a server whose KV pool already owns all free HBM, a plugin inside a framework that owns
every allocation).  Its split partials live in a fixed array inside the library instead of a
caller workspace.

Checked here, through the C ABI: two calls in a row give the same output and LSE as
vb200_decode_fwd with a caller workspace (same kernels, so the results must agree to the
last bit; the gate is the decode tests' 1e-2 / 1e-3) and stay within that gate of the
oracle, the shared array's stale contents from the first call do not leak into the second
(different lengths), the cache append and length advance behave identically, and a plan
larger than the array is refused with VB200_ERR_WORKSPACE.  This file sorts last so a stop-at-first-failure run has already
exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_decode_matches_workspace_decode(lib, cuda, oracle):
    import torch
    from vesper_b200 import capi
    from helpers import from_torch, maxabs
    B, Hq, Hkv, D, cap = 3, 8, 2, 128, 1200
    g = torch.Generator(device="cpu").manual_seed(77)
    kc_a = torch.randn(B, Hkv, cap, D, generator=g).to(torch.bfloat16).to(cuda)
    vc_a = torch.randn(B, Hkv, cap, D, generator=g).to(torch.bfloat16).to(cuda)
    kc_b, vc_b = kc_a.clone(), vc_a.clone()
    seq_a = torch.tensor([1000, 17, 513], dtype=torch.int32, device=cuda)
    seq_b = seq_a.clone()
    scale = float(1.0 / np.sqrt(D))
    for call in range(2):                      # second call reuses the array the first one dirtied
        q = torch.randn(B, Hq, 1, D, generator=g).to(torch.bfloat16).to(cuda)
        kn = torch.randn(B, Hkv, 1, D, generator=g).to(torch.bfloat16).to(cuda)
        vn = torch.randn(B, Hkv, 1, D, generator=g).to(torch.bfloat16).to(cuda)
        o_a, o_b = torch.empty_like(q), torch.empty_like(q)
        lse_a = torch.empty(B, Hq, dtype=torch.float32, device=cuda)
        lse_b = torch.empty_like(lse_a)
        # existing entry point, caller workspace
        capi.decode(q, o_a, kc_a, vc_a, scale=scale, k_new=kn, v_new=vn, lse=lse_a, theta=10000.0,
                    seq_lens=seq_a, advance_lens=True, max_len=1100)
        # the oracle's answer for sequence 2 (all heads), from the cache as it stands before the step
        L2 = int(seq_b[2].item())
        want_o, want_lse, _ = oracle.gqa_attention_cached(from_torch(q[2:3]), from_torch(kn[2:3]), from_torch(vn[2:3]),
                                                          from_torch(kc_b[2:3]), from_torch(vc_b[2:3]), L2, L2)
        # new entry point: no workspace pointer at all
        a = capi.decode_args(q, o_b, kc_b, vc_b, scale=scale, k_new=kn, v_new=vn, lse=lse_b, theta=10000.0,
                             seq_lens=seq_b, advance_lens=True, max_len=1100)
        assert a.workspace is None and a.workspace_bytes == 0
        capi.check(lib.vb200_decode_fwd_static(C.byref(a)))
        torch.cuda.synchronize()
        capi.check_kernel_status(0)
        assert (o_a.float() - o_b.float()).abs().max().item() <= 1e-2
        assert (lse_a - lse_b).abs().max().item() <= 1e-3
        assert torch.equal(o_a, o_b) and torch.equal(lse_a, lse_b)      # same kernels, same plan
        assert maxabs(from_torch(o_b[2]), want_o[0]) <= 1e-2
        assert maxabs(from_torch(lse_b[2]), want_lse[0, :, 0]) <= 1e-3
        assert torch.equal(seq_a, seq_b)
        # make the next call see different lengths than the stale header holds
        seq_a[1] += 40
        seq_b[1] += 40
    assert torch.equal(kc_a, kc_b) and torch.equal(vc_a, vc_b)
    assert seq_a.tolist() == [1002, 17 + 2 + 80, 515]


def test_static_scratch_rejects_plans_beyond_the_array(lib, cuda):
    import torch
    from vesper_b200 import capi
    # 256 sequences x 8 kv heads x 33 splits x 4 heads x 130 floats = 140 MB of partials > 16 MiB
    B, Hq, Hkv, D, cap = 256, 32, 8, 128, 64
    q = torch.zeros(B, Hq, 1, D, dtype=torch.bfloat16, device=cuda)
    kc = torch.zeros(B, Hkv, cap, D, dtype=torch.bfloat16, device=cuda)
    a = capi.decode_args(q, torch.empty_like(q), kc, kc, scale=1.0, uniform_len=10, max_len=16384 + 512)
    a.num_splits = 33                 # asked for explicitly: with one common length the planner would pick far fewer
    need = lib.vb200_decode_workspace_bytes(C.byref(a))
    assert need > 16 * 1024 * 1024
    assert lib.vb200_decode_fwd_static(C.byref(a)) == -4
    assert b"scratch" in lib.vb200_last_error_detail()
    a.struct_size = 12
    assert lib.vb200_decode_fwd_static(C.byref(a)) == -1
    torch.cuda.synchronize()


def test_static_scratch_on_a_device_that_is_not_current(lib, cuda):
    """The array's address is looked up per device with that device made current inside the call: a caller whose
    current device is GPU 0 steps a cache that lives on GPU 1 (needs two GPUs)."""
    import torch
    from vesper_b200 import capi
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    dev1 = torch.device("cuda", 1)
    B, Hq, Hkv, D, cap, L = 2, 8, 2, 128, 400, 333
    g = torch.Generator(device="cpu").manual_seed(78)
    kc = torch.randn(B, Hkv, cap, D, generator=g).to(torch.bfloat16).to(dev1)
    vc = torch.randn(B, Hkv, cap, D, generator=g).to(torch.bfloat16).to(dev1)
    q = torch.randn(B, Hq, 1, D, generator=g).to(torch.bfloat16).to(dev1)
    o_a, o_b = torch.empty_like(q), torch.empty_like(q)
    scale = float(1.0 / np.sqrt(D))
    torch.cuda.set_device(0)
    s1 = torch.cuda.Stream(device=dev1)
    capi.decode(q, o_a, kc, vc, scale=scale, uniform_len=L, max_len=L, stream=s1)
    a = capi.decode_args(q, o_b, kc, vc, scale=scale, uniform_len=L, max_len=L, stream=s1)
    assert a.device == 1 and torch.cuda.current_device() == 0
    capi.check(lib.vb200_decode_fwd_static(C.byref(a)))
    assert torch.cuda.current_device() == 0
    s1.synchronize()
    capi.check_kernel_status(1, s1)
    assert torch.equal(o_a, o_b)
