"""The C-ABI library loads and exports every symbol include/vesper_b200.h declares
(no compute calls: this runs without a GPU)."""
import ctypes as C
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header="vesper_b200.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vb200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    from vesper_b200 import capi
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/vesper_b200.h but not exported"
    assert sorted(capi.EXPORTS) == names
    block = declared_symbols("vesper_b200_block.h")
    for n in block:
        assert hasattr(lib, n), f"{n} declared in include/vesper_b200_block.h but not exported"
    assert sorted(capi.BLOCK_EXPORTS) == block


def test_struct_layout_and_host_helpers(lib):
    from vesper_b200 import capi
    assert lib.vb200_abi_version() == 1
    assert lib.vb200_strerror(0) == b"ok" and b"workspace" in lib.vb200_strerror(-4)
    # a struct_size mismatch is rejected before anything touches a device
    a = capi.PrefillArgs()
    a.struct_size = 4
    assert lib.vb200_prefill_fwd(C.byref(a)) == -1
    assert lib.vb200_prefill_workspace_bytes(C.byref(a)) == 0
    d = capi.DecodeArgs()
    assert lib.vb200_decode_fwd(C.byref(d)) == -1
    # inv_freq is the reference's fp32 expression pow(theta, -2i/D) (src/nn/functional.cpp:433)
    f = capi.inv_freq(10000.0, 128)
    from oracle.binding import Oracle
    want = Oracle().rope_frequencies(2, 128, 1, 10000.0)[0]     # position 1 -> angle == inv_freq
    assert np.array_equal(np.array(list(f), np.float32), want)


def test_decode_plan_for_one_common_length(lib):
    """Without per-sequence lengths the split plan aims at one or two CTAs per SM (not four): the long-context decode
    of 8 groups of 8 heads over 131072 keys gets 148 // 8 = 18 splits, a 16384-key shard 2 * 148 / 8 = 37."""
    from vesper_b200 import capi
    d = capi.DecodeArgs()
    d.struct_size = C.sizeof(capi.DecodeArgs)
    d.B, d.Hq, d.Hkv, d.D = 1, 64, 8, 128
    for max_len, splits in ((131072, 18), (16384, 37)):
        d.cache_cap, d.max_len, d.uniform_len = max_len, max_len, max_len
        n = lib.vb200_decode_workspace_bytes(C.byref(d))
        want = (64 + 1 * 8 * splits * 8 * 130) * 4
        assert n == (want + 255) // 256 * 256, (max_len, n, want)


def test_decode_workspace_plan_is_consistent(lib):
    from vesper_b200 import capi
    d = capi.DecodeArgs()
    d.struct_size = C.sizeof(capi.DecodeArgs)
    d.B, d.Hq, d.Hkv, d.D, d.cache_cap, d.max_len = 32, 32, 8, 128, 8448, 8193
    d.seq_lens = 0x1000          # per-sequence lengths (only its presence matters for the plan): splits of at most 2048 keys
    n = lib.vb200_decode_workspace_bytes(C.byref(d))
    # [B,Hkv,splits,n_rep,D+2] fp32 with 2048-key splits of 8193 keys -> 5 splits
    assert n >= 32 * 8 * 5 * 4 * 130 * 4 and n % 256 == 0
    d.seq_lens = None            # one common length: longer chunks, fewer splits
    assert lib.vb200_decode_workspace_bytes(C.byref(d)) < n
    d.seq_lens = 0x1000
    d.num_splits = 1
    assert lib.vb200_decode_workspace_bytes(C.byref(d)) < n


def test_decode_workspace_max_covers_every_step_of_a_generation(lib):
    """The split plan is not monotone in max_len (chunks round up to 64 keys and are capped at 512 with
    per-sequence lengths), so a buffer sized for max_len == cache capacity can be too small for a shorter
    step.  vb200_decode_workspace_bytes_max is what the model's buffers are sized with: no step it can be
    asked for -- a common length start_pos (max_len = start_pos + 1) or the device length array with any
    max_len up to the capacity -- may need more."""
    from vesper_b200 import capi
    found_non_monotone = False
    for B, Hq, Hkv, cap in ((8, 32, 8, 1024), (8, 32, 8, 2048), (4, 16, 4, 4096), (1, 64, 8, 8192), (2, 8, 2, 777), (32, 32, 8, 8448)):
        d = capi.DecodeArgs()
        d.struct_size = C.sizeof(capi.DecodeArgs)
        d.B, d.Hq, d.Hkv, d.D, d.cache_cap = B, Hq, Hkv, 128, cap
        worst = lib.vb200_decode_workspace_bytes_max(C.byref(d))
        d.max_len = cap
        at_cap = lib.vb200_decode_workspace_bytes(C.byref(d))
        assert worst >= at_cap > 0
        step = 1 if cap <= 2048 else 7
        for pos in list(range(1, cap + 1, step)) + [cap]:
            d.max_len = pos
            d.seq_lens = None
            n0 = lib.vb200_decode_workspace_bytes(C.byref(d))
            d.seq_lens = 0x1000
            n1 = lib.vb200_decode_workspace_bytes(C.byref(d))
            assert n0 <= worst and n1 <= worst, (B, Hkv, cap, pos)
            found_non_monotone |= max(n0, n1) > at_cap
        d.seq_lens = None
    assert found_non_monotone          # the case the helper exists for does occur
    bad = capi.DecodeArgs()
    bad.struct_size = C.sizeof(capi.DecodeArgs)
    bad.B, bad.Hq, bad.Hkv, bad.D, bad.cache_cap = 1, 8, 2, 0, 64
    assert lib.vb200_decode_workspace_bytes(C.byref(bad)) == 0 and lib.vb200_decode_workspace_bytes_max(C.byref(bad)) == 0


def test_host_layer_facade_exports(lib):
    """libvesper_b200_host.so (models::TransformerLM / generation::Generator behind a C facade) loads without
    a GPU and exports what vesper_b200/model.py binds."""
    from vesper_b200 import model
    from vesper_b200.build import build_host
    build_host()
    L = model.load_host()
    for n in model.HOST_EXPORTS:
        assert hasattr(L, n), n
    shapes = model.param_shapes(32000, 2048, 24, 16, 4, 5632)
    assert shapes["layers.23.attention.wqkv.weight"] == (3072, 2048) and shapes["output.weight"] == (32000, 2048)
    assert sum(int(np.prod(s)) for s in shapes.values()) == 1213302784          # the C5 decoder
