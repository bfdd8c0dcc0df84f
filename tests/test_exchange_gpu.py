"""vb200_exchange_combine (the fused peer-memory exchange + LSE merge of sequence-sharded decode) on ONE
GPU: the other ranks are emulated by writing what they would have pushed (8-byte words {value, call number})
into this rank's buffer before the launch, so no launch ever waits for another one.  The real multi-GPU run is
tests/test_exchange_multi_gpu.py."""
import numpy as np
import pytest

from helpers import from_torch

pytestmark = pytest.mark.gpu

SLOT_BASE = 4096 + 2 * 16 * 64 * 4


def _partials(rng, world, rows, D):
    """Records (O/l, m, l) as a split of one softmax over `world` shards."""
    p = np.empty((world, rows, D + 2), np.float32)
    p[:, :, :D] = rng.standard_normal((world, rows, D))
    p[:, :, D] = 3.0 * rng.standard_normal((world, rows))
    p[:, :, D + 1] = rng.uniform(0.5, 20.0, size=(world, rows))
    return p


def _want(oracle, p):
    world, rows, D2 = p.shape
    D = D2 - 2
    o, lse = oracle.lse_combine(p[:, :, D].copy(), p[:, :, D + 1].copy(), p[:, :, :D].copy())
    return o, lse


ONE_LAUNCH_TAG = 0x80000000      # the numbers vb200_decode_exchange_fwd's words carry have bit 31 set


def _seed_peer(buf, world, rows, D, src, step, record, tag=0):
    """What rank `src` would have pushed into this buffer for call number `step`."""
    import torch
    parity = step & 1
    n = rows * (D + 2)
    off = SLOT_BASE + (parity * world + src) * n * 8
    words = np.empty((n, 2), np.uint32)
    words[:, 0] = record.reshape(-1).astype(np.float32).view(np.uint32)
    words[:, 1] = step | tag
    buf[off:off + n * 8].view(torch.int32).copy_(torch.from_numpy(words.reshape(-1).view(np.int32)).to(buf.device))


def _pushed(buf, world, rows, D, src, step):
    """(values, call numbers) of the words rank `src` pushed into this buffer for call number `step`."""
    import torch
    n = rows * (D + 2)
    off = SLOT_BASE + ((step & 1) * world + src) * n * 8
    w = buf[off:off + n * 8].view(torch.int32).cpu().numpy().view(np.uint32).reshape(n, 2)
    return w[:, 0].copy().view(np.float32), w[:, 1]


def test_buffer_size_and_argument_checks(lib):
    from vesper_b200 import capi
    assert capi.exchange_buffer_bytes(8, 64, 128) == SLOT_BASE + 2 * 8 * 64 * 130 * 8
    assert capi.exchange_buffer_bytes(17, 64, 128) == 0 and capi.exchange_buffer_bytes(0, 64, 128) == 0
    a = capi.ExchangeArgs()
    assert lib.vb200_exchange_combine(None) == -1
    a.struct_size = 8
    assert lib.vb200_exchange_combine(a) == -1


def test_single_rank_equals_lse_combine(cuda, oracle):
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(0)
    rows, D = 64, 128
    p = _partials(rng, 1, rows, D)
    buf = torch.zeros(capi.exchange_buffer_bytes(1, rows, D), dtype=torch.uint8, device=cuda)
    out = torch.empty(rows, D, dtype=torch.bfloat16, device=cuda)
    lse = torch.empty(rows, dtype=torch.float32, device=cuda)
    for _ in range(3):                                   # call numbers 1, 2, 3 from the buffer's own counter
        capi.exchange_combine(torch.from_numpy(p[0]).to(cuda), [buf.data_ptr()], 0, out, lse)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    o, l = _want(oracle, p)
    assert np.abs(from_torch(out) - o).max() <= 2.0 ** -8 * np.abs(o).max() and np.abs(from_torch(lse) - l).max() <= 1e-5


# (8, 1024, 128): 16 rows per block, whose words of 8 ranks do not fit the shared-memory staging area -- the blocks poll and merge from global memory
@pytest.mark.parametrize("world,rows,D", [(2, 64, 128), (4, 7, 64), (8, 64, 128), (3, 300, 128), (8, 1024, 128)])
def test_emulated_peers_receive_side_and_push_side(cuda, oracle, world, rows, D):
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(world * 1000 + rows)
    rank = 1 % world
    nbytes = capi.exchange_buffer_bytes(world, rows, D)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=cuda) for _ in range(world)]     # bufs[rank] is "ours", the rest stand in for the peers' memory
    out = torch.empty(rows, D, dtype=torch.bfloat16, device=cuda)
    lse = torch.empty(rows, dtype=torch.float32, device=cuda)
    for step in (1, 2, 3):
        p = _partials(rng, world, rows, D)
        for src in range(world):
            if src != rank:
                _seed_peer(bufs[rank], world, rows, D, src, step, p[src])
        capi.exchange_combine(torch.from_numpy(p[rank]).to(cuda), [b.data_ptr() for b in bufs], rank, out, lse)
        torch.cuda.synchronize()
        capi.check_kernel_status(0)
        o, l = _want(oracle, p)
        assert np.abs(from_torch(out) - o).max() <= 2.0 ** -8 * max(1.0, np.abs(o).max()), step
        assert np.abs(from_torch(lse) - l).max() <= 1e-4, step
        # push side: every stand-in peer buffer now holds our records in slot[parity][rank], every word with the call number
        for dst in range(world):
            got, numbers = _pushed(bufs[dst], world, rows, D, rank, step)
            assert np.array_equal(got, p[rank].reshape(-1)) and bool((numbers == step).all())


def test_absent_peer_times_out_with_a_status_not_a_hang(cuda, oracle):
    """Words that nothing writes: the bounded wait (here 2e6 cycles, about a millisecond) gives up, the
    output stays untouched, the status word reports it, and the next call works."""
    import torch
    from vesper_b200 import capi
    rng = np.random.default_rng(5)
    world, rows, D = 2, 16, 128
    p = _partials(rng, world, rows, D)
    nbytes = capi.exchange_buffer_bytes(world, rows, D)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=cuda) for _ in range(world)]
    out = torch.full((rows, D), 7.0, dtype=torch.bfloat16, device=cuda)
    capi.exchange_combine(torch.from_numpy(p[0]).to(cuda), [b.data_ptr() for b in bufs], 0, out, timeout_cycles=2_000_000)
    torch.cuda.synchronize()
    with pytest.raises(capi.Vb200Error, match="bounded in-kernel wait"):
        capi.check_kernel_status(0)
    assert bool((out == 7.0).all())
    # the peer "arrives" for the next call number (2): the same buffers keep working
    _seed_peer(bufs[0], world, rows, D, 1, 2, p[1])
    capi.exchange_combine(torch.from_numpy(p[0]).to(cuda), [b.data_ptr() for b in bufs], 0, out, timeout_cycles=2_000_000)
    torch.cuda.synchronize()
    capi.check_kernel_status(0)
    o, _ = _want(oracle, p)
    assert np.abs(from_torch(out) - o).max() <= 2.0 ** -8 * max(1.0, np.abs(o).max())


@pytest.mark.parametrize("n_rep,L,num_splits", [(8, 4096, 0), (4, 4096, 0), (8, 8192, 64), (4, 8192, 64)])
def test_decode_and_exchange_in_one_launch_with_an_emulated_peer(cuda, oracle, n_rep, L, num_splits):
    """vb200_decode_exchange_fwd: rank 0 of a 2-way sequence-sharded decode runs its shard, merges its splits and
    exchanges in ONE launch; rank 1 is emulated by seeding what it would have pushed (its record comes from a
    vb200_decode_fwd(partial_out) over the second shard).  Result against the oracle's attention over the whole
    context, query rotated at the absolute position; push side: the stand-in peer buffer received this rank's record
    (compared with the two-call form's record).  With 64 splits of 64 keys the group's records do not fit one staging
    round of the in-kernel split merge (20 records for 8-head groups, 44 for 4-head groups): the later rounds fold in
    with a rescale."""
    import torch
    from helpers import bf16_round, maxabs, to_torch
    from vesper_b200 import capi
    B, Hkv, D = 1, 2, 128
    Hq = Hkv * n_rep
    rows = B * Hq
    rng = np.random.default_rng(70 + n_rep)
    k = bf16_round(rng.standard_normal((B, Hkv, L, D), dtype=np.float32))
    v = bf16_round(rng.standard_normal((B, Hkv, L, D), dtype=np.float32))
    scale = float(1.0 / np.sqrt(D))
    half = L // 2
    k0, v0 = to_torch(k[:, :, :half], torch.bfloat16, cuda), to_torch(v[:, :, :half], torch.bfloat16, cuda)
    k1, v1 = to_torch(k[:, :, half:], torch.bfloat16, cuda), to_torch(v[:, :, half:], torch.bfloat16, cuda)
    qpos = torch.tensor([L], dtype=torch.int32, device=cuda)
    nbytes = capi.exchange_buffer_bytes(2, rows, D)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=cuda) for _ in range(2)]
    out = torch.empty(rows, D, dtype=torch.bfloat16, device=cuda)
    lse = torch.empty(rows, dtype=torch.float32, device=cuda)
    for step in (1, 2, 3):                                   # the call number advances in the buffer; slots alternate
        q = bf16_round(rng.standard_normal((B, Hq, 1, D), dtype=np.float32))
        tq = to_torch(q, torch.bfloat16, cuda)
        rec1 = torch.empty(rows, D + 2, dtype=torch.float32, device=cuda)
        capi.decode(tq, None, k1, v1, scale=scale, theta=10000.0, uniform_len=half, max_len=half, pos_offset=half,
                    q_positions=qpos, partial_out=rec1)
        rec0 = torch.empty_like(rec1)
        capi.decode(tq, None, k0, v0, scale=scale, theta=10000.0, uniform_len=half, max_len=half, pos_offset=0,
                    q_positions=qpos, partial_out=rec0)
        torch.cuda.synchronize()
        _seed_peer(bufs[0], 2, rows, D, 1, step, rec1.cpu().numpy(), tag=ONE_LAUNCH_TAG)
        capi.decode_exchange(tq, k0, v0, [b.data_ptr() for b in bufs], 0, out, lse, scale=scale, theta=10000.0,
                             uniform_len=half, max_len=half, pos_offset=0, q_positions=qpos, num_splits=num_splits)
        torch.cuda.synchronize()
        capi.check_kernel_status(0)
        q_rot = oracle.apply_rope(q, L, 10000.0)
        want_o, want_lse = oracle.decode_ragged(q_rot[:, :, 0], k, v, [L])
        assert maxabs(from_torch(out), want_o[0]) <= 1e-2, step
        assert maxabs(from_torch(lse), want_lse[0]) <= 1e-3, step
        # push side: our merged record in the stand-in peer's slot[parity][0]; same numbers as the two-call form up to
        # the summation order of the split merge
        got, numbers = _pushed(bufs[1], 2, rows, D, 0, step)
        got = got.reshape(rows, D + 2)
        assert bool((numbers == (step | ONE_LAUNCH_TAG)).all())
        ref = rec0.cpu().numpy()
        # (for 4-head groups the two-call form at this length runs the CUDA-core split kernel, the one-launch form the
        # warp-MMA one, whose P is rounded to 16 bits: a few 1e-4 apart on records of size ~0.1)
        # (m is a reference maximum, raised lazily, not necessarily the true one: only m + ln l is determined)
        assert np.abs(got[:, :D] - ref[:, :D]).max() <= 1e-3
        assert np.abs((got[:, D] + np.log(got[:, D + 1])) - (ref[:, D] + np.log(ref[:, D + 1]))).max() <= 1e-3


def test_decode_exchange_refuses_shapes_it_does_not_take(cuda):
    import torch
    from vesper_b200 import capi
    B, Hq, Hkv, D, L = 1, 4, 2, 128, 256                     # two query heads per KV head: the two-call form applies
    q = torch.zeros(B, Hq, 1, D, dtype=torch.bfloat16, device=cuda)
    kc = torch.zeros(B, Hkv, L, D, dtype=torch.bfloat16, device=cuda)
    buf = torch.zeros(capi.exchange_buffer_bytes(1, B * Hq, D), dtype=torch.uint8, device=cuda)
    out = torch.empty(B * Hq, D, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(capi.Vb200Error) as e:
        capi.decode_exchange(q, kc, kc, [buf.data_ptr()], 0, out, scale=1.0, uniform_len=L, max_len=L)
    assert e.value.status == -2
    torch.cuda.synchronize()
    capi.check_kernel_status(0)


@pytest.mark.gpu
@pytest.mark.parametrize("n_rep", [8, 4])
def test_one_launch_step_on_a_ragged_batch_single_rank(cuda, oracle, n_rep):
    """vb200_decode_exchange_fwd with per-sequence lengths (world 1, so the exchange is the rank with itself): groups
    of different sequences have different numbers of live splits -- a one-key sequence has a single one, splits past a
    sequence's end take no ticket -- and every group's last CTA must still find its count.  Against the oracle's ragged
    decode; three consecutive calls (the ticket words return to zero)."""
    import torch
    from helpers import bf16_round, maxabs, to_torch
    from vesper_b200 import capi
    B, Hkv, D, cap = 4, 2, 128, 3072
    Hq = Hkv * n_rep
    rows = B * Hq
    lens = np.array([3000, 700, 1, 2049], dtype=np.int32)
    rng = np.random.default_rng(91 + n_rep)
    k = bf16_round(rng.standard_normal((B, Hkv, cap, D), dtype=np.float32))
    v = bf16_round(rng.standard_normal((B, Hkv, cap, D), dtype=np.float32))
    for b in range(B):
        k[b, :, lens[b]:] = 0
        v[b, :, lens[b]:] = 0
    tk, tv = to_torch(k, torch.bfloat16, cuda), to_torch(v, torch.bfloat16, cuda)
    tl = torch.from_numpy(lens).to(cuda)
    buf = torch.zeros(capi.exchange_buffer_bytes(1, rows, D), dtype=torch.uint8, device=cuda)
    out = torch.empty(rows, D, dtype=torch.bfloat16, device=cuda)
    lse = torch.empty(rows, dtype=torch.float32, device=cuda)
    scale = float(1.0 / np.sqrt(D))
    for step in range(3):
        q = bf16_round(rng.standard_normal((B, Hq, 1, D), dtype=np.float32))
        capi.decode_exchange(to_torch(q, torch.bfloat16, cuda), tk, tv, [buf.data_ptr()], 0, out, lse, scale=scale,
                             seq_lens=tl, max_len=int(lens.max()))
        torch.cuda.synchronize()
        capi.check_kernel_status(0)
        want_o, want_lse = oracle.decode_ragged(q[:, :, 0], k, v, lens)
        assert maxabs(from_torch(out).reshape(B, Hq, D), want_o) <= 1e-2, step
        assert maxabs(from_torch(lse).reshape(B, Hq), want_lse) <= 1e-3, step
