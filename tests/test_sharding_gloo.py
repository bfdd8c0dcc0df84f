"""Multi-rank host logic of the sequence-sharded decode on CPU: two gloo ranks each
compute their shard's partial with the oracle, all-gather, combine, and must
reproduce the single-device attention.  Also a rank that contributes a
wrong-size partial must be detected on the host (no GPU involved)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, L, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.binding import Oracle
        from vesper_b200.sharded import ShardedDecodeStep
        orc = Oracle()
        rng = np.random.default_rng(0)          # same stream on every rank: replicated q, global K/V
        Hq, Hkv, D = 8, 2, 32
        q = rng.standard_normal((1, Hq, 1, D), dtype=np.float32)
        k = rng.standard_normal((1, Hkv, L, D), dtype=np.float32)
        v = rng.standard_normal((1, Hkv, L, D), dtype=np.float32)
        q_rot = orc.apply_rope(q, L, 10000.0)

        def local_partial(begin, end, qpos):
            ks, vs = np.ascontiguousarray(k[:, :, begin:end]), np.ascontiguousarray(v[:, :, begin:end])
            kr, vr = orc.repeat_kv(ks, Hq // Hkv), orc.repeat_kv(vs, Hq // Hkv)
            o, sc = orc.sdpa_standard(q_rot, kr, vr, False, want_scores=True)
            m = sc[0, :, 0].max(-1)
            l = np.exp(sc[0, :, 0] - m[:, None]).sum(-1)
            return torch.from_numpy(np.concatenate([o[0, :, 0], m[:, None], l[:, None]], axis=1).astype(np.float32))

        def combine(g):
            g = g.numpy()
            out, lse = orc.lse_combine(g[:, :, D], g[:, :, D + 1], g[:, :, :D])
            return out, lse

        out, lse = ShardedDecodeStep(world, rank, L).run(local_partial, combine, dist)
        kr, vr = orc.repeat_kv(k, Hq // Hkv), orc.repeat_kv(v, Hq // Hkv)
        want = orc.sdpa_standard(q_rot, kr, vr, False)
        ret[rank] = float(np.abs(out - want[0, :, 0]).max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("L", [64, 101])
def test_two_rank_sharded_decode_matches_single_device(L):
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, 29500 + L % 200, L, ret), nprocs=world, join=True)
    assert len(ret) == world and all(err < 1e-5 for err in ret.values()), dict(ret)


def test_shard_ranges_cover_sequence_exactly():
    from vesper_b200.sharded import owner_of_row, shard_range, unit_range
    for total in (0, 1, 7, 64, 131072, 131073):
        for world in (1, 2, 4, 8):
            edges = [shard_range(total, world, r) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == total
            assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in edges]
            assert max(sizes) - min(sizes) <= 1
    assert shard_range(131072, 8, 3) == (49152, 65536)
    assert unit_range(32, 8, 7) == (28, 32)
    assert owner_of_row(100, 4, 99) == 3 and owner_of_row(100, 4, 100) == 3 and owner_of_row(100, 4, 0) == 0
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)


def _bad_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from vesper_b200.sharded import ShardedDecodeStep
        rows = 4 if rank == 0 else 3          # rank 1 contributes a wrong-size partial
        try:
            ShardedDecodeStep(world, rank, 16, validate=True).run(lambda b, e, p: torch.zeros(rows, 6), lambda g: g, dist)
            ret[rank] = "no error"
        except ValueError as e:               # detected on the host before the data all-gather
            ret[rank] = "ValueError"
    finally:
        dist.destroy_process_group()


def test_wrong_size_partial_is_a_host_error():
    ret = mp.Manager().dict()
    mp.spawn(_bad_worker, args=(2, 29733, ret), nprocs=2, join=True)
    assert dict(ret) == {0: "ValueError", 1: "ValueError"}


def _absent_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    import time
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from vesper_b200.sharded import ShardedDecodeStep, ShardExchangeError
    if rank == 1:
        time.sleep(6)                         # the failing rank: joined the group, never contributes its partial
        ret[rank] = "absent"
        os._exit(0)
    try:
        ShardedDecodeStep(world, rank, 16, timeout_s=2.0).run(lambda b, e, p: torch.zeros(4, 6), lambda g: g, dist)
        ret[rank] = "no error"
    except ShardExchangeError:
        ret[rank] = "ShardExchangeError"
    os._exit(0)                               # the group is unusable after the failure: leave without a collective


def test_rank_that_never_contributes_is_a_host_timeout():
    """Failure made on the host: one rank never issues its all-gather; the other must get an
    error within the host-side limit instead of hanging."""
    ret = mp.Manager().dict()
    mp.spawn(_absent_worker, args=(2, 29761, ret), nprocs=2, join=True)
    assert ret.get(0) == "ShardExchangeError", dict(ret)
