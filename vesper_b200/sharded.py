"""Sequence-sharded long-context decode across the GPUs of one node.

The KV sequence of each (batch, kv_head) is split into ``world`` contiguous
shards, shard r living on GPU r.  One decode step is

    local split-KV decode  ->  partial (O/l, m, l) per query head   [vb200_decode_fwd, partial_out]
    exchange of the partials (Hq*(D+2) floats per rank) and log-sum-exp merge, identical on every rank:
      either ONE kernel over NVLink peer memory                     [vb200_exchange_combine, PeerExchange]
      or an all-gather followed by the merge                        [NCCL via torch.distributed, vb200_lse_combine]

There is no other exchange on the attention path; prefill and batched decode
partition by (batch x kv_head) with no collective at all (``unit_range``).
The reference has no multi-device code; numerically the result must equal the
single-device attention (src/ops/flash_attention.cpp:309-345 is the combine
algebra).
"""
from __future__ import annotations

from dataclasses import dataclass


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [begin, end) of a length-``total`` sequence owned by ``rank``: equal
    contiguous shards, the remainder spread over the first ranks."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def unit_range(n_units: int, world: int, rank: int) -> tuple[int, int]:
    """Independent (batch x kv_head) units [begin, end) owned by ``rank``."""
    return shard_range(n_units, world, rank)


def owner_of_row(total: int, world: int, row: int) -> int:
    """Rank whose shard contains ``row`` (rows past the end belong to the last rank,
    which is where new tokens are appended)."""
    for r in range(world):
        b, e = shard_range(total, world, r)
        if b <= row < e:
            return r
    return world - 1


class ShardExchangeError(RuntimeError):
    """The all-gather of the partials did not complete (a rank is missing, slow or failed)."""


def guarded_all_gather(dist, out, inp, timeout_s=None):
    """all_gather_into_tensor supervised from the host: with a timeout the collective is issued
    asynchronously and waited for at most ``timeout_s`` seconds; a rank that never contributes its
    partial turns into a ShardExchangeError on the others instead of a hang.  No GPU state is
    touched by the failure path (the process group is left for the caller to abort or rebuild)."""
    if timeout_s is None:
        dist.all_gather_into_tensor(out, inp)
        return
    import datetime
    work = dist.all_gather_into_tensor(out, inp, async_op=True)
    try:
        done = work.wait(timeout=datetime.timedelta(seconds=timeout_s))
    except RuntimeError as e:                      # gloo / NCCL report an expired wait as an exception
        raise ShardExchangeError(f"partial all-gather failed or timed out after {timeout_s} s: {e}") from e
    if done is False:
        raise ShardExchangeError(f"partial all-gather timed out after {timeout_s} s")


@dataclass
class ShardedDecodeStep:
    """One rank's view of a sequence-sharded decode step.

    ``local_partial(rank_begin, q_position) -> tensor [B*Hq, D+2]`` computes this
    rank's partial; ``combine(gathered [world, B*Hq, D+2]) -> (out, lse)`` merges.
    On GPUs they are the C-ABI calls (see ``cuda_step``); the CPU tests plug in the
    oracle to exercise the sharding and gather logic under gloo.
    """
    world: int
    rank: int
    context_len: int
    validate: bool = False   # exchange the partial's shape first and fail on the host if ranks disagree
    timeout_s: float | None = None   # host-side limit on the all-gather (None: wait without limit)

    def run(self, local_partial, combine, dist=None):
        import torch
        begin, end = shard_range(self.context_len, self.world, self.rank)
        part = local_partial(begin, end, self.context_len)
        if self.world == 1:
            gathered = part.unsqueeze(0)
        else:
            part = part.contiguous()
            if self.validate:
                mine = torch.tensor(list(part.shape) + [0] * (4 - part.dim()), dtype=torch.int64, device=part.device)
                shapes = torch.empty(self.world * 4, dtype=torch.int64, device=part.device)
                dist.all_gather_into_tensor(shapes, mine)
                if not all(torch.equal(shapes[4 * r:4 * r + 4], mine) for r in range(self.world)):
                    raise ValueError(f"rank {self.rank}: partial shapes differ across ranks: {shapes.view(self.world, 4).tolist()}")
            flat = torch.empty((self.world * part.shape[0],) + tuple(part.shape[1:]), dtype=part.dtype, device=part.device)
            guarded_all_gather(dist, flat, part, self.timeout_s)       # rank-major concatenation along dim 0
            gathered = flat.view((self.world,) + tuple(part.shape))
        return combine(gathered)


class PeerExchange:
    """Exchange buffers of all ranks mapped into every process (torch symmetric memory supplies the
    allocation and the address exchange: plumbing only) for ``vb200_exchange_combine``, which pushes
    this rank's partial records into every peer's buffer over NVLink, waits for the peers' records and
    merges -- one kernel instead of all-gather + combine.  Collective: every rank constructs it with
    the same (rows, D) at the same point."""

    def __init__(self, dist, world, rank, rows, D, device, group=None):
        import torch
        import torch.distributed._symmetric_memory as symm_mem
        from . import capi
        self.world, self.rank, self.rows, self.D = world, rank, rows, D
        nbytes = capi.exchange_buffer_bytes(world, rows, D)
        # one set of buffers per entry point: vb200_exchange_combine (`ptrs`) and vb200_decode_exchange_fwd (`ptrs_one`)
        # number their calls per exchanging block and cut the rows into blocks differently
        self._bufs, self._handles, sets = [], [], []
        for _ in range(2):
            buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            buf.zero_()
            handle = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in handle.buffer_ptrs]
            if len(ptrs) != world or ptrs[rank] != buf.data_ptr():
                raise ShardExchangeError("symmetric memory rendezvous returned an unexpected set of buffers")
            self._bufs.append(buf); self._handles.append(handle); sets.append(ptrs)
        self.buf, self.ptrs, self.ptrs_one = self._bufs[0], sets[0], sets[1]
        torch.cuda.synchronize(device)          # every rank's buffer is zero before anybody stores into it
        dist.barrier()

    def combine(self, partial, out, lse=None, *, timeout_cycles=0, stream=None):
        from . import capi
        return capi.exchange_combine(partial, self.ptrs, self.rank, out, lse, timeout_cycles=timeout_cycles, stream=stream)

    def supports_one_launch(self, B, Hq, Hkv):
        """Whether vb200_decode_exchange_fwd takes this shape (else: decode call + combine())."""
        return Hq % Hkv == 0 and Hq // Hkv in (4, 8) and B * Hkv <= 64


def cuda_step(step: ShardedDecodeStep, q, k_shard, v_shard, *, scale, theta, partial_buf, out, lse=None,
              gathered=None, workspace=None, dist=None, stream=None, exchange: PeerExchange | None = None, qpos=None,
              one_launch=False):
    """GPU implementation of one step on this rank.  ``k_shard``/``v_shard`` hold rows
    [begin, end) of the sequence; ``q`` is the unrotated query [B,Hq,1,D] (replicated).
    With ``exchange`` the partial records travel and merge in one peer-memory kernel -- with ``one_launch`` as the
    tail of the decode kernel itself (vb200_decode_exchange_fwd); without ``exchange`` they go through a
    host-supervised all-gather followed by ``vb200_lse_combine``."""
    import torch
    from . import capi
    begin, end = shard_range(step.context_len, step.world, step.rank)
    B, Hq, _, D = q.shape
    if qpos is None:
        qpos = torch.full((B,), step.context_len, dtype=torch.int32, device=q.device)
    if exchange is not None and one_launch:
        capi.decode_exchange(q, k_shard, v_shard, exchange.ptrs_one, exchange.rank, out, lse, scale=scale, theta=theta,
                             uniform_len=end - begin, max_len=end - begin, pos_offset=begin, q_positions=qpos,
                             workspace=workspace, stream=stream)
        return out
    if step.world == 1 and exchange is None:
        # one shard: nothing to exchange or merge, the decode call writes the result itself
        capi.decode(q, out.view(B, Hq, 1, D), k_shard, v_shard, scale=scale, theta=theta, uniform_len=end - begin, max_len=end - begin,
                    pos_offset=begin, q_positions=qpos, lse=lse, workspace=workspace, stream=stream)
        return out
    capi.decode(q, None, k_shard, v_shard, scale=scale, theta=theta, uniform_len=end - begin, max_len=end - begin,
                pos_offset=begin, q_positions=qpos, partial_out=partial_buf, workspace=workspace, stream=stream)
    if exchange is not None:
        exchange.combine(partial_buf.view(B * Hq, D + 2), out, lse, stream=stream)
        return out
    if step.world == 1:
        g = partial_buf.view(1, B * Hq, D + 2)
    else:
        g = gathered if gathered is not None else torch.empty(step.world, B * Hq, D + 2, dtype=torch.float32, device=q.device)
        guarded_all_gather(dist, g.view(step.world * B * Hq, D + 2), partial_buf.view(B * Hq, D + 2), step.timeout_s)
    capi.lse_combine(g, out, lse, stream=stream)
    return out
