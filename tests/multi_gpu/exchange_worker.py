"""One rank of the multi-GPU check of the fused exchange (run under torch.distributed.run by
tests/test_exchange_multi_gpu.py): sequence-sharded decode steps through PeerExchange must give the
result of the all-gather + vb200_lse_combine path and of the single-GPU attention over the whole
context (computed by rank 0 with the same library)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from vesper_b200 import capi  # noqa: E402
from vesper_b200.sharded import PeerExchange, ShardedDecodeStep, cuda_step, shard_range  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    capi.load()
    B, Hq, Hkv, D, L = 1, 64, 8, 128, 8192
    g = torch.Generator().manual_seed(5)
    k_all = torch.randn(B, Hkv, L, D, generator=g).to(torch.bfloat16)
    v_all = torch.randn(B, Hkv, L, D, generator=g).to(torch.bfloat16)
    begin, end = shard_range(L, world, rank)
    ks, vs = k_all[:, :, begin:end].contiguous().to(dev), v_all[:, :, begin:end].contiguous().to(dev)
    step = ShardedDecodeStep(world, rank, L)
    ex = PeerExchange(dist, world, rank, B * Hq, D, dev)
    part = torch.empty(B * Hq, D + 2, dtype=torch.float32, device=dev)
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    scale = float(1.0 / np.sqrt(D))
    worst = 0.0
    for it in range(6):
        q = torch.randn(B, Hq, 1, D, generator=torch.Generator().manual_seed(100 + it)).to(torch.bfloat16).to(dev)
        out_fused = torch.empty(B * Hq, D, dtype=torch.bfloat16, device=dev)
        lse_fused = torch.empty(B * Hq, dtype=torch.float32, device=dev)
        out_nccl = torch.empty_like(out_fused)
        lse_nccl = torch.empty_like(lse_fused)
        cuda_step(step, q, ks, vs, scale=scale, theta=10000.0, partial_buf=part, out=out_fused, lse=lse_fused, workspace=ws, exchange=ex)
        cuda_step(step, q, ks, vs, scale=scale, theta=10000.0, partial_buf=part, out=out_nccl, lse=lse_nccl, workspace=ws, dist=dist)
        # decode + split merge + exchange in ONE launch
        out_one_launch = torch.empty_like(out_fused)
        lse_one_launch = torch.empty_like(lse_fused)
        cuda_step(step, q, ks, vs, scale=scale, theta=10000.0, partial_buf=part, out=out_one_launch, lse=lse_one_launch, workspace=ws,
                  exchange=ex, one_launch=True)
        torch.cuda.synchronize()
        capi.check_kernel_status(local)
        assert torch.equal(out_fused, out_nccl), f"rank {rank} step {it}: fused exchange differs from all-gather + combine"
        assert torch.allclose(lse_fused, lse_nccl, atol=1e-6, rtol=0)
        # (its split merge sums in another order: equal up to one rounding of the 16-bit output)
        assert (out_one_launch.float() - out_fused.float()).abs().max().item() <= 2e-3, f"rank {rank} step {it}: one-launch step differs"
        assert torch.allclose(lse_one_launch, lse_fused, atol=1e-5, rtol=0)
        if rank == 0:
            # single-GPU attention over the whole context through the same library (q rotated at position L)
            one = ShardedDecodeStep(1, 0, L)
            out_one = torch.empty_like(out_fused)
            cuda_step(one, q, k_all.to(dev), v_all.to(dev), scale=scale, theta=10000.0, partial_buf=part, out=out_one, workspace=ws)
            torch.cuda.synchronize()
            worst = max(worst, float((out_one.float() - out_fused.float()).abs().max()))
    if rank == 0:
        assert worst <= 1e-2, worst
        print(f"exchange ok: world {world}, fused == all-gather path bit for bit, max-abs vs one GPU {worst:.2e}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
