"""Shared helpers for the parity tests."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def bf16_round(x):
    """Round-to-nearest-even fp32 -> bf16 -> fp32 (include/vesper/core/half.h:162-173)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(x.shape)


def fp16_round(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def to_torch(x, dtype, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device=device, dtype=dtype)


def from_torch(t):
    return t.detach().float().cpu().numpy()


def maxabs(a, b):
    return float(np.max(np.abs(np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64))))
