"""The opt-in two-SM prefill kernel (prefill_pair_sm100.cu, selected with VB200_PREFILL_KERNEL=pair) against the same
oracle cases as the default kernel.  The switch is read once per process, so the cases run in a child pytest."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# the head_dim-128, 16-bit cases of tests/test_prefill_gpu.py (the only shapes the two-SM kernel takes; everything
# else stays on the default kernels whatever the switch says)
CASES = "16bit or rope or far_position or aligned_to or sdpa or config2"


@pytest.mark.gpu
def test_pair_kernel_passes_the_prefill_parity_cases(lib, cuda):
    env = dict(os.environ, VB200_PREFILL_KERNEL="pair")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_prefill_gpu.py"), "-m", "gpu", "-q", "--tb=short",
                        "-x", "-k", CASES, "-p", "no:cacheprovider"], capture_output=True, text=True, timeout=900, cwd=ROOT, env=env)
    tail = r.stdout[-3000:] + r.stderr[-2000:]
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and "failed" not in r.stdout, tail


PROBE = """
import sys
import numpy as np, torch
sys.path.insert(0, {root!r})
from vesper_b200 import capi
L = capi.load()
dev = torch.device("cuda:0")
q = torch.randn(1, 4, 256, 128, device=dev).to(torch.bfloat16); k = torch.randn(1, 2, 256, 128, device=dev).to(torch.bfloat16)
o = torch.empty_like(q)
import ctypes as C
a = capi.prefill_args(q, k, k, o, None, scale=0.088, causal=True)
ws = torch.empty(max(256, L.vb200_prefill_workspace_bytes(C.byref(a))), dtype=torch.uint8, device=dev)
a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
capi.check(L.vb200_prefill_fwd(C.byref(a))); torch.cuda.synchronize()
print("KERNEL", L.vb200_last_prefill_kernel().decode())
"""


@pytest.mark.gpu
@pytest.mark.parametrize("switch,kernel", [("pair", "prefill_pair_kernel"), ("single", "prefill_sm100_kernel"), (None, "prefill_sm100_kernel")])
def test_the_switch_selects_the_kernel(lib, cuda, switch, kernel):
    env = dict(os.environ)
    env.pop("VB200_PREFILL_KERNEL", None)
    if switch:
        env["VB200_PREFILL_KERNEL"] = switch
    r = subprocess.run([sys.executable, "-c", PROBE.format(root=ROOT)], capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    assert f"KERNEL {kernel}" in r.stdout, r.stdout[-500:]
