"""The literal drop-in: the reference's OWN test programs, unmodified, linked with the reference's host library
(compiled with -DUSE_CUDA_BACKEND=1 from the reference tree, never copied) and with
vesper_b200/dropin/vesper_cuda_backend.cu as its CUDA backend, i.e. onto libvesper_b200's kernels.

    tests/test_flash_attention.cpp   GPU section :195-284 (basic non-causal B2 H4 N64 D64 and causal B2 H8 N128 D64
                                     against the CPU reference attention at rtol 1e-2 / atol 1e-3; N=1024 finite)
                                     and :547-576 (dropout arguments accepted)
    tests/test_attention.cpp         scaled_dot_product_attention on Device::CUDA: shapes, causality, CPU vs GPU 1e-4
                                     (the standard path: gemm_batch / div / add / softmax seams)

The programs are built by `make -C oracle dropin` where the reference tree is present (oracle/_ref/dropin, which
travels to the GPU machine as a built artefact); the GPU test runs them and reads the PASSED lines they print, not
the exit code (the reference's static destructors can fault after main returns).
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DROPIN = os.path.join(ROOT, "oracle", "_ref", "dropin")
REF = os.path.abspath(os.path.join(ROOT, "..", "reference"))

FLASH_LINES = [
    "Flash Attention basic (GPU): PASSED",
    "Flash Attention causal (GPU): PASSED",
    "Flash Attention long sequence (GPU): PASSED",
    "Flash Attention with dropout (GPU): PASSED",
    "All Flash Attention tests PASSED!",
]
ATTENTION_LINES = ["Attention Shapes Passed!", "Attention Causality Passed!", "Attention CPU vs GPU Passed!"]


def test_dropin_programs_build_against_the_reference_tree(lib):
    if not os.path.isdir(os.path.join(REF, "src")):
        pytest.skip("the reference tree is not present on this machine")
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("nvcc is needed to compile the backend")
    from oracle.binding import build_oracle
    build_oracle(ref=False, dropin=True)
    for name in ("test_flash_attention", "test_attention"):
        assert os.access(os.path.join(DROPIN, name), os.X_OK)
    # the backend defines every *_cuda* symbol the reference's host objects leave open: the link above is the proof;
    # the hot-path ones are real adapters, not stubs
    src = open(os.path.join(ROOT, "vesper_b200", "dropin", "vesper_cuda_backend.cu")).read()
    for sym in ("vb200_prefill_fwd", "vb200_attention_bwd", "vb200_repeat_kv", "vb200_apply_rope"):
        assert sym in src


def run_program(name):
    exe = os.path.join(DROPIN, name)
    if not os.access(exe, os.X_OK):
        pytest.skip(f"{exe} was not built (needs the reference tree at build time)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:], r.stderr[-2000:])
    return r.stdout


@pytest.mark.gpu
def test_reference_flash_attention_program_passes_on_this_backend(lib, cuda):
    out = run_program("test_flash_attention")
    for line in FLASH_LINES:
        assert line in out, line


@pytest.mark.gpu
def test_reference_attention_program_passes_on_this_backend(lib, cuda):
    out = run_program("test_attention")
    for line in ATTENTION_LINES:
        assert line in out, line
