"""Build libvesper_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m vesper_b200.build            # incremental
    python -m vesper_b200.build --force    # rebuild everything
    python -m vesper_b200.build --verbose  # also print ptxas resource usage

nvcc cross-compiles without a GPU; the resulting vesper_b200/lib/libvesper_b200.so
links the static CUDA runtime and has no link-time dependency on the driver.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")
LIB = os.path.join(LIBDIR, "libvesper_b200.so")

SOURCES = ["api.cu", "rope_append.cu", "prefill_f32.cu", "prefill_sm100.cu", "prefill_pair_sm100.cu", "decode_splitkv.cu", "decode_generic.cu", "decode_static.cu",
           "linear_sm100.cu", "block_ops.cu", "decode_exchange.cu", "decode_gqa_mma.cu", "flash_bwd_f32.cu"]
HEADERS = ["common.cuh", "kernels.h", os.path.join("..", "..", "include", "vesper_b200.h"),
           os.path.join("..", "..", "include", "vesper_b200_block.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-O2",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = _nvcc()
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + hdrs):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        list(ex.map(run, jobs))
    objs = [os.path.join(OBJDIR, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        run([nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"])
    return LIB


HOST_DIR = os.path.join(PKG, "host")
HOST_LIB = os.path.join(LIBDIR, "libvesper_b200_host.so")
HOST_SOURCES = ["tensor.cpp", "attention.cpp", "attention_modules.cpp", "transformer.cpp", "generator.cpp", "modules.cpp", "c_api.cpp"]


def build_host(force: bool = False) -> str:
    """C++17 host layer with Vesper's class and function names (vesper_b200/host) on top of the C ABI."""
    build(force=False)
    nvcc = _nvcc()
    srcs = [os.path.join(HOST_DIR, "src", s) for s in HOST_SOURCES]
    hdrs = []
    for root, _, files in os.walk(os.path.join(HOST_DIR, "include")):
        hdrs += [os.path.join(root, f) for f in files]
    if force or _stale(HOST_LIB, srcs + hdrs + [LIB, os.path.join(PKG, "..", "include", "vesper_b200.h")]):
        cmd = [nvcc, "-shared", "-std=c++17", "-O2", "-Xcompiler", "-fPIC,-Wall",
               "-I", os.path.join(HOST_DIR, "include"), "-I", os.path.join(PKG, "..", "include")] + srcs + \
              ["-o", HOST_LIB, "-L", LIBDIR, "-lvesper_b200", "-Xlinker", "-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("host layer build failed")
    return HOST_LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    print(build_host(a.force))
