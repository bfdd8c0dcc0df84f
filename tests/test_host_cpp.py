"""The C++17 host layer (vesper_b200/host: Vesper's class and function names over the C ABI).

CPU part: it compiles and links, and the headers keep the reference's signatures.
GPU part: the assert-style executable tests/cpp/test_attention_b200.cpp, written like the
reference's own tests (flash op GPU-vs-CPU, KV cache, cached == uncached, RoPE, repeat_kv),
with the CPU oracle linked in as the checker.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "tests", "cpp", "_build")
EXE = os.path.join(BUILD, "test_attention_b200")


def build_exe():
    from oracle.binding import ORACLE_SO, build_oracle
    from vesper_b200.build import LIBDIR, build_host
    build_host()
    if not os.path.exists(ORACLE_SO):
        build_oracle(ref=False)
    os.makedirs(BUILD, exist_ok=True)
    src = os.path.join(ROOT, "tests", "cpp", "test_attention_b200.cpp")
    deps = [src, os.path.join(LIBDIR, "libvesper_b200_host.so"), ORACLE_SO]
    if os.path.exists(EXE) and all(os.path.getmtime(d) <= os.path.getmtime(EXE) for d in deps):
        return EXE
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "vesper_b200", "host", "include"),
           "-I", os.path.join(ROOT, "include"), src, "-o", EXE,
           "-L", LIBDIR, "-lvesper_b200_host", "-lvesper_b200", "-L", os.path.dirname(ORACLE_SO), "-l:liboracle.so",
           f"-Wl,-rpath,{LIBDIR}", f"-Wl,-rpath,{os.path.dirname(ORACLE_SO)}"]
    subprocess.check_call(cmd)
    return EXE


def test_host_layer_builds_and_links(lib):
    exe = build_exe()
    assert os.access(exe, os.X_OK)


def test_headers_keep_reference_signatures():
    inc = os.path.join(ROOT, "vesper_b200", "host", "include", "vesper")
    fa = open(os.path.join(inc, "ops", "flash_attention.h")).read()
    assert "Tensor flash_attention(const Tensor& q, const Tensor& k, const Tensor& v, float scale," in fa
    assert "bool is_causal = true, float dropout_p = 0.0f, bool training = false);" in fa
    assert "void flash_attention_cuda_dispatch(const Tensor& q, const Tensor& k, const Tensor& v," in fa
    kv = open(os.path.join(inc, "nn", "transformer.h")).read()
    assert "std::pair<Tensor, Tensor> update(const Tensor& new_k, const Tensor& new_v, int start_pos);" in kv
    assert "int current_seq_len() const" in kv and "int get_max_seq_len() const" in kv and "void reset();" in kv
    fn = open(os.path.join(inc, "nn", "functional.h")).read()
    assert "Tensor scaled_dot_product_attention(const Tensor& query, const Tensor& key, const Tensor& value," in fn
    assert "Tensor compute_rope_frequencies(int seq_len, int head_dim, int start_pos = 0, float theta = 10000.0f," in fn
    assert "Tensor apply_rotary_emb(const Tensor& x, const Tensor& freqs);" in fn
    assert "std::tuple<Tensor, Tensor, Tensor> flash_attention_backward(const Tensor& grad_output, const Tensor& q, const Tensor& k," in fa
    tm = open(os.path.join(inc, "models", "transformer.h")).read()
    assert "explicit TransformerLM(const TransformerConfig& config);" in tm
    assert "Tensor forward_with_cache(const Tensor& tokens, int64_t start_pos" in tm
    assert "void init_cache(int64_t batch_size, Device device);" in tm and "void clear_cache();" in tm
    gn = open(os.path.join(inc, "generation", "generator.h")).read()
    assert "explicit Generator(models::TransformerLM* model)" in gn
    assert "Tensor generate(const Tensor& prompt_ids, const SamplingParams& params);" in gn


@pytest.mark.gpu
def test_cpp_attention_suite_on_gpu(lib, cuda):
    exe = build_exe()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:], r.stderr[-2000:])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "All B200 host-layer tests passed" in r.stdout
