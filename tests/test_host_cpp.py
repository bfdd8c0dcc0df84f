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


REF_INCLUDE = os.path.abspath(os.path.join(ROOT, "..", "reference", "include", "vesper"))
HOST_INCLUDE = os.path.join(ROOT, "vesper_b200", "host", "include", "vesper")

# (header, text that starts the declaration) of every reference interface the host layer stands behind
SIGNATURES = [
    ("ops/flash_attention.h", "Tensor flash_attention("),
    ("ops/flash_attention.h", "std::tuple<Tensor, Tensor, Tensor> flash_attention_backward("),
    ("ops/attention_ops.h", "Tensor repeat_kv("),
    ("nn/transformer.h", "std::pair<Tensor, Tensor> update("),
    ("nn/transformer.h", "void reset("),
    ("nn/transformer.h", "int current_seq_len("),
    ("nn/transformer.h", "int get_max_seq_len("),
    ("nn/transformer.h", "Tensor forward(const Tensor& x, KVCache* cache, int start_pos"),
    ("nn/gqa_attention.h", "Tensor forward(const Tensor& x, bool causal"),
    ("nn/gqa_attention.h", "Tensor forward(const Tensor& x, KVCache* cache, int64_t start_pos"),
    ("nn/functional.h", "Tensor scaled_dot_product_attention("),
    ("nn/functional.h", "Tensor compute_rope_frequencies("),
    ("nn/functional.h", "Tensor apply_rotary_emb("),
    ("models/transformer.h", "explicit TransformerLM("),
    ("models/transformer.h", "void init_cache("),
    ("models/transformer.h", "void clear_cache("),
    ("generation/generator.h", "explicit Generator("),
    ("generation/generator.h", "Tensor generate("),
]
# constructors the host layer extends with one trailing defaulted argument (dtype): the reference's argument list
# must be a prefix of ours
CONSTRUCTORS = [
    ("nn/transformer.h", "KVCache(int batch_size"),
    ("nn/transformer.h", "MultiHeadAttention(int embed_dim"),
    ("nn/gqa_attention.h", "GroupedQueryAttention("),
]


def declaration(text, start):
    """The declaration that begins with `start`: up to the closing parenthesis of its parameter list, comments and
    line breaks removed, default values kept, blanks collapsed."""
    import re
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"\s+", " ", text)
    text = re.sub(r"\s*([(),])\s*", r"\1", text)        # no blanks around brackets and commas
    text = re.sub(r"\s*=\s*", " = ", text)               # one blank around a default value's "="
    start = re.sub(r"\s*([(),])\s*", r"\1", re.sub(r"\s+", " ", start))
    i = text.find(start)
    if i < 0:
        return None
    depth, j = 0, i + start.index("(")
    while True:
        depth += text[j] == "("
        depth -= text[j] == ")"
        if depth == 0:
            return text[i:j + 1]
        j += 1


def test_headers_keep_reference_signatures():
    """Every interface of the path is declared in the host layer exactly as in the reference's header of the same
    name (parsed out of the reference tree when it is present; on a machine without it the comparison falls back to
    the declarations recorded below)."""
    recorded = {
        "Tensor flash_attention(": "Tensor flash_attention(const Tensor& q,const Tensor& k,const Tensor& v,float scale,bool is_causal = true,float dropout_p = 0.0f,bool training = false)",
        "Tensor scaled_dot_product_attention(": "Tensor scaled_dot_product_attention(const Tensor& query,const Tensor& key,const Tensor& value,bool is_causal = false,double dropout_p = 0.0)",
        "std::pair<Tensor, Tensor> update(": "std::pair<Tensor,Tensor> update(const Tensor& new_k,const Tensor& new_v,int start_pos)",
        "Tensor generate(": "Tensor generate(const Tensor& prompt_ids,const SamplingParams& params)",
    }
    have_ref = os.path.isdir(REF_INCLUDE)
    for header, start in SIGNATURES:
        ours = declaration(open(os.path.join(HOST_INCLUDE, header)).read(), start)
        assert ours is not None, f"{start} not declared in the host layer's {header}"
        if have_ref:
            theirs = declaration(open(os.path.join(REF_INCLUDE, header)).read(), start)
            assert theirs is not None, f"{start} not found in the reference's {header}"
            assert ours == theirs, f"{header}: {ours!r} differs from the reference's {theirs!r}"
        elif start in recorded:
            assert ours == recorded[start]
    for header, start in CONSTRUCTORS:
        ours = declaration(open(os.path.join(HOST_INCLUDE, header)).read(), start)
        assert ours is not None, f"{start} not declared in the host layer's {header}"
        if have_ref:
            theirs = declaration(open(os.path.join(REF_INCLUDE, header)).read(), start)
            assert theirs is not None
            assert ours[:len(theirs) - 1] == theirs[:-1], f"{header}: {ours!r} does not extend the reference's {theirs!r}"
            assert ours[len(theirs) - 1:] in (")", ",DType dtype = DType::Float32)", ",DType dtype = DType::BFloat16)")


@pytest.mark.gpu
def test_cpp_attention_suite_on_gpu(lib, cuda):
    exe = build_exe()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:], r.stderr[-2000:])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "All B200 host-layer tests passed" in r.stdout
