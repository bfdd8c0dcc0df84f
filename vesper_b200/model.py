"""ctypes binding of the C facade of the host layer (libvesper_b200_host.so: models::TransformerLM
and generation::Generator, vesper_b200/host/src/c_api.cpp) for the Python tests and the benchmark.
Every computation happens in the CUDA library underneath; there is no fallback."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

PKG = os.path.dirname(os.path.abspath(__file__))
HOST_LIB_PATH = os.path.join(PKG, "lib", "libvesper_b200_host.so")

HOST_EXPORTS = ["vbh_last_error", "vbh_model_new", "vbh_model_free", "vbh_model_set_param", "vbh_model_init_cache",
                "vbh_model_forward_with_cache", "vbh_generate_greedy", "vbh_attn_new", "vbh_attn_free", "vbh_attn_load",
                "vbh_kvcache_new", "vbh_kvcache_free", "vbh_kvcache_len", "vbh_attn_forward"]

_host = None
_i64 = C.c_int64
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)


def load_host():
    global _host
    if _host is not None:
        return _host
    if not os.path.exists(HOST_LIB_PATH):
        raise FileNotFoundError(f"{HOST_LIB_PATH} is missing: run `python -m vesper_b200.build`")
    from . import capi
    capi.load()                               # the C-ABI library the host layer links against
    L = C.CDLL(HOST_LIB_PATH)
    L.vbh_last_error.restype = C.c_char_p
    L.vbh_model_new.argtypes = [_i64] * 7 + [C.c_float, C.c_float]
    L.vbh_model_new.restype = C.c_void_p
    L.vbh_model_free.argtypes = [C.c_void_p]
    L.vbh_model_set_param.argtypes = [C.c_void_p, C.c_char_p, _f32p, _i64]
    L.vbh_model_init_cache.argtypes = [C.c_void_p, _i64]
    L.vbh_model_forward_with_cache.argtypes = [C.c_void_p, _i32p, _i64, _i64, _i64, C.c_int, _f32p]
    L.vbh_generate_greedy.argtypes = [C.c_void_p, _i32p, _i64, _i64, _i64, C.POINTER(_i64), _i64, _i64, C.c_int, _i32p, C.POINTER(C.c_double)]
    L.vbh_generate_greedy.restype = _i64
    L.vbh_attn_new.argtypes = [C.c_int, _i64, _i64, _i64, _i64, C.c_float, C.c_int, C.c_int, C.c_int]
    L.vbh_attn_new.restype = C.c_void_p
    L.vbh_attn_free.argtypes = [C.c_void_p]
    L.vbh_attn_load.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, _f32p]
    L.vbh_kvcache_new.argtypes = [_i64, _i64, _i64, _i64, C.c_int]
    L.vbh_kvcache_new.restype = C.c_void_p
    L.vbh_kvcache_free.argtypes = [C.c_void_p]
    L.vbh_kvcache_len.argtypes = [C.c_void_p]
    L.vbh_attn_forward.argtypes = [C.c_void_p, _f32p, _i64, _i64, _i64, C.c_int, C.c_int, C.c_void_p, _i64, _f32p]
    _host = L
    return L


def param_shapes(vocab, dim, n_layers, n_heads, n_kv_heads, ffn_hidden):
    """Parameter names and shapes of the Llama-style TransformerLM (the reference's named_parameters)."""
    D = dim // n_heads
    out = {"tok_embeddings.weight": (vocab, dim), "norm.weight": (dim,), "output.weight": (vocab, dim)}
    for l in range(n_layers):
        p = f"layers.{l}."
        out[p + "attention_norm.weight"] = (dim,)
        out[p + "attention.wqkv.weight"] = ((n_heads + 2 * n_kv_heads) * D, dim)
        out[p + "attention.wo.weight"] = (dim, n_heads * D)
        out[p + "ffn_norm.weight"] = (dim,)
        out[p + "feed_forward.gate_proj.weight"] = (ffn_hidden, dim)
        out[p + "feed_forward.up_proj.weight"] = (ffn_hidden, dim)
        out[p + "feed_forward.down_proj.weight"] = (dim, ffn_hidden)
    return out


class TransformerLM:
    def __init__(self, vocab, dim, n_layers, n_heads, n_kv_heads, ffn_hidden, max_seq_len, norm_eps=1e-6, rope_base=10000.0):
        self.L = load_host()
        self.vocab = vocab
        self.cfg = dict(vocab=vocab, dim=dim, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_kv_heads, ffn_hidden=ffn_hidden)
        self.h = self.L.vbh_model_new(vocab, dim, n_layers, n_heads, n_kv_heads, ffn_hidden, max_seq_len, norm_eps, rope_base)
        if not self.h:
            raise RuntimeError(self.L.vbh_last_error().decode())

    def _chk(self, rc):
        if rc < 0:
            raise RuntimeError(self.L.vbh_last_error().decode())
        return rc

    def param_shapes(self):
        return param_shapes(**self.cfg)

    def set_param(self, name, value):
        value = np.ascontiguousarray(value, dtype=np.float32)
        self._chk(self.L.vbh_model_set_param(self.h, name.encode(), value.ctypes.data_as(_f32p), value.size))

    def init_cache(self, B):
        self._chk(self.L.vbh_model_init_cache(self.h, B))

    def forward_with_cache(self, ids, start_pos, last_only=False):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        B, T = ids.shape
        y = np.empty((B, 1 if last_only else T, self.vocab), np.float32)
        self._chk(self.L.vbh_model_forward_with_cache(self.h, ids.ctypes.data_as(_i32p), B, T, start_pos, int(last_only), y.ctypes.data_as(_f32p)))
        return y

    def generate_greedy(self, prompt, max_new, stop_ids=(), min_new=0, use_graph=True):
        """Returns (tokens [B, P + generated] int32, timings dict)."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        B, P = prompt.shape
        out = np.zeros((B, P + max_new), np.int32)
        stop = np.ascontiguousarray(list(stop_ids), dtype=np.int64)
        t = (C.c_double * 4)()
        cols = self._chk(self.L.vbh_generate_greedy(self.h, prompt.ctypes.data_as(_i32p), B, P, max_new, stop.ctypes.data_as(C.POINTER(_i64)),
                                                     stop.size, min_new, int(use_graph), out.ctypes.data_as(_i32p), t))
        toks = out.reshape(-1)[: B * cols].reshape(B, cols)
        return toks, {"prefill_ms": t[0], "decode_ms": t[1], "decode_steps": int(t[2]), "graph_replay": bool(t[3])}

    def close(self):
        if getattr(self, "h", None):
            self.L.vbh_model_free(self.h)
            self.h = None

    def __del__(self):
        self.close()


def _fp(a):
    return None if a is None else a.ctypes.data_as(_f32p)


class KVCache:
    """nn::KVCache of the host layer ([B, H, max_seq_len, D] on the GPU; dtype "f32" or "bf16")."""

    def __init__(self, B, H, max_seq_len, D, dtype="bf16"):
        self.L = load_host()
        self.h = self.L.vbh_kvcache_new(B, H, max_seq_len, D, 0 if dtype == "f32" else 1)
        if not self.h:
            raise RuntimeError(self.L.vbh_last_error().decode())

    def __len__(self):
        return self.L.vbh_kvcache_len(self.h)

    def __del__(self):
        if getattr(self, "h", None):
            self.L.vbh_kvcache_free(self.h)
            self.h = None


class AttentionModule:
    """nn::GroupedQueryAttention (kind "gqa") or nn::MultiHeadAttention (kind "mha") of the host layer, with the
    reference's constructor arguments and forward overloads; host fp32 arrays in and out."""

    def __init__(self, kind, embed_dim, num_heads, num_kv_heads=None, max_seq_len=4096, rope_base=10000.0, bias=False,
                 use_rope=True, dtype="bf16"):
        self.L = load_host()
        self.C = embed_dim
        self.h = self.L.vbh_attn_new(0 if kind == "gqa" else 1, embed_dim, num_heads, num_kv_heads or num_heads, max_seq_len, rope_base,
                                     int(bias), int(use_rope), 0 if dtype == "f32" else 1)
        if not self.h:
            raise RuntimeError(self.L.vbh_last_error().decode())

    def load(self, w_in, w_out, b_in=None, b_out=None):
        arrs = [None if a is None else np.ascontiguousarray(a, np.float32) for a in (w_in, b_in, w_out, b_out)]
        if self.L.vbh_attn_load(self.h, *[_fp(a) for a in arrs]) != 0:
            raise RuntimeError(self.L.vbh_last_error().decode())

    def _run(self, x, mode, causal, cache, start_pos):
        x = np.ascontiguousarray(x, np.float32)
        B, T, C_ = x.shape
        y = np.empty_like(x)
        if self.L.vbh_attn_forward(self.h, _fp(x), B, T, C_, mode, int(causal), cache.h if cache is not None else None, start_pos, _fp(y)) != 0:
            raise RuntimeError(self.L.vbh_last_error().decode())
        return y

    def forward(self, x, causal=None):
        return self._run(x, 0, False, None, 0) if causal is None else self._run(x, 1, causal, None, 0)

    def forward_cached(self, cache, x, start_pos):
        return self._run(x, 2, False, cache, start_pos)

    def __del__(self):
        if getattr(self, "h", None):
            self.L.vbh_attn_free(self.h)
            self.h = None
