"""ctypes bindings for the two CPU checkers -- TEST INFRASTRUCTURE ONLY.

``Oracle``  wraps ``oracle/liboracle.so``  (the plain-C restatement).
``Ref``     wraps ``oracle/_ref/libvesper_ref.so`` (the unmodified reference CPU
            code behind ``ref_shim.cpp``); present only where it was built.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import
this module; the CUDA product path never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libvesper_ref.so")

_f32p = C.POINTER(C.c_float)
_i64 = C.c_int64


def _fp(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def build_oracle(ref: bool = True, dropin: bool = False) -> None:
    """Compile liboracle.so (always), _ref (only when the reference tree exists) and, on request, the reference's
    own test programs linked against this repository's CUDA backend (_ref/dropin; needs nvcc and the built library)."""
    targets = ["oracle"] + (["ref"] if ref else []) + (["dropin"] if dropin else [])
    subprocess.check_call(["make", "-s", "-C", HERE, "-j8"] + targets)


def ref_available() -> bool:
    return os.path.exists(REF_SO)


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build_oracle(ref=False)
        self.lib = C.CDLL(ORACLE_SO)
        L = self.lib
        L.vo_flash_attention_fwd.argtypes = [_f32p] * 5 + [_i64] * 4 + [C.c_float, C.c_int]
        L.vo_sdpa_standard.argtypes = [_f32p] * 5 + [_i64] * 5 + [C.c_int]
        L.vo_sdpa.argtypes = [_f32p] * 4 + [_i64] * 5 + [C.c_int]
        L.vo_sdpa.restype = C.c_int
        L.vo_rope_frequencies.argtypes = [C.c_int, C.c_int, C.c_int, C.c_float, _f32p]
        L.vo_apply_rotary_emb.argtypes = [_f32p] * 3 + [_i64] * 4
        L.vo_repeat_kv.argtypes = [_f32p] * 2 + [_i64] * 5
        L.vo_kv_cache_update.argtypes = [_f32p] * 4 + [_i64] * 6 + [C.POINTER(_i64)]
        L.vo_cache_active.argtypes = [_f32p] * 2 + [_i64] * 5
        L.vo_gqa_attention_cached.argtypes = [_f32p] * 7 + [_i64] * 7 + [C.c_float, C.c_int, C.POINTER(_i64)]
        L.vo_gqa_attention_cached.restype = C.c_int
        L.vo_decode_ragged.argtypes = [_f32p] * 3 + [C.POINTER(C.c_int32)] + [_f32p] * 2 + [_i64] * 5
        L.vo_lse_combine.argtypes = [_f32p] * 5 + [_i64] * 3
        L.vo_bf16_round_array.argtypes = [_f32p, _f32p, _i64]
        L.vo_flash_attention_bwd.argtypes = [_f32p] * 9 + [_i64] * 4 + [C.c_float, C.c_int]
        _i32p = C.POINTER(C.c_int32)
        L.vo_linear.argtypes = [_f32p] * 3 + [_i64] * 3
        L.vo_rms_norm.argtypes = [_f32p] * 3 + [_i64] * 2 + [C.c_float]
        L.vo_silu_mul.argtypes = [_f32p] * 3 + [_i64]
        L.vo_embedding.argtypes = [_i32p, _f32p, _f32p] + [_i64] * 3
        L.vo_embedding.restype = C.c_int
        L.vo_argmax.argtypes = [_f32p, _i32p, _i64, _i64]
        L.vo_check_stop_tokens.argtypes = [_i32p, _i32p, _i64, C.POINTER(_i64), _i64, _i64, _i64]

    def flash_attention(self, q, k, v, scale, causal=True):
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, H, N, D = q.shape
        o = np.empty_like(q)
        lse = np.empty((B, H, N), np.float32)
        self.lib.vo_flash_attention_fwd(_fp(q), _fp(k), _fp(v), _fp(o), _fp(lse), B, H, N, D, scale, int(causal))
        return o, lse

    def sdpa_standard(self, q, k, v, causal=False, want_scores=False):
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, H, Tq, D = q.shape
        Tk = k.shape[2]
        o = np.empty_like(q)
        sc = np.empty((B, H, Tq, Tk), np.float32) if want_scores else None
        self.lib.vo_sdpa_standard(_fp(q), _fp(k), _fp(v), _fp(o), _fp(sc), B, H, Tq, Tk, D, int(causal))
        return (o, sc) if want_scores else o

    def sdpa(self, q, k, v, causal=False):
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, H, Tq, D = q.shape
        o = np.empty_like(q)
        rc = self.lib.vo_sdpa(_fp(q), _fp(k), _fp(v), _fp(o), B, H, Tq, k.shape[2], D, int(causal))
        if rc != 0:
            raise RuntimeError("flash_attention: Q, K, V must have same shape")
        return o

    def rope_frequencies(self, T, D, start_pos=0, theta=10000.0):
        f = np.empty((T, D // 2), np.float32)
        self.lib.vo_rope_frequencies(T, D, start_pos, theta, _fp(f))
        return f

    def apply_rope(self, x, start_pos=0, theta=10000.0):
        x = _f32(x)
        B, H, S, D = x.shape
        f = self.rope_frequencies(S, D, start_pos, theta)
        out = np.empty_like(x)
        self.lib.vo_apply_rotary_emb(_fp(x), _fp(f), _fp(out), B, H, S, D)
        return out

    def repeat_kv(self, x, n_rep):
        x = _f32(x)
        B, H, S, D = x.shape
        out = np.empty((B, H * n_rep, S, D), np.float32)
        self.lib.vo_repeat_kv(_fp(x), _fp(out), B, H, S, D, n_rep)
        return out

    def kv_cache_update(self, k_cache, v_cache, new_k, new_v, start_pos, current_len):
        new_k, new_v = _f32(new_k), _f32(new_v)
        B, H, cap, D = k_cache.shape
        T = new_k.shape[2]
        cl = _i64(current_len)
        self.lib.vo_kv_cache_update(_fp(k_cache), _fp(v_cache), _fp(new_k), _fp(new_v), B, H, cap, D, T, start_pos, C.byref(cl))
        return cl.value

    def gqa_attention_cached(self, q, k_new, v_new, k_cache, v_cache, start_pos, current_len,
                             theta=10000.0, use_rope=True, want_lse=True):
        q, k_new, v_new = _f32(q), _f32(k_new), _f32(v_new)
        B, Hq, T, D = q.shape
        Hkv, cap = k_cache.shape[1], k_cache.shape[2]
        out = np.empty_like(q)
        lse = np.empty((B, Hq, T), np.float32) if want_lse else None
        cl = _i64(current_len)
        self.lib.vo_gqa_attention_cached(_fp(q), _fp(k_new), _fp(v_new), _fp(k_cache), _fp(v_cache),
                                         _fp(out), _fp(lse), B, Hq, Hkv, T, D, cap, start_pos,
                                         theta, int(use_rope), C.byref(cl))
        return out, lse, cl.value

    def decode_ragged(self, q, k_cache, v_cache, lens):
        q = _f32(q)
        B, Hq, D = q.shape
        Hkv, cap = k_cache.shape[1], k_cache.shape[2]
        lens = np.ascontiguousarray(lens, dtype=np.int32)
        out = np.empty_like(q)
        lse = np.empty((B, Hq), np.float32)
        self.lib.vo_decode_ragged(_fp(q), _fp(k_cache), _fp(v_cache), lens.ctypes.data_as(C.POINTER(C.c_int32)),
                                  _fp(out), _fp(lse), B, Hq, Hkv, cap, D)
        return out, lse

    def lse_combine(self, m, l, o):
        m, l, o = _f32(m), _f32(l), _f32(o)
        R, rows, D = o.shape
        out = np.empty((rows, D), np.float32)
        lse = np.empty((rows,), np.float32)
        self.lib.vo_lse_combine(_fp(m), _fp(l), _fp(o), _fp(out), _fp(lse), R, rows, D)
        return out, lse

    def bf16_round(self, x):
        x = _f32(x)
        out = np.empty_like(x)
        self.lib.vo_bf16_round_array(_fp(x), _fp(out), x.size)
        return out

    def flash_attention_bwd(self, d_out, q, k, v, out, lse, scale, causal=True):
        d_out, q, k, v, out, lse = _f32(d_out), _f32(q), _f32(k), _f32(v), _f32(out), _f32(lse)
        B, H, N, D = q.shape
        dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(q)
        self.lib.vo_flash_attention_bwd(_fp(d_out), _fp(q), _fp(k), _fp(v), _fp(out), _fp(lse), _fp(dq), _fp(dk), _fp(dv), B, H, N, D, scale, int(causal))
        return dq, dk, dv

    # ---- decoder-block operators (vesper_block_oracle.c) ----
    def linear(self, x, w):
        x, w = _f32(x), _f32(w)
        M, K = x.shape
        N = w.shape[0]
        y = np.empty((M, N), np.float32)
        self.lib.vo_linear(_fp(x), _fp(w), _fp(y), M, N, K)
        return y

    def rms_norm(self, x, w, eps):
        x, w = _f32(x), _f32(w)
        y = np.empty_like(x)
        self.lib.vo_rms_norm(_fp(x), _fp(w), _fp(y), x.size // x.shape[-1], x.shape[-1], eps)
        return y

    def silu_mul(self, gate, up):
        gate, up = _f32(gate), _f32(up)
        y = np.empty_like(gate)
        self.lib.vo_silu_mul(_fp(gate), _fp(up), _fp(y), gate.size)
        return y

    def embedding(self, ids, table):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        table = _f32(table)
        y = np.empty(ids.shape + (table.shape[1],), np.float32)
        rc = self.lib.vo_embedding(ids.ctypes.data_as(C.POINTER(C.c_int32)), _fp(table), _fp(y), ids.size, table.shape[0], table.shape[1])
        if rc != 0:
            raise IndexError("embedding index out of bounds")
        return y

    def argmax(self, logits):
        logits = _f32(logits)
        out = np.empty(logits.shape[0], np.int32)
        self.lib.vo_argmax(_fp(logits), out.ctypes.data_as(C.POINTER(C.c_int32)), logits.shape[0], logits.shape[1])
        return out

    def check_stop_tokens(self, tokens, stop_ids, min_generated, generated_count):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        stop = np.ascontiguousarray(stop_ids, dtype=np.int64)
        out = np.empty(tokens.shape, np.int32)
        self.lib.vo_check_stop_tokens(tokens.ctypes.data_as(C.POINTER(C.c_int32)), out.ctypes.data_as(C.POINTER(C.c_int32)),
                                      tokens.size, stop.ctypes.data_as(C.POINTER(_i64)), stop.size, min_generated, generated_count)
        return out



class Ref:
    """The unmodified reference CPU implementation (only where it was built)."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        self.lib = C.CDLL(REF_SO)
        L = self.lib
        L.ref_last_error.restype = C.c_char_p
        L.ref_randn.argtypes = [C.c_uint64, _i64, _f32p]
        L.ref_randn_seq.argtypes = [C.c_uint64, C.c_int, C.POINTER(_i64), C.POINTER(_f32p)]
        L.ref_flash_attention.argtypes = [_f32p] * 5 + [_i64] * 4 + [C.c_float, C.c_int]
        L.ref_flash_attention_op.argtypes = [_f32p] * 4 + [_i64] * 4 + [C.c_float, C.c_int]
        L.ref_sdpa.argtypes = [_f32p] * 4 + [_i64] * 5 + [C.c_int]
        L.ref_rope_frequencies.argtypes = [C.c_int, C.c_int, C.c_int, C.c_float, _f32p]
        L.ref_apply_rope.argtypes = [_f32p, _f32p] + [_i64] * 4 + [C.c_int, C.c_float]
        L.ref_repeat_kv.argtypes = [_f32p, _f32p] + [_i64] * 5
        L.ref_kvcache_new.argtypes = [C.c_int] * 4
        L.ref_kvcache_new.restype = C.c_void_p
        L.ref_kvcache_free.argtypes = [C.c_void_p]
        L.ref_kvcache_len.argtypes = [C.c_void_p]
        L.ref_kvcache_reset.argtypes = [C.c_void_p]
        L.ref_kvcache_update.argtypes = [C.c_void_p, _f32p, _f32p] + [_i64] * 4 + [C.c_int, _f32p, _f32p]
        L.ref_gqa_attention_cached.argtypes = [C.c_void_p] + [_f32p] * 4 + [_i64] * 5 + [C.c_int, C.c_float, C.c_int]
        L.ref_gqa_new.argtypes = [_i64] * 4 + [C.c_float, _f32p, _f32p]
        L.ref_gqa_new.restype = C.c_void_p
        L.ref_gqa_free.argtypes = [C.c_void_p]
        L.ref_gqa_forward.argtypes = [C.c_void_p, _f32p, _f32p] + [_i64] * 3 + [C.c_int]
        L.ref_gqa_forward_cached.argtypes = [C.c_void_p, C.c_void_p, _f32p, _f32p] + [_i64] * 4
        _i32p = C.POINTER(C.c_int32)
        L.ref_flash_attention_backward.argtypes = [_f32p] * 9 + [_i64] * 4 + [C.c_float, C.c_int]
        L.ref_linear.argtypes = [_f32p] * 3 + [_i64] * 3
        L.ref_rms_norm.argtypes = [_f32p] * 3 + [_i64] * 2 + [C.c_float]
        L.ref_silu_mul.argtypes = [_f32p] * 3 + [_i64]
        L.ref_embedding.argtypes = [_i32p, _f32p, _f32p] + [_i64] * 3
        L.ref_argmax.argtypes = [_f32p, _i32p, _i64, _i64]
        L.ref_model_new.argtypes = [_i64] * 7 + [C.c_float, C.c_float]
        L.ref_model_new.restype = C.c_void_p
        L.ref_model_free.argtypes = [C.c_void_p]
        L.ref_model_param_names.argtypes = [C.c_void_p, C.c_char_p, _i64]
        L.ref_model_param_names.restype = _i64
        L.ref_model_set_param.argtypes = [C.c_void_p, C.c_char_p, _f32p, _i64]
        L.ref_model_forward.argtypes = [C.c_void_p, _i32p, _i64, _i64, _f32p]
        L.ref_model_init_cache.argtypes = [C.c_void_p, _i64]
        L.ref_model_forward_with_cache.argtypes = [C.c_void_p, _i32p, _i64, _i64, _i64, _f32p]
        L.ref_generate_greedy.argtypes = [C.c_void_p, _i32p, _i64, _i64, _i64, C.POINTER(_i64), _i64, _i64, _i32p]
        L.ref_generate_greedy.restype = _i64

    def _chk(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def randn_seq(self, seed, shapes):
        outs = [np.empty(s, np.float32) for s in shapes]
        sizes = (_i64 * len(shapes))(*[int(np.prod(s)) for s in shapes])
        ptrs = (_f32p * len(shapes))(*[_fp(o) for o in outs])
        self._chk(self.lib.ref_randn_seq(seed, len(shapes), sizes, ptrs))
        return outs

    def flash_attention(self, q, k, v, scale, causal=True):
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, H, N, D = q.shape
        o = np.empty_like(q)
        lse = np.empty((B, H, N), np.float32)
        self._chk(self.lib.ref_flash_attention(_fp(q), _fp(k), _fp(v), _fp(o), _fp(lse), B, H, N, D, scale, int(causal)))
        return o, lse

    def flash_attention_op(self, q, k, v, scale, causal=True):
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, H, N, D = q.shape
        o = np.empty_like(q)
        self._chk(self.lib.ref_flash_attention_op(_fp(q), _fp(k), _fp(v), _fp(o), B, H, N, D, scale, int(causal)))
        return o

    def sdpa(self, q, k, v, causal=False):
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, H, Tq, D = q.shape
        o = np.empty_like(q)
        self._chk(self.lib.ref_sdpa(_fp(q), _fp(k), _fp(v), _fp(o), B, H, Tq, k.shape[2], D, int(causal)))
        return o

    def rope_frequencies(self, T, D, start_pos=0, theta=10000.0):
        f = np.empty((T, D // 2), np.float32)
        self._chk(self.lib.ref_rope_frequencies(T, D, start_pos, theta, _fp(f)))
        return f

    def apply_rope(self, x, start_pos=0, theta=10000.0):
        x = _f32(x)
        B, H, S, D = x.shape
        out = np.empty_like(x)
        self._chk(self.lib.ref_apply_rope(_fp(x), _fp(out), B, H, S, D, start_pos, theta))
        return out

    def repeat_kv(self, x, n_rep):
        x = _f32(x)
        B, H, S, D = x.shape
        out = np.empty((B, H * n_rep, S, D), np.float32)
        self._chk(self.lib.ref_repeat_kv(_fp(x), _fp(out), B, H, S, D, n_rep))
        return out

    class KVCache:
        def __init__(self, ref, B, H, cap, D):
            self.ref, self.shape = ref, (B, H, cap, D)
            self.h = ref.lib.ref_kvcache_new(B, H, cap, D)
            if not self.h:
                raise RuntimeError(ref.lib.ref_last_error().decode())

        def update(self, new_k, new_v, start_pos):
            new_k, new_v = _f32(new_k), _f32(new_v)
            B, H, T, D = new_k.shape
            n = max(self.len, start_pos + T)
            ko, vo = np.empty((B, H, n, D), np.float32), np.empty((B, H, n, D), np.float32)
            self.ref._chk(self.ref.lib.ref_kvcache_update(self.h, _fp(new_k), _fp(new_v), B, H, T, D, start_pos, _fp(ko), _fp(vo)))
            return ko, vo

        @property
        def len(self):
            return self.ref.lib.ref_kvcache_len(self.h)

        def reset(self):
            self.ref._chk(self.ref.lib.ref_kvcache_reset(self.h))

        def __del__(self):
            if getattr(self, "h", None):
                self.ref.lib.ref_kvcache_free(self.h)
                self.h = None

    def kvcache(self, B, H, cap, D):
        return Ref.KVCache(self, B, H, cap, D)

    def gqa_attention_cached(self, cache, q, k_new, v_new, start_pos, theta=10000.0, use_rope=True):
        q, k_new, v_new = _f32(q), _f32(k_new), _f32(v_new)
        B, Hq, T, D = q.shape
        out = np.empty_like(q)
        self._chk(self.lib.ref_gqa_attention_cached(cache.h, _fp(q), _fp(k_new), _fp(v_new), _fp(out),
                                                    B, Hq, k_new.shape[1], T, D, start_pos, theta, int(use_rope)))
        return out

    class GQA:
        def __init__(self, ref, C_, Hq, Hkv, max_seq, theta, wqkv, wo):
            self.ref = ref
            wqkv, wo = _f32(wqkv), _f32(wo)
            self.h = ref.lib.ref_gqa_new(C_, Hq, Hkv, max_seq, theta, _fp(wqkv), _fp(wo))
            if not self.h:
                raise RuntimeError(ref.lib.ref_last_error().decode())

        def forward(self, x, causal=True):
            x = _f32(x)
            B, T, C_ = x.shape
            y = np.empty_like(x)
            self.ref._chk(self.ref.lib.ref_gqa_forward(self.h, _fp(x), _fp(y), B, T, C_, int(causal)))
            return y

        def forward_cached(self, cache, x, start_pos):
            x = _f32(x)
            B, T, C_ = x.shape
            y = np.empty_like(x)
            self.ref._chk(self.ref.lib.ref_gqa_forward_cached(self.h, cache.h, _fp(x), _fp(y), B, T, C_, start_pos))
            return y

        def __del__(self):
            if getattr(self, "h", None):
                self.ref.lib.ref_gqa_free(self.h)
                self.h = None

    def gqa(self, C_, Hq, Hkv, max_seq, theta, wqkv, wo):
        return Ref.GQA(self, C_, Hq, Hkv, max_seq, theta, wqkv, wo)

    class MHA:
        """nn::MultiHeadAttention (src/nn/transformer.cpp:97-216) with caller-set c_attn / c_proj weights and biases."""

        def __init__(self, ref, C_, H, use_rope, w_attn, b_attn, w_proj, b_proj):
            self.ref = ref
            L = ref.lib
            L.ref_mha_new.restype = C.c_void_p
            L.ref_mha_new.argtypes = [C.c_int, C.c_int, C.c_int] + [_f32p] * 4
            L.ref_mha_free.argtypes = [C.c_void_p]
            L.ref_mha_forward.argtypes = [C.c_void_p, _f32p, _f32p, _i64, _i64, _i64, C.c_int, C.c_int, C.c_void_p, C.c_int]
            arrs = [_f32(a) for a in (w_attn, b_attn, w_proj, b_proj)]
            self.h = L.ref_mha_new(C_, H, int(use_rope), *[_fp(a) for a in arrs])
            if not self.h:
                raise RuntimeError(L.ref_last_error().decode())

        def _run(self, x, mode, causal=False, cache=None, start_pos=0):
            x = _f32(x)
            B, T, C_ = x.shape
            y = np.empty_like(x)
            self.ref._chk(self.ref.lib.ref_mha_forward(self.h, _fp(x), _fp(y), B, T, C_, mode, int(causal), cache.h if cache else None, start_pos))
            return y

        def forward(self, x, causal=None):
            return self._run(x, 0) if causal is None else self._run(x, 1, causal)

        def forward_cached(self, cache, x, start_pos):
            return self._run(x, 2, False, cache, start_pos)

        def __del__(self):
            if getattr(self, "h", None):
                self.ref.lib.ref_mha_free(self.h)
                self.h = None

    def mha(self, C_, H, use_rope, w_attn, b_attn, w_proj, b_proj):
        return Ref.MHA(self, C_, H, use_rope, w_attn, b_attn, w_proj, b_proj)

    def flash_attention_bwd(self, d_out, q, k, v, out, lse, scale, causal=True):
        d_out, q, k, v, out, lse = _f32(d_out), _f32(q), _f32(k), _f32(v), _f32(out), _f32(lse)
        B, H, N, D = q.shape
        dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(q)
        self._chk(self.lib.ref_flash_attention_backward(_fp(d_out), _fp(q), _fp(k), _fp(v), _fp(out), _fp(lse), _fp(dq), _fp(dk), _fp(dv),
                                                        B, H, N, D, scale, int(causal)))
        return dq, dk, dv

    # ---- decoder-block operators and the model, through the reference's own classes ----
    def linear(self, x, w):
        x, w = _f32(x), _f32(w)
        y = np.empty((x.shape[0], w.shape[0]), np.float32)
        self._chk(self.lib.ref_linear(_fp(x), _fp(w), _fp(y), x.shape[0], w.shape[0], x.shape[1]))
        return y

    def rms_norm(self, x, w, eps):
        x, w = _f32(x), _f32(w)
        y = np.empty_like(x)
        self._chk(self.lib.ref_rms_norm(_fp(x), _fp(w), _fp(y), x.size // x.shape[-1], x.shape[-1], eps))
        return y

    def silu_mul(self, gate, up):
        gate, up = _f32(gate), _f32(up)
        y = np.empty_like(gate)
        self._chk(self.lib.ref_silu_mul(_fp(gate), _fp(up), _fp(y), gate.size))
        return y

    def embedding(self, ids, table):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        table = _f32(table)
        y = np.empty(ids.shape + (table.shape[1],), np.float32)
        self._chk(self.lib.ref_embedding(ids.ctypes.data_as(C.POINTER(C.c_int32)), _fp(table), _fp(y), ids.size, table.shape[0], table.shape[1]))
        return y

    def argmax(self, logits):
        logits = _f32(logits)
        out = np.empty(logits.shape[0], np.int32)
        self._chk(self.lib.ref_argmax(_fp(logits), out.ctypes.data_as(C.POINTER(C.c_int32)), logits.shape[0], logits.shape[1]))
        return out

    class Model:
        """models::TransformerLM (Llama style: RMSNorm, RoPE, SwiGLU, no bias, untied head)."""

        def __init__(self, ref, vocab, dim, n_layers, n_heads, n_kv_heads, ffn_hidden, max_seq_len, norm_eps=1e-6, rope_base=10000.0):
            self.ref = ref
            self.vocab = vocab
            self.h = ref.lib.ref_model_new(vocab, dim, n_layers, n_heads, n_kv_heads, ffn_hidden, max_seq_len, norm_eps, rope_base)
            if not self.h:
                raise RuntimeError(ref.lib.ref_last_error().decode())

        def param_shapes(self):
            n = self.ref.lib.ref_model_param_names(self.h, None, 0)
            buf = C.create_string_buffer(int(n))
            self.ref.lib.ref_model_param_names(self.h, buf, n)
            out = {}
            for line in buf.value.decode().splitlines():
                parts = line.split()
                out[parts[0]] = tuple(int(p) for p in parts[1:])
            return out

        def set_param(self, name, value):
            value = _f32(value)
            self.ref._chk(self.ref.lib.ref_model_set_param(self.h, name.encode(), _fp(value), value.size))

        def forward(self, ids):
            ids = np.ascontiguousarray(ids, dtype=np.int32)
            B, T = ids.shape
            y = np.empty((B, T, self.vocab), np.float32)
            self.ref._chk(self.ref.lib.ref_model_forward(self.h, ids.ctypes.data_as(C.POINTER(C.c_int32)), B, T, _fp(y)))
            return y

        def init_cache(self, B):
            self.ref._chk(self.ref.lib.ref_model_init_cache(self.h, B))

        def forward_with_cache(self, ids, start_pos):
            ids = np.ascontiguousarray(ids, dtype=np.int32)
            B, T = ids.shape
            y = np.empty((B, T, self.vocab), np.float32)
            self.ref._chk(self.ref.lib.ref_model_forward_with_cache(self.h, ids.ctypes.data_as(C.POINTER(C.c_int32)), B, T, start_pos, _fp(y)))
            return y

        def generate_greedy(self, prompt, max_new, stop_ids=(), min_new=0):
            prompt = np.ascontiguousarray(prompt, dtype=np.int32)
            B, P = prompt.shape
            out = np.zeros((B, P + max_new), np.int32)
            stop = np.ascontiguousarray(list(stop_ids), dtype=np.int64)
            cols = self.ref.lib.ref_generate_greedy(self.h, prompt.ctypes.data_as(C.POINTER(C.c_int32)), B, P, max_new,
                                                    stop.ctypes.data_as(C.POINTER(_i64)), stop.size, min_new,
                                                    out.ctypes.data_as(C.POINTER(C.c_int32)))
            if cols < 0:
                raise RuntimeError(self.ref.lib.ref_last_error().decode())
            return out.reshape(-1)[: B * cols].reshape(B, cols)

        def __del__(self):
            if getattr(self, "h", None):
                self.ref.lib.ref_model_free(self.h)
                self.h = None

    def model(self, *args, **kw):
        return Ref.Model(self, *args, **kw)
