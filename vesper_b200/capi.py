"""ctypes binding of libvesper_b200.so (include/vesper_b200.h) for the Python
test / benchmark harness.  Device buffers are torch CUDA tensors (plumbing
only: memory, streams); every computation goes through the C ABI.

The library must be present: there is no fallback path.  ``load()`` raises
when the shared object is missing.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libvesper_b200.so")

F32, BF16, F16 = 0, 1, 2
OK = 0


class Tensor4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_s", C.c_int64)]


class Rope(C.Structure):
    _fields_ = [("enabled", C.c_int32), ("inv_freq_host", C.POINTER(C.c_float))]


class PrefillArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("device", C.c_int32), ("stream", C.c_void_p), ("dtype", C.c_int32),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("T", C.c_int32), ("D", C.c_int32),
        ("start_pos", C.c_int32), ("causal", C.c_int32), ("scale", C.c_float),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4), ("lse", C.c_void_p),
        ("rope", Rope), ("k_cache", Tensor4), ("v_cache", Tensor4), ("cache_cap", C.c_int32),
        ("cache_read_only", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("device", C.c_int32), ("stream", C.c_void_p), ("dtype", C.c_int32),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32), ("scale", C.c_float),
        ("q", Tensor4), ("k_new", Tensor4), ("v_new", Tensor4), ("o", Tensor4), ("lse", C.c_void_p),
        ("rope", Rope), ("k_cache", Tensor4), ("v_cache", Tensor4), ("cache_cap", C.c_int32),
        ("seq_lens", C.c_void_p), ("uniform_len", C.c_int32), ("advance_lens", C.c_int32),
        ("max_len", C.c_int32), ("num_splits", C.c_int32), ("pos_offset", C.c_int64),
        ("append_enabled", C.c_int32), ("q_positions", C.c_void_p), ("partial_out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


EXPORTS = [
    "vb200_prefill_workspace_bytes", "vb200_prefill_fwd", "vb200_decode_workspace_bytes", "vb200_decode_workspace_bytes_max", "vb200_decode_fwd",
    "vb200_decode_fwd_static", "vb200_exchange_buffer_bytes", "vb200_exchange_combine", "vb200_decode_exchange_fwd",
    "vb200_attention_bwd_workspace_bytes", "vb200_attention_bwd",
    "vb200_lse_combine", "vb200_kv_append", "vb200_apply_rope", "vb200_repeat_kv", "vb200_rope_inv_freq",
    "vb200_strerror", "vb200_last_error_detail", "vb200_abi_version", "vb200_launch_count",
    "vb200_reset_launch_count", "vb200_last_prefill_kernel", "vb200_check_kernel_status", "vb200_profile_enable", "vb200_profile_read",
]
BLOCK_EXPORTS = [
    "vb200_linear", "vb200_linear_bias", "vb200_linear_f32", "vb200_linear_ex", "vb200_row_inv_rms", "vb200_embedding_scaled", "vb200_linear_add_rmsnorm", "vb200_embedding_rmsnorm", "vb200_interleave_rows", "vb200_rms_norm", "vb200_silu_mul", "vb200_embedding", "vb200_greedy_step",
]


class AttnBwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t), ("device", C.c_int32), ("stream", C.c_void_p), ("dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("N", C.c_int32), ("D", C.c_int32), ("causal", C.c_int32), ("scale", C.c_float),
        ("d_out", C.c_void_p), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class ExchangeArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t), ("device", C.c_int32), ("stream", C.c_void_p), ("world", C.c_int32), ("rank", C.c_int32),
        ("peer_buffers", C.POINTER(C.c_void_p)), ("partial", C.c_void_p), ("rows", C.c_int64), ("D", C.c_int32), ("dtype", C.c_int32),
        ("out", C.c_void_p), ("lse", C.c_void_p), ("step", C.c_uint32), ("timeout_cycles", C.c_int64),
    ]


class LinearArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t), ("device", C.c_int32), ("stream", C.c_void_p),
        ("x", C.c_void_p), ("ldx", C.c_int64), ("w", C.c_void_p), ("ldw", C.c_int64), ("out", C.c_void_p), ("ldo", C.c_int64),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("epilogue", C.c_int32), ("splits", C.c_int32),
        ("bias", C.c_void_p), ("scaled_copy", C.c_void_p), ("copy_scale", C.c_void_p),
        ("rms_rows", C.c_void_p), ("rms_ld", C.c_int64), ("rms_dim", C.c_int32), ("rms_eps", C.c_float), ("row_scale", C.c_void_p),
    ]


class GreedyArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_size_t), ("device", C.c_int32), ("stream", C.c_void_p),
        ("logits", C.c_void_p), ("ld_logits", C.c_int64), ("B", C.c_int32), ("vocab", C.c_int32),
        ("out_ids", C.c_void_p), ("history", C.c_void_p), ("history_ld", C.c_int64), ("step", C.c_int32),
        ("stop_ids", C.c_void_p), ("n_stop", C.c_int32), ("min_new_tokens", C.c_int32), ("done", C.c_void_p),
        ("pos_dev", C.c_void_p), ("pos_base", C.c_int32),
    ]


EPI_BF16, EPI_F32, EPI_ADD_F32, EPI_SWIGLU = 0, 1, 2, 3

_lib = None


class Vb200Error(RuntimeError):
    def __init__(self, status, text):
        super().__init__(text)
        self.status = status


def load():
    """dlopen the C-ABI library (raises if it has not been built)."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("VESPER_B200_LIB", LIB_PATH)     # override: a differently tuned build of the same library
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} is missing: run `python -m vesper_b200.build` (needs nvcc)")
    L = C.CDLL(path)
    L.vb200_prefill_workspace_bytes.argtypes = [C.POINTER(PrefillArgs)]
    L.vb200_prefill_workspace_bytes.restype = C.c_size_t
    L.vb200_prefill_fwd.argtypes = [C.POINTER(PrefillArgs)]
    L.vb200_decode_workspace_bytes.argtypes = [C.POINTER(DecodeArgs)]
    L.vb200_decode_workspace_bytes.restype = C.c_size_t
    L.vb200_decode_workspace_bytes_max.argtypes = [C.POINTER(DecodeArgs)]
    L.vb200_decode_workspace_bytes_max.restype = C.c_size_t
    L.vb200_decode_fwd.argtypes = [C.POINTER(DecodeArgs)]
    L.vb200_decode_fwd_static.argtypes = [C.POINTER(DecodeArgs)]
    L.vb200_lse_combine.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    L.vb200_kv_append.argtypes = [C.c_int, C.c_void_p, C.c_int32] + [C.c_int32] * 5 + [C.POINTER(Tensor4)] * 4 + [C.c_int32, C.POINTER(Rope)]
    L.vb200_apply_rope.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int32] * 4
    L.vb200_repeat_kv.argtypes = [C.c_int, C.c_void_p, C.c_int32, C.POINTER(Tensor4), C.c_void_p] + [C.c_int32] * 5
    L.vb200_rope_inv_freq.argtypes = [C.c_float, C.c_int32, C.POINTER(C.c_float)]
    L.vb200_rope_inv_freq.restype = None
    L.vb200_strerror.argtypes = [C.c_int]
    L.vb200_strerror.restype = C.c_char_p
    L.vb200_last_error_detail.restype = C.c_char_p
    L.vb200_launch_count.restype = C.c_uint64
    L.vb200_last_prefill_kernel.restype = C.c_char_p
    L.vb200_reset_launch_count.restype = None
    L.vb200_check_kernel_status.argtypes = [C.c_int, C.c_void_p]
    L.vb200_profile_enable.argtypes = [C.c_int]
    L.vb200_profile_read.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_uint64)]
    L.vb200_attention_bwd_workspace_bytes.argtypes = [C.POINTER(AttnBwdArgs)]
    L.vb200_attention_bwd_workspace_bytes.restype = C.c_size_t
    L.vb200_attention_bwd.argtypes = [C.POINTER(AttnBwdArgs)]
    L.vb200_exchange_buffer_bytes.argtypes = [C.c_int32, C.c_int64, C.c_int32]
    L.vb200_exchange_buffer_bytes.restype = C.c_size_t
    L.vb200_exchange_combine.argtypes = [C.POINTER(ExchangeArgs)]
    L.vb200_decode_exchange_fwd.argtypes = [C.POINTER(DecodeArgs), C.POINTER(ExchangeArgs)]
    # decoder-block operators (include/vesper_b200_block.h)
    L.vb200_linear.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64] + [C.c_int32] * 5
    L.vb200_linear_bias.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64] + [C.c_int32] * 5
    L.vb200_linear_f32.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64] + [C.c_int32] * 3
    L.vb200_linear_ex.argtypes = [C.POINTER(LinearArgs)]
    L.vb200_row_inv_rms.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_float]
    L.vb200_embedding_scaled.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_void_p, C.c_void_p]
    L.vb200_linear_add_rmsnorm.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                           C.c_void_p, C.c_float, C.c_void_p, C.c_int32]
    L.vb200_embedding_rmsnorm.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                          C.c_void_p, C.c_float, C.c_void_p]
    L.vb200_interleave_rows.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]
    L.vb200_rms_norm.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_float]
    L.vb200_silu_mul.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]
    L.vb200_embedding.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32]
    L.vb200_greedy_step.argtypes = [C.POINTER(GreedyArgs)]
    _lib = L
    return L


def check(rc):
    if rc != OK:
        L = load()
        raise Vb200Error(rc, f"vb200 status {rc} ({L.vb200_strerror(rc).decode()}): {L.vb200_last_error_detail().decode()}")


def dtype_code(t):
    import torch
    return {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}[t.dtype]


def view4(t):
    """[B,H,S,D] torch tensor (any strides, D contiguous) -> Tensor4."""
    if t is None:
        return Tensor4(None, 0, 0, 0)
    assert t.dim() == 4 and t.stride(3) == 1
    return Tensor4(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def inv_freq(theta, D):
    arr = (C.c_float * (D // 2))()
    load().vb200_rope_inv_freq(theta, D, arr)
    return arr


def _stream_ptr(stream):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def prefill_args(q, k, v, o, lse=None, *, scale, causal=True, start_pos=0, theta=None,
                 k_cache=None, v_cache=None, workspace=None, stream=None, cache_read_only=False):
    B, Hq, T, D = q.shape
    a = PrefillArgs()
    a.struct_size = C.sizeof(PrefillArgs)
    a.device = q.device.index if q.device.index is not None else -1
    a.stream = _stream_ptr(stream)
    a.dtype = dtype_code(q)
    a.B, a.Hq, a.Hkv, a.T, a.D = B, Hq, (k if k is not None else k_cache).shape[1], T, D
    a.cache_read_only = int(cache_read_only)
    a.start_pos, a.causal, a.scale = start_pos, int(causal), scale
    a.q, a.k, a.v, a.o = view4(q), view4(k), view4(v), view4(o)
    a.lse = _ptr(lse)
    keep = None
    if theta is not None:
        keep = inv_freq(theta, D)
        a.rope = Rope(1, keep)
    else:
        a.rope = Rope(0, None)
    a.k_cache, a.v_cache = view4(k_cache), view4(v_cache)
    a.cache_cap = k_cache.shape[2] if k_cache is not None else 0
    a.workspace = _ptr(workspace)
    a.workspace_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    a._keep = keep
    return a


def prefill(q, k, v, o, lse=None, *, scale, causal=True, start_pos=0, theta=None,
            k_cache=None, v_cache=None, workspace=None, stream=None, cache_read_only=False):
    """vb200_prefill_fwd on torch CUDA tensors.  Allocates a workspace with torch when none is given."""
    import torch
    L = load()
    a = prefill_args(q, k, v, o, lse, scale=scale, causal=causal, start_pos=start_pos, theta=theta,
                     k_cache=k_cache, v_cache=v_cache, workspace=workspace, stream=stream, cache_read_only=cache_read_only)
    need = L.vb200_prefill_workspace_bytes(C.byref(a))
    if need > a.workspace_bytes:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
        a.workspace, a.workspace_bytes = _ptr(workspace), need
    check(L.vb200_prefill_fwd(C.byref(a)))
    return workspace


def decode_args(q, o, k_cache, v_cache, *, scale, k_new=None, v_new=None, lse=None, theta=None,
                seq_lens=None, uniform_len=0, advance_lens=False, max_len=0, num_splits=0,
                pos_offset=0, append_enabled=True, q_positions=None, partial_out=None,
                workspace=None, stream=None):
    B, Hq, _, D = q.shape
    a = DecodeArgs()
    a.struct_size = C.sizeof(DecodeArgs)
    a.device = q.device.index if q.device.index is not None else -1
    a.stream = _stream_ptr(stream)
    a.dtype = dtype_code(q)
    a.B, a.Hq, a.Hkv, a.D, a.scale = B, Hq, k_cache.shape[1], D, scale
    a.q, a.k_new, a.v_new, a.o = view4(q), view4(k_new), view4(v_new), view4(o)
    a.lse = _ptr(lse)
    keep = None
    if theta is not None:
        keep = inv_freq(theta, D)
        a.rope = Rope(1, keep)
    else:
        a.rope = Rope(0, None)
    a.k_cache, a.v_cache = view4(k_cache), view4(v_cache)
    a.cache_cap = k_cache.shape[2]
    a.seq_lens = _ptr(seq_lens)
    a.uniform_len, a.advance_lens, a.max_len, a.num_splits = uniform_len, int(advance_lens), max_len, num_splits
    a.pos_offset, a.append_enabled = pos_offset, int(append_enabled)
    a.q_positions, a.partial_out = _ptr(q_positions), _ptr(partial_out)
    a.workspace = _ptr(workspace)
    a.workspace_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    a._keep = keep
    return a


def decode(q, o, k_cache, v_cache, **kw):
    """vb200_decode_fwd on torch CUDA tensors.  Allocates a workspace with torch when none is given."""
    import torch
    L = load()
    a = decode_args(q, o, k_cache, v_cache, **kw)
    need = L.vb200_decode_workspace_bytes(C.byref(a))
    ws = kw.get("workspace")
    if need > a.workspace_bytes:
        ws = torch.empty(need, dtype=torch.uint8, device=q.device)
        a.workspace, a.workspace_bytes = _ptr(ws), need
    check(L.vb200_decode_fwd(C.byref(a)))
    return ws


def lse_combine(partials, out, lse=None, stream=None):
    """partials [R, rows, D+2] fp32 -> out [rows, D] (bf16/fp16), lse [rows]."""
    R, rows, Dp2 = partials.shape
    check(load().vb200_lse_combine(partials.device.index, _stream_ptr(stream), _ptr(partials), R, rows, Dp2 - 2,
                                   dtype_code(out), _ptr(out), _ptr(lse)))


def check_kernel_status(device=0, stream=None):
    check(load().vb200_check_kernel_status(device, _stream_ptr(stream)))


def profile_enable(on=True):
    check(load().vb200_profile_enable(int(on)))


def profile_read():
    """(summed dominant-kernel milliseconds, number of bracketed launches) since profile_enable(True)."""
    ms, n = C.c_double(0.0), C.c_uint64(0)
    check(load().vb200_profile_read(C.byref(ms), C.byref(n)))
    return ms.value, n.value


def attention_bwd(d_out, q, k, v, out, lse, *, scale, causal=True, stream=None):
    """fp32 contiguous [B,H,N,D] tensors; returns (dq, dk, dv)."""
    import torch
    B, H, N, D = q.shape
    a = AttnBwdArgs()
    a.struct_size = C.sizeof(AttnBwdArgs)
    a.device = q.device.index or 0
    a.stream = _stream_ptr(stream)
    a.dtype = dtype_code(q)
    a.B, a.H, a.N, a.D, a.causal, a.scale = B, H, N, D, int(causal), scale
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    for name, t in (("d_out", d_out), ("q", q), ("k", k), ("v", v), ("out", out), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert t.is_contiguous()
        setattr(a, name, _ptr(t))
    need = load().vb200_attention_bwd_workspace_bytes(C.byref(a))
    ws = torch.empty(need, dtype=torch.uint8, device=q.device)
    a.workspace, a.workspace_bytes = _ptr(ws), need
    check(load().vb200_attention_bwd(C.byref(a)))
    return dq, dk, dv


def exchange_buffer_bytes(world, rows, D):
    return int(load().vb200_exchange_buffer_bytes(world, rows, D))


def exchange_args(peer_ptrs, rank, out, lse=None, *, partial=None, rows=None, D=None, step=0, timeout_cycles=0, stream=None):
    a = ExchangeArgs()
    a.struct_size = C.sizeof(ExchangeArgs)
    a.device = out.device.index or 0
    a.stream = _stream_ptr(stream)
    a.world, a.rank = len(peer_ptrs), rank
    arr = (C.c_void_p * len(peer_ptrs))(*[C.c_void_p(int(p)) for p in peer_ptrs])
    a.peer_buffers = arr
    a._keep = arr
    a.partial = _ptr(partial)
    a.rows = rows if rows is not None else partial.shape[0]
    a.D = D if D is not None else partial.shape[1] - 2
    a.dtype = dtype_code(out)
    a.out = _ptr(out)
    a.lse = _ptr(lse)
    a.step = step
    a.timeout_cycles = timeout_cycles
    return a


def exchange_combine(partial, peer_ptrs, rank, out, lse=None, *, step=0, timeout_cycles=0, stream=None):
    """partial [rows, D+2] fp32 (local), peer_ptrs: device address of every rank's exchange buffer."""
    a = exchange_args(peer_ptrs, rank, out, lse, partial=partial, step=step, timeout_cycles=timeout_cycles, stream=stream)
    check(load().vb200_exchange_combine(C.byref(a)))
    return out


def decode_exchange(q, k_cache, v_cache, peer_ptrs, rank, out, lse=None, *, timeout_cycles=0, step=0, workspace=None, **kw):
    """vb200_decode_exchange_fwd: this rank's shard of a sequence-sharded decode step, split merge and exchange in one
    launch.  out [B*Hq, D] (bf16/fp16), lse [B*Hq]; kw as for decode_args (scale, theta, uniform_len, max_len, pos_offset,
    q_positions, ...)."""
    import torch
    L = load()
    B, Hq, _, D = q.shape
    stream = kw.get("stream")
    a = decode_args(q, None, k_cache, v_cache, workspace=workspace, **kw)
    need = L.vb200_decode_workspace_bytes(C.byref(a))
    if need > a.workspace_bytes:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
        a.workspace, a.workspace_bytes = _ptr(workspace), need
    x = exchange_args(peer_ptrs, rank, out, lse, rows=B * Hq, D=D, step=step, timeout_cycles=timeout_cycles, stream=stream)
    check(L.vb200_decode_exchange_fwd(C.byref(a), C.byref(x)))
    return workspace


def linear(x, w, out, epilogue=EPI_BF16, splits=0, stream=None, bias=None):
    """out = epilogue(x @ w.T [+ bias]): x [M,K] bf16, w [N,K] bf16 (row strides honoured), bias fp32 [N]."""
    M, K = x.shape
    N = w.shape[0]
    check(load().vb200_linear_bias(x.device.index or 0, _stream_ptr(stream), _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias),
                                   _ptr(out), out.stride(0), M, N, K, epilogue, splits))
    return out


def linear_ex(x, w, out, *, epilogue=EPI_BF16, splits=0, bias=None, scaled_copy=None, copy_scale=None, rms_rows=None, rms_eps=0.0,
              row_scale=None, stream=None):
    """vb200_linear_ex: the GEMM with bias and the two halves of a deferred RMSNorm."""
    a = LinearArgs()
    a.struct_size = C.sizeof(LinearArgs)
    a.device = x.device.index or 0
    a.stream = _stream_ptr(stream)
    a.x, a.ldx, a.w, a.ldw, a.out, a.ldo = _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0)
    a.M, a.K = x.shape
    a.N = w.shape[0]
    a.epilogue, a.splits = epilogue, splits
    a.bias, a.scaled_copy, a.copy_scale, a.row_scale = _ptr(bias), _ptr(scaled_copy), _ptr(copy_scale), _ptr(row_scale)
    if rms_rows is not None:
        a.rms_rows, a.rms_ld, a.rms_dim, a.rms_eps = _ptr(rms_rows), rms_rows.stride(0), rms_rows.shape[1], rms_eps
    check(load().vb200_linear_ex(C.byref(a)))
    return out


def row_inv_rms(h, out, eps, stream=None):
    check(load().vb200_row_inv_rms(h.device.index or 0, _stream_ptr(stream), _ptr(h), h.stride(0), _ptr(out), h.shape[0], h.shape[1], eps))
    return out


def embedding_scaled(ids, table, out, scale, scaled_out, stream=None):
    import torch
    ids64 = 1 if ids.dtype == torch.int64 else 0
    check(load().vb200_embedding_scaled(table.device.index or 0, _stream_ptr(stream), _ptr(ids), ids64, _ptr(table), _ptr(out), ids.numel(),
                                        table.shape[1], table.shape[0], _ptr(scale), _ptr(scaled_out)))
    return out, scaled_out


def linear_add_rmsnorm(x, w, h, norm_weight, eps, xn_out, splits=0, stream=None):
    """h += x @ w.T; xn_out = rmsnorm(h) * norm_weight (bf16)."""
    M, K = x.shape
    N = w.shape[0]
    check(load().vb200_linear_add_rmsnorm(x.device.index or 0, _stream_ptr(stream), _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(h), M, N, K,
                                          _ptr(norm_weight), eps, _ptr(xn_out), splits))
    return h, xn_out


def embedding_rmsnorm(ids, table, out, norm_weight, eps, xn_out, stream=None):
    import torch
    ids64 = 1 if ids.dtype == torch.int64 else 0
    check(load().vb200_embedding_rmsnorm(table.device.index or 0, _stream_ptr(stream), _ptr(ids), ids64, _ptr(table), _ptr(out), ids.numel(),
                                         table.shape[1], table.shape[0], _ptr(norm_weight), eps, _ptr(xn_out)))
    return out, xn_out


def interleave_rows(a, b, out, stream=None):
    check(load().vb200_interleave_rows(a.device.index or 0, _stream_ptr(stream), _ptr(a), _ptr(b), _ptr(out), a.shape[0], a.shape[1]))
    return out


def rms_norm(x, weight, out, eps, stream=None):
    M, dim = x.shape
    check(load().vb200_rms_norm(x.device.index or 0, _stream_ptr(stream), _ptr(x), _ptr(weight), _ptr(out), M, dim, eps))
    return out


def silu_mul(gate, up, out, stream=None):
    check(load().vb200_silu_mul(gate.device.index or 0, _stream_ptr(stream), _ptr(gate), _ptr(up), _ptr(out), gate.numel()))
    return out


def embedding(ids, table, out, stream=None):
    import torch
    ids64 = 1 if ids.dtype == torch.int64 else 0
    check(load().vb200_embedding(table.device.index or 0, _stream_ptr(stream), _ptr(ids), ids64, _ptr(table), _ptr(out),
                                 ids.numel(), table.shape[1], table.shape[0]))
    return out


def greedy_step(logits, out_ids, *, history=None, step=0, stop_ids=None, min_new_tokens=0, done=None, pos_dev=None,
                pos_base=0, stream=None):
    a = GreedyArgs()
    a.struct_size = C.sizeof(GreedyArgs)
    a.device = logits.device.index or 0
    a.stream = _stream_ptr(stream)
    a.logits = _ptr(logits)
    a.ld_logits = logits.stride(0)
    a.B, a.vocab = logits.shape
    a.out_ids = _ptr(out_ids)
    if history is not None:
        a.history = _ptr(history)
        a.history_ld = history.stride(0)
    a.step = step
    if stop_ids is not None and stop_ids.numel() > 0:
        a.stop_ids = _ptr(stop_ids)
        a.n_stop = stop_ids.numel()
    a.min_new_tokens = min_new_tokens
    if done is not None:
        a.done = _ptr(done)
    if pos_dev is not None:
        a.pos_dev = _ptr(pos_dev)
        a.pos_base = pos_base
    check(load().vb200_greedy_step(C.byref(a)))
    return out_ids
