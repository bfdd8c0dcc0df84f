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


# ---- decoder model: seeded weights and the oracle composition -------------------------------
def model_weights(shapes, seed, std=0.02, single=False):
    """N(0, std) matrices and (1 + 0.1 N(0,1)) norm weights, seeded per parameter name order;
    matrices are rounded to bf16 so the GPU (bf16 storage) and the CPU checkers see the same values.
    single=True draws in float32 (a different, faster stream: for large models without fixtures)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name in sorted(shapes):
        shape = shapes[name]
        if len(shape) == 1:
            out[name] = (1.0 + 0.1 * rng.standard_normal(shape)).astype(np.float32)
        elif single:
            out[name] = bf16_round(np.float32(std) * rng.standard_normal(shape, dtype=np.float32))
        else:
            out[name] = bf16_round((std * rng.standard_normal(shape)).astype(np.float32))
    return out


class OracleDecoder:
    """TransformerLM::forward_with_cache (src/models/transformer.cpp:152-188) composed from the CPU
    oracle's operators: embedding -> blocks (src/models/transformer_block.cpp:183-205: RMSNorm, fused
    QKV, RoPE + cache + GQA attention, wo, residual, RMSNorm, SwiGLU, residual) -> RMSNorm -> head."""

    def __init__(self, oracle, weights, *, n_layers, n_heads, n_kv_heads, max_seq_len, norm_eps=1e-6, rope_base=10000.0):
        self.o, self.w = oracle, weights
        self.n_layers, self.Hq, self.Hkv = n_layers, n_heads, n_kv_heads
        self.dim = weights["tok_embeddings.weight"].shape[1]
        self.D = self.dim // n_heads
        self.cap, self.eps, self.theta = max_seq_len, norm_eps, rope_base
        self.caches = None

    def init_cache(self, B):
        self.caches = [(np.zeros((B, self.Hkv, self.cap, self.D), np.float32), np.zeros((B, self.Hkv, self.cap, self.D), np.float32))
                       for _ in range(self.n_layers)]
        self.cur = 0

    def forward_with_cache(self, ids, start_pos):
        o, w = self.o, self.w
        B, T = ids.shape
        h = o.embedding(ids.reshape(-1), w["tok_embeddings.weight"])                # [B*T, dim]
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        for l in range(self.n_layers):
            p = f"layers.{l}."
            x = o.rms_norm(h, w[p + "attention_norm.weight"], self.eps)
            qkv = o.linear(x, w[p + "attention.wqkv.weight"]).reshape(B, T, Hq + 2 * Hkv, D)
            q = np.ascontiguousarray(qkv[:, :, :Hq].transpose(0, 2, 1, 3))
            k = np.ascontiguousarray(qkv[:, :, Hq:Hq + Hkv].transpose(0, 2, 1, 3))
            v = np.ascontiguousarray(qkv[:, :, Hq + Hkv:].transpose(0, 2, 1, 3))
            kc, vc = self.caches[l]
            att, _, _ = o.gqa_attention_cached(q, k, v, kc, vc, start_pos, self.cur, theta=self.theta, want_lse=False)
            att = np.ascontiguousarray(att.transpose(0, 2, 1, 3)).reshape(B * T, Hq * D)
            h = h + o.linear(att, w[p + "attention.wo.weight"])
            x = o.rms_norm(h, w[p + "ffn_norm.weight"], self.eps)
            act = o.silu_mul(o.linear(x, w[p + "feed_forward.gate_proj.weight"]), o.linear(x, w[p + "feed_forward.up_proj.weight"]))
            h = h + o.linear(act, w[p + "feed_forward.down_proj.weight"])
        self.cur = max(self.cur, start_pos + T)
        x = o.rms_norm(h, w["norm.weight"], self.eps)
        return o.linear(x, w["output.weight"]).reshape(B, T, -1)

    def generate_greedy(self, prompt, max_new):
        """Generator::generate with greedy picks (src/generation/generator.cpp:62-131); also returns
        the logits every pick was made from."""
        B, P = prompt.shape
        self.init_cache(B)
        logits = self.forward_with_cache(prompt, 0)[:, -1]
        toks, all_logits = [prompt], []
        for i in range(max_new):
            nxt = self.o.argmax(logits)
            all_logits.append(logits)
            toks.append(nxt.reshape(B, 1))
            if i + 1 < max_new:
                logits = self.forward_with_cache(nxt.reshape(B, 1), P + i)[:, -1]
        return np.concatenate(toks, axis=1).astype(np.int32), np.stack(all_logits, axis=1)
