"""CPU restatement (numpy, f32) of the reference's OLMoE forward pass — TEST INFRASTRUCTURE.

Follows crates/mummu/src/models/olmoe.rs:522-587 (embed, per layer: input RMSNorm, attention,
residual, post-attention RMSNorm, MoE, residual; final norm; lm_head on the last position),
nn/attention.rs:182-295 (q/k RMSNorm over the whole projection, rotate-half RoPE, cache append,
f32 scores scaled by 1/sqrt(head_dim), additive -1e4 causal mask, softmax, value matmul, o_proj)
and nn/rope.rs:21-105.  The MoE block is the C oracle's.  Small shapes only."""
from __future__ import annotations

import numpy as np

from . import oracle as O


def rms(x, gamma, eps):
    x = x.astype(np.float32)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + np.float32(eps)) * gamma


def rope_tables(positions, head_dim, theta):
    half = head_dim // 2
    k = np.arange(half, dtype=np.float32)
    inv = (np.float32(1.0) / np.power(np.float32(theta), np.float32(2.0) * k / np.float32(head_dim))).astype(np.float32)
    ang = np.asarray(positions, np.float32)[:, None] * inv[None, :]
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    return np.concatenate([c, c], 1), np.concatenate([s, s], 1)


def apply_rope(x, cos, sin):                       # x [nh, t, hd]
    half = x.shape[-1] // 2
    rh = np.concatenate([-x[..., half:], x[..., :half]], -1)
    return x * cos + rh * sin


class RefOlmoe:
    def __init__(self, cfg, state, q4k: bool):
        self.cfg, self.s, self.q4k = cfg, state, q4k
        self.cache = [dict(k=None, v=None) for _ in range(cfg.num_hidden_layers)]

    def forward(self, ids, past):
        """ids: list of new token ids (one sequence); returns logits [vocab] of the last position."""
        c, s = self.cfg, self.s
        nh, nkv, hd = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        t = len(ids)
        x = s["embed"][np.asarray(ids)].astype(np.float32)
        cos, sin = rope_tables(np.arange(past, past + t), hd, c.rope_theta)
        for l in range(c.num_hidden_layers):
            g = lambda n: s[f"l{l}.{n}"]
            h = rms(x, g("in_norm"), c.rms_norm_eps)
            q = rms(h @ g("q").T, g("q_norm"), c.rms_norm_eps).reshape(t, nh, hd).transpose(1, 0, 2)
            k = rms(h @ g("k").T, g("k_norm"), c.rms_norm_eps).reshape(t, nkv, hd).transpose(1, 0, 2)
            v = (h @ g("v").T).reshape(t, nkv, hd).transpose(1, 0, 2)
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
            kv = self.cache[l]
            kv["k"] = k if kv["k"] is None else np.concatenate([kv["k"], k], 1)
            kv["v"] = v if kv["v"] is None else np.concatenate([kv["v"], v], 1)
            keys, vals = np.repeat(kv["k"], nh // nkv, 0), np.repeat(kv["v"], nh // nkv, 0)
            scores = (q @ keys.transpose(0, 2, 1)) * np.float32(1.0 / np.sqrt(hd))
            if t > 1:
                kc = past + t
                mask = np.zeros((t, kc), np.float32)
                for i in range(t):
                    mask[i, past + i + 1:] = -1e4
                scores = scores + mask
            scores = scores - scores.max(-1, keepdims=True)
            p = np.exp(scores)
            p = p / p.sum(-1, keepdims=True)
            ctx = (p @ vals).transpose(1, 0, 2).reshape(t, nh * hd)
            x = x + ctx @ g("o").T
            h2 = rms(x, g("post_norm"), c.rms_norm_eps)
            y, _, _ = O.moe_forward(h2, g("router"), g("gate"), g("up"), g("down"), c.num_experts_per_tok,
                                    c.norm_topk_prob, q4k=self.q4k)
            x = x + y
        last = rms(x[-1:], s["norm"], c.rms_norm_eps)
        return (last @ s["lm_head"].T)[0]
