"""OLMoE decoder around the CUDA expert bank — the caller of the hot path
(crates/mummu/src/models/olmoe.rs:522-587) restated minimally so that whole-model decode can be
measured.  The trunk (embedding, RMSNorm, attention projections, RoPE, attention, lm_head, argmax)
is plain torch on the GPU (library kernels): it is not the path this repository accelerates.  Each
layer's MLP is a `mummu_b200.moe.SparseMoe`, called exactly as the reference calls it:
`mlp.forward(h2, num_experts_per_tok, norm_topk_prob)` (olmoe.rs:566-571).

Differences from the reference, on purpose: `forward` takes a batch of B independent sequences of
equal length (the reference's forward is batch 1, olmoe.rs:545-549); the KV cache is preallocated
(the reference concatenates, nn/attention.rs `kv_append`)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from . import _lib as L
from . import moe as moe_mod


@dataclass
class OlmoeConfig:
    """`OlmoeConfig` (models/olmoe.rs:40-80) — the fields the forward pass uses."""
    vocab_size: int = 50304
    hidden_size: int = 2048
    intermediate_size: int = 1024
    num_hidden_layers: int = 16
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    num_experts: int = 64
    num_experts_per_tok: int = 8
    norm_topk_prob: bool = False
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


def rope_tables(positions: np.ndarray, head_dim: int, theta: float):
    """cos/sin [len, head_dim], both halves equal — nn/rope.rs:21-63, f32 arithmetic."""
    half = head_dim // 2
    k = np.arange(half, dtype=np.float32)
    inv = (np.float32(1.0) / np.power(np.float32(theta), np.float32(2.0) * k / np.float32(head_dim))).astype(np.float32)
    ang = positions.astype(np.float32)[:, None] * inv[None, :]
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    return np.concatenate([c, c], 1), np.concatenate([s, s], 1)


class OlmoeDecoder:
    def __init__(self, cfg: OlmoeConfig, device: int = 0, expert_dtype: int = L.Q4_K, max_batch: int = 1,
                 max_ctx: int = 1024, max_tokens: int = 0):
        import torch
        self.torch, self.cfg = torch, cfg
        self.dev = torch.device("cuda", device)
        self.dtype = torch.float16
        self.max_batch, self.max_ctx = max_batch, max_ctx
        self.expert_dtype = expert_dtype
        c = cfg
        hd = c.head_dim
        self.embed = None
        self.lm_head = None
        self.final_norm = None
        self.layers = []
        mcfg = moe_mod.SparseMoeConfig(c.hidden_size, c.intermediate_size, c.num_experts, c.num_experts_per_tok)
        for l in range(c.num_hidden_layers):
            mlp = mcfg.init(device=device, act_dtype=L.F16, weight_dtype=expert_dtype,
                            max_tokens=max(max_tokens, max_batch * 64) if l == 0 else 0)
            if l:
                mlp.adopt_scratch(self.layers[0]["mlp"])
            self.layers.append(dict(mlp=mlp))
        cos, sin = rope_tables(np.arange(max_ctx), hd, c.rope_theta)
        self.cos = torch.from_numpy(cos).to(self.dev)
        self.sin = torch.from_numpy(sin).to(self.dev)
        self._arange = torch.arange(max_ctx, device=self.dev)
        self.k_cache = torch.zeros(c.num_hidden_layers, max_batch, c.num_key_value_heads, max_ctx, hd,
                                   dtype=self.dtype, device=self.dev)
        self.v_cache = torch.zeros_like(self.k_cache)

    # ---- weights ------------------------------------------------------------------------------
    def load_state(self, state: dict) -> None:
        """state: numpy arrays named as the HF / GGUF-mapped checkpoint (models/olmoe.rs:319-349):
        embed [V,H], lm_head [V,H], norm [H]; per layer l: in_norm, post_norm [H], q,k,v,o [H,H],
        q_norm, k_norm [H], router [H,E] (burn order), gate/up [E,I,H], down [E,H,I] (f32 or Q4_K bytes)."""
        t = self.torch
        f16 = lambda a: t.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(self.dev, self.dtype)
        f32 = lambda a: t.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(self.dev)
        self.embed, self.lm_head, self.final_norm = f16(state["embed"]), f16(state["lm_head"]), f32(state["norm"])
        for l, lay in enumerate(self.layers):
            g = lambda n: state[f"l{l}.{n}"]
            lay.update(in_norm=f32(g("in_norm")), post_norm=f32(g("post_norm")), q=f16(g("q")), k=f16(g("k")),
                       v=f16(g("v")), o=f16(g("o")), q_norm=f32(g("q_norm")), k_norm=f32(g("k_norm")))
            lay["mlp"].set_router(g("router"))
            banks = [g("gate"), g("up"), g("down")]
            if self.expert_dtype != L.Q4_K:
                banks = [np.ascontiguousarray(b, dtype=np.float32).astype(np.float16) for b in banks]
            lay["mlp"].set_banks(*banks)

    def random_init(self, seed: int = 0) -> None:
        """Random weights of the right shapes on the device (benchmark use)."""
        t, c = self.torch, self.cfg
        gen = t.Generator(device=self.dev)
        gen.manual_seed(seed)
        rnd = lambda *s: t.randn(*s, generator=gen, device=self.dev) * 0.02
        H, E, I = c.hidden_size, c.num_experts, c.intermediate_size
        self.embed, self.lm_head = rnd(c.vocab_size, H).to(self.dtype), rnd(c.vocab_size, H).to(self.dtype)
        self.final_norm = t.ones(H, device=self.dev)
        for lay in self.layers:
            lay.update(in_norm=t.ones(H, device=self.dev), post_norm=t.ones(H, device=self.dev),
                       q=rnd(H, H).to(self.dtype), k=rnd(H, H).to(self.dtype), v=rnd(H, H).to(self.dtype),
                       o=rnd(H, H).to(self.dtype), q_norm=t.ones(H, device=self.dev), k_norm=t.ones(H, device=self.dev))
            lay["mlp"].set_router(rnd(H, E).cpu().numpy())
            for which, shape in ((L.BANK_GATE, (E, I, H)), (L.BANK_UP, (E, I, H)), (L.BANK_DOWN, (E, H, I))):
                w = rnd(*shape)
                lay["mlp"].set_bank(which, moe_mod.q4k_quantize_device(w) if self.expert_dtype == L.Q4_K
                                    else w.to(self.dtype))
                del w

    # ---- forward ------------------------------------------------------------------------------
    def _rms(self, x, gamma):
        xf = x.float()
        return (xf * self.torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps) * gamma).to(self.dtype)

    def _rope(self, x, cos, sin):                      # x [B, nh, t, hd]; rotate-half (nn/rope.rs:66-105)
        half = x.shape[-1] // 2
        rh = self.torch.cat([-x[..., half:], x[..., :half]], -1)
        return (x.float() * cos + rh.float() * sin).to(self.dtype)

    def forward(self, ids, past: int):
        """ids [B, t] int64 on the device; appends to the cache at `past`; logits [B, vocab] (f32) of
        the last position — LoadedOlmoe::forward (models/olmoe.rs:522-587)."""
        t_, c = self.torch, self.cfg
        F = t_.nn.functional
        B, t = ids.shape
        nh, nkv, hd, H = c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.hidden_size
        x = self.embed[ids]                                                         # [B, t, H]
        cos, sin = self.cos[past:past + t], self.sin[past:past + t]
        for l, lay in enumerate(self.layers):
            h = self._rms(x, lay["in_norm"])
            q = self._rms(F.linear(h, lay["q"]), lay["q_norm"]).view(B, t, nh, hd).transpose(1, 2)
            k = self._rms(F.linear(h, lay["k"]), lay["k_norm"]).view(B, t, nkv, hd).transpose(1, 2)
            v = F.linear(h, lay["v"]).view(B, t, nkv, hd).transpose(1, 2)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
            self.k_cache[l, :B, :, past:past + t] = k
            self.v_cache[l, :B, :, past:past + t] = v
            keys, vals = self.k_cache[l, :B, :, :past + t], self.v_cache[l, :B, :, :past + t]
            if nkv != nh:
                keys = keys.repeat_interleave(nh // nkv, 1)
                vals = vals.repeat_interleave(nh // nkv, 1)
            # f32 scores and softmax, additive -1e4 causal mask (nn/attention.rs:28-48, 275-289)
            if t == 1 or past == 0:
                from torch.nn.attention import SDPBackend, sdpa_kernel
                # flash / memory-efficient kernels only: no per-shape planning while the cache grows
                with sdpa_kernel([SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]):
                    ctx = F.scaled_dot_product_attention(q, keys, vals, is_causal=(t > 1 and past == 0))
            else:
                ctx = self._attn_masked(q, keys, vals, past)
            x = x + F.linear(ctx.transpose(1, 2).reshape(B, t, H), lay["o"])
            h2 = self._rms(x, lay["post_norm"])
            x = x + lay["mlp"].forward(h2.reshape(B * t, H), c.num_experts_per_tok, c.norm_topk_prob).view(B, t, H)
        x = self._rms(x[:, -1], self.final_norm)
        return F.linear(x, self.lm_head).float()

    def _attn_masked(self, q, keys, vals, past):
        t_ = self.torch
        t, kc = q.shape[2], keys.shape[2]
        mask = t_.zeros(t, kc, device=self.dev)
        mask.masked_fill_(t_.arange(kc, device=self.dev)[None, :] > (past + t_.arange(t, device=self.dev))[:, None], -1e4)
        scores = (q.float() @ keys.float().transpose(2, 3)) / math.sqrt(q.shape[-1]) + mask
        return (t_.softmax(scores, -1).to(self.dtype) @ vals)

    # ---- shape-static decode step (one token per sequence), capturable in a CUDA graph ----------
    def _decode_static(self, ids_buf, pos_buf):
        """ids_buf [B, 1] int64, pos_buf [1] int64 (the position being written), both on the device.
        Same arithmetic as forward() with t == 1, but every shape is fixed: the new k/v are written
        at pos by index, attention runs over the whole preallocated cache with the reference's
        additive -1e4 mask on positions > pos (nn/attention.rs:28-48), scores and softmax in f32."""
        t_, c = self.torch, self.cfg
        F = t_.nn.functional
        B = ids_buf.shape[0]
        nh, nkv, hd, H = c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.hidden_size
        x = self.embed[ids_buf]
        cos, sin = self.cos.index_select(0, pos_buf), self.sin.index_select(0, pos_buf)
        mask = (self._arange > pos_buf).float() * -1e4                                  # [max_ctx]
        scale = 1.0 / math.sqrt(hd)
        for l, lay in enumerate(self.layers):
            h = self._rms(x, lay["in_norm"])
            q = self._rms(F.linear(h, lay["q"]), lay["q_norm"]).view(B, 1, nh, hd).transpose(1, 2)
            k = self._rms(F.linear(h, lay["k"]), lay["k_norm"]).view(B, 1, nkv, hd).transpose(1, 2)
            v = F.linear(h, lay["v"]).view(B, 1, nkv, hd).transpose(1, 2)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
            kc, vc = self.k_cache[l, :B], self.v_cache[l, :B]
            kc.index_copy_(2, pos_buf, k)
            vc.index_copy_(2, pos_buf, v)
            keys, vals = kc, vc
            if nkv != nh:
                keys, vals = keys.repeat_interleave(nh // nkv, 1), vals.repeat_interleave(nh // nkv, 1)
            scores = t_.matmul(q, keys.transpose(2, 3)).float() * scale + mask
            ctx = t_.matmul(t_.softmax(scores, -1).to(self.dtype), vals)
            x = x + F.linear(ctx.transpose(1, 2).reshape(B, 1, H), lay["o"])
            h2 = self._rms(x, lay["post_norm"])
            x = x + lay["mlp"].forward(h2.reshape(B, H), c.num_experts_per_tok, c.norm_topk_prob).view(B, 1, H)
        x = self._rms(x[:, -1], self.final_norm)
        return F.linear(x, self.lm_head).float()

    def decode_step(self, ids, past: int):
        """One shape-static decode step, eagerly: ids [B, 1] int64 at position `past` for every
        sequence; logits [B, vocab].  The same code a captured step replays."""
        pos = self.torch.tensor([past], device=self.dev)
        return self._decode_static(ids, pos)

    def make_decode_graph(self, B: int):
        """Captures one decode step for batch B; returns (graph, ids_buf, pos_buf, logits_buf)."""
        t_ = self.torch
        ids_buf = t_.zeros(B, 1, dtype=t_.int64, device=self.dev)
        pos_buf = t_.zeros(1, dtype=t_.int64, device=self.dev)
        pos_buf.fill_(self.max_ctx - 1)                 # warm-up writes land in the last slot
        s = t_.cuda.Stream(self.dev)
        s.wait_stream(t_.cuda.current_stream())
        with t_.cuda.stream(s):
            for _ in range(2):
                self._decode_static(ids_buf, pos_buf)
        t_.cuda.current_stream().wait_stream(s)
        t_.cuda.synchronize()
        g = t_.cuda.CUDAGraph()
        with t_.cuda.graph(g):
            logits_buf = self._decode_static(ids_buf, pos_buf)
        self.k_cache[:, :B, :, self.max_ctx - 1].zero_()
        self.v_cache[:, :B, :, self.max_ctx - 1].zero_()
        return g, ids_buf, pos_buf, logits_buf

    def greedy_generate(self, prompt_ids, n_new: int, chunk: int = 1024):
        """Greedy decode (decode.rs:33-48 argmax picker; prompt fed in chunks of 1024, decode.rs:311-346)."""
        t_ = self.torch
        B, P = prompt_ids.shape
        past, logits = 0, None
        while past < P:
            n = min(chunk, P - past)
            logits = self.forward(prompt_ids[:, past:past + n], past)
            past += n
        out = []
        for _ in range(n_new):
            nxt = logits.argmax(-1)
            out.append(nxt)
            logits = self.forward(nxt[:, None], past)
            past += 1
        return t_.stack(out, 1)

    def close(self):
        for lay in reversed(self.layers):
            lay["mlp"].close()
