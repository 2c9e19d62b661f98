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

import ctypes as C
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


BUCKET = 256          # the smallest key bucket (nn/static_kv.rs: BUCKET); buckets above it double


def bucket(keys: int, max_ctx: int) -> int:
    """Keys a step attends over: the smallest bucket that holds `keys`, never past the cache."""
    b = BUCKET
    while b < keys:
        b *= 2
    return min(b, max_ctx)


class StaticState:
    """`StaticDecode::State` (capture.rs:48-52): the preallocated cache of a static decode plus the
    step's fixed buffers.  The cache lives in a trunk handle of the CUDA library together with the
    trunk weights; tokens / positions are the two small buffers a driver refreshes in place
    between replays (nn/static_kv.rs)."""

    def __init__(self, dec: "OlmoeDecoder", slots: int, max_ctx: int):
        t_, c = dec.torch, dec.cfg
        self.slots, self.max_ctx, self.dec = slots, max_ctx, dec
        cfg = dec._trunk_config(slots, max_ctx)
        self.handle = C.c_void_p()
        moe_mod._check(L.lib.mummu_trunk_create(C.byref(cfg), C.byref(self.handle)))
        dev = dec.dev
        self.tokens = t_.zeros(slots, 1, dtype=t_.int32, device=dev)
        self.positions = t_.zeros(slots, dtype=t_.int32, device=dev)
        self.x = t_.zeros(slots, c.hidden_size, dtype=t_.float16, device=dev)
        self.h2 = t_.zeros(slots, c.hidden_size, dtype=t_.float16, device=dev)
        self.logits = t_.zeros(slots, c.vocab_size, dtype=t_.float32, device=dev)
        self.argmax = t_.zeros(slots, dtype=t_.int32, device=dev)

        def put(which, layer, tensor, f32=False):
            tt = tensor.to(t_.float32 if f32 else t_.float16).contiguous()
            moe_mod._check(L.lib.mummu_trunk_set_weight(self.handle, which, layer, tt.data_ptr(),
                                                        tt.numel() * tt.element_size(), 1))
        put(L.TRUNK_EMBED, 0, dec.embed)
        put(L.TRUNK_LM_HEAD, 0, dec.lm_head)
        put(L.TRUNK_FINAL_NORM, 0, dec.final_norm, True)
        for l, lay in enumerate(dec.layers):
            put(L.TRUNK_IN_NORM, l, lay["in_norm"], True)
            put(L.TRUNK_POST_NORM, l, lay["post_norm"], True)
            put(L.TRUNK_Q_NORM, l, lay["q_norm"], True)
            put(L.TRUNK_K_NORM, l, lay["k_norm"], True)
            for which, name in ((L.TRUNK_Q, "q"), (L.TRUNK_K, "k"), (L.TRUNK_V, "v"), (L.TRUNK_O, "o")):
                put(which, l, lay[name])

    # `StaticState::{mark, rewind}` (capture.rs:109-122): a KV write is an assignment (the same row,
    # the same values however often it runs), and this model carries no recurrent state
    def mark(self):
        return (self.tokens.clone(), self.positions.clone())

    def rewind(self, mark) -> None:
        self.tokens.copy_(mark[0])
        self.positions.copy_(mark[1])

    def close(self) -> None:
        if self.handle and self.handle.value:
            L.lib.mummu_trunk_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


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

    # ---- `StaticDecode` (capture.rs:48-107): the fixed-shape decode step -----------------------
    def static_supported(self, device=None) -> bool:
        """Whether the model, as loaded, can take the static path: f16 trunk on this device with
        projection widths the trunk kernels take (multiples of 128 rows)."""
        c = self.cfg
        nqkv = (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
        return (self.embed is not None and c.hidden_size % 128 == 0 and nqkv % 128 == 0 and c.vocab_size % 128 == 0
                and c.head_dim % 8 == 0)

    def static_capturable(self, device=None) -> bool:
        """Every buffer the step touches is on the device and nothing is uploaded inside it."""
        return self.static_supported(device)

    def trained_context(self):
        return None

    def _trunk_config(self, slots: int, max_ctx: int) -> "L.MummuTrunkConfig":
        c = self.cfg
        return L.MummuTrunkConfig(device=self.dev.index, hidden=c.hidden_size, heads=c.num_attention_heads,
                                  kv_heads=c.num_key_value_heads, head_dim=c.head_dim, layers=c.num_hidden_layers,
                                  vocab=c.vocab_size, slots=slots, max_ctx=max_ctx, rope_theta=c.rope_theta,
                                  rms_eps=c.rms_norm_eps)

    def static_bytes(self, slots: int, max_ctx: int, device=None) -> int:
        cfg = self._trunk_config(slots, max_ctx)
        return int(L.lib.mummu_trunk_static_bytes(C.byref(cfg)))

    def static_state(self, slots: int, max_ctx: int, device=None) -> "StaticState":
        """A zeroed static state for `slots` sequences of up to `max_ctx` positions: the preallocated
        cache [slots, kv_heads, max_ctx, head_dim] per layer (nn/static_kv.rs:36-72) inside a trunk
        handle that also holds this model's trunk weights."""
        assert self.static_supported(), "the static path needs loaded weights and 128-row projection widths"
        return StaticState(self, slots, max_ctx)

    def forward_static(self, tokens, positions, state: "StaticState", length: int):
        """One decode step for the state's first k slots: tokens [k, 1] at positions [k] (device
        int32), attending over a bucket of `length` keys; logits [k, vocab] (f32).  Touches nothing
        but device buffers; every buffer of `state` it advances it advances in place
        (capture.rs:93-103)."""
        t_, c = self.torch, self.cfg
        k = tokens.shape[0]
        assert tokens.dtype == t_.int32 and positions.dtype == t_.int32 and k <= state.slots
        h = state.handle
        stream = moe_mod._torch_stream()
        x, h2, logits = state.x[:k], state.h2[:k], state.logits[:k]
        moe_mod._check(L.lib.mummu_trunk_embed(h, tokens.data_ptr(), k, x.data_ptr(), stream))
        y = None
        for l, lay in enumerate(self.layers):
            moe_mod._check(L.lib.mummu_trunk_attention_step(h, l, x.data_ptr(), None if y is None else y.data_ptr(),
                                                            positions.data_ptr(), k, length, h2.data_ptr(), stream))
            y = lay["mlp"].forward(h2, c.num_experts_per_tok, c.norm_topk_prob)
        moe_mod._check(L.lib.mummu_trunk_head(h, x.data_ptr(), y.data_ptr(), k, logits.data_ptr(),
                                              state.argmax.data_ptr(), stream))
        return logits

    def seed_static(self, state: "StaticState", slot: int, cache_len: int, src_slot: int = None) -> None:
        """Copy the first `cache_len` positions of a prefilled sequence (this decoder's growing
        cache, sequence `src_slot`) into `slot` of the static state (capture.rs:105-106)."""
        b = slot if src_slot is None else src_slot
        stream = moe_mod._torch_stream()
        for l in range(self.cfg.num_hidden_layers):
            k = self.k_cache[l, b, :, :cache_len].contiguous()
            v = self.v_cache[l, b, :, :cache_len].contiguous()
            moe_mod._check(L.lib.mummu_trunk_kv_write(state.handle, l, slot, 0, cache_len, k.data_ptr(), v.data_ptr(),
                                                      stream))

    def decode_step(self, ids, past: int, state: "StaticState" = None):
        """One static decode step, eagerly: ids [B, 1] at position `past` for every sequence; logits
        [B, vocab].  Without a state one is made (and seeded from the growing cache) and kept."""
        t_ = self.torch
        B = ids.shape[0]
        if state is None:
            if getattr(self, "_own_state", None) is None or self._own_state.slots < B:
                self._own_state = self.static_state(B, self.max_ctx)
                self._own_next = -1
            state = self._own_state
            if self._own_next != past:          # not the continuation of the previous call: seed afresh
                for b in range(B):
                    self.seed_static(state, b, past)
            self._own_next = past + 1
        tokens = ids.reshape(B, 1).to(t_.int32)
        positions = t_.full((B,), past, dtype=t_.int32, device=self.dev)
        return self.forward_static(tokens, positions, state, bucket(past + 1, self.max_ctx)).clone()

    def make_decode_graph(self, state: "StaticState", B: int, length: int):
        """Captures one decode step of B slots over a bucket of `length` keys; returns the graph.
        The step reads state.tokens / state.positions and leaves state.logits / state.argmax."""
        t_ = self.torch
        s = t_.cuda.Stream(self.dev)
        s.wait_stream(t_.cuda.current_stream())
        mark = state.mark()
        with t_.cuda.stream(s):
            for _ in range(2):              # settle one-time attribute calls and the layers' scratch
                self.forward_static(state.tokens[:B], state.positions[:B], state, length)
        t_.cuda.current_stream().wait_stream(s)
        t_.cuda.synchronize()
        g = t_.cuda.CUDAGraph()
        with t_.cuda.graph(g):
            self.forward_static(state.tokens[:B], state.positions[:B], state, length)
        state.rewind(mark)
        return g

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

    def greedy_generate_static(self, prompt_ids, n_new: int, chunk: int = 1024, timed: bool = False):
        """Greedy decode on the static path: the prompt goes through `forward` in chunks
        (decode.rs:311-346) and seeds a static state; then every new token is one replay of the
        graph captured for its key bucket, the pick (argmax, decode.rs:33-48) made on the device
        and fed back without leaving it.  Returns the tokens [B, n_new]; with timed=True also the
        device time of the n_new decode steps in ms (CUDA events) and the launches of one step."""
        t_ = self.torch
        B, P = prompt_ids.shape
        past, logits = 0, None
        while past < P:
            n = min(chunk, P - past)
            logits = self.forward(prompt_ids[:, past:past + n], past)
            past += n
        state = self.static_state(B, self.max_ctx)
        for b in range(B):
            self.seed_static(state, b, past)
        state.tokens[:B, 0] = logits.argmax(-1).to(t_.int32)
        state.positions[:B] = past
        graphs, out = {}, []
        launches = None
        a, b_ev = t_.cuda.Event(enable_timing=True), t_.cuda.Event(enable_timing=True)
        lengths = sorted({bucket(p + 1, self.max_ctx) for p in range(past, past + n_new)})
        moe0 = sum(l["mlp"].launch_count() for l in self.layers)
        for length in lengths:                   # capture outside the timed region
            graphs[length] = self.make_decode_graph(state, B, length)
        moe_per_step = (sum(l["mlp"].launch_count() for l in self.layers) - moe0) // (3 * len(lengths))
        launches = moe_per_step + 7 * self.cfg.num_hidden_layers + 4           # + trunk kernels (7 per layer, head)
        t_.cuda.synchronize()
        a.record()
        for i in range(n_new):
            out.append(state.tokens[:B, 0].clone())
            graphs[bucket(past + 1, self.max_ctx)].replay()
            state.tokens[:B, 0] = state.argmax[:B]           # device to device: the pick feeds the next step
            state.positions[:B] += 1
            past += 1
        b_ev.record()
        t_.cuda.synchronize()
        toks = t_.stack(out, 1).to(t_.int64)
        ms = a.elapsed_time(b_ev)
        state.close()
        return (toks, ms, launches) if timed else toks

    def close(self):
        if getattr(self, "_own_state", None) is not None:
            self._own_state.close()
            self._own_state = None
        for lay in reversed(self.layers):
            lay["mlp"].close()
