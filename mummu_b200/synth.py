"""Seeded synthetic inputs for the MoE layer.

Generator: SplitMix64 (the generator the reference's own tests use,
crates/mummu/src/nn/packed_gemv.rs:1557-1566 and models/qwen4exp/experts.rs:1162-1171), 53-bit
uniforms, Box-Muller in f64, narrowed to f32.  SplitMix64 is counter based (output n is a mix of
seed + n*gamma), so the stream vectorises in numpy.  Draw order for one layer: router weight,
gate bank, up bank, down bank, activations, each from its own sub-stream.
"""
from __future__ import annotations

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix64(seed: int, start: int, count: int) -> np.ndarray:
    """Outputs start+1 .. start+count of SplitMix64(seed) as uint64."""
    with np.errstate(over="ignore"):
        n = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + n * _GAMMA
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def normal(seed: int, shape, std: float = 1.0, chunk: int = 1 << 22) -> np.ndarray:
    """N(0, std) f32 array of `shape`, reproducible from `seed` alone."""
    total = int(np.prod(shape))
    out = np.empty(total, dtype=np.float32)
    pairs = (total + 1) // 2
    done = 0
    while done < pairs:
        n = min(chunk, pairs - done)
        z = splitmix64(seed, 2 * done, 2 * n)
        u1 = ((z[0::2] >> np.uint64(11)).astype(np.float64) + 1.0) * (2.0 ** -53)
        u2 = (z[1::2] >> np.uint64(11)).astype(np.float64) * (2.0 ** -53)
        r = np.sqrt(-2.0 * np.log(u1))
        th = 2.0 * np.pi * u2
        pair = np.empty(2 * n, dtype=np.float64)
        pair[0::2] = r * np.cos(th)
        pair[1::2] = r * np.sin(th)
        lo = 2 * done
        hi = min(total, lo + 2 * n)
        out[lo:hi] = (pair[: hi - lo] * std).astype(np.float32)
        done += n
    return out.reshape(shape)


def permutation(seed: int, n: int) -> np.ndarray:
    """A seeded permutation of 0..n-1 (argsort of one SplitMix64 draw per element)."""
    return np.argsort(splitmix64(seed, 0, n), kind="stable").astype(np.int64)


def layer_seed(cfg_seed: int, layer: int, stream: int) -> int:
    """One sub-stream per (config seed, layer, tensor)."""
    return ((cfg_seed << 32) + (layer << 8) + stream) & 0xFFFFFFFFFFFFFFFF


def moe_layer(hidden: int, inter: int, experts: int, tokens: int, cfg_seed: int = 0,
              layer: int = 0, w_std: float = 0.02, x_std: float = 1.0):
    """(router [H, E], gate [E, I, H], up [E, I, H], down [E, H, I], x [T, H]) in f32."""
    router = normal(layer_seed(cfg_seed, layer, 0), (hidden, experts), w_std)
    gate = normal(layer_seed(cfg_seed, layer, 1), (experts, inter, hidden), w_std)
    up = normal(layer_seed(cfg_seed, layer, 2), (experts, inter, hidden), w_std)
    down = normal(layer_seed(cfg_seed, layer, 3), (experts, hidden, inter), w_std)
    x = normal(layer_seed(cfg_seed, layer, 4), (tokens, hidden), x_std)
    return router, gate, up, down, x


def zipf_router_bias(experts: int, alpha: float, s: float = 1.1, seed: int = 0) -> np.ndarray:
    """Additive router-logit bias that skews expert load: b_e = -alpha * s * ln(rank_e), rank a
    seeded permutation of 1..experts.  A benchmark construct (the reference's router has no
    bias, crates/mummu/src/nn/moe.rs:92)."""
    rank = permutation(layer_seed(seed, 0, 9), experts) + 1
    return (-alpha * s * np.log(rank.astype(np.float64))).astype(np.float32)
