"""The reference tests' toy layer (crates/mummu/src/nn/moe.rs:1617-1651, 2088-2093): HIDDEN=4,
INTER=3, EXPERTS=4, TOP_K=2, closed-form sinusoid weights and inputs."""
import numpy as np

HIDDEN, INTER, EXPERTS, TOP_K = 4, 3, 4, 2


def _fill(seed: float, dims):
    n = int(np.prod(dims))
    i = np.arange(n, dtype=np.float64)
    # f32 fused multiply-add of (i, 0.37f32, seed): exact in f64, rounded once to f32
    arg = (i * np.float64(np.float32(0.37)) + np.float64(np.float32(seed))).astype(np.float32)
    return (np.sin(arg.astype(np.float64)).astype(np.float32) * np.float32(0.5)).reshape(dims)


def router():
    i = np.arange(HIDDEN * EXPERTS, dtype=np.float64)
    arg = (i * np.float64(np.float32(0.61)) + 1.0).astype(np.float32)
    return (np.cos(arg.astype(np.float64)).astype(np.float32) * np.float32(0.5)).reshape(HIDDEN, EXPERTS)


def banks():
    return (_fill(0.1, (EXPERTS, INTER, HIDDEN)), _fill(1.7, (EXPERTS, INTER, HIDDEN)),
            _fill(3.3, (EXPERTS, HIDDEN, INTER)))


def inputs(t: int, seed: float):
    i = np.arange(t * HIDDEN, dtype=np.float32)
    arg = (i + np.float32(seed)) * np.float32(0.9)
    return np.sin(arg.astype(np.float64)).astype(np.float32).reshape(t, HIDDEN)
