"""ctypes front end of the CPU oracle (``mummu_oracle.c``).

TEST INFRASTRUCTURE, NOT PRODUCT: imported only by ``tests/``, by the smoke check and by the
benchmark's CPU-baseline leg.  Every function takes and returns numpy arrays; all arithmetic is the
C file's, which restates the reference (physics515/Mummu) and cites its lines.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmummu_oracle.so")

SUM_LANES8 = 0      # 8 lanes in the order of models/qwen4exp/experts.rs:463-478 (router: fused steps)
SUM_SEQUENTIAL = 1  # left to right, the reference tests' scalar loop (nn/moe.rs:2136)

ERR_NONFINITE = 5


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc, OpenMP, -ffp-contract=off)."""
    src = os.path.join(_HERE, "mummu_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B"], env=env)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_exp.restype = C.c_float
        L.orc_exp.argtypes = [C.c_float]
        L.orc_silu.restype = C.c_float
        L.orc_silu.argtypes = [C.c_float]
        L.orc_dot8.restype = C.c_float
        L.orc_dot8.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        L.orc_dequant_q4_k_blocks.restype = None
        L.orc_dequant_q4_k_blocks.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        L.orc_dequant_blocks.restype = C.c_int
        L.orc_dequant_blocks.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p]
        L.orc_router_logits.restype = None
        L.orc_router_logits.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                        C.c_int64, C.c_int, C.c_void_p]
        L.orc_route.restype = C.c_int
        L.orc_route.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int,
                                C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
        L.orc_expert_ffn.restype = None
        L.orc_expert_ffn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                     C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
        L.orc_moe_routed.restype = C.c_int
        L.orc_moe_routed.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                     C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.orc_moe_dense_mask.restype = C.c_int
        L.orc_moe_dense_mask.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                         C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_int, C.c_void_p]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.restype = None
        L.orc_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """Size the OpenMP pool (a launcher may have exported OMP_NUM_THREADS=1 for its ranks)."""
    lib().orc_set_num_threads(int(n))


def exp(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    L = lib()
    flat_in, flat_out = x.reshape(-1), out.reshape(-1)
    for i in range(flat_in.size):
        flat_out[i] = L.orc_exp(float(flat_in[i]))
    return out


def silu(x: float) -> float:
    return float(lib().orc_silu(float(x)))


def f16_to_f32(bits: int) -> float:
    return float(lib().orc_f16_to_f32(int(bits)))


def dot8(a, b) -> float:
    a, b = _f32(a), _f32(b)
    assert a.size == b.size
    return float(lib().orc_dot8(_p(a), _p(b), a.size))


def dequant_q4_k(raw) -> np.ndarray:
    """Q4_K bytes (multiple of 144) -> f32, gguf.rs:1701-1726."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    assert raw.size % 144 == 0, "whole super-blocks"
    nb = raw.size // 144
    out = np.empty(nb * 256, dtype=np.float32)
    lib().orc_dequant_q4_k_blocks(_p(raw), nb, _p(out))
    return out


BLOCK_FORMATS = {"Q4_K": (3, 256, 144), "Q8_0": (4, 32, 34), "Q5_K": (5, 256, 176), "Q6_K": (6, 256, 210)}


def dequant_blocks(raw, kind: str) -> np.ndarray:
    """Whole blocks of a GGUF block format -> f32 (gguf.rs:1535-1543 Q8_0, 1701-1726 Q4_K,
    1731-1765 Q5_K, 1769-1797 Q6_K)."""
    code, elems, nbytes = BLOCK_FORMATS[kind]
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    assert raw.size % nbytes == 0, "whole blocks"
    nb = raw.size // nbytes
    out = np.empty(nb * elems, dtype=np.float32)
    rc = lib().orc_dequant_blocks(code, _p(raw), nb, _p(out))
    assert rc == 0
    return out


def router_logits(x, w_in_out, bias=None, order: int = SUM_LANES8) -> np.ndarray:
    """x [T, H] f32, w [H, E] f32 (burn Linear order) -> logits [T, E]."""
    x, w = _f32(x), _f32(w_in_out)
    T, H = x.shape
    assert w.shape[0] == H
    E = w.shape[1]
    b = None if bias is None else _f32(bias)
    out = np.empty((T, E), dtype=np.float32)
    lib().orc_router_logits(_p(x), _p(w), None if b is None else _p(b), T, H, E, order, _p(out))
    return out


def route(logits, top_k: int, norm_topk_prob: bool = False, exp_kind: int = 0):
    """logits [T, E] -> (ids [T, k] int32, weights [T, k] f32).  Raises ValueError like the
    reference's `route` on bad k or a non-finite logit (experts.rs:547-560)."""
    logits = _f32(logits)
    T, E = logits.shape
    ids = np.empty((T, max(top_k, 0)), dtype=np.int32)
    w = np.empty((T, max(top_k, 0)), dtype=np.float32)
    bad = C.c_int64(-1)
    rc = lib().orc_route(_p(logits), T, E, top_k, int(bool(norm_topk_prob)), exp_kind, _p(ids),
                         _p(w), C.byref(bad))
    if rc == ERR_NONFINITE:
        raise ValueError(f"router logit for token {bad.value // E} expert {bad.value % E} is "
                         f"{logits.reshape(-1)[bad.value]}")
    if rc != 0:
        raise ValueError(f"top-{top_k} of {E} experts is not a routing")
    return ids, w


def expert_ffn(gate, up, down, x, order: int = SUM_LANES8) -> np.ndarray:
    """gate, up [I, H]; down [H, I]; x [rows, H] -> [rows, H]."""
    gate, up, down, x = _f32(gate), _f32(up), _f32(down), _f32(x)
    I, H = gate.shape
    rows = x.shape[0]
    y = np.empty((rows, H), dtype=np.float32)
    lib().orc_expert_ffn(_p(gate), _p(up), _p(down), H, I, _p(x), rows, order, _p(y))
    return y


def moe_routed(x, ids, weights, gate, up, down, hidden: int, inter: int, experts: int,
               q4k: bool = False, order: int = SUM_LANES8, hits=None) -> np.ndarray:
    """Routed bank + ascending-expert scatter-add.  Banks: f32 [E, out, in] or Q4_K bytes."""
    x = _f32(x)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    weights = _f32(weights)
    T, k = ids.shape
    if q4k:
        gate, up, down = (np.ascontiguousarray(b, dtype=np.uint8) for b in (gate, up, down))
        nbytes = experts * inter * hidden // 256 * 144
        assert gate.size == nbytes and up.size == nbytes and down.size == nbytes
    else:
        gate, up, down = _f32(gate), _f32(up), _f32(down)
        assert gate.size == experts * inter * hidden
    out = np.empty((T, hidden), dtype=np.float32)
    rc = lib().orc_moe_routed(_p(x), _p(ids), _p(weights), T, k, hidden, inter, experts, _p(gate),
                              _p(up), _p(down), int(q4k), order, _p(out),
                              None if hits is None else _p(hits))
    if rc != 0:
        raise ValueError("orc_moe_routed: bad argument")
    return out


def moe_dense_mask(x, ids, weights, gate, up, down, hidden: int, inter: int, experts: int,
                   order: int = SUM_LANES8) -> np.ndarray:
    x = _f32(x)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    weights = _f32(weights)
    gate, up, down = _f32(gate), _f32(up), _f32(down)
    T, k = ids.shape
    out = np.empty((T, hidden), dtype=np.float32)
    rc = lib().orc_moe_dense_mask(_p(x), _p(ids), _p(weights), T, k, hidden, inter, experts,
                                  _p(gate), _p(up), _p(down), order, _p(out))
    if rc != 0:
        raise ValueError("orc_moe_dense_mask: bad argument")
    return out


def moe_forward(x, router_w, gate, up, down, top_k: int, norm_topk_prob: bool = False,
                bias=None, q4k: bool = False, order: int = SUM_LANES8, dense_mask: bool = False):
    """The whole layer: router -> routed (or dense-mask) bank.  Returns (out, ids, weights)."""
    x = _f32(x)
    H, E = np.asarray(router_w).shape
    logits = router_logits(x, router_w, bias, order)
    ids, w = route(logits, top_k, norm_topk_prob)
    if q4k:
        inter = np.asarray(gate).size // (E * (H // 256) * 144)
    else:
        inter = np.asarray(gate).shape[1]
    if dense_mask:
        out = moe_dense_mask(x, ids, w, gate, up, down, H, inter, E, order)
    else:
        out = moe_routed(x, ids, w, gate, up, down, H, inter, E, q4k, order)
    return out, ids, w
