"""GGUF Q4_K encoder (host, numpy).

The reference only decodes Q4_K (crates/mummu/src/gguf.rs:1685-1726); its own quantisers produce a
different block-32 format.  Parity is defined on the decoded values of whatever bytes are fed to
both sides, so any valid encoder serves.  This one is a plain min/max affine fit per 32-value
sub-block, written with operations whose results are fixed by IEEE-754 (min, max, divide, round
half to even), so the CUDA encoder `mummu_q4k_quantize` produces the same bytes.

Super-block layout (144 bytes for 256 values): f16 d, f16 dmin, 12 bytes of packed 6-bit
(scale, min) pairs for 8 sub-blocks, 128 bytes of 4-bit quants; chunk c of 64 values stores
sub-block 2c in the low nibbles and sub-block 2c+1 in the high nibbles of 32 bytes.
value = d*scale*q - dmin*min.
"""
from __future__ import annotations

import numpy as np

BLOCK_ELEMS = 256
BLOCK_BYTES = 144


def quantize(values: np.ndarray) -> np.ndarray:
    """f32 array whose size is a multiple of 256 -> uint8 array of size/256*144 bytes."""
    x = np.ascontiguousarray(values, dtype=np.float32).reshape(-1, 8, 32)
    nb = x.shape[0]
    zero = np.float32(0.0)
    lo = np.minimum(x.min(axis=2), zero)                       # [nb, 8]
    hi = np.maximum(x.max(axis=2), lo)
    scale = (hi - lo) / np.float32(15.0)
    mn = -lo
    d = (scale.max(axis=1) / np.float32(63.0)).astype(np.float16)
    dmin = (mn.max(axis=1) / np.float32(63.0)).astype(np.float16)
    df = d.astype(np.float32)[:, None]
    dminf = dmin.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(df > 0, np.clip(np.rint(scale / df), 0, 63), 0).astype(np.float32)
        m = np.where(dminf > 0, np.clip(np.rint(mn / dminf), 0, 63), 0).astype(np.float32)
        dsc = (df * sc)[:, :, None]
        dm = (dminf * m)[:, :, None]
        q = np.where(dsc > 0, np.clip(np.rint((x + dm) / dsc), 0, 15), 0).astype(np.uint8)
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    out = np.empty((nb, BLOCK_BYTES), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(nb, 2)
    out[:, 4:8] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)
    out[:, 8:12] = m[:, 0:4] | ((m[:, 4:8] >> 4) << 6)
    out[:, 12:16] = (sc[:, 4:8] & 0x0F) | ((m[:, 4:8] & 0x0F) << 4)
    q = q.reshape(nb, 4, 2, 32)                                # [block, chunk, low/high, byte]
    out[:, 16:144] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(nb, 128)
    return out.reshape(-1)


def bank_bytes(experts: int, out_dim: int, in_dim: int) -> int:
    assert in_dim % BLOCK_ELEMS == 0, "Q4_K rows hold whole 256-value super-blocks"
    return experts * out_dim * (in_dim // BLOCK_ELEMS) * BLOCK_BYTES
