"""Sibling GGUF block formats Q8_0, Q5_K, Q6_K (crates/mummu/src/gguf.rs:1535-1543, 1731-1797): the
oracle against the reference's hand-computed super-blocks, the device decoders bit for bit against
the oracle, and a layer over such banks (generic bank) against the oracle's f32 layer."""
import numpy as np
import pytest

from oracle import oracle as O
from mummu_b200 import synth

F16_ONE = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
FORMATS = {"Q8_0": (32, 34), "Q5_K": (256, 176), "Q6_K": (256, 210)}


def test_q6_k_superblock_matches_hand_computation():
    # gguf.rs:2432-2449
    b = np.zeros(210, np.uint8)
    b[0], b[128], b[192], b[194] = 0x0F, 0b11, 2, 1
    b[208:210] = F16_ONE
    out = O.dequant_blocks(b, "Q6_K")
    assert out.size == 256
    assert out[0] == 62.0          # q1 = (15 | 3<<4) - 32 = 31, scale 2
    assert out[32] == -32.0        # q2 = -32, scale sc[2] = 1
    assert out[64] == 0.0          # zero scale zeroes the value


def test_q5_k_superblock_matches_hand_computation():
    # gguf.rs:2638-2653
    b = np.zeros(176, np.uint8)
    b[0:2], b[2:4] = F16_ONE, F16_ONE
    b[4], b[5], b[8], b[16], b[48] = 2, 3, 1, 1, 0x21
    out = O.dequant_blocks(b, "Q5_K")
    assert out.size == 256
    assert out[0] == 33.0          # sc*(q + 16) - dmin*m = 2*17 - 1
    assert out[1] == -1.0          # zero quant still subtracts the min
    assert out[32] == 6.0          # bit-plane 1 unset: no +16; m1 = 0


def test_q8_0_block():
    # gguf.rs:1535-1543: x = d * i8
    b = np.zeros(34, np.uint8)
    b[0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    b[2], b[3], b[33] = 4, 0xFF, 0x80
    out = O.dequant_blocks(b, "Q8_0")
    assert out[0] == 2.0 and out[1] == -0.5 and out[31] == -64.0 and out[2] == 0.0


def random_blocks(kind, n_blocks, seed, d_scale=1.0):
    """Every byte pattern is a valid block; f16 scales kept small and finite."""
    elems, nbytes = FORMATS[kind]
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(n_blocks, nbytes), dtype=np.uint8)
    d = np.frombuffer(rng.uniform(0.0005 * d_scale, 0.003 * d_scale, n_blocks).astype(np.float16).tobytes(), np.uint8).reshape(n_blocks, 2)
    if kind == "Q6_K":
        raw[:, 208:210] = d
    else:
        raw[:, 0:2] = d
    if kind == "Q5_K":
        raw[:, 2:4] = np.frombuffer(rng.uniform(0.0005 * d_scale, 0.003 * d_scale, n_blocks).astype(np.float16).tobytes(), np.uint8).reshape(n_blocks, 2)
    return raw


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["Q8_0", "Q5_K", "Q6_K"])
def test_sibling_format_layer(kind):
    from mummu_b200 import _lib as L, moe as M
    H, I, E, K, T = 512, 256, 4, 2, 13
    elems, nbytes = FORMATS[kind]
    code = {"Q8_0": L.Q8_0, "Q5_K": L.Q5_K, "Q6_K": L.Q6_K}[kind]
    router, _, _, _, x = synth.moe_layer(H, 16, E, T, cfg_seed=23)
    gate = random_blocks(kind, E * I * H // elems, 1)
    up = random_blocks(kind, E * I * H // elems, 2)
    down = random_blocks(kind, E * H * I // elems, 3)
    m = M.SparseMoeConfig(H, I, E, K).init(act_dtype=L.F32, weight_dtype=code)
    m.set_router(router)
    m.set_banks(gate, up, down)
    gf = O.dequant_blocks(gate, kind).reshape(E, I, H)
    uf = O.dequant_blocks(up, kind).reshape(E, I, H)
    df = O.dequant_blocks(down, kind).reshape(E, H, I)
    for which, ref in ((L.BANK_GATE, gf), (L.BANK_UP, uf), (L.BANK_DOWN, df)):
        for e in (0, E - 1):
            got = m.dequant_bank(which, e)
            assert np.array_equal(got.view(np.uint32), ref[e].view(np.uint32))     # bit for bit
    y = m.forward(x, K, False)
    want, oid, ow = O.moe_forward(x, router, gf, uf, df, K, False)
    ids, w = m.route_flat(x, K, False)
    assert np.array_equal(ids, oid) and np.array_equal(w.view(np.uint32), ow.view(np.uint32))
    err = np.linalg.norm(y - want) / np.linalg.norm(want)
    assert err < 1e-4
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["Q8_0", "Q5_K", "Q6_K"])
@pytest.mark.parametrize("T", [13, 300])
def test_sibling_format_layer_f16_takes_the_tensor_cores(kind, T):
    """With f16 activations a bank in a sibling format is expanded to f16 (experts with rows only;
    the same element decoders, one more rounding) and runs the tcgen05 grouped GEMMs instead of
    the generic bank.  Against the oracle's f32 layer over the exactly dequantised weights."""
    from mummu_b200 import _lib as L, moe as M
    H, I, E, K = 512, 256, 4, 2
    elems, nbytes = FORMATS[kind]
    code = {"Q8_0": L.Q8_0, "Q5_K": L.Q5_K, "Q6_K": L.Q6_K}[kind]
    router, _, _, _, x = synth.moe_layer(H, 16, E, T, cfg_seed=29)
    # random scale bytes make weights of magnitude d * 63 * 31: scales small enough that the 16-bit
    # intermediate stays far from its range
    gate = random_blocks(kind, E * I * H // elems, 4, d_scale=0.05)
    up = random_blocks(kind, E * I * H // elems, 5, d_scale=0.05)
    down = random_blocks(kind, E * H * I // elems, 6, d_scale=0.05)
    xh = x.astype(np.float16)
    m = M.SparseMoeConfig(H, I, E, K).init(act_dtype=L.F16, weight_dtype=code)
    m.set_router(router)
    m.set_banks(gate, up, down)
    m.set_profiling(True)
    y = m.forward(xh, K, True).astype(np.float32)
    names = set(m.take_profile())
    assert {"block_expand", "tc_gate_up", "tc_down"} <= names, names
    gf = O.dequant_blocks(gate, kind).reshape(E, I, H)
    uf = O.dequant_blocks(up, kind).reshape(E, I, H)
    df = O.dequant_blocks(down, kind).reshape(E, H, I)
    want, _, _ = O.moe_forward(xh.astype(np.float32), router, gf, uf, df, K, True)
    assert np.abs(y - want).max() / np.abs(want).max() < 2e-2
    m.set_switch("NO_TC", 1)                                   # the generic bank on the same call
    y2 = m.forward(xh, K, True).astype(np.float32)
    assert np.abs(y2 - want).max() / np.abs(want).max() < 2e-2
    m.close()
