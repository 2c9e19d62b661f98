"""CPU tests: the oracle against every known-answer vector the reference's tests hold for this
path, against the committed golden fixtures, and against itself (properties the reference
asserts)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import toy  # noqa: E402
from oracle import oracle as O  # noqa: E402
from mummu_b200 import q4k, synth  # noqa: E402


def f16_bytes(v):
    return np.frombuffer(np.float16(v).tobytes(), np.uint8)


# ---- Q4_K ---------------------------------------------------------------------------------

def test_q4k_superblock_known_answer():
    """crates/mummu/src/gguf.rs:2408-2429, literal for literal."""
    block = np.zeros(144, np.uint8)
    block[0:2] = f16_bytes(1.0)
    block[2:4] = f16_bytes(0.5)
    block[4], block[5], block[8] = 2, 3, 1
    block[12] = 0x21
    block[16] = 0x51
    block[16 + 64] = 0x04
    out = O.dequant_q4_k(block)
    assert out.size == 256
    assert out[0] == 1.5
    assert out[32] == 15.0
    assert out[128] == 3.0
    assert out[1] == -0.5


def test_f16_widening_is_exact_for_every_bit_pattern():
    """gguf.rs:1464-1468 checks its conversion exhaustively against the `half` crate; numpy's
    float16 is the same IEEE type."""
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([O.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_q4k_decode_matches_gguf_package():
    gguf = pytest.importorskip("gguf")
    rng = np.random.default_rng(3)
    raw = rng.integers(0, 256, size=64 * 144, dtype=np.uint8).reshape(64, 144)
    for b in range(64):  # sane scales, as the reference's synthetic blocks (experts.rs:1225-1229)
        raw[b, 0:2] = f16_bytes(rng.uniform(0.0005, 0.003))
        raw[b, 2:4] = f16_bytes(rng.uniform(0.0005, 0.003))
    want = gguf.quants.dequantize(raw, gguf.GGMLQuantizationType.Q4_K).reshape(-1)
    got = O.dequant_q4_k(raw)
    assert np.array_equal(got.view(np.uint32), want.astype(np.float32).view(np.uint32))


def test_q4k_encoder_round_trip():
    w = synth.normal(11, (64, 256), 0.02)
    raw = q4k.quantize(w)
    assert raw.size == 64 * 144
    back = O.dequant_q4_k(raw).reshape(64, 256)
    # 4-bit affine fit per 32 values: error below one quantisation step of the widest sub-block
    step = (w.reshape(64, 8, 32).max(2) - np.minimum(w.reshape(64, 8, 32).min(2), 0)).max() / 15
    assert np.abs(back - w).max() <= 1.01 * step
    # encoding what was decoded changes nothing any more (idempotent on its own grid)
    again = O.dequant_q4_k(q4k.quantize(back)).reshape(64, 256)
    assert np.abs(again - back).max() <= 0.51 * step


# ---- router -------------------------------------------------------------------------------

def test_router_picks_most_probable():
    """models/qwen4exp/experts.rs:1366-1378 (ids; weights there are renormalised)."""
    logits = np.array([[0.0, 3.0, 1.0, 2.5, -2.0, 2.0, 0.5, 2.9]], np.float32)
    ids, w = O.route(logits, 3, True)
    assert ids.tolist() == [[1, 7, 3]]
    z = np.exp(3.0) + np.exp(2.9) + np.exp(2.5)
    want = [np.exp(3.0) / z, np.exp(2.9) / z, np.exp(2.5) / z]
    assert np.allclose(w[0], want, atol=1e-6)
    assert abs(w.sum() - 1.0) < 1e-6


def test_router_ties_go_to_lowest_expert_id():
    """experts.rs:1381-1388."""
    ids, w = O.route(np.full((1, 8), 0.5, np.float32), 3, True)
    assert ids.tolist() == [[0, 1, 2]]
    assert np.allclose(w, 1.0 / 3.0, atol=1e-6)
    ids, _ = O.route(np.array([[1.0, 0.0, 2.0, 1.0]], np.float32), 2, False)
    assert ids.tolist() == [[2, 0]]


def test_router_huge_logits_and_many_tokens():
    """experts.rs:1391-1408."""
    logits = np.full((3, 16), -1000.0, np.float32)
    logits[0, 5] = 1000.0
    logits[1, 9] = 999.0
    logits[1, 3] = 998.0
    logits[2, 15] = 30.0
    ids, w = O.route(logits, 2, True)
    assert ids[0, 0] == 5
    assert ids[1].tolist() == [9, 3]
    assert ids[2, 0] == 15
    assert np.isfinite(w).all()
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)
    e = np.e
    assert abs(w[1, 0] - e / (e + 1.0)) < 1e-6


def test_router_refuses_nonfinite_and_bad_k():
    """experts.rs:1411-1417."""
    with pytest.raises(ValueError, match="token 0 expert 1"):
        O.route(np.array([[0.0, np.nan], [1.0, 2.0]], np.float32), 1)
    for k in (0, 5):
        with pytest.raises(ValueError):
            O.route(np.zeros((1, 4), np.float32), k)


def test_exp_within_one_ulp_of_libm():
    xs = np.concatenate([np.linspace(-104.0, 0.0, 20001), -np.abs(np.random.default_rng(0).normal(size=20000)) * 10])
    xs = xs.astype(np.float32)
    got = O.exp(xs).astype(np.float64)
    ref = np.exp(xs.astype(np.float64))
    ulp = np.spacing(np.maximum(ref, 2.0 ** -149).astype(np.float32)).astype(np.float64)
    assert (np.abs(got - ref) / ulp).max() <= 1.0
    assert O.exp(np.array([0.0], np.float32))[0] == 1.0


def test_routing_same_with_libm_exp_on_gaussian_logits():
    """The deterministic exp changes no routing decision on the benchmark's input distribution."""
    router, _, _, _, x = synth.moe_layer(256, 8, 64, 512, cfg_seed=3)
    logits = O.router_logits(x, router)
    a, wa = O.route(logits, 8, False, exp_kind=0)
    b, wb = O.route(logits, 8, False, exp_kind=1)
    assert np.array_equal(a, b)
    assert np.allclose(wa, wb, rtol=1e-6)


def test_dot8_order():
    """experts.rs:463-478: 8 lanes, fixed fold, leftovers one by one."""
    rng = np.random.default_rng(5)
    a = rng.normal(size=27).astype(np.float32)
    b = rng.normal(size=27).astype(np.float32)
    acc = np.zeros(8, np.float32)
    for c in range(3):
        for l in range(8):
            acc[l] = np.float32(acc[l] + np.float32(a[c * 8 + l] * b[c * 8 + l]))
    s = np.float32(np.float32(np.float32(acc[0] + acc[4]) + np.float32(acc[1] + acc[5])) +
                   np.float32(np.float32(acc[2] + acc[6]) + np.float32(acc[3] + acc[7])))
    for i in range(24, 27):
        s = np.float32(s + np.float32(a[i] * b[i]))
    assert O.dot8(a, b) == s


# ---- the layer ------------------------------------------------------------------------------

GOLD = np.load(os.path.join(HERE, "golden", "toy_moe.npz"))


@pytest.mark.parametrize("t,seed,norm", [(5, 2.0, False), (5, 2.0, True), (1, 2.0, False),
                                         (1, 2.0, True), (5, 7.0, False), (5, 7.0, True)])
def test_toy_layer_matches_committed_golden(t, seed, norm):
    """nn/moe.rs:2177-2202 shapes (t in {5, 1}, both norm settings) on the reference's toy layer."""
    rw = toy.router()
    g, u, d = toy.banks()
    x = toy.inputs(t, seed)
    key = f"t{t}_s{seed}_n{int(norm)}_k{toy.TOP_K}"
    for order in (O.SUM_SEQUENTIAL, O.SUM_LANES8):
        y, ids, w = O.moe_forward(x, rw, g, u, d, toy.TOP_K, norm, order=order)
        assert np.array_equal(ids, GOLD[key + "_ids"])
        assert np.abs(w - GOLD[key + "_w"]).max() < 1e-6
        assert np.abs(y - GOLD[key + "_y"]).max() < 1e-5   # the reference's own tolerance


def test_dense_mask_equals_routed():
    """nn/moe.rs:1655-1700: routed == dense-mask < 1e-5."""
    rw = toy.router()
    g, u, d = toy.banks()
    for t, seed, norm in [(1, 2.0, False), (5, 7.0, False), (5, 7.0, True)]:
        x = toy.inputs(t, seed)
        a, _, _ = O.moe_forward(x, rw, g, u, d, toy.TOP_K, norm, dense_mask=True)
        b, _, _ = O.moe_forward(x, rw, g, u, d, toy.TOP_K, norm, dense_mask=False)
        assert np.abs(a - b).max() < 1e-5


def test_top_k_equal_to_num_experts():
    """nn/moe.rs:2204-2230: k == E without renorm is the full softmax mixture."""
    rw = toy.router()
    g, u, d = toy.banks()
    x = toy.inputs(3, 0.5)
    y, ids, w = O.moe_forward(x, rw, g, u, d, toy.EXPERTS, False)
    assert sorted(ids[0].tolist()) == [0, 1, 2, 3]
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)
    assert np.abs(y - GOLD[f"t3_s0.5_n0_k{toy.EXPERTS}_y"]).max() < 1e-5


def test_renorm_changes_output_and_position_independence_and_zero():
    """nn/moe.rs:2297-2352."""
    rw = toy.router()
    g, u, d = toy.banks()
    x = toy.inputs(4, 7.0)
    a, _, _ = O.moe_forward(x, rw, g, u, d, toy.TOP_K, False)
    b, _, _ = O.moe_forward(x, rw, g, u, d, toy.TOP_K, True)
    assert (np.abs(a - b) > 1e-7).any()
    row = toy.inputs(1, 11.0)
    s, _, _ = O.moe_forward(row, rw, g, u, d, toy.TOP_K, False)
    dd, _, _ = O.moe_forward(np.concatenate([row, row]), rw, g, u, d, toy.TOP_K, False)
    assert np.array_equal(s[0], dd[0]) and np.array_equal(s[0], dd[1])
    z, _, _ = O.moe_forward(np.zeros((2, toy.HIDDEN), np.float32), rw, g, u, d, toy.TOP_K, False)
    assert (z == 0).all()


def test_q4k_small_matches_committed_golden():
    gold = np.load(os.path.join(HERE, "golden", "q4k_small.npz"))
    y, ids, w = O.moe_forward(gold["x"], gold["router"], gold["gate_q"], gold["up_q"], gold["down_q"],
                              2, False, q4k=True)
    assert np.array_equal(ids, gold["ids"])
    assert np.array_equal(w.view(np.uint32), gold["w"].view(np.uint32))
    assert np.array_equal(y.view(np.uint32), gold["y"].view(np.uint32))
    assert np.array_equal(O.dequant_q4_k(gold["gate_q"][: 4 * 144]).view(np.uint32),
                          gold["gate_deq_rows"].view(np.uint32))


def test_q4k_matvec_equals_dequantise_then_f64_matmul():
    """experts.rs:1273-1309: packed-bytes path == dequantise then f64 matmul at 1e-5."""
    H, I, E = 256, 256, 2
    _, gate, up, down, x = synth.moe_layer(H, I, E, 3, cfg_seed=5)
    gq, uq, dq = (q4k.quantize(b) for b in (gate, up, down))
    ids = np.array([[0], [1], [0]], np.int32)
    w = np.ones((3, 1), np.float32)
    got = O.moe_routed(x, ids, w, gq, uq, dq, H, I, E, q4k=True)
    gd, ud, dd = (O.dequant_q4_k(b).astype(np.float64) for b in (gq, uq, dq))
    gd, ud, dd = gd.reshape(E, I, H), ud.reshape(E, I, H), dd.reshape(E, H, I)
    for t in range(3):
        e = ids[t, 0]
        xv = x[t].astype(np.float64)
        a = gd[e] @ xv
        h = a / (1 + np.exp(-a)) * (ud[e] @ xv)
        want = dd[e] @ h
        assert np.abs(got[t] - want).max() / np.abs(want).max() < 1e-5


def test_hits_count_rows_per_expert():
    """nn/moe.rs:1562-1564: hits[e] += rows served."""
    rw = toy.router()
    g, u, d = toy.banks()
    x = toy.inputs(6, 2.0)
    ids, w = O.route(O.router_logits(x, rw), toy.TOP_K)
    hits = np.zeros(toy.EXPERTS, np.uint64)
    O.moe_routed(x, ids, w, g, u, d, toy.HIDDEN, toy.INTER, toy.EXPERTS, hits=hits)
    assert hits.sum() == 12
    assert np.array_equal(hits, np.bincount(ids.reshape(-1), minlength=toy.EXPERTS).astype(np.uint64))
