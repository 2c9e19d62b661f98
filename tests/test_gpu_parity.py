"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Bars: routing ids, routing weights and dequantised weights bit-exact; layer
outputs within 1e-4 (f32) / 2e-2 (f16, bf16, Q4_K) relative, measured as max|a-b| / max|b|
(the reference's convention, crates/mummu/src/nn/packed_gemv.rs:1610-1622)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import toy  # noqa: E402
from oracle import oracle as O  # noqa: E402
from mummu_b200 import q4k, synth  # noqa: E402

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-4
TOL_16 = 2e-2


def rel_err(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(np.abs(b).max(), 1e-30))


@pytest.fixture(scope="module")
def M(cuda_lib):
    from mummu_b200 import moe
    return moe


def make_layer(M, L, H, I, E, K, act, wdt, router, gate, up, down, bias=None, max_tokens=0):
    m = M.SparseMoeConfig(H, I, E, K).init(act_dtype=act, weight_dtype=wdt, max_tokens=max_tokens)
    m.set_router(router, bias=bias)
    m.set_banks(gate, up, down)
    return m


def bf16_bits(a):
    """f32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


# ---- toy layer: the reference's own unit-test shapes --------------------------------------------

@pytest.mark.parametrize("t,seed,norm,k", [(5, 2.0, False, 2), (5, 2.0, True, 2), (1, 2.0, False, 2),
                                            (1, 2.0, True, 2), (5, 7.0, True, 2), (3, 0.5, False, 4)])
def test_toy_layer(M, cuda_lib, t, seed, norm, k):
    """nn/moe.rs:2177-2230 on HIDDEN=4, INTER=3, EXPERTS=4 (ragged: nothing divides a tile)."""
    L = cuda_lib
    rw = toy.router()
    g, u, d = toy.banks()
    x = toy.inputs(t, seed)
    m = make_layer(M, L, toy.HIDDEN, toy.INTER, toy.EXPERTS, toy.EXPERTS, L.F32, L.F32, rw, g, u, d)
    y = m.forward(x.reshape(1, t, toy.HIDDEN), k, norm).reshape(t, toy.HIDDEN)
    ids, w = m.route_flat(x, k, norm)
    want, wid, ww = O.moe_forward(x, rw, g, u, d, k, norm)
    assert np.array_equal(ids, wid)
    assert np.array_equal(w.view(np.uint32), ww.view(np.uint32))
    assert np.abs(y - want).max() < 1e-5
    gold = np.load(os.path.join(HERE, "golden", "toy_moe.npz"))
    key = f"t{t}_s{seed}_n{int(norm)}_k{k}"
    assert np.array_equal(ids, gold[key + "_ids"])
    assert np.abs(y - gold[key + "_y"]).max() < 1e-5
    m.close()


def test_toy_properties(M, cuda_lib):
    """Position independence bit-exact, zero in -> zero out, renorm changes the mixture, top_k
    contract (nn/moe.rs:2297-2361)."""
    L = cuda_lib
    rw = toy.router()
    g, u, d = toy.banks()
    m = make_layer(M, L, toy.HIDDEN, toy.INTER, toy.EXPERTS, toy.EXPERTS, L.F32, L.F32, rw, g, u, d)
    row = toy.inputs(1, 11.0)
    s = m.forward(row, 2, False)
    dd = m.forward(np.concatenate([row, row]), 2, False)
    assert np.array_equal(s[0], dd[0]) and np.array_equal(s[0], dd[1])
    z = m.forward(np.zeros((2, toy.HIDDEN), np.float32), 2, False)
    assert (z == 0).all()
    x = toy.inputs(4, 7.0)
    assert (np.abs(m.forward(x, 2, False) - m.forward(x, 2, True)) > 1e-7).any()
    with pytest.raises(M.MoeContractError, match="top_k"):
        m.forward(row, toy.EXPERTS + 1, False)
    with pytest.raises(M.MoeContractError, match="top_k"):
        m.forward(row, 0, False)
    with pytest.raises(M.MoeContractError, match="hidden"):
        m.forward(np.zeros((1, 5), np.float32), 2, False)
    assert m.forward(np.zeros((0, toy.HIDDEN), np.float32), 2, False).shape == (0, toy.HIDDEN)
    m.close()


def test_router_known_answers_on_device(M, cuda_lib):
    """The reference's router vectors (models/qwen4exp/experts.rs:1366-1408) through the CUDA
    router: an identity-like router weight turns activations into the listed logits."""
    L = cuda_lib
    E = 8
    eye = np.eye(E, dtype=np.float32)
    z = np.zeros((E, 1, E), np.float32)
    m = make_layer(M, L, E, 1, E, E, L.F32, L.F32, eye, z, z, np.zeros((E, E, 1), np.float32))
    ids, w = m.route_flat(np.array([[0.0, 3.0, 1.0, 2.5, -2.0, 2.0, 0.5, 2.9]], np.float32), 3, True)
    assert ids.tolist() == [[1, 7, 3]]
    assert abs(w.sum() - 1.0) < 1e-6
    ids, w = m.route_flat(np.full((1, E), 0.5, np.float32), 3, True)
    assert ids.tolist() == [[0, 1, 2]]
    assert np.allclose(w, 1 / 3, atol=1e-6)
    m.close()
    m = make_layer(M, L, 4, 1, 4, 4, L.F32, L.F32, np.eye(4, dtype=np.float32), np.zeros((4, 1, 4), np.float32),
                   np.zeros((4, 1, 4), np.float32), np.zeros((4, 4, 1), np.float32))
    ids, _ = m.route_flat(np.array([[1.0, 0.0, 2.0, 1.0]], np.float32), 2, False)
    assert ids.tolist() == [[2, 0]]
    m.close()
    m = make_layer(M, L, 16, 1, 16, 16, L.F32, L.F32, np.eye(16, dtype=np.float32), np.zeros((16, 1, 16), np.float32),
                   np.zeros((16, 1, 16), np.float32), np.zeros((16, 16, 1), np.float32))
    logits = np.full((3, 16), -1000.0, np.float32)
    logits[0, 5], logits[1, 9], logits[1, 3], logits[2, 15] = 1000.0, 999.0, 998.0, 30.0
    ids, w = m.route_flat(logits, 2, True)
    oid, ow = O.route(logits, 2, True)
    assert np.array_equal(ids, oid) and np.array_equal(w.view(np.uint32), ow.view(np.uint32))
    assert ids[0, 0] == 5 and ids[1].tolist() == [9, 3] and ids[2, 0] == 15
    # non-finite logits are refused (experts.rs:1411-1417)
    bad = logits.copy()
    bad[1, 1] = np.nan
    with pytest.raises(M.MoeNumericError):
        m.route_flat(bad, 2, True)
    ids, _ = m.route_flat(logits, 2, True)      # the handle stays usable
    assert np.array_equal(ids, oid)
    m.close()


# ---- routing bit-exactness at the benchmark shapes ---------------------------------------------

@pytest.mark.parametrize("T,H,E,K,norm,act", [(16, 2048, 64, 8, False, "f32"), (333, 2048, 64, 8, True, "f32"),
                                              (4096, 2048, 64, 8, False, "bf16"), (64, 2048, 64, 8, False, "f16"),
                                              (257, 2048, 128, 8, False, "f32"), (7, 100, 20, 5, True, "f32"),
                                              # the register-tiled kernel: 32-token tiles and two expert passes;
                                              # a partial second pass with a k tail; f16 with a ragged last tile
                                              (9601, 2048, 128, 8, True, "bf16"), (300, 2116, 72, 6, True, "f32"),
                                              (1027, 1024, 64, 8, False, "f16")])
def test_routing_bit_exact(M, cuda_lib, T, H, E, K, norm, act):
    L = cuda_lib
    router = synth.normal(synth.layer_seed(1, 0, 0), (H, E), 0.02)
    x = synth.normal(synth.layer_seed(1, 0, 4), (T, H), 1.0)
    bias = synth.zipf_router_bias(E, 1.0) if T == 4096 else None
    code = {"f32": L.F32, "f16": L.F16, "bf16": L.BF16}[act]
    if act == "f16":
        xin = x.astype(np.float16)
        x = xin.astype(np.float32)
    elif act == "bf16":
        xin = bf16_bits(x)
        x = bf16_to_f32(xin)
    else:
        xin = x
    z = np.zeros((E, 1, H), np.float32)
    m = M.SparseMoeConfig(H, 1, E, K).init(act_dtype=code, weight_dtype=L.F32)
    m.set_router(router, bias=bias)
    ids, w = m.route_flat(xin, K, norm)
    oid, ow = O.route(O.router_logits(x, router, bias), K, norm)
    assert np.array_equal(ids, oid)
    assert np.array_equal(w.view(np.uint32), ow.view(np.uint32))
    hits = m.take_hits()
    assert np.array_equal(hits, np.bincount(oid.reshape(-1), minlength=E).astype(np.uint64))
    assert m.take_hits().sum() == 0
    m.close()


# ---- Q4_K -----------------------------------------------------------------------------------

def test_q4k_dequant_bit_exact_and_quantiser_parity(M, cuda_lib):
    import torch
    L = cuda_lib
    H, I, E = 512, 256, 3
    _, gate, up, down, _ = synth.moe_layer(H, I, E, 1, cfg_seed=2)
    gq, uq, dq = (q4k.quantize(b) for b in (gate, up, down))
    m = M.SparseMoeConfig(H, I, E, 2).init(act_dtype=L.F16, weight_dtype=L.Q4_K)
    m.set_banks(gq, uq, dq)
    for which, raw, shape in ((L.BANK_GATE, gq, (E, I, H)), (L.BANK_UP, uq, (E, I, H)), (L.BANK_DOWN, dq, (E, H, I))):
        want = O.dequant_q4_k(raw).reshape(shape)
        for e in range(E):
            got = m.dequant_bank(which, e)
            assert np.array_equal(got.view(np.uint32), want[e].view(np.uint32))
    m.close()
    # random bytes (every scale/nibble pattern), sane f16 scales as the reference's synthetic blocks
    rng = np.random.default_rng(9)
    raw = rng.integers(0, 256, size=(4096, 144), dtype=np.uint8)
    raw[:, 0:2] = np.frombuffer(rng.uniform(0.0005, 0.003, 4096).astype(np.float16).tobytes(), np.uint8).reshape(4096, 2)
    raw[:, 2:4] = np.frombuffer(rng.uniform(0.0005, 0.003, 4096).astype(np.float16).tobytes(), np.uint8).reshape(4096, 2)
    got = M.q4k_dequantize_device(torch.from_numpy(raw.reshape(-1)).cuda()).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), O.dequant_q4_k(raw).view(np.uint32))
    # device encoder == host encoder, byte for byte
    w = synth.normal(77, (2048, 256), 0.02)
    dev = M.q4k_quantize_device(torch.from_numpy(w).cuda()).cpu().numpy()
    assert np.array_equal(dev, q4k.quantize(w))


@pytest.mark.parametrize("T", [1, 2, 3, 7, 8, 9, 16, 17, 33, 64, 65, 130, 256])
def test_q4k_decode_layer(M, cuda_lib, T):
    """Decode regime, Q4_K experts, f16 activations, the ragged token counts included."""
    L = cuda_lib
    H, I, E, K = 1024, 512, 16, 4
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=4)
    gq, uq, dq = (q4k.quantize(b) for b in (gate, up, down))
    xh = x.astype(np.float16)
    m = make_layer(M, L, H, I, E, K, L.F16, L.Q4_K, router, gq, uq, dq)
    y = m.forward(xh, K, False).astype(np.float32)
    want, oid, ow = O.moe_forward(xh.astype(np.float32), router, gq, uq, dq, K, False, q4k=True)
    ids, w = m.route_flat(xh, K, False)
    assert np.array_equal(ids, oid) and np.array_equal(w.view(np.uint32), ow.view(np.uint32))
    assert rel_err(y, want) < TOL_16
    # position independence, bit-exact: token 0 alone == token 0 in the batch (nn/moe.rs:2318-2338)
    alone = m.forward(xh[:1], K, False)
    assert np.array_equal(alone[0], m.forward(xh, K, False)[0])
    m.close()


def test_q4k_decode_all_tokens_one_expert(M, cuda_lib):
    """Collision edge: every token routed to the same experts (more rows than one token tile)."""
    L = cuda_lib
    H, I, E, K, T = 512, 256, 8, 2, 40
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=6)
    bias = np.zeros(E, np.float32)
    bias[3], bias[5] = 50.0, 40.0
    gq, uq, dq = (q4k.quantize(b) for b in (gate, up, down))
    xh = x.astype(np.float16)
    m = make_layer(M, L, H, I, E, K, L.F16, L.Q4_K, router, gq, uq, dq, bias=bias)
    y = m.forward(xh, K, True).astype(np.float32)
    want, oid, _ = O.moe_forward(xh.astype(np.float32), router, gq, uq, dq, K, True, bias=bias, q4k=True)
    assert set(oid.reshape(-1).tolist()) == {3, 5}
    assert rel_err(y, want) < TOL_16
    m.close()


@pytest.fixture(scope="module")
def olmoe_q4k_layer(M, cuda_lib):
    """One OLMoE-sized Q4_K layer (hidden 2048, intermediate 1024, 64 experts): large enough that
    the decode path takes its streaming kernels."""
    import torch
    L = cuda_lib
    H, I, E, K = 2048, 1024, 64, 8
    router, _, _, _, x = synth.moe_layer(H, 16, E, 256, cfg_seed=12)
    banks = []
    for i, shape in enumerate(((E * I, H), (E * I, H), (E * H, I))):
        w = synth.normal(900 + i, shape, 0.02)
        banks.append(M.q4k_quantize_device(torch.from_numpy(w).cuda()).cpu().numpy())
    return H, I, E, K, router, banks, x.astype(np.float16)


@pytest.mark.parametrize("T", [9, 40, 64, 200])
def test_q4k_decode_olmoe_shape(M, cuda_lib, olmoe_q4k_layer, T):
    L = cuda_lib
    H, I, E, K, router, (gq, uq, dq), xh = olmoe_q4k_layer
    m = make_layer(M, L, H, I, E, K, L.F16, L.Q4_K, router, gq, uq, dq)
    y = m.forward(xh[:T], K, False).astype(np.float32)
    want, oid, ow = O.moe_forward(xh[:T].astype(np.float32), router, gq, uq, dq, K, False, q4k=True)
    ids, w = m.route_flat(xh[:T], K, False)
    assert np.array_equal(ids, oid) and np.array_equal(w.view(np.uint32), ow.view(np.uint32))
    assert rel_err(y, want) < TOL_16
    # a token's result does not depend on its batch-mates or on the kernel variant that ran
    # (streaming for large batches, split-K for one token): bit for bit (nn/moe.rs:2318-2338)
    if T == 64:
        y40 = m.forward(xh[:40], K, False)
        y64 = m.forward(xh, K, False)
        assert np.array_equal(y40[:40], y64[:40])
        assert np.array_equal(m.forward(xh[:1], K, False)[0], y64[0])
    m.close()


def test_q4k_decode_olmoe_shape_crowded_experts(M, cuda_lib, olmoe_q4k_layer):
    """Every token on the same experts: 64 rows per expert = four passes of the 16-token tile."""
    L = cuda_lib
    H, I, E, K, router, (gq, uq, dq), xh = olmoe_q4k_layer
    bias = np.zeros(E, np.float32)
    bias[[3, 5, 11, 17, 23, 31, 42, 63]] = 60.0
    m = make_layer(M, L, H, I, E, K, L.F16, L.Q4_K, router, gq, uq, dq, bias=bias)
    T = 64
    y = m.forward(xh[:T], K, True).astype(np.float32)
    want, oid, _ = O.moe_forward(xh[:T].astype(np.float32), router, gq, uq, dq, K, True, bias=bias, q4k=True)
    assert set(oid.reshape(-1).tolist()) == {3, 5, 11, 17, 23, 31, 42, 63}
    assert rel_err(y, want) < TOL_16
    m.close()


def test_q4k_grouped_rows_many_passes(M, cuda_lib, olmoe_q4k_layer):
    """`experts_grouped` on already sorted rows with ragged segments (0 .. 64 rows per expert, the
    shape an expert-parallel rank sees): several passes of the token tile, shared between CTAs."""
    import torch
    L = cuda_lib
    H, I, E, K, router, (gq, uq, dq), _ = olmoe_q4k_layer
    counts = np.full(E, 8, np.int32)
    counts[[0, 5, 9, 20, 33, 47, 63]] = [17, 0, 33, 64, 1, 40, 16]
    rows = int(counts.sum())
    xs = synth.normal(31, (rows, H), 1.0).astype(np.float16)
    m = make_layer(M, L, H, I, E, K, L.F16, L.Q4_K, router, gq, uq, dq)
    ys = torch.zeros(rows, H, dtype=torch.float16, device="cuda")
    # the row bound an expert-parallel caller passes (capacity, not the exact count) sets the split
    cap = torch.zeros(4 * rows, H, dtype=torch.float16, device="cuda")
    cap[:rows] = torch.from_numpy(xs).cuda()
    ycap = torch.zeros(4 * rows, H, dtype=torch.float16, device="cuda")
    m.experts_grouped(torch.from_numpy(xs).cuda(), torch.from_numpy(counts).cuda(), ys)
    m.experts_grouped(cap, torch.from_numpy(counts).cuda(), ycap)
    torch.cuda.synchronize()
    m.sync()
    assert torch.equal(ys, ycap[:rows])            # same bits whatever the pass split
    off = np.concatenate([[0], np.cumsum(counts)])
    got = ys.cpu().numpy().astype(np.float32)
    rb_gate, rb_down = H // 256 * 144, I // 256 * 144
    for e in (0, 9, 20, 33, 47):
        g = O.dequant_q4_k(gq.reshape(E, I, rb_gate)[e]).reshape(I, H)
        u = O.dequant_q4_k(uq.reshape(E, I, rb_gate)[e]).reshape(I, H)
        d = O.dequant_q4_k(dq.reshape(E, H, rb_down)[e]).reshape(H, I)
        want = O.expert_ffn(g, u, d, xs[off[e]:off[e + 1]].astype(np.float32))
        assert rel_err(got[off[e]:off[e + 1]], want) < TOL_16
    assert not got[off[5]:off[6]].size
    m.close()


def test_host_pointer_calls_replay_a_graph(M, cuda_lib):
    """Host-pointer decode calls: the first runs eagerly, the second is captured, later ones are
    replayed.  Same bits every time, on new inputs, into a caller-provided output array, and after
    the router or a bank changed (which drops the captured graphs)."""
    L = cuda_lib
    H, I, E, K, T = 1024, 512, 16, 4, 24
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=4)
    banks = [q4k.quantize(b) for b in (gate, up, down)]
    a = make_layer(M, L, H, I, E, K, L.F16, L.Q4_K, router, *banks)
    b = make_layer(M, L, H, I, E, K, L.F16, L.Q4_K, router, *banks)     # only ever called once per state
    xh = x.astype(np.float16)
    first = b.forward(xh, K, False)
    for _ in range(5):
        assert np.array_equal(a.forward(xh, K, False), first)
    x2 = (xh * 0.5).astype(np.float16)
    out = np.empty_like(x2)
    got = a.forward(x2, K, False, out=out)
    assert got.base is out or got is out
    assert np.array_equal(out, b.forward(x2, K, False))
    a.set_router(router * 2.0)
    b.set_router(router * 2.0)
    assert np.array_equal(a.forward(x2, K, False), b.forward(x2, K, False))
    swapped = np.ascontiguousarray(banks[2].reshape(E, -1)[::-1])          # experts in reverse order
    a.set_bank(L.BANK_DOWN, swapped)
    b.set_bank(L.BANK_DOWN, swapped)
    for _ in range(3):
        ya = a.forward(x2, K, False)
    assert np.array_equal(ya, b.forward(x2, K, False))
    with pytest.raises(M.MoeContractError):
        a.forward(x2, K, False, out=np.empty((3, 3), np.float16))
    a.close()
    b.close()


def test_q4k_prompt_sized_calls_take_the_tensor_cores(M, cuda_lib, olmoe_q4k_layer):
    """More than 256 tokens on Q4_K experts (a prompt): the experts with rows are expanded to f16
    and the tcgen05 grouped GEMMs run on them.  Small shape in full against the oracle; the OLMoE
    shape at 600 tokens on sampled tokens (tokens are independent), and against the generic bank
    (NO_TC) on every token; the kernel list shows which path ran."""
    L = cuda_lib
    H, I, E, K, T = 512, 256, 8, 2, 300
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=23)
    gq, uq, dq = (q4k.quantize(b) for b in (gate, up, down))
    xh = x.astype(np.float16)
    m = make_layer(M, L, H, I, E, K, L.F16, L.Q4_K, router, gq, uq, dq)
    m.set_profiling(True)
    y = m.forward(xh, K, True).astype(np.float32)
    names = set(m.take_profile())
    assert {"q4k_expand", "tc_gate_up", "tc_down"} <= names, names
    want, _, _ = O.moe_forward(xh.astype(np.float32), router, gq, uq, dq, K, True, q4k=True)
    assert rel_err(y, want) < TOL_16
    m.close()
    H, I, E, K, router, (gq, uq, dq), xh = olmoe_q4k_layer
    T = 600
    rng = np.random.default_rng(4)
    xl = np.concatenate([xh, (rng.standard_normal((T - xh.shape[0], H))).astype(np.float16)])
    m = make_layer(M, L, H, I, E, K, L.F16, L.Q4_K, router, gq, uq, dq)
    y = m.forward(xl, K, False).astype(np.float32)
    pick = [0, 1, 255, 256, 300, 599]
    want, _, _ = O.moe_forward(xl[pick].astype(np.float32), router, gq, uq, dq, K, False, q4k=True)
    assert rel_err(y[pick], want) < TOL_16
    m.set_switch("NO_TC", 1)
    y_generic = m.forward(xl, K, False).astype(np.float32)
    assert rel_err(y, y_generic) < TOL_16
    m.close()


def test_q4k_small_golden(M, cuda_lib):
    L = cuda_lib
    gold = np.load(os.path.join(HERE, "golden", "q4k_small.npz"))
    m = make_layer(M, L, 256, 256, 4, 2, L.F16, L.Q4_K, gold["router"], gold["gate_q"], gold["up_q"], gold["down_q"])
    xh = gold["x"].astype(np.float16)
    ids, w = m.route_flat(xh, 2, False)
    assert np.array_equal(ids, gold["ids"]) and np.array_equal(w.view(np.uint32), gold["w"].view(np.uint32))
    assert rel_err(m.forward(xh, 2, False).astype(np.float32), gold["y"]) < TOL_16
    assert np.array_equal(m.dequant_bank(L.BANK_GATE, 0)[:4].reshape(-1).view(np.uint32),
                          gold["gate_deq_rows"].view(np.uint32))
    m.close()


# ---- float banks ------------------------------------------------------------------------------

def test_config1_f32_layer(M, cuda_lib):
    """T=16, hidden 2048, 64 experts, top-8 without renormalisation, intermediate 1024, f32
    N(0, 0.02) weights, N(0, 1) activations, seed 0; checked against both the routed and the
    dense-mask form of the reference (nn/moe.rs:116-177, 296-328)."""
    L = cuda_lib
    H, I, E, K, T = 2048, 1024, 64, 8, 16
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=0)
    m = make_layer(M, L, H, I, E, K, L.F32, L.F32, router, gate, up, down)
    y = m.forward(x.reshape(1, T, H), K, False).reshape(T, H)
    want, oid, ow = O.moe_forward(x, router, gate, up, down, K, False)
    ids, w = m.route_flat(x, K, False)
    assert np.array_equal(ids, oid) and np.array_equal(w.view(np.uint32), ow.view(np.uint32))
    assert rel_err(y, want) < TOL_F32
    dense, _, _ = O.moe_forward(x, router, gate, up, down, K, False, dense_mask=True)
    assert rel_err(y, dense) < TOL_F32
    # ExpertExec::run and SparseMoePerExpert::{route, run_local}
    e = int(oid[0, 0])
    got = M.CudaExpert(m, e).run(x[:3].reshape(-1), 3, H).reshape(3, H)
    assert rel_err(got, O.expert_ffn(gate[e], up[e], down[e], x[:3])) < TOL_F32
    routing = m.route(x, K, False)
    assert sum(len(r) for r, _ in routing.per_expert) == T * K
    assert rel_err(m.run_local(x, routing), want) < TOL_F32
    m.close()


@pytest.mark.parametrize("act", ["f16", "bf16"])
def test_half_precision_layer(M, cuda_lib, act):
    L = cuda_lib
    H, I, E, K, T = 512, 256, 16, 4, 50
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=8)
    if act == "f16":
        conv = lambda a: a.astype(np.float16)
        back = lambda a: a.astype(np.float32)
        code = L.F16
    else:
        conv, back, code = bf16_bits, bf16_to_f32, L.BF16
    gq, uq, dq, xq = conv(gate), conv(up), conv(down), conv(x)
    m = make_layer(M, L, H, I, E, K, code, code, router, gq, uq, dq)
    y = back(m.forward(xq, K, False))
    want, _, _ = O.moe_forward(back(xq), router, back(gq), back(uq), back(dq), K, False)
    assert rel_err(y, want) < TOL_16
    m.close()


@pytest.mark.parametrize("T", [1, 24, 128, 300])
def test_route_grouped_equals_route_then_permute(M, cuda_lib, T):
    """The fused router + grouping launch (and its two-launch fallback for large T) give exactly
    the (ids, weights, counts, offsets, row_token, pos) of route followed by permute."""
    import torch
    L = cuda_lib
    H, I, E, K = 512, 64, 16, 4
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=17)
    m = make_layer(M, L, H, I, E, K, L.F16, L.F16, router, *(b.astype(np.float16) for b in (gate, up, down)))
    xd = torch.from_numpy(x.astype(np.float16)).cuda()
    ids, w = m.route_flat(xd, K, False)
    i32 = dict(dtype=torch.int32, device="cuda")
    counts, offsets = torch.empty(E, **i32), torch.empty(E + 1, **i32)
    row_token, pos = torch.empty(T * K, **i32), torch.empty(T * K, **i32)
    m.permute(ids, counts, offsets, row_token, pos)
    got = m.route_grouped(xd, K, False)
    torch.cuda.synchronize()
    for a, b in zip(got, (ids, w, counts, offsets, row_token, pos)):
        assert torch.equal(a, b)
    m.close()


@pytest.mark.parametrize("T,E,K", [(1100, 64, 8), (9001, 128, 8), (22000, 20, 3)])
def test_permute_of_a_large_call_is_the_stable_sort_by_expert(M, cuda_lib, T, E, K):
    """From 65536 (token, slot) pairs on, grouping is a three-launch counting sort (the last two
    shapes); it must give what the one-launch kernel gives: rows ordered by expert, ascending token
    inside an expert (`Routing.per_expert` of nn/moe.rs:275-289), counts and offsets."""
    import torch
    L = cuda_lib
    H = 256
    router, gate, up, down, x = synth.moe_layer(H, 16, E, T, cfg_seed=19)
    m = make_layer(M, L, H, 16, E, K, L.F32, L.F32, router, gate, up, down)
    xd = torch.from_numpy(x).cuda()
    ids, w, counts, offsets, row_token, pos = m.route_grouped(xd, K, False)
    m.sync()
    idn = ids.cpu().numpy().reshape(-1)
    want_counts = np.bincount(idn, minlength=E)
    assert np.array_equal(counts.cpu().numpy(), want_counts)
    assert np.array_equal(offsets.cpu().numpy(), np.concatenate([[0], np.cumsum(want_counts)]))
    order = np.argsort(idn, kind="stable")
    assert np.array_equal(row_token.cpu().numpy(), order // K)
    assert np.array_equal(pos.cpu().numpy()[order], np.arange(T * K))
    y = m.forward(xd, K, False)                      # and the layer that runs on this plan
    want, _, _ = O.moe_forward(x[:64], router, gate, up, down, K, False)
    assert rel_err(y[:64].cpu().numpy(), want) < TOL_F32
    m.close()


def test_staged_calls_match_whole_layer(M, cuda_lib):
    """permute -> experts_grouped -> combine on device tensors == forward."""
    import torch
    L = cuda_lib
    H, I, E, K, T = 256, 128, 8, 2, 37
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=12)
    m = make_layer(M, L, H, I, E, K, L.F32, L.F32, router, gate, up, down)
    xd = torch.from_numpy(x).cuda()
    whole = m.forward(xd, K, False)
    ids, w = m.route_flat(xd, K, False)
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    row_token = torch.zeros(T * K, dtype=torch.int32, device="cuda")
    pos = torch.zeros(T * K, dtype=torch.int32, device="cuda")
    m.permute(ids, counts, offsets, row_token, pos)
    idn = ids.cpu().numpy()
    assert np.array_equal(counts.cpu().numpy(), np.bincount(idn.reshape(-1), minlength=E))
    order = np.argsort(idn.reshape(-1), kind="stable")
    assert np.array_equal(row_token.cpu().numpy(), order // K)
    assert np.array_equal(pos.cpu().numpy()[order], np.arange(T * K))
    xs = xd[row_token.long()]
    ys = torch.empty_like(xs)
    m.experts_grouped(xs, counts, ys)
    out = torch.empty_like(xd)
    m.combine(ys, ids, w, pos, out)
    m.sync()
    assert torch.equal(out, whole)
    m.close()


# ---- tensor-core (tcgen05) prefill path ---------------------------------------------------------

@pytest.mark.parametrize("act,T,H,I,E,K", [("bf16", 300, 512, 256, 8, 2), ("f16", 129, 256, 128, 4, 2),
                                           ("bf16", 1, 256, 128, 4, 2), ("bf16", 700, 1024, 512, 16, 4)])
def test_tensor_core_layer_against_oracle(M, cuda_lib, act, T, H, I, E, K):
    """Ragged per-expert segments (not multiples of the 128-row tile), several tiles per expert,
    experts with no rows; outputs against the f32 oracle on the same 16-bit inputs."""
    L = cuda_lib
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=31)
    if act == "f16":
        conv, back, code = (lambda a: a.astype(np.float16)), (lambda a: a.astype(np.float32)), L.F16
    else:
        conv, back, code = bf16_bits, bf16_to_f32, L.BF16
    bias = np.zeros(E, np.float32)
    bias[1] = -1000.0                      # an expert nobody picks
    bias[0] = 3.0                          # a hot one
    gq, uq, dq, xq = conv(gate), conv(up), conv(down), conv(x)
    m = make_layer(M, L, H, I, E, K, code, code, router, gq, uq, dq, bias=bias)
    y = back(m.forward(xq, K, False))
    want, oid, _ = O.moe_forward(back(xq), router, back(gq), back(uq), back(dq), K, False, bias=bias)
    assert 1 not in set(oid.reshape(-1).tolist())
    assert rel_err(y, want) < TOL_16
    prof_names = None
    m.set_profiling(True)
    m.forward(xq, K, False)
    prof_names = set(m.take_profile())
    assert "tc_gate_up" in prof_names and "tc_down" in prof_names, prof_names   # the tensor-core path ran
    m.close()


def test_tensor_core_prefill_config_shape(M, cuda_lib):
    """The prefill configuration's shape (T=4096, hidden 2048, 64 experts, top-8, intermediate 1024,
    bf16, Zipf-skewed router bias).  Routing of every token against the oracle, bit for bit; layer
    outputs of a sample of tokens against the oracle (tokens are independent, so 40 rows of y cost
    the oracle seconds): tokens of the hottest and of the coldest expert, the first and last rows,
    a row present at two positions; and the whole output against the SIMT path of the library."""
    import torch
    L = cuda_lib
    H, I, E, K, T = 2048, 1024, 64, 8, 4096
    g = torch.Generator(device="cuda").manual_seed(5)
    rnd = lambda *s: torch.randn(*s, generator=g, device="cuda") * 0.02
    router = rnd(H, E).cpu().numpy()
    bias = synth.zipf_router_bias(E, alpha=1.0)
    m = M.SparseMoeConfig(H, I, E, K).init(act_dtype=L.BF16, weight_dtype=L.BF16, max_tokens=T)
    m.set_router(router, bias=bias)
    banks = [rnd(E, I, H).to(torch.bfloat16), rnd(E, I, H).to(torch.bfloat16), rnd(E, H, I).to(torch.bfloat16)]
    m.set_banks(*banks)
    x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    x[7] = x[3000]                                   # same row at two positions
    y = m.forward(x, K, False)
    m.sync()
    m.set_profiling(True)
    m.forward(x, K, False)
    assert {"tc_gate_up", "tc_down"} <= set(m.take_profile())      # the tensor-core path ran
    m.set_profiling(False)
    ids, w = m.route_flat(x, K, False)
    xf = x.float().cpu().numpy()
    oid, ow = O.route(O.router_logits(xf, router, bias), K, False)
    assert np.array_equal(ids.cpu().numpy(), oid)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), ow.view(np.uint32))
    load = np.bincount(oid.reshape(-1), minlength=E)
    assert load.max() > 3 * load.mean()              # skewed: ragged, many-tile segments
    assert torch.equal(y[7], y[3000])
    # sampled rows against the oracle
    hot, cold = int(load.argmax()), int(np.where(load > 0, load, load.max() + 1).argmin())
    rows_of = lambda e: np.nonzero((oid == e).any(1))[0]
    pick = sorted(set([0, 1, 7, 3000, T - 1] + rows_of(hot)[[0, len(rows_of(hot)) // 2, -1]].tolist()
                      + rows_of(cold)[:3].tolist() + list(range(100, 4000, 150))))
    gate, up, down = (b.float().cpu().numpy() for b in banks)
    want, _, _ = O.moe_forward(xf[pick], router, gate, up, down, K, False, bias=bias)
    got = y[pick].float().cpu().numpy()
    assert rel_err(got, want) < TOL_16
    assert len(pick) >= 32
    m.set_switch("NO_TC", 1)
    y_simt = m.forward(x, K, False)
    m.sync()
    m.set_switch("NO_TC", 0)
    err = (y.float() - y_simt.float()).abs().max().item() / y_simt.float().abs().max().item()
    assert err < TOL_16
    m.close()


# ---- ExpertExec: one expert on its own -----------------------------------------------------------

@pytest.mark.parametrize("kind", ["f32", "bf16", "q4k"])
def test_expert_exec_methods(M, cuda_lib, kind):
    """`ExpertExec` (nn/moe.rs:348-419): run (host f32 rows), run_tensor / run_tensor_resident (device
    rows), gate_energy, resident_bytes, tier, and the pinned-executor defaults."""
    import torch
    L = cuda_lib
    H, I, E, K, rows = 512, 256, 6, 2, 21
    router, gate, up, down, x = synth.moe_layer(H, I, E, rows, cfg_seed=33)
    if kind == "f32":
        act, wdt, banks, per = L.F32, L.F32, (gate, up, down), 4.0
        deq = (gate, up, down)
        tdt = torch.float32
    elif kind == "bf16":
        act, wdt = L.BF16, L.BF16
        banks = tuple(bf16_bits(b) for b in (gate, up, down))
        deq = tuple(bf16_to_f32(b) for b in banks)
        per, tdt = 2.0, torch.bfloat16
    else:
        act, wdt = L.F16, L.Q4_K
        banks = tuple(q4k.quantize(b) for b in (gate, up, down))
        deq = (O.dequant_q4_k(banks[0]).reshape(E, I, H), O.dequant_q4_k(banks[1]).reshape(E, I, H),
               O.dequant_q4_k(banks[2]).reshape(E, H, I))
        per, tdt = 144.0 / 256.0, torch.float16
    m = make_layer(M, L, H, I, E, K, act, wdt, router, *banks)
    e = 4
    ex = M.CudaExpert(m, e)
    xin = x if kind == "f32" else (bf16_to_f32(bf16_bits(x)) if kind == "bf16" else x.astype(np.float16).astype(np.float32))
    want = O.expert_ffn(deq[0][e], deq[1][e], deq[2][e], xin)
    tol = TOL_F32 if kind == "f32" else TOL_16
    got = ex.run(xin.reshape(-1), rows, H).reshape(rows, H)
    assert rel_err(got, want) < tol
    assert np.array_equal(got, ex.run(xin.reshape(-1), rows, H).reshape(rows, H))     # staging is reused
    xd = torch.from_numpy(xin).cuda().to(tdt)
    yd = ex.run_tensor(xd)
    yr = ex.run_tensor_resident(xd)
    torch.cuda.synchronize()
    assert rel_err(yd.float().cpu().numpy(), want) < tol and torch.equal(yd, yr)
    energy = ex.gate_energy(xin.reshape(-1), rows, H)
    g = xin.astype(np.float64) @ deq[0][e].astype(np.float64).T
    ref_energy = ((g / (1.0 + np.exp(-g))) ** 2).sum(1)
    assert np.abs(energy - ref_energy).max() / ref_energy.max() < 1e-4
    assert ex.resident_bytes() == int(3 * H * I * per)
    t = ex.tier()
    assert t.device == 0 and t.precision == wdt
    assert ex.is_staged() and ex.stage() is None and ex.evict() is None and ex.disable_native() is None
    with pytest.raises(M.MoeContractError):
        M.CudaExpert(m, E).run(xin.reshape(-1), rows, H)
    m.close()


# ---- checked mode -------------------------------------------------------------------------------

def test_checked_mode_passes_good_plans_and_reports_bad_ones(M, cuda_lib):
    """Switch CHECKED: the routing plan behind every computed address is verified on the device.
    Good plans give bit-identical results with no report; a caller-given index outside its buffer
    is made safe, the call completes, and the next sync reports it.  (The buffers here have slack
    behind their stated size, so not even an unchecked build would leave allocated memory.)"""
    import torch
    L = cuda_lib
    for act, wdt, T in ((L.F16, L.Q4_K, 40), (L.BF16, L.BF16, 300), (L.F32, L.F32, 33)):
        H, I, E, K = 512, 256, 8, 2
        router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=31)
        if wdt == L.Q4_K:
            banks = [q4k.quantize(b) for b in (gate, up, down)]
            xin = x.astype(np.float16)
        elif wdt == L.BF16:
            banks = [bf16_bits(b) for b in (gate, up, down)]
            xin = bf16_bits(x)
        else:
            banks, xin = [gate, up, down], x
        m = make_layer(M, L, H, I, E, K, act, wdt, router, *banks)
        plain = m.forward(xin, K, True)
        m.set_switch("CHECKED", 1)
        checked = m.forward(xin, K, True)
        m.sync()                                         # nothing to report
        assert np.array_equal(np.asarray(plain).view(np.uint8), np.asarray(checked).view(np.uint8))
        m.close()
    H, I, E, K, T = 256, 128, 8, 2, 37
    router, gate, up, down, x = synth.moe_layer(H, I, E, T, cfg_seed=12)
    m = make_layer(M, L, H, I, E, K, L.F32, L.F32, router, gate, up, down)
    m.set_switch("CHECKED", 1)
    xd = torch.from_numpy(x).cuda()
    ids, w, counts, offsets, row_token, pos = m.route_grouped(xd, K, False)
    m.sync()
    slack = 8
    xs = torch.zeros(T * K + slack, H, device="cuda")
    xs[:T * K] = xd[row_token.long()]
    ys = torch.zeros_like(xs)
    m.experts_grouped(xs[:T * K], counts, ys[:T * K])
    out = torch.empty_like(xd)
    m.combine(ys[:T * K], ids, w, pos, out)
    m.sync()
    assert torch.equal(out, m.forward(xd, K, False))
    bad_pos = pos.clone()
    bad_pos[5] = T * K + 1                               # behind the rows the call states
    m.combine(ys[:T * K], ids, w, bad_pos, out)
    with pytest.raises(M.MoeContractError, match="left its buffer"):
        m.sync()
    assert torch.isfinite(out).all()
    bad_counts = counts.clone()
    bad_counts[E - 1] += 3                               # segments run past the rows the call states
    m.experts_grouped(xs[:T * K], bad_counts, ys[:T * K])
    with pytest.raises(M.MoeContractError, match="left its buffer"):
        m.sync()
    m.sync()
    m.close()
