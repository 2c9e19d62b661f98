"""GGUF container: the reader's limits and refusals (crates/mummu/src/gguf.rs:1124-1376), the
OLMoE keys and tensor names (models/olmoe.rs:116-179, 319-349), and verbatim Q4_K expert banks."""
import os
import struct

import numpy as np
import pytest

from mummu_b200 import gguf, q4k, synth

META = {"general.architecture": "olmoe", "olmoe.embedding_length": 256, "olmoe.expert_feed_forward_length": 256,
        "olmoe.expert_count": 4, "olmoe.expert_used_count": 2, "olmoe.block_count": 2,
        "tokenizer.ggml.tokens": ["a", "b", "c"], "olmoe.rope.freq_base": 10000.0}


def synthetic_file(path, alignment=32, layers=2, extra_meta=None):
    H, I, E = 256, 256, 4
    tensors, truth = [], {}
    for l in range(layers):
        router, gate, up, down, _ = synth.moe_layer(H, I, E, 1, cfg_seed=50 + l)
        banks = {"gate": q4k.quantize(gate), "up": q4k.quantize(up), "down": q4k.quantize(down)}
        truth[l] = (router, banks)
        tensors.append((f"blk.{l}.ffn_gate_inp.weight", [H, E], "F32", np.ascontiguousarray(router.T)))
        tensors.append((f"blk.{l}.ffn_gate_exps.weight", [H, I, E], "Q4_K", banks["gate"]))
        tensors.append((f"blk.{l}.ffn_up_exps.weight", [H, I, E], "Q4_K", banks["up"]))
        tensors.append((f"blk.{l}.ffn_down_exps.weight", [I, H, E], "Q4_K", banks["down"]))
    meta = dict(META)
    meta.update(extra_meta or {})
    gguf.write_gguf(path, meta, tensors, alignment=alignment)
    return truth


@pytest.mark.parametrize("alignment", [32, 64, 4096])
def test_round_trip_verbatim_banks(tmp_path, alignment):
    p = str(tmp_path / "m.gguf")
    truth = synthetic_file(p, alignment)
    f = gguf.GgufFile.open(p)
    assert f.version == 3 and f.alignment == alignment and f.data_offset % alignment == 0
    assert f.architecture() == "olmoe" and f.get("tokenizer.ggml.tokens") == ["a", "b", "c"]
    assert abs(f.get("olmoe.rope.freq_base") - 10000.0) < 1e-3
    shp = gguf.olmoe_moe_shape(f)
    assert (shp.hidden_size, shp.expert_intermediate_size, shp.num_experts, shp.num_experts_per_tok,
            shp.norm_topk_prob, shp.num_hidden_layers) == (256, 256, 4, 2, False, 2)
    for l, (router, banks) in truth.items():
        t = f.tensor(f"blk.{l}.ffn_gate_exps.weight")
        assert t.dtype == "Q4_K" and t.shape == (4, 256, 256) and t.byte_len == 4 * 256 * 144 and t.offset % alignment == 0
        for which in ("gate", "up", "down"):
            got = f.tensor_bytes(f"blk.{l}.ffn_{which}_exps.weight")
            assert np.array_equal(got, banks[which].reshape(-1))          # byte for byte
        assert np.array_equal(f.tensor_array(f"blk.{l}.ffn_gate_inp.weight"), router.T)
    f.close()


def test_feed_forward_length_spelling_and_norm_key(tmp_path):
    p = str(tmp_path / "m.gguf")
    meta = dict(META)
    del meta["olmoe.expert_feed_forward_length"]
    meta.update({"olmoe.feed_forward_length": 256, "olmoe.expert_weights_norm": True})
    gguf.write_gguf(p, meta, [("x", [32], "F32", np.zeros(32, np.float32))])
    shp = gguf.olmoe_moe_shape(gguf.GgufFile.open(p))
    assert shp.expert_intermediate_size == 256 and shp.norm_topk_prob is True
    meta["general.architecture"] = "llama"
    gguf.write_gguf(p, meta, [("x", [32], "F32", np.zeros(32, np.float32))])
    with pytest.raises(ValueError, match="is not olmoe"):
        gguf.olmoe_moe_shape(gguf.GgufFile.open(p))


def _header(version=3, tensors=0, kvs=0, magic=b"GGUF"):
    return magic + struct.pack("<IQQ", version, tensors, kvs)


def _str(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _tensor(name, dims, type_id, offset):
    return _str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", type_id, offset)


def _write(tmp_path, blob):
    p = str(tmp_path / "bad.gguf")
    with open(p, "wb") as fh:
        fh.write(blob + b"\0" * 4096)
    return p


@pytest.mark.parametrize("blob,exc,text", [
    (_header(magic=b"GGML"), gguf.BadMagic, "bad magic"),
    (_header(version=1), gguf.UnsupportedVersion, "unsupported version 1"),
    (_header(version=4), gguf.UnsupportedVersion, "unsupported version 4"),
    (_header(tensors=65_537), gguf.OverBound, "tensor count 65537"),
    (_header(kvs=4097), gguf.OverBound, "metadata kv count 4097"),
    (_header(kvs=1) + struct.pack("<Q", (1 << 20) + 1), gguf.OverBound, "metadata key"),
    (_header(kvs=1) + _str("k") + struct.pack("<IB", 7, 2), gguf.BadValue, "bool byte 2"),
    (_header(kvs=1) + _str("k") + struct.pack("<I", 13), gguf.BadValue, "unknown value type 13"),
    (_header(kvs=1) + _str("k") + struct.pack("<IIQ", 9, 9, 1) + struct.pack("<IQ", 9, 1) + struct.pack("<IQ", 4, 0),
     gguf.BadValue, "nested deeper than 2"),
    (_header(kvs=1) + _str("k") + struct.pack("<IIQ", 9, 4, (1 << 22) + 1), gguf.OverBound, "metadata array"),
    (_header(kvs=1) + _str("general.alignment") + struct.pack("<II", 4, 24), gguf.BadValue, "24 is not a power of two"),
    (_header(kvs=1) + _str("general.alignment") + struct.pack("<II", 4, 0), gguf.BadValue, "0 is not a power of two"),
    (_header(tensors=1) + _tensor("t", [], 0, 0), gguf.BadTensor, "0 dims"),
    (_header(tensors=1) + _tensor("t", [2, 2, 2, 2, 2], 0, 0), gguf.BadTensor, "5 dims"),
    (_header(tensors=1) + _tensor("t", [32], 99, 0), gguf.BadTensor, "unknown ggml type id 99"),
    (_header(tensors=1) + _tensor("t", [32], 0, 16), gguf.BadTensor, "offset 16 not 32-aligned"),
    (_header(tensors=1) + _tensor("t", [255], 12, 0), gguf.BadTensor, "255 elements is not whole Q4_K blocks"),
    (_header(tensors=1) + _tensor("t", [0], 0, 0), gguf.BadTensor, "0 elements"),
    (_header(tensors=2) + _tensor("t", [32], 0, 0) + _tensor("t", [32], 0, 128), gguf.BadTensor, "duplicate tensor name 't'"),
    (_header(tensors=2) + _tensor("a", [64], 0, 0) + _tensor("b", [32], 0, 128), gguf.BadTensor, "overlaps 'a'"),
])
def test_refusals(tmp_path, blob, exc, text):
    with pytest.raises(exc, match=text):
        gguf.GgufFile.open(_write(tmp_path, blob))


def test_truncated_and_arrays(tmp_path):
    p = str(tmp_path / "t.gguf")
    with open(p, "wb") as fh:
        fh.write(_header(kvs=1) + _str("k"))
    with pytest.raises(gguf.GgufError, match="unexpected end of file"):
        gguf.GgufFile.open(p)
    # two levels of arrays are allowed; every scalar type round-trips
    blob = (_header(kvs=3, version=2) + _str("nest") + struct.pack("<IIQ", 9, 9, 1) + struct.pack("<IQ", 5, 2) + struct.pack("<ii", -1, 7)
            + _str("f64") + struct.pack("<Id", 12, 2.5) + _str("u8") + struct.pack("<IB", 0, 200))
    f = gguf.GgufFile.open(_write(tmp_path, blob))
    assert f.version == 2 and f.get("nest") == [[-1, 7]] and f.get("f64") == 2.5 and f.get("u8") == 200


@pytest.mark.gpu
def test_layer_from_gguf_equals_direct_upload(tmp_path):
    """`ffn_*_exps` Q4_K bytes go from the file to the device verbatim: the layer built from the
    file gives the bits of the layer built from the same arrays in memory."""
    from mummu_b200 import _lib as L, moe
    p = str(tmp_path / "m.gguf")
    truth = synthetic_file(p)
    f = gguf.GgufFile.open(p)
    x = synth.normal(5, (9, 256), 1.0).astype(np.float16)
    for l, (router, banks) in truth.items():
        from_file, shp = gguf.load_moe_layer(f, l)
        direct = moe.SparseMoeConfig(256, 256, 4, 2).init(act_dtype=L.F16, weight_dtype=L.Q4_K)
        direct.set_router(router)
        direct.set_banks(banks["gate"], banks["up"], banks["down"])
        a = from_file.forward(x, shp.num_experts_per_tok, shp.norm_topk_prob)
        b = direct.forward(x, 2, False)
        assert np.array_equal(a, b)
        assert np.array_equal(from_file.dequant_bank(L.BANK_DOWN, 3), direct.dequant_bank(L.BANK_DOWN, 3))
        from_file.close()
        direct.close()


def test_loader_refuses_what_the_bank_cannot_take(tmp_path):
    """Shape and type checks of `load_moe_layer` happen before anything touches a device."""
    H, I, E = 256, 256, 4
    p = str(tmp_path / "m.gguf")
    z = lambda n: np.zeros(n, np.uint8)
    q = E * I * H // 256 * 144
    base = [("blk.0.ffn_gate_inp.weight", [H, E], "F32", np.zeros((E, H), np.float32)),
            ("blk.0.ffn_gate_exps.weight", [H, I, E], "Q4_K", z(q)),
            ("blk.0.ffn_up_exps.weight", [H, I, E], "Q4_K", z(q)),
            ("blk.0.ffn_down_exps.weight", [I, H, E], "Q4_K", z(q))]
    # a bank stored as Q3_K: a real type, but not one this path computes from
    t = list(base)
    t[3] = ("blk.0.ffn_down_exps.weight", [I, H, E], "Q3_K", z(E * I * H // 256 * 110))
    gguf.write_gguf(p, META, t)
    with pytest.raises(NotImplementedError, match="Q3_K"):
        gguf.load_moe_layer(gguf.GgufFile.open(p), 0)
    # mixed bank types
    t = list(base)
    t[2] = ("blk.0.ffn_up_exps.weight", [H, I, E], "F16", np.zeros(E * I * H, np.float16))
    gguf.write_gguf(p, META, t)
    with pytest.raises(NotImplementedError, match="mixes bank types"):
        gguf.load_moe_layer(gguf.GgufFile.open(p), 0)
    # wrong dims and a missing tensor
    t = list(base)
    t[1] = ("blk.0.ffn_gate_exps.weight", [I, H, E], "Q4_K", z(q))
    meta = dict(META)
    meta["olmoe.expert_feed_forward_length"] = 512
    gguf.write_gguf(p, meta, t)
    with pytest.raises(ValueError, match="do not match"):
        gguf.load_moe_layer(gguf.GgufFile.open(p), 0)
    gguf.write_gguf(p, META, base[:3])
    with pytest.raises(KeyError, match="ffn_down_exps"):
        gguf.load_moe_layer(gguf.GgufFile.open(p), 0)


# ---- cross-check with the independent `gguf` package (llama.cpp's gguf-py) ------------------------

def _gguf_py():
    return pytest.importorskip("gguf", reason="the gguf package is not installed")


def test_reads_a_file_written_by_the_gguf_package(tmp_path):
    """The reader against a writer it shares no code with: metadata of several types, an array, and
    F32 / F16 / Q4_K tensors placed by gguf-py's own alignment logic.  Q4_K bytes must come back
    verbatim and decode (oracle) to what gguf-py's own dequantizer gives."""
    g = _gguf_py()
    from oracle import oracle as O
    H, I, E = 256, 256, 4
    router, gate, up, down, _ = synth.moe_layer(H, I, E, 1, cfg_seed=77)
    gq = q4k.quantize(gate)                                   # uint8 [E, I, H/256*144]
    p = str(tmp_path / "pkg.gguf")
    w = g.GGUFWriter(p, "olmoe")
    w.add_uint32("olmoe.embedding_length", H)
    w.add_uint32("olmoe.expert_feed_forward_length", I)
    w.add_uint32("olmoe.expert_count", E)
    w.add_uint32("olmoe.expert_used_count", 2)
    w.add_uint32("olmoe.block_count", 1)
    w.add_bool("olmoe.expert_weights_norm", True)
    w.add_float32("olmoe.rope.freq_base", 10000.0)
    w.add_array("tokenizer.ggml.tokens", ["a", "bc", "def"])
    w.add_tensor("blk.0.ffn_gate_inp.weight", np.ascontiguousarray(router.T))
    w.add_tensor("blk.0.attn_norm.weight", np.linspace(0, 1, H, dtype=np.float16))
    w.add_tensor("blk.0.ffn_gate_exps.weight", gq.reshape(E, I, -1), raw_dtype=g.GGMLQuantizationType.Q4_K)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    f = gguf.GgufFile.open(p)
    assert f.architecture() == "olmoe" and f.version == 3
    assert f.get("olmoe.expert_count") == E and f.get("olmoe.expert_weights_norm") is True
    assert abs(f.get("olmoe.rope.freq_base") - 10000.0) < 1e-3
    assert f.get("tokenizer.ggml.tokens") == ["a", "bc", "def"]
    shape = gguf.olmoe_moe_shape(f)
    assert (shape.hidden_size, shape.expert_intermediate_size, shape.num_experts, shape.num_experts_per_tok,
            shape.norm_topk_prob, shape.num_hidden_layers) == (H, I, E, 2, True, 1)
    t = f.tensor("blk.0.ffn_gate_exps.weight")
    assert t.dtype == "Q4_K" and t.shape == (E, I, H) and t.offset % f.alignment == 0
    raw = f.tensor_bytes("blk.0.ffn_gate_exps.weight")
    assert np.array_equal(raw.reshape(-1), gq.reshape(-1))
    want = g.quants.dequantize(gq.reshape(E * I, -1), g.GGMLQuantizationType.Q4_K).reshape(E, I, H)
    got = O.dequant_q4_k(raw).reshape(E, I, H)
    assert np.array_equal(got.view(np.uint32), np.asarray(want, np.float32).view(np.uint32))
    assert np.array_equal(f.tensor_array("blk.0.ffn_gate_inp.weight"), np.ascontiguousarray(router.T))
    assert f.tensor("blk.0.attn_norm.weight").dtype == "F16"
    f.close()


def test_the_gguf_package_reads_a_file_written_here(tmp_path):
    """The other direction: the writer used by the other tests produces files gguf-py's reader
    accepts, with the same keys, tensor types, shapes and bytes."""
    g = _gguf_py()
    p = str(tmp_path / "ours.gguf")
    truth = synthetic_file(p, alignment=64, layers=1)
    r = g.GGUFReader(p)
    assert r.alignment == 64
    arch = r.fields["general.architecture"]
    assert bytes(arch.parts[arch.data[0]]).decode() == "olmoe"
    assert int(r.fields["olmoe.expert_count"].parts[-1][0]) == 4
    by_name = {t.name: t for t in r.tensors}
    gate = by_name["blk.0.ffn_gate_exps.weight"]
    assert gate.tensor_type == g.GGMLQuantizationType.Q4_K
    assert list(gate.shape) == [256, 256, 4]                      # ggml order, innermost first
    assert np.array_equal(np.asarray(gate.data).reshape(-1), truth[0][1]["gate"].reshape(-1))
    inp = by_name["blk.0.ffn_gate_inp.weight"]
    assert inp.tensor_type == g.GGMLQuantizationType.F32
    assert np.array_equal(np.asarray(inp.data).reshape(4, 256), np.ascontiguousarray(truth[0][0].T))
