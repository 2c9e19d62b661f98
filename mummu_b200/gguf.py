"""GGUF container reader (and a small writer) for the expert-bank path.

What the reference's reader does for this path (crates/mummu/src/gguf.rs:1124-1376: header, typed
metadata, tensor table, alignment; :298-384: the ggml type table; crates/mummu/src/models/olmoe.rs
:116-179 config keys, :319-349 tensor names), with the same limits and the same refusals, so that
the `ffn_{gate,up,down}_exps` tensors of an OLMoE file reach the device **verbatim**: a Q4_K bank is
handed to `SparseMoe.set_bank` as the bytes in the file (the reference dequantises them to f32
first).  Nothing here touches a GPU; tensors come back as numpy views of a memory map.

File layout (little endian): magic "GGUF", u32 version (2 or 3), u64 tensor count, u64 key-value
count, the key-values (string key, u32 type id, value), the tensor table (string name, u32 n_dims,
u64 dims[n_dims] innermost first, u32 ggml type id, u64 offset relative to the data section), then
padding to `general.alignment` (default 32) and the tensor data.
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

MAGIC = b"GGUF"
SUPPORTED_VERSIONS = (2, 3)
DEFAULT_ALIGNMENT = 32
MAX_KVS = 4096
MAX_TENSORS = 65_536
MAX_STRING_BYTES = 1 << 20
MAX_ARRAY_LEN = 1 << 22
MAX_DIMS = 4

# ggml type id -> (name, elements per block, bytes per block)   (gguf.rs:298-384)
GGML_TYPES: Dict[int, Tuple[str, int, int]] = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2_K", 256, 84),
    11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210),
    15: ("Q8_K", 256, 292), 17: ("IQ2_XS", 256, 74), 18: ("IQ3_XXS", 256, 98), 20: ("IQ4_NL", 32, 18),
    21: ("IQ3_S", 256, 110), 22: ("IQ2_S", 256, 82), 23: ("IQ4_XS", 256, 136), 30: ("BF16", 1, 2),
    41: ("Q1_0", 128, 18), 42: ("Q2_0", 64, 18), 142: ("PQ2_0", 128, 34), 143: ("PTQ1_0", 128, 28),
}
TYPE_ID = {name: tid for tid, (name, _, _) in GGML_TYPES.items()}


class GgufError(Exception):
    """Base of every refusal; the message starts with 'gguf <path>:' like the reference's."""


class BadMagic(GgufError):
    pass


class UnsupportedVersion(GgufError):
    pass


class OverBound(GgufError):
    pass


class BadValue(GgufError):
    pass


class BadTensor(GgufError):
    pass


@dataclass
class TensorInfo:
    """One entry of the tensor table.  `dims` are ggml's (innermost first); `offset` is relative to
    the data section."""
    name: str
    dims: List[int]
    type_id: int
    offset: int

    @property
    def dtype(self) -> str:
        return GGML_TYPES[self.type_id][0]

    @property
    def elements(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    @property
    def byte_len(self) -> int:
        _, block, nbytes = GGML_TYPES[self.type_id]
        return self.elements // block * nbytes

    @property
    def shape(self) -> Tuple[int, ...]:
        """Row-major shape (outermost first) = ggml dims reversed."""
        return tuple(reversed(self.dims))


class _Reader:
    def __init__(self, buf, path: str):
        self.buf, self.path, self.pos = buf, path, 0

    def take(self, n: int) -> bytes:
        if self.pos + n > len(self.buf):
            raise GgufError(f"gguf {self.path}: unexpected end of file at byte {len(self.buf)}")
        out = self.buf[self.pos:self.pos + n]
        self.pos += n
        return out

    def num(self, fmt: str):
        return struct.unpack("<" + fmt, self.take(struct.calcsize("<" + fmt)))[0]

    def string(self, what: str) -> str:
        n = self.num("Q")
        if n > MAX_STRING_BYTES:
            raise OverBound(f"gguf {self.path}: {what} count {n} exceeds bound {MAX_STRING_BYTES}")
        raw = bytes(self.take(n))
        try:
            return raw.decode("utf-8")
        except UnicodeDecodeError as exc:
            raise BadValue(f"gguf {self.path}: {what}: invalid UTF-8: {exc}") from None

    _SCALARS = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 10: "Q", 11: "q", 12: "d"}

    def value(self, key: str, type_id: int, depth: int):
        if type_id in self._SCALARS:
            return self.num(self._SCALARS[type_id])
        if type_id == 7:
            b = self.num("B")
            if b > 1:
                raise BadValue(f"gguf {self.path}: key '{key}': bool byte {b}")
            return bool(b)
        if type_id == 8:
            return self.string("metadata string")
        if type_id == 9:
            if depth >= 2:
                raise BadValue(f"gguf {self.path}: key '{key}': arrays nested deeper than 2")
            elem_type = self.num("I")
            n = self.num("Q")
            if n > MAX_ARRAY_LEN:
                raise OverBound(f"gguf {self.path}: metadata array count {n} exceeds bound {MAX_ARRAY_LEN}")
            return [self.value(key, elem_type, depth + 1) for _ in range(n)]
        raise BadValue(f"gguf {self.path}: key '{key}': unknown value type {type_id}")


@dataclass
class GgufFile:
    path: str
    version: int
    metadata: List[Tuple[str, Any]]
    tensors: List[TensorInfo]
    alignment: int
    data_offset: int
    _map: Any = field(default=None, repr=False)

    # -- construction ------------------------------------------------------------------------
    @classmethod
    def open(cls, path: str) -> "GgufFile":
        path = os.fspath(path)
        with open(path, "rb") as fh:
            size = os.fstat(fh.fileno()).st_size
            if size == 0:
                raise GgufError(f"gguf {path}: unexpected end of file at byte 0")
            mm = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        r = _Reader(memoryview(mm), path)
        magic = bytes(r.take(4))
        if magic != MAGIC:
            raise BadMagic(f"gguf {path}: bad magic {magic!r}")
        version = r.num("I")
        if version not in SUPPORTED_VERSIONS:
            raise UnsupportedVersion(f"gguf {path}: unsupported version {version} (supported: {list(SUPPORTED_VERSIONS)})")
        tensor_count, kv_count = r.num("Q"), r.num("Q")
        for what, count, bound in (("tensor", tensor_count, MAX_TENSORS), ("metadata kv", kv_count, MAX_KVS)):
            if count > bound:
                raise OverBound(f"gguf {path}: {what} count {count} exceeds bound {bound}")
        metadata = []
        for _ in range(kv_count):
            key = r.string("metadata key")
            metadata.append((key, r.value(key, r.num("I"), 0)))
        alignment = DEFAULT_ALIGNMENT
        for k, v in metadata:
            if k == "general.alignment" and isinstance(v, int) and not isinstance(v, bool) and v >= 0:
                alignment = v
                break
        if alignment == 0 or alignment & (alignment - 1):
            raise BadValue(f"gguf {path}: key 'general.alignment': {alignment} is not a power of two")
        tensors = cls._tensor_table(r, tensor_count, alignment, path)
        data_offset = -(-r.pos // alignment) * alignment
        return cls(path, version, metadata, tensors, alignment, data_offset, mm)

    @staticmethod
    def _tensor_table(r: _Reader, count: int, alignment: int, path: str) -> List[TensorInfo]:
        tensors: List[TensorInfo] = []
        names = set()
        for index in range(count):
            def bad(reason: str) -> BadTensor:
                return BadTensor(f"gguf {path}: tensor {index}: {reason}")
            name = r.string("tensor name")
            n_dims = r.num("I")
            if n_dims == 0 or n_dims > MAX_DIMS:
                raise bad(f"{n_dims} dims (1..={MAX_DIMS})")
            dims = [r.num("Q") for _ in range(n_dims)]
            type_id = r.num("I")
            if type_id not in GGML_TYPES:
                raise bad(f"unknown ggml type id {type_id}")
            offset = r.num("Q")
            if offset % alignment:
                raise bad(f"offset {offset} not {alignment}-aligned")
            elements = 1
            for d in dims:
                elements *= d
            tname, block, _ = GGML_TYPES[type_id]
            if elements == 0 or elements % block:
                raise bad(f"{elements} elements is not whole {tname} blocks")
            if name in names:
                raise bad(f"duplicate tensor name '{name}'")
            names.add(name)
            tensors.append(TensorInfo(name, dims, type_id, offset))
        # payloads must not overlap (a table whose dtypes are not the file's real packing)
        order = sorted(range(len(tensors)), key=lambda i: tensors[i].offset)
        for ia, ib in zip(order, order[1:]):
            a, b = tensors[ia], tensors[ib]
            end = a.offset + a.byte_len
            if end > b.offset:
                raise BadTensor(f"gguf {path}: tensor {ib}: '{b.name}' at offset {b.offset} overlaps '{a.name}' "
                                f"({a.dtype}, {a.byte_len} bytes ending at {end})")
        return tensors

    # -- access --------------------------------------------------------------------------------
    def get(self, key: str, default=None):
        for k, v in self.metadata:
            if k == key:
                return v
        return default

    def architecture(self) -> Optional[str]:
        v = self.get("general.architecture")
        return v if isinstance(v, str) else None

    def tensor(self, name: str) -> Optional[TensorInfo]:
        for t in self.tensors:
            if t.name == name:
                return t
        return None

    def tensor_bytes(self, name: str) -> np.ndarray:
        """The tensor's bytes exactly as stored (uint8 view of the memory map)."""
        t = self.tensor(name)
        if t is None:
            raise KeyError(f"gguf {self.path}: no tensor '{name}'")
        start = self.data_offset + t.offset
        if start + t.byte_len > len(self._map):
            raise BadTensor(f"gguf {self.path}: '{name}' ({t.byte_len} bytes at {start}) runs past the end of the file")
        return np.frombuffer(self._map, dtype=np.uint8, count=t.byte_len, offset=start)

    def tensor_array(self, name: str) -> np.ndarray:
        """Float tensors (F32 / F16 / BF16-as-uint16) as row-major arrays of `shape`."""
        t = self.tensor(name)
        raw = self.tensor_bytes(name)
        if t.dtype == "F32":
            return raw.view(np.float32).reshape(t.shape)
        if t.dtype == "F16":
            return raw.view(np.float16).reshape(t.shape)
        if t.dtype == "BF16":
            return raw.view(np.uint16).reshape(t.shape)
        raise TypeError(f"gguf {self.path}: '{name}' is {t.dtype}, not a float tensor")

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:        # views still alive: the map goes with them
                pass
            self._map = None


# ---------------------------------------------------------------------------------------------
# writer (synthetic files for tests and for packing a model's expert banks)
# ---------------------------------------------------------------------------------------------
def _pack_value(v) -> Tuple[int, bytes]:
    if isinstance(v, bool):
        return 7, struct.pack("<B", int(v))
    if isinstance(v, int):
        return (4, struct.pack("<I", v)) if 0 <= v < 2 ** 32 else (11, struct.pack("<q", v))
    if isinstance(v, float):
        return 6, struct.pack("<f", v)
    if isinstance(v, str):
        raw = v.encode("utf-8")
        return 8, struct.pack("<Q", len(raw)) + raw
    if isinstance(v, (list, tuple)):
        if not v:
            return 9, struct.pack("<IQ", 4, 0)
        packed = [_pack_value(x) for x in v]
        elem_type = packed[0][0]
        if any(t != elem_type for t, _ in packed):
            raise TypeError("GGUF arrays hold one element type")
        return 9, struct.pack("<IQ", elem_type, len(v)) + b"".join(b for _, b in packed)
    raise TypeError(f"cannot store {type(v).__name__} in GGUF metadata")


def write_gguf(path: str, metadata: Dict[str, Any], tensors: List[Tuple[str, List[int], str, np.ndarray]],
               alignment: int = DEFAULT_ALIGNMENT, version: int = 3) -> None:
    """tensors: (name, ggml dims innermost first, type name, raw bytes or array).  Data are laid
    out in the order given, each padded to `alignment`."""
    meta = dict(metadata)
    if alignment != DEFAULT_ALIGNMENT:
        meta["general.alignment"] = alignment
    head = bytearray(MAGIC + struct.pack("<IQQ", version, len(tensors), len(meta)))
    for k, v in meta.items():
        kb = k.encode("utf-8")
        tid, payload = _pack_value(v)
        head += struct.pack("<Q", len(kb)) + kb + struct.pack("<I", tid) + payload
    blobs, offset = [], 0
    for name, dims, tname, data in tensors:
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        _, block, nbytes = GGML_TYPES[TYPE_ID[tname]]
        elements = int(np.prod(dims))
        if elements % block or raw.size != elements // block * nbytes:
            raise ValueError(f"{name}: {raw.size} bytes do not hold {elements} {tname} elements")
        nb = name.encode("utf-8")
        head += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(dims))
        head += b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", TYPE_ID[tname], offset)
        blobs.append((offset, raw))
        offset += -(-raw.size // alignment) * alignment
    data_offset = -(-len(head) // alignment) * alignment
    with open(path, "wb") as fh:
        fh.write(head)
        fh.write(b"\0" * (data_offset - len(head)))
        for off, raw in blobs:
            fh.seek(data_offset + off)
            fh.write(raw.tobytes())
        fh.truncate(data_offset + offset)


# ---------------------------------------------------------------------------------------------
# OLMoE: config keys and the expert-bank tensors of one layer
# ---------------------------------------------------------------------------------------------
@dataclass
class OlmoeMoeShape:
    hidden_size: int
    expert_intermediate_size: int
    num_experts: int
    num_experts_per_tok: int
    norm_topk_prob: bool
    num_hidden_layers: int


def olmoe_moe_shape(f: GgufFile) -> OlmoeMoeShape:
    """The MoE part of `OlmoeConfig::from_gguf` (models/olmoe.rs:116-179)."""
    arch = f.architecture() or "<missing>"
    if arch != "olmoe":
        raise ValueError(f"GGUF architecture '{arch}' is not olmoe")

    def need(key: str) -> int:
        v = f.get(key)
        if not isinstance(v, int) or isinstance(v, bool) or v < 0:
            raise ValueError(f"GGUF key '{key}' is missing or not an unsigned integer")
        return v

    try:
        inter = need("olmoe.expert_feed_forward_length")
    except ValueError:
        inter = need("olmoe.feed_forward_length")
    norm = f.get("olmoe.expert_weights_norm")
    return OlmoeMoeShape(need("olmoe.embedding_length"), inter, need("olmoe.expert_count"),
                         need("olmoe.expert_used_count"), norm if isinstance(norm, bool) else False,
                         need("olmoe.block_count"))


_BANK_CODES = {"Q4_K": "Q4_K", "Q8_0": "Q8_0", "Q5_K": "Q5_K", "Q6_K": "Q6_K", "F32": "F32", "F16": "F16", "BF16": "BF16"}


def load_moe_layer(f: GgufFile, layer: int, device: int = 0, act_dtype: Optional[int] = None, max_tokens: int = 0):
    """Build the `SparseMoe` of `blk.<layer>` from the file: router from `ffn_gate_inp.weight`
    (ggml dims [hidden, experts] = rows per expert, the GGUF order), banks from
    `ffn_{gate,up,down}_exps.weight` (ggml dims [in, out, experts] = row-major [E, out, in], the
    `MoeExperts` layout, models/olmoe.rs:339-345) uploaded as stored."""
    from . import _lib as L, moe
    shp = olmoe_moe_shape(f)
    H, I, E = shp.hidden_size, shp.expert_intermediate_size, shp.num_experts
    pre = f"blk.{layer}."
    want = {"ffn_gate_exps.weight": [H, I, E], "ffn_up_exps.weight": [H, I, E], "ffn_down_exps.weight": [I, H, E]}
    kinds = set()
    for name, dims in want.items():
        t = f.tensor(pre + name)
        if t is None:
            raise KeyError(f"gguf {f.path}: no tensor '{pre + name}'")
        if t.dims != dims:
            raise ValueError(f"'{pre + name}' dims {t.dims} do not match {dims}")
        if t.dtype not in _BANK_CODES:
            raise NotImplementedError(f"'{pre + name}' is {t.dtype}: this path takes Q4_K, Q8_0, Q5_K, Q6_K, F32, F16 and BF16 banks")
        kinds.add(t.dtype)
    if len(kinds) != 1:
        raise NotImplementedError(f"layer {layer} mixes bank types {sorted(kinds)}")
    kind = kinds.pop()
    wcode = {"Q4_K": L.Q4_K, "Q8_0": L.Q8_0, "Q5_K": L.Q5_K, "Q6_K": L.Q6_K, "F32": L.F32, "F16": L.F16,
             "BF16": L.BF16}[kind]
    if act_dtype is None:
        act_dtype = {"F32": L.F32, "BF16": L.BF16}.get(kind, L.F16)
    rt = f.tensor(pre + "ffn_gate_inp.weight")
    if rt is None or rt.dims != [H, E] or rt.dtype not in ("F32", "F16"):
        raise ValueError(f"'{pre}ffn_gate_inp.weight' must be an F32 or F16 [hidden={H}, experts={E}] tensor")
    layer_moe = moe.SparseMoeConfig(H, I, E, shp.num_experts_per_tok).init(
        device=device, act_dtype=act_dtype, weight_dtype=wcode, max_tokens=max_tokens)
    router = np.asarray(f.tensor_array(pre + "ffn_gate_inp.weight"), dtype=np.float32)      # [E, H]
    layer_moe.set_router(np.ascontiguousarray(router.T))                                   # [H, E]
    banks = []
    for name in want:
        raw = f.tensor_bytes(pre + name)
        if kind in ("Q4_K", "Q8_0", "Q5_K", "Q6_K"):
            banks.append(raw)
        elif kind == "F32":
            banks.append(raw.view(np.float32).reshape(f.tensor(pre + name).shape))
        else:
            banks.append(raw.view(np.float16 if kind == "F16" else np.uint16).reshape(f.tensor(pre + name).shape))
    layer_moe.set_banks(*banks)
    return layer_moe, shp
