"""Host-side mirror of the reference's expert-bank interface (crates/mummu/src/nn/moe.rs), over
the C ABI of libmummu_cuda.so.

Names, argument meaning and error behaviour follow the reference: `SparseMoeConfig.init`,
`SparseMoe.forward(x, top_k, norm_topk_prob)`, `SparseMoePerExpert.{forward, route, run_local}`,
`Routing`, `ExpertExec.run` (as `CudaExpert.run`), `ExpertPool.take_hits`.  Where the reference
panics on a contract violation this raises `MoeContractError` with the reference's message.
Inputs are numpy arrays (host path: copied in and out inside the call) or torch CUDA tensors
(device path: queued on the current torch stream, nothing is copied).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import numpy as np

from . import _lib as L

_NP_DTYPES = {np.dtype(np.float32): L.F32, np.dtype(np.float16): L.F16}


class MoeContractError(AssertionError):
    """The reference panics here (assert!/expect); message kept."""


class MoeDeviceError(RuntimeError):
    pass


class MoeNumericError(ValueError):
    """Non-finite router logit (the reference's host router returns Err, experts.rs:553-560)."""


def _check(rc: int) -> None:
    if rc == L.OK:
        return
    msg = L.last_error()
    if rc == L.ERR_CONTRACT:
        raise MoeContractError(msg)
    if rc == L.ERR_NUMERIC:
        raise MoeNumericError(msg)
    if rc == L.ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    if rc == L.ERR_TIMEOUT:
        raise TimeoutError(msg)
    raise MoeDeviceError(msg)


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


def _torch_dtype_code(t) -> int:
    import torch
    return {torch.float32: L.F32, torch.float16: L.F16, torch.bfloat16: L.BF16}[t.dtype]


def _torch_stream():
    """The current torch stream as a cudaStream_t.  torch's default stream has handle 0, which the
    C ABI reads as "the handle's own stream", so it is passed as cudaStreamLegacy (0x1)."""
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream or 1)


@dataclass
class Routing:
    """`Routing` of nn/moe.rs:333-337: per expert, the token rows it serves and their weights."""
    tokens: int
    per_expert: List[Tuple[List[int], List[float]]] = field(default_factory=list)


@dataclass
class SparseMoeConfig:
    """`SparseMoeConfig` of nn/moe.rs:42-50."""
    hidden_size: int
    expert_intermediate_size: int
    num_experts: int
    num_experts_per_tok: int

    def init(self, device: int = 0, act_dtype: int = L.F32, weight_dtype: Optional[int] = None,
             max_tokens: int = 0, expert_first: int = 0,
             experts_local: Optional[int] = None) -> "SparseMoe":
        """nn/moe.rs:61-99.  Weights are left undefined until set (the reference draws a uniform
        init that every loader overwrites)."""
        return SparseMoe(self, device, act_dtype, act_dtype if weight_dtype is None else weight_dtype,
                         max_tokens, expert_first, experts_local)


class SparseMoe:
    """Router + expert bank on one B200 — `SparseMoe` (nn/moe.rs:34-39, 102-177) and, through
    `route`/`run_local`, `SparseMoePerExpert` (nn/moe.rs:201-329)."""

    def __init__(self, cfg: SparseMoeConfig, device: int, act_dtype: int, weight_dtype: int,
                 max_tokens: int, expert_first: int, experts_local: Optional[int]):
        self.cfg = cfg
        self.device = device
        self.act_dtype = act_dtype
        self.weight_dtype = weight_dtype
        self._h = C.c_void_p()
        c = L.MummuMoeConfig(
            device=device, hidden=cfg.hidden_size, inter=cfg.expert_intermediate_size,
            experts=cfg.num_experts, top_k=cfg.num_experts_per_tok, act_dtype=act_dtype,
            weight_dtype=weight_dtype, expert_first=expert_first,
            experts_local=cfg.num_experts if experts_local is None else experts_local,
            max_tokens=max_tokens)
        self.experts_local = c.experts_local
        self.expert_first = expert_first
        _check(L.lib.mummu_moe_create(C.byref(c), C.byref(self._h)))

    # -- life cycle -------------------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "_h", None) and self._h.value:
            L.lib.mummu_moe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def adopt_scratch(self, donor: "SparseMoe") -> None:
        """Use `donor`'s per-call scratch (layers of one stack run one after another)."""
        _check(L.lib.mummu_moe_adopt_scratch(self._h, donor._h))

    # -- weights ----------------------------------------------------------------------------
    def set_router(self, weight, layout: int = L.ROUTER_IN_OUT, bias=None) -> None:
        """`gate: Linear` weight, [hidden, experts] (burn, nn/moe.rs:1642) or [experts, hidden]
        (GGUF ffn_gate_inp, models/olmoe.rs:338-339)."""
        w = np.ascontiguousarray(weight)
        if w.dtype not in _NP_DTYPES:
            w = w.astype(np.float32)
        assert w.size == self.cfg.hidden_size * self.cfg.num_experts, "router weight size"
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        _check(L.lib.mummu_moe_set_router(self._h, w.ctypes.data, _NP_DTYPES[w.dtype], layout,
                                          None if b is None else b.ctypes.data))

    def set_bank(self, which: int, data) -> None:
        """One of `MoeExperts::{gate, up, down}` (nn/moe.rs:22-30), [experts, out, in]; numpy
        (f32/f16, uint16 bit patterns for bf16, uint8 bytes of a block format) or a torch CUDA
        tensor."""
        if _is_torch(data):
            t = data.contiguous()
            _check(L.lib.mummu_moe_set_bank(self._h, which, t.data_ptr(),
                                            t.numel() * t.element_size(), 1))
            return
        a = np.ascontiguousarray(data)
        _check(L.lib.mummu_moe_set_bank(self._h, which, a.ctypes.data, a.nbytes, 0))

    def set_banks(self, gate, up, down) -> None:
        self.set_bank(L.BANK_GATE, gate)
        self.set_bank(L.BANK_UP, up)
        self.set_bank(L.BANK_DOWN, down)

    # -- the layer ----------------------------------------------------------------------------
    def forward(self, x, top_k: int, norm_topk_prob: bool, out=None):
        """[b, t, hidden] -> [b, t, hidden] (nn/moe.rs:116-177, 214-219).  `out`: optional host
        array for the result of a host-pointer call (e.g. pinned memory; same shape and dtype)."""
        shape = tuple(x.shape)
        h = shape[-1]
        if h != self.cfg.hidden_size:
            raise MoeContractError(
                f"MoE forward: input hidden {h} does not match expert hidden {self.cfg.hidden_size}")
        tokens = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
        if _is_torch(x):
            import torch
            assert x.is_cuda and _torch_dtype_code(x) == self.act_dtype
            xc = x.contiguous()
            y = torch.empty_like(xc)
            _check(L.lib.mummu_moe_forward(self._h, xc.data_ptr(), y.data_ptr(), tokens, top_k,
                                           int(bool(norm_topk_prob)), 1, _torch_stream()))
            return y.view(shape)
        xa = self._host_act(x)
        if out is None:
            y = np.empty_like(xa)
        else:
            y = out
            if y.dtype != xa.dtype or y.size != xa.size or not y.flags["C_CONTIGUOUS"]:
                raise MoeContractError("MoE forward: `out` must be a contiguous array of the input's dtype and size")
        _check(L.lib.mummu_moe_forward(self._h, xa.ctypes.data, y.ctypes.data, tokens, top_k,
                                       int(bool(norm_topk_prob)), 0, None))
        return y.reshape(shape)

    def _host_act(self, x) -> np.ndarray:
        want = {L.F32: np.float32, L.F16: np.float16, L.BF16: np.uint16}[self.act_dtype]
        a = np.ascontiguousarray(x)
        if self.act_dtype != L.BF16 and a.dtype != want:
            a = a.astype(want)
        assert a.dtype == want, "bf16 host activations are passed as uint16 bit patterns"
        return a

    def route_flat(self, xt, top_k: int, norm_topk_prob: bool):
        """ids [tokens, top_k] int32 and weights [tokens, top_k] f32 (descending probability)."""
        tokens = xt.shape[0]
        if _is_torch(xt):
            import torch
            xc = xt.contiguous()
            ids = torch.empty((tokens, top_k), dtype=torch.int32, device=xc.device)
            w = torch.empty((tokens, top_k), dtype=torch.float32, device=xc.device)
            _check(L.lib.mummu_moe_route(self._h, xc.data_ptr(), tokens, top_k,
                                         int(bool(norm_topk_prob)), ids.data_ptr(), w.data_ptr(), 1,
                                         _torch_stream()))
            return ids, w
        xa = self._host_act(xt)
        ids = np.empty((tokens, max(top_k, 0)), dtype=np.int32)
        w = np.empty((tokens, max(top_k, 0)), dtype=np.float32)
        _check(L.lib.mummu_moe_route(self._h, xa.ctypes.data, tokens, top_k,
                                     int(bool(norm_topk_prob)), ids.ctypes.data, w.ctypes.data, 0,
                                     None))
        return ids, w

    def route(self, xt, top_k: int, norm_topk_prob: bool) -> Routing:
        """`SparseMoePerExpert::route` (nn/moe.rs:247-290): the per-expert (rows, weights) lists,
        token-major."""
        ids, w = self.route_flat(xt, top_k, norm_topk_prob)
        if _is_torch(ids):
            ids, w = ids.cpu().numpy(), w.cpu().numpy()
        routed: List[Tuple[List[int], List[float]]] = [([], []) for _ in range(self.cfg.num_experts)]
        for token in range(ids.shape[0]):
            for slot in range(ids.shape[1]):
                e = int(ids[token, slot])
                routed[e][0].append(token)
                routed[e][1].append(float(w[token, slot]))
        return Routing(tokens=ids.shape[0], per_expert=routed)

    def run_local(self, xt: np.ndarray, routing: Routing) -> np.ndarray:
        """`SparseMoePerExpert::run_local` (nn/moe.rs:296-328): ascending expert id, gather rows,
        run the expert, scatter-add `y * scale` (two roundings)."""
        xt = np.ascontiguousarray(xt, dtype=np.float32)
        out = np.zeros_like(xt)
        for expert, (rows, weights) in enumerate(routing.per_expert):
            if not rows:
                continue
            y = CudaExpert(self, expert).run(xt[rows].reshape(-1), len(rows), xt.shape[1])
            y = y.reshape(len(rows), xt.shape[1])
            scaled = y * np.asarray(weights, dtype=np.float32)[:, None]
            np.add.at(out, rows, scaled)
        return out

    # -- taps -------------------------------------------------------------------------------
    def dequant_bank(self, which: int, expert: int) -> np.ndarray:
        out_dim = self.cfg.hidden_size if which == L.BANK_DOWN else self.cfg.expert_intermediate_size
        in_dim = self.cfg.expert_intermediate_size if which == L.BANK_DOWN else self.cfg.hidden_size
        out = np.empty((out_dim, in_dim), dtype=np.float32)
        _check(L.lib.mummu_moe_dequant_bank(self._h, which, expert, out.ctypes.data))
        return out

    def take_hits(self) -> np.ndarray:
        """`ExpertPool::take_hits` (nn/moe.rs:1527-1535) for this layer."""
        out = np.zeros(self.cfg.num_experts, dtype=np.uint64)
        _check(L.lib.mummu_moe_take_hits(self._h, out.ctypes.data))
        return out

    def sync(self) -> None:
        stream = None
        try:
            import torch
            if torch.cuda.is_available():
                stream = _torch_stream()
        except ImportError:
            pass
        _check(L.lib.mummu_moe_sync(self._h, stream))

    def set_profiling(self, enabled: bool) -> None:
        _check(L.lib.mummu_moe_set_profiling(self._h, int(enabled)))

    def take_profile(self) -> dict:
        buf = C.create_string_buffer(4096)
        _check(L.lib.mummu_moe_take_profile(self._h, buf, 4096))
        out = {}
        for item in buf.value.decode().split(";"):
            if "=" in item:
                name, rest = item.split("=")
                n, ms = rest.split(":")
                out[name] = (int(n), float(ms))
        return out

    def launch_count(self) -> int:
        return int(L.lib.mummu_moe_launch_count(self._h))

    def set_switch(self, name: str, value: int) -> None:
        """One kernel-variant switch of this layer (the handle read MUMMU_CUDA_<name> when it was
        created; the reference reads its MUMMU_* switches once too, nn/packed_gemv.rs:85-92)."""
        _check(L.lib.mummu_moe_set_switch(self._h, name.encode(), int(value)))

    # -- staged calls (device tensors), used by the expert-parallel layer -----------------------
    def route_grouped(self, xt, top_k: int, norm_topk_prob: bool):
        """`route_flat` + `permute` on device tensors; one launch for decode-sized calls.
        Returns (ids, w, counts, offsets, row_token, pos)."""
        import torch
        xc = xt.contiguous()
        tokens, E = xc.shape[0], self.cfg.num_experts
        i32 = dict(dtype=torch.int32, device=xc.device)
        ids = torch.empty((tokens, top_k), **i32)
        w = torch.empty((tokens, top_k), dtype=torch.float32, device=xc.device)
        counts, offsets = torch.empty(E, **i32), torch.empty(E + 1, **i32)
        row_token, pos = torch.empty(tokens * top_k, **i32), torch.empty(tokens * top_k, **i32)
        _check(L.lib.mummu_moe_route_grouped(self._h, xc.data_ptr(), tokens, top_k, int(bool(norm_topk_prob)),
                                             ids.data_ptr(), w.data_ptr(), counts.data_ptr(), offsets.data_ptr(),
                                             row_token.data_ptr(), pos.data_ptr(), _torch_stream()))
        return ids, w, counts, offsets, row_token, pos

    def permute(self, ids, counts=None, offsets=None, row_token=None, pos=None) -> None:
        tokens, top_k = ids.shape
        p = lambda t: None if t is None else t.data_ptr()
        _check(L.lib.mummu_moe_permute(self._h, ids.data_ptr(), tokens, top_k, p(counts), p(offsets),
                                       p(row_token), p(pos), _torch_stream()))

    def experts_grouped(self, xs, counts, ys) -> None:
        _check(L.lib.mummu_moe_experts_grouped(self._h, xs.data_ptr(), counts.data_ptr(),
                                               xs.shape[0], ys.data_ptr(), _torch_stream()))

    def experts_grouped_raw(self, xs_ptr: int, counts, rows: int, ys_ptr: int) -> None:
        _check(L.lib.mummu_moe_experts_grouped(self._h, xs_ptr, counts.data_ptr(), rows, ys_ptr,
                                               _torch_stream()))

    # stages of the expert-parallel layer (peer memory; see include/mummu_cuda.h)
    def ep_gather_tokens(self, x, sync_table, gx_table, rank: int, world: int) -> None:
        _check(L.lib.mummu_ep_gather_tokens(self._h, x.data_ptr(), x.shape[0], sync_table, gx_table, rank, world,
                                            _torch_stream()))

    def ep_wait(self, sync_table, rank: int, world: int, channel: int) -> None:
        _check(L.lib.mummu_ep_wait(self._h, sync_table, rank, world, channel, _torch_stream()))

    def ep_experts_gathered(self, sync_table, back_table, gx_ptr: int, row_token, counts, offsets, rank: int, world: int,
                            tokens_per_rank: int, top_k: int, back_rows: int) -> None:
        _check(L.lib.mummu_ep_experts_gathered(self._h, sync_table, back_table, gx_ptr, row_token.data_ptr(),
                                               counts.data_ptr(), offsets.data_ptr(), rank, world, tokens_per_rank, top_k,
                                               back_rows, _torch_stream()))

    def route_grouped_ptr(self, x_ptr: int, tokens: int, top_k: int, norm_topk_prob: bool, device):
        """`route_grouped` over activations given as a device address (a buffer the library allocated)."""
        import torch
        E = self.cfg.num_experts
        i32 = dict(dtype=torch.int32, device=device)
        ids = torch.empty((tokens, top_k), **i32)
        w = torch.empty((tokens, top_k), dtype=torch.float32, device=device)
        counts, offsets = torch.empty(E, **i32), torch.empty(E + 1, **i32)
        row_token, pos = torch.empty(tokens * top_k, **i32), torch.empty(tokens * top_k, **i32)
        _check(L.lib.mummu_moe_route_grouped(self._h, x_ptr, tokens, top_k, int(bool(norm_topk_prob)),
                                             ids.data_ptr(), w.data_ptr(), counts.data_ptr(), offsets.data_ptr(),
                                             row_token.data_ptr(), pos.data_ptr(), _torch_stream()))
        return ids, w, counts, offsets, row_token, pos

    def ep_place(self, ids, table, experts_real: int, ids_out) -> None:
        _check(L.lib.mummu_ep_place(self._h, ids.data_ptr(), table.data_ptr(), experts_real, ids.numel(),
                                    ids_out.data_ptr(), _torch_stream()))

    def ep_post_counts(self, counts, sync_table, rank: int, world: int) -> None:
        _check(L.lib.mummu_ep_post_counts(self._h, counts.data_ptr(), sync_table, rank, world, _torch_stream()))

    def ep_dispatch(self, x, row_token, offsets, sync_table, recv_table, rank: int, world: int, cap_rows: int,
                    dst_base, local_counts) -> None:
        _check(L.lib.mummu_ep_dispatch(self._h, x.data_ptr(), row_token.data_ptr(), offsets.data_ptr(),
                                       sync_table, recv_table, rank, world, row_token.numel(), cap_rows,
                                       dst_base.data_ptr(), local_counts.data_ptr(), _torch_stream()))

    def ep_experts(self, sync_table, back_table, rank: int, world: int, recv_ptr: int, local_counts, rows_cap: int,
                   ys_ptr: int, back_rows: int) -> None:
        _check(L.lib.mummu_ep_experts(self._h, sync_table, back_table, rank, world, recv_ptr, local_counts.data_ptr(),
                                      rows_cap, ys_ptr, back_rows, _torch_stream()))

    def ep_combine(self, sync_table, back_ptr: int, ids, w, pos, rank: int, world: int, out, order_ids=None) -> None:
        tokens, top_k = ids.shape
        _check(L.lib.mummu_ep_combine(self._h, sync_table, back_ptr, ids.data_ptr(),
                                      None if order_ids is None else order_ids.data_ptr(), w.data_ptr(), pos.data_ptr(),
                                      rank, world, tokens, top_k, out.data_ptr(), _torch_stream()))

    def combine(self, ys, ids, w, pos, out) -> None:
        tokens, top_k = ids.shape
        _check(L.lib.mummu_moe_combine(self._h, ys.data_ptr(), ids.data_ptr(), w.data_ptr(),
                                       pos.data_ptr(), tokens, top_k, out.data_ptr(),
                                       _torch_stream()))


SparseMoePerExpert = SparseMoe


@dataclass
class Tier:
    """`tier::Tier` as far as this path uses it (nn/moe.rs:349-350): where an expert is resident and
    at which stored precision."""
    device: int
    precision: int          # a weight dtype code of this library (F32 .. Q6_K)


class CudaExpert:
    """`ExpertExec` (nn/moe.rs:348-419) for one expert of a bank on a B200: all ten methods.  The
    expert is pinned to its device, so `stage`/`evict` are the trait's no-op defaults and
    `is_staged` is always true; `disable_native` has nothing to switch off (there is no
    dequantise-first fallback here)."""

    def __init__(self, moe: SparseMoe, expert: int):
        self.moe = moe
        self.expert = expert

    def tier(self) -> Tier:
        c = L.MummuMoeConfig()
        _check(L.lib.mummu_moe_get_config(self.moe._h, C.byref(c)))
        return Tier(device=c.device, precision=c.weight_dtype)

    def resident_bytes(self) -> int:
        return int(L.lib.mummu_expert_resident_bytes(self.moe._h, self.expert))

    def run(self, x: np.ndarray, rows: int, hidden: int) -> np.ndarray:
        if hidden != self.moe.cfg.hidden_size:
            raise MoeContractError(f"expert input hidden {hidden} != {self.moe.cfg.hidden_size}")
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        if x.size != rows * hidden:
            raise MoeContractError(f"expert input holds {x.size} values, wants {rows} x {hidden}")
        y = np.empty(rows * hidden, dtype=np.float32)
        _check(L.lib.mummu_expert_run(self.moe._h, self.expert, x.ctypes.data, rows, y.ctypes.data))
        return y

    def run_tensor(self, x):
        """[rows, hidden] torch CUDA tensor of the layer's activation dtype -> the same, no host
        round trip (nn/moe.rs:399-412)."""
        import torch
        assert x.is_cuda and _torch_dtype_code(x) == self.moe.act_dtype and x.shape[1] == self.moe.cfg.hidden_size
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _check(L.lib.mummu_expert_run_device(self.moe._h, self.expert, xc.data_ptr(), xc.shape[0], y.data_ptr(),
                                             _torch_stream()))
        return y

    def run_tensor_resident(self, x):
        """The result stays on the expert's device and nothing waits (nn/moe.rs:358-367): here the
        same call, since `run_tensor` already returns without synchronising."""
        return self.run_tensor(x)

    def gate_energy(self, x: np.ndarray, rows: int, hidden: int) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        if hidden != self.moe.cfg.hidden_size or x.size != rows * hidden:
            raise MoeContractError(f"gate_energy input holds {x.size} values, wants {rows} x {self.moe.cfg.hidden_size}")
        out = np.empty(rows, dtype=np.float32)
        _check(L.lib.mummu_expert_gate_energy(self.moe._h, self.expert, x.ctypes.data, rows, out.ctypes.data))
        return out

    def disable_native(self) -> None:
        pass

    def stage(self, device=None) -> None:
        pass

    def evict(self) -> None:
        pass

    def is_staged(self) -> bool:
        return True


def q4k_quantize_device(src):
    """f32 torch CUDA tensor (size % 256 == 0) -> uint8 tensor of Q4_K bytes, on the device."""
    import torch
    assert src.is_cuda and src.dtype == torch.float32 and src.numel() % 256 == 0
    src = src.contiguous()
    nb = src.numel() // 256
    dst = torch.empty(nb * 144, dtype=torch.uint8, device=src.device)
    _check(L.lib.mummu_q4k_quantize(src.data_ptr(), dst.data_ptr(), nb, src.device.index,
                                    _torch_stream()))
    return dst


def q4k_dequantize_device(raw):
    import torch
    assert raw.is_cuda and raw.dtype == torch.uint8 and raw.numel() % 144 == 0
    nb = raw.numel() // 144
    dst = torch.empty(nb * 256, dtype=torch.float32, device=raw.device)
    _check(L.lib.mummu_q4k_dequantize(raw.contiguous().data_ptr(), dst.data_ptr(), nb,
                                      raw.device.index, _torch_stream()))
    return dst
