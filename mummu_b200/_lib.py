"""ctypes binding of libmummu_cuda.so — the C ABI declared in include/mummu_cuda.h.

There is no CPU fallback: if the shared library has not been built (python -m mummu_b200.build)
the import of this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libmummu_cuda.so")

OK, ERR_CONTRACT, ERR_DEVICE, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_NUMERIC = 0, 1, 2, 3, 4, 5
F32, F16, BF16, Q4_K = 0, 1, 2, 3
Q8_0, Q5_K, Q6_K = 4, 5, 6       # sibling GGUF block formats: generic bank only
BANK_GATE, BANK_UP, BANK_DOWN = 0, 1, 2
ROUTER_IN_OUT, ROUTER_OUT_IN = 0, 1


class MummuMoeConfig(C.Structure):
    _fields_ = [
        ("device", C.c_int32), ("hidden", C.c_int32), ("inter", C.c_int32),
        ("experts", C.c_int32), ("top_k", C.c_int32), ("act_dtype", C.c_int32),
        ("weight_dtype", C.c_int32), ("expert_first", C.c_int32),
        ("experts_local", C.c_int32), ("max_tokens", C.c_int32),
    ]


class MummuTrunkConfig(C.Structure):
    _fields_ = [
        ("device", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("layers", C.c_int32), ("vocab", C.c_int32), ("slots", C.c_int32),
        ("max_ctx", C.c_int32), ("rope_theta", C.c_float), ("rms_eps", C.c_float),
    ]


(TRUNK_EMBED, TRUNK_LM_HEAD, TRUNK_FINAL_NORM, TRUNK_IN_NORM, TRUNK_POST_NORM, TRUNK_Q, TRUNK_K, TRUNK_V, TRUNK_O,
 TRUNK_Q_NORM, TRUNK_K_NORM) = range(11)

# name -> (restype, argtypes); every symbol include/mummu_cuda.h declares
SYMBOLS = {
    "mummu_moe_create": (C.c_int32, [C.POINTER(MummuMoeConfig), C.POINTER(C.c_void_p)]),
    "mummu_moe_destroy": (C.c_int32, [C.c_void_p]),
    "mummu_moe_set_router": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "mummu_moe_set_bank": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_size_t, C.c_int32]),
    "mummu_moe_adopt_scratch": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "mummu_moe_forward": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                      C.c_int32, C.c_int32, C.c_void_p]),
    "mummu_moe_route": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                    C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "mummu_moe_route_grouped": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "mummu_moe_permute": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "mummu_moe_experts_grouped": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                              C.c_void_p, C.c_void_p]),
    "mummu_moe_experts_planned": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                              C.c_void_p, C.c_void_p]),
    "mummu_moe_combine": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "mummu_ep_alloc": (C.c_int32, [C.c_int32, C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p]),
    "mummu_ep_open": (C.c_int32, [C.c_int32, C.c_char_p, C.POINTER(C.c_void_p)]),
    "mummu_ep_close": (C.c_int32, [C.c_void_p]),
    "mummu_ep_free": (C.c_int32, [C.c_void_p]),
    "mummu_ep_sync_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "mummu_ep_reset": (C.c_int32, [C.c_int32, C.c_void_p, C.c_int32, C.c_int32]),
    "mummu_ep_gather_tokens": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                           C.c_int32, C.c_int32, C.c_void_p]),
    "mummu_ep_wait": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "mummu_ep_experts_gathered": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                              C.c_int32, C.c_int64, C.c_void_p]),
    "mummu_ep_place": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p]),
    "mummu_ep_post_counts": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.c_int32,
                                         C.c_void_p]),
    "mummu_ep_dispatch": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p),
                                      C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int32, C.c_int64,
                                      C.c_void_p, C.c_void_p, C.c_void_p]),
    "mummu_ep_experts": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int32, C.c_int32,
                                     C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p]),
    "mummu_ep_combine": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                     C.c_void_p]),
    "mummu_expert_run": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "mummu_expert_run_device": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "mummu_expert_gate_energy": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "mummu_expert_resident_bytes": (C.c_uint64, [C.c_void_p, C.c_int32]),
    "mummu_moe_get_config": (C.c_int32, [C.c_void_p, C.POINTER(MummuMoeConfig)]),
    "mummu_moe_dequant_bank": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "mummu_moe_take_hits": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "mummu_moe_sync": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "mummu_moe_set_profiling": (C.c_int32, [C.c_void_p, C.c_int32]),
    "mummu_moe_take_profile": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "mummu_moe_launch_count": (C.c_int64, [C.c_void_p]),
    "mummu_moe_set_switch": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_int32]),
    "mummu_q4k_quantize": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]),
    "mummu_q4k_dequantize": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]),
    "mummu_moe_route_noalloc": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32,
                                            C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                            C.c_void_p, C.c_int32, C.c_void_p]),
    "mummu_trunk_static_bytes": (C.c_uint64, [C.POINTER(MummuTrunkConfig)]),
    "mummu_trunk_create": (C.c_int32, [C.POINTER(MummuTrunkConfig), C.POINTER(C.c_void_p)]),
    "mummu_trunk_destroy": (C.c_int32, [C.c_void_p]),
    "mummu_trunk_set_weight": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_int32]),
    "mummu_trunk_embed": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "mummu_trunk_attention_step": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                               C.c_int32, C.c_void_p, C.c_void_p]),
    "mummu_trunk_head": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p,
                                     C.c_void_p]),
    "mummu_trunk_kv_write": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                         C.c_void_p, C.c_void_p]),
    "mummu_cuda_last_error": (C.c_char_p, []),
    "mummu_cuda_version": (C.c_char_p, []),
}

if not os.path.exists(SO_PATH):
    raise ImportError(
        f"{SO_PATH} is missing: build the CUDA library first (python -m mummu_b200.build). "
        "This package has no CPU fallback.")

lib = C.CDLL(SO_PATH)
for _name, (_res, _args) in SYMBOLS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return (lib.mummu_cuda_last_error() or b"").decode(errors="replace")
