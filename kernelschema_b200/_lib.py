"""ctypes binding of libb200moe.so (the C ABI declared in include/b200moe.h).

The library is the product: if it is missing or fails to load this module raises, it never falls
back to another implementation.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200moe.so")

ABI_VERSION = 3
SF_ROW_MAJOR, SF_TILED = 0, 1


class Config(C.Structure):
    _fields_ = [("struct_size", C.c_int32), ("hidden", C.c_int32), ("intermediate", C.c_int32), ("num_experts", C.c_int32),
                ("top_k", C.c_int32), ("num_shared_experts", C.c_int32), ("max_tokens", C.c_int32), ("tile_n", C.c_int32),
                ("sm_margin", C.c_int32), ("graph_cache", C.c_int32), ("tma_gather", C.c_int32),
                ("reserved", C.c_int32 * 5)]


class Args(C.Structure):
    _fields_ = [("struct_size", C.c_int32), ("num_tokens", C.c_int32), ("topk_ids", C.c_void_p), ("topk_weights", C.c_void_p),
                ("hidden_states", C.c_void_p), ("hidden_states_scale", C.c_void_p), ("hidden_states_scale_layout", C.c_int32),
                ("activation_type", C.c_int32), ("gemm1_weights", C.c_void_p), ("gemm1_weights_scale", C.c_void_p),
                ("gemm2_weights", C.c_void_p), ("gemm2_weights_scale", C.c_void_p), ("gemm1_alpha", C.c_void_p),
                ("gemm1_beta", C.c_void_p), ("gemm1_clamp_limit", C.c_void_p), ("output1_scale_scalar", C.c_void_p),
                ("output1_scale_gate_scalar", C.c_void_p), ("output2_scale_scalar", C.c_void_p),
                ("local_expert_offset", C.c_int32), ("direct_rows", C.c_int32), ("output", C.c_void_p),
                ("output_stride", C.c_int64), ("hidden_states_stride", C.c_int64), ("hidden_states_scale_stride", C.c_int64),
                ("topk_stride", C.c_int64)]


EP_MAX_RANKS = 16
EP_CTRL_INTS = 4 * EP_MAX_RANKS
EP_FLAG_DISPATCH, EP_FLAG_RETURN = 2 * EP_MAX_RANKS, 3 * EP_MAX_RANKS


class EpPeers(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("recv", C.c_void_p * EP_MAX_RANKS), ("ctrl", C.c_void_p * EP_MAX_RANKS),
                ("ret", C.c_void_p * EP_MAX_RANKS)]


class StepArgs(C.Structure):
    _fields_ = [("struct_size", C.c_int32), ("num_tokens", C.c_int32), ("x", C.c_void_p), ("x_stride", C.c_int64),
                ("gate_weight", C.c_void_p), ("gate_bias", C.c_void_p), ("activation_global_scale", C.c_float),
                ("activation_type", C.c_int32), ("gemm1_weights", C.c_void_p), ("gemm1_weights_scale", C.c_void_p),
                ("gemm2_weights", C.c_void_p), ("gemm2_weights_scale", C.c_void_p), ("gemm1_alpha", C.c_void_p),
                ("gemm1_beta", C.c_void_p), ("gemm1_clamp_limit", C.c_void_p), ("output1_scale_scalar", C.c_void_p),
                ("output1_scale_gate_scalar", C.c_void_p), ("output2_scale_scalar", C.c_void_p), ("output", C.c_void_p),
                ("output_stride", C.c_int64)]


class Stats(C.Structure):
    _fields_ = [("runs", C.c_int64), ("graph_replays", C.c_int64), ("graph_captures", C.c_int64), ("graph_evictions", C.c_int64),
                ("eager_in_capture", C.c_int64), ("workspace_bytes", C.c_int64)]


class WorkspaceView(C.Structure):
    _fields_ = [("counts", C.c_void_p), ("seg_start", C.c_void_p), ("tile_expert", C.c_void_p), ("tile_row0", C.c_void_p),
                ("tile_rows", C.c_void_p), ("totals", C.c_void_p), ("row_of", C.c_void_p), ("tok_of_row", C.c_void_p),
                ("weight_of_row", C.c_void_p), ("a_q", C.c_void_p), ("a_sf", C.c_void_p), ("act_q", C.c_void_p),
                ("act_sf", C.c_void_p), ("rout", C.c_void_p), ("row_capacity", C.c_int64), ("tile_capacity", C.c_int64),
                ("pair_expert", C.c_void_p), ("pair_row0", C.c_void_p), ("pair_rows", C.c_void_p), ("step_ids", C.c_void_p),
                ("step_weights", C.c_void_p)]


#: every exported symbol with (restype, argtypes); the CPU test checks the library exports exactly these
SIGNATURES = {
    "b200moe_abi_version": (C.c_int, []),
    "b200moe_last_error": (C.c_char_p, []),
    "b200moe_quantize_nvfp4": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_float, C.c_void_p, C.c_void_p,
                                         C.c_int32, C.c_void_p]),
    "b200moe_scales_to_tiles": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200moe_route_topk": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                     C.c_void_p]),
    "b200moe_router_logits": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200moe_gemm_nvfp4": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_int64,
                                     C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200moe_create": (C.c_int, [C.POINTER(Config), C.POINTER(C.c_void_p)]),
    "b200moe_destroy": (C.c_int, [C.c_void_p]),
    "b200moe_workspace_bytes": (C.c_int64, [C.POINTER(Config)]),
    "b200moe_workspace": (C.c_int, [C.c_void_p, C.POINTER(WorkspaceView)]),
    "b200moe_route_map": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "b200moe_gemm_bf16_nvfp4_workspace_bytes": (C.c_int64, [C.c_int64, C.c_int64, C.c_int64]),
    "b200moe_gemm_bf16_nvfp4": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                          C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200moe_ep_visits": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200moe_ep_pack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_int64, C.c_void_p, C.c_void_p]),
    "b200moe_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_int64,
                                  C.c_void_p]),
    "b200moe_route_map_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32]
                                  + [C.c_void_p] * 9 + [C.c_int64, C.c_void_p]),
    "b200moe_ep_shared_alloc": (C.c_int, [C.c_int64, C.POINTER(C.c_void_p), C.c_void_p]),
    "b200moe_ep_shared_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "b200moe_ep_shared_close": (C.c_int, [C.c_void_p]),
    "b200moe_ep_shared_free": (C.c_int, [C.c_void_p]),
    "b200moe_ep_dispatch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                      C.c_int32, C.c_int64, C.POINTER(EpPeers), C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200moe_ep_wait": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "b200moe_ep_post": (C.c_int, [C.POINTER(EpPeers), C.c_int32, C.c_int32, C.c_void_p]),
    "b200moe_run_ep": (C.c_int, [C.c_void_p, C.POINTER(Args), C.POINTER(EpPeers), C.c_void_p, C.c_int32, C.c_void_p]),
    "b200moe_run": (C.c_int, [C.c_void_p, C.POINTER(Args), C.c_void_p]),
    "b200moe_run_profiled": (C.c_int, [C.c_void_p, C.POINTER(Args), C.c_void_p, C.POINTER(C.c_float)]),
    "b200moe_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]),
    "b200moe_get_stats": (C.c_int, [C.c_void_p, C.POINTER(Stats)]),
    "b200moe_step": (C.c_int, [C.c_void_p, C.POINTER(StepArgs), C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (built by ``python -m kernelschema_b200.build``); raise if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m kernelschema_b200.build` (needs nvcc). "
                               "There is no fallback implementation.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        if lib.b200moe_abi_version() != ABI_VERSION:
            raise RuntimeError("libb200moe.so ABI version mismatch; rebuild it")
        _lib = lib
    return _lib


def check(code: int, what: str) -> None:
    """Mirror of the reference host's error behaviour (candidate/solution.py:1560-1562): raise on non-zero."""
    if code != 0:
        msg = load().b200moe_last_error().decode(errors="replace")
        if 700 <= code < 800:
            raise ValueError(f"{what}: {msg} (code {code})")
        raise RuntimeError(f"{what} failed: {msg} (code {code})")
