"""ctypes binding of libdmoq.so (the C ABI declared in include/dmoq.h).

The library is the only compute path: if it is missing or fails to load the
import raises, there is no fallback.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# DMOQ_LIB points at another build of the same library (tuning builds); default: the in-tree one
LIB_PATH = os.environ.get("DMOQ_LIB") or os.path.join(HERE, "libdmoq.so")

MAX_POOLS = 8
A16, A8, FP8, FP4 = 0, 1, 2, 3
EPI_SILU, EPI_WEIGHTED, EPI_PLAIN = 0, 1, 2
TILE_M = 128

MODE_NAMES = {"wxa16": A16, "wxa8": A8, "wxfp8": FP8, "wxfp4": FP4}


class Pool(C.Structure):
    """Mirror of dmoq_pool_t."""
    _fields_ = [
        ("bit", C.c_int32), ("mode", C.c_int32), ("n_members", C.c_int32), ("inter", C.c_int32),
        ("hoisted", C.c_int32), ("act_cap_rows", C.c_int32),
        ("gu_idx", C.c_void_p), ("gu_norm", C.c_void_p), ("dn_idx", C.c_void_p), ("dn_norm", C.c_void_p),
        ("gu_lut", C.c_void_p), ("dn_lut", C.c_void_p),
        ("identity_lut", C.c_int32), ("gu_e0", C.c_int32), ("dn_e0", C.c_int32),
        ("gu_act_scale", C.c_float), ("dn_act_scale", C.c_float),
        ("gu_rot", C.c_void_p), ("dn_rot", C.c_void_p),
        ("act_codes", C.c_void_p), ("act_scales", C.c_void_p),
        ("gu_idx_wide", C.c_void_p), ("dn_idx_wide", C.c_void_p),
        ("gu_img", C.c_void_p), ("dn_img", C.c_void_p), ("gu_norm_img", C.c_void_p), ("dn_norm_img", C.c_void_p),
    ]


class Route(C.Structure):
    """Mirror of dmoq_route_t."""
    _fields_ = [
        ("T", C.c_int32), ("top_k", C.c_int32), ("E", C.c_int32), ("has_shared", C.c_int32),
        ("tile_m", C.c_int32), ("n_pools", C.c_int32),
        ("expert_pool", C.c_void_p), ("expert_rank", C.c_void_p), ("expert_rows", C.c_void_p),
        ("sorted_tokens", C.c_void_p), ("sorted_weights", C.c_void_p), ("row_of", C.c_void_p),
        ("a_row", C.c_void_p), ("pool_rows", C.c_void_p), ("pool_src", C.c_void_p),
        ("pool_src_base", C.c_void_p), ("tiles", C.c_void_p), ("n_tiles", C.c_void_p),
        ("tile_cap", C.c_int32), ("pool_hoisted", C.c_void_p),
    ]


EXPORTS = {
    "dmoq_version": (C.c_int, []),
    "dmoq_strerror": (C.c_char_p, [C.c_int]),
    "dmoq_route_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "dmoq_route_build": (C.c_int, [C.POINTER(Route), C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_size_t, C.c_void_p]),
    "dmoq_router_topk": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                   C.c_void_p]),
    "dmoq_router_topk_gate": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p]),
    "dmoq_route_static_max_bytes": (C.c_size_t, []),
    "dmoq_route_build_static": (C.c_int, [C.POINTER(Route), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "dmoq_rotate_quant": (C.c_int, [C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_int32, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p,
                                    C.c_void_p]),
    "dmoq_rotate_quant_down": (C.c_int, [C.POINTER(Route), C.POINTER(Pool), C.c_int32, C.c_void_p, C.c_int32,
                                         C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "dmoq_grouped_gemm": (C.c_int, [C.POINTER(Route), C.POINTER(Pool), C.c_int32, C.c_int32, C.c_int32,
                                    C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                                    C.c_void_p, C.c_void_p]),
    "dmoq_grouped_gemm_pools": (C.c_int, [C.POINTER(Route), C.POINTER(Pool), C.POINTER(C.c_int32), C.c_int32, C.c_int32,
                                          C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                                          C.c_void_p]),
    "dmoq_tc_status": (C.c_int, [C.POINTER(C.c_int32)]),
    "dmoq_combine": (C.c_int, [C.POINTER(Route), C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "dmoq_combine_weighted": (C.c_int, [C.POINTER(Route), C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "dmoq_convert_group_first": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "dmoq_widen_indices": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
    "dmoq_moe_decode_rotate": (C.c_int, [C.POINTER(Route), C.POINTER(Pool), C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                         C.c_void_p]),
    "dmoq_moe_decode_rotate_down": (C.c_int, [C.POINTER(Route), C.POINTER(Pool), C.c_int32, C.c_void_p, C.c_int32,
                                              C.c_void_p, C.c_int32, C.c_void_p]),
    "dmoq_moe_decode_gateup": (C.c_int, [C.POINTER(Route), C.POINTER(Pool), C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                         C.c_void_p]),
    "dmoq_moe_decode_down": (C.c_int, [C.POINTER(Route), C.POINTER(Pool), C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                       C.c_void_p, C.c_void_p]),
    "dmoq_quantize_packed": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_void_p]),
    "dmoq_gather_rows": (C.c_int, [C.POINTER(Route), C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                   C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "dmoq_weight_image_bytes": (C.c_size_t, [C.POINTER(Pool), C.c_int32, C.c_int32]),
    "dmoq_expand_weights": (C.c_int, [C.POINTER(Pool), C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


class DmoqError(RuntimeError):
    pass


def load():
    """Load libdmoq.so once and declare every prototype; raises if the library is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise DmoqError(
            f"{LIB_PATH} not found: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no CPU or eager fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().dmoq_strerror(code).decode()
        raise DmoqError(f"{what}: {msg} ({code})")


def ptr(t):
    """Device (or host) address of a torch tensor, or None."""
    return None if t is None else C.c_void_p(t.data_ptr())
