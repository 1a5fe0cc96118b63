"""ctypes binding of libbitsmoe_b200.so (the C ABI declared in include/bitsmoe_b200.h).

There is no fallback: if the shared library is missing, ``lib()`` raises and so does every
op built on it.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "_lib", "libbitsmoe_b200.so")

BM_OK = 0
BM_F16, BM_BF16, BM_F32 = 0, 1, 2
ROUND_NONE, ROUND_F16, ROUND_BF16 = 0, 1, 2
PATH_AUTO, PATH_GENERIC, PATH_DECODE, PATH_TENSOR = 0, 1, 2, 3
GATE, UP, DOWN = 0, 1, 2

_DTYPES = {torch.float16: BM_F16, torch.bfloat16: BM_BF16, torch.float32: BM_F32}
_ROUND = {None: ROUND_NONE, torch.float32: ROUND_NONE, torch.float16: ROUND_F16, torch.bfloat16: ROUND_BF16}


class BitsMoEError(RuntimeError):
    """A non-zero status from the C ABI (the reference raises RuntimeError from TORCH_CHECK)."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class Matrix(C.Structure):
    _fields_ = [
        ("payload", C.c_void_p), ("payload_words", C.c_int64),
        ("rank_idx", C.c_void_p), ("n_rows", C.c_int32),
        ("tile_meta", C.c_void_p), ("n_tile_rows", C.c_int32),
        ("slab_meta", C.c_void_p), ("n_slabs", C.c_int32),
        ("scale", C.c_void_p), ("n_scales", C.c_int64),
        ("s", C.c_void_p),
    ]


class LayerDesc(C.Structure):
    _fields_ = [
        ("num_experts", C.c_int32), ("hidden", C.c_int32), ("intermediate", C.c_int32),
        ("rank_in", C.c_int32), ("rank_out", C.c_int32), ("act_type", C.c_int32),
        ("gate", C.POINTER(Matrix)), ("up", C.POINTER(Matrix)), ("down", C.POINTER(Matrix)),
        ("vh_gate", C.c_void_p), ("vh_up", C.c_void_p), ("u_down", C.c_void_p),
    ]


_SIGS = {
    "bm_abi_version": (C.c_int, []),
    "bm_launch_count": (C.c_uint64, []),
    "bm_arena_layout_version": (C.c_int, []),
    "bm_last_error": (C.c_char_p, []),
    "bm_status_string": (C.c_char_p, [C.c_int]),
    "bm_pack_bitplanes_i8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "bm_quantize_pack_slab": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p]),
    "bm_unpack_bitplanes_i8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "bm_layer_plan": (C.c_int, [C.POINTER(LayerDesc), C.POINTER(C.c_size_t)]),
    "bm_layer_create": (C.c_int, [C.POINTER(LayerDesc), C.c_void_p, C.c_size_t, C.c_void_p, C.POINTER(C.c_void_p)]),
    "bm_layer_destroy": (C.c_int, [C.c_void_p]),
    "bm_layer_expert_bytes": (C.c_int64, [C.c_void_p, C.c_int32]),
    "bm_layer_decode_codes": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "bm_layer_has_fast_layout": (C.c_int, [C.c_void_p]),
    "bm_layer_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "bm_layer_set_option": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32]),
    "bm_layer_selftest_wait": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "bm_gate_logits": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int, C.c_void_p]),
    "bm_dense_mlp_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "bm_dense_mlp_forward": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                       C.c_int32, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]),
    "bm_ep_flag_bytes": (C.c_size_t, []),
    "bm_ep_barrier": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "bm_ep_push": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "bm_ep_pull_reduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                    C.c_void_p, C.c_void_p]),
    "bm_route_topk": (C.c_int, [C.c_void_p, C.c_int, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                C.c_void_p, C.c_void_p, C.c_void_p]),
    "bm_route_build_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "bm_route_max_tiles": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "bm_route_build": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                 C.c_void_p]),
    "bm_route_build_static_capacity": (C.c_size_t, []),
    "bm_route_build_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                        C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "bm_route": (C.c_int, [C.c_void_p, C.c_int, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                           C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                           C.c_void_p, C.c_size_t, C.c_void_p]),
    "bm_basis_project": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "bm_experts_workspace_bytes": (C.c_size_t, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32]),
    "bm_experts_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                     C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p]),
    "bm_combine_down_basis": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "bm_layer_workspace_bytes": (C.c_size_t, [C.c_void_p, C.c_int32, C.c_int32]),
    "bm_layer_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int32, C.c_int32, C.c_int32,
                                   C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                   C.c_size_t, C.c_void_p]),
}

_lib: Optional[C.CDLL] = None


def exported_symbols():
    return tuple(_SIGS)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"bitsmoe_b200 CUDA library not found at {LIB_PATH}; build it with "
                "`python -m bitsmoe_b200._build` (there is no Python or CPU fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != BM_OK:
        raise BitsMoEError(status, lib().bm_last_error().decode("utf-8", "replace"))


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported activation dtype {dt}") from None


def round_code(dt) -> int:
    return _ROUND[dt]


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream
