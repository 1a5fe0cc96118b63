"""``moe_packed_forward`` with the reference's 26-argument signature.

Stands in for the pybind module ``bitsmoe.algorithms._mlp_forward_cuda``
(bitsmoe/algorithms/cpp/mlp_forward_binding.cpp:53-189): same argument order, same dtype and
shape checks raising RuntimeError, same result (fp32 ``[tokens, rank_out]``).  The prepared
per-layer device state is cached on the identity of the buffer lists the caller passes (the
block keeps those tuples alive), not on raw device pointers.
"""
from __future__ import annotations

import weakref
from typing import Dict, Sequence, Tuple

import torch

from bitsmoe_b200.layer import PackedLayer

_FIELDS = ("payload", "rank_idx", "tile_meta", "slab_meta", "scale", "s")
_cache: Dict[Tuple, PackedLayer] = {}
_CACHE_LIMIT = 256


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_cuda_contig(t: torch.Tensor, name: str) -> None:
    _check(t.is_cuda, f"{name} must be CUDA tensor")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _layer_key(lists: Sequence[Sequence[torch.Tensor]], rank_out: int, intermediate_size: int, h_rank: int, device):
    # data pointers + lengths of every payload identify the weights; sizes guard against reuse of freed memory
    first = tuple((t.data_ptr(), t.numel()) for t in lists[0])
    last = tuple((t.data_ptr(), t.numel()) for t in lists[12])
    mid = tuple((t.data_ptr(), t.numel()) for t in lists[6])
    return (first, mid, last, rank_out, intermediate_size, h_rank, str(device))


def clear_cache() -> None:
    for layer in _cache.values():
        layer.close()
    _cache.clear()


def moe_packed_forward(h_gate, h_up, token_indices, expert_offsets, route_weights,
                       gate_payload, gate_rank_idx, gate_tile_meta, gate_slab_meta, gate_scale, gate_s,
                       up_payload, up_rank_idx, up_tile_meta, up_slab_meta, up_scale, up_s,
                       down_payload, down_rank_idx, down_tile_meta, down_slab_meta, down_scale, down_s,
                       rank_out, intermediate_size, act_type, path: int = 0):
    _check(h_gate.dim() == 2, "h_gate must be 2D [tokens, rank]")
    _check(h_up.dim() == 2, "h_up must be 2D [tokens, rank]")
    _check(h_gate.shape[0] == h_up.shape[0], "h_gate/h_up token dim mismatch")
    _check(token_indices.dim() == 1, "token_indices must be 1D")
    _check(expert_offsets.dim() == 1, "expert_offsets must be 1D")
    _check(route_weights.dim() == 1, "route_weights must be 1D")
    for t, n in ((h_gate, "h_gate"), (h_up, "h_up"), (token_indices, "token_indices"),
                 (expert_offsets, "expert_offsets"), (route_weights, "route_weights")):
        _check_cuda_contig(t, n)
    _check(h_gate.dtype == torch.float16, "h_gate must be float16")
    _check(h_up.dtype == torch.float16, "h_up must be float16")
    _check(token_indices.dtype == torch.int32, "token_indices must be int32")
    _check(expert_offsets.dtype == torch.int32, "expert_offsets must be int32")
    _check(route_weights.dtype == torch.float32, "route_weights must be float32")
    num_experts = expert_offsets.numel() - 1
    _check(num_experts >= 0, "expert_offsets must have length >= 1")
    _check(token_indices.numel() == route_weights.numel(), "token_indices/route_weights size mismatch")
    lists = (gate_payload, gate_rank_idx, gate_tile_meta, gate_slab_meta, gate_scale, gate_s,
             up_payload, up_rank_idx, up_tile_meta, up_slab_meta, up_scale, up_s,
             down_payload, down_rank_idx, down_tile_meta, down_slab_meta, down_scale, down_s)
    names = [f"{m}_{f}" for m in ("gate", "up", "down") for f in _FIELDS]
    for xs, n in zip(lists, names):
        _check(len(xs) == num_experts, f"{n} size mismatch, expected {num_experts}, got {len(xs)}")
    _check(intermediate_size > 0, "intermediate_size must be > 0")
    _check(rank_out > 0, "rank_out must be > 0")
    _check(act_type == 0, "only SiLU act_type=0 is currently supported")

    tokens = h_gate.shape[0]
    if token_indices.numel() == 0 or num_experts == 0:
        return torch.zeros((tokens, rank_out), dtype=torch.float32, device=h_gate.device)
    key = _layer_key(lists, int(rank_out), int(intermediate_size), int(h_gate.shape[1]), h_gate.device)
    layer = _cache.get(key)
    if layer is None:
        if len(_cache) >= _CACHE_LIMIT:
            clear_cache()
        tabs = [{f: lists[6 * m + i] for i, f in enumerate(_FIELDS)} for m in range(3)]
        layer = PackedLayer(tabs[0], tabs[1], tabs[2], int(intermediate_size), int(rank_out),
                            rank_in=int(h_gate.shape[1]), act_type=int(act_type), device=h_gate.device)
        _cache[key] = layer
    return layer.experts_forward(h_gate, h_up, token_indices, expert_offsets, route_weights, path=path)
