"""Container of one packed expert: 10 persistent buffers for each of gate / up / down.

Same surface as ``bitsmoe.models.base_mlp.BitsMoE_BaseMoeMLP`` (bitsmoe/models/base_mlp.py:84-402):
buffer names ``{gate,up,down}_{payload_buffer,rank_idx_buffer,tile_meta_buffer,slab_meta_buffer,
scale_buffer,s_buffer,segments,original_indices,groupsize,original_rank}`` (they are the checkpoint
schema), ``load_runtime_packed_from_state`` accepting the packer's keys
(``{prefix}.{mtype}.{u|vh}.payload_buffer`` …) or the materialised module keys
(``{prefix}.{tag}_payload_buffer`` …), a ``_load_from_state_dict`` that re-shapes or binds the
initially empty buffers, and ``forward`` that refuses to run: compute happens in the block.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

_PROGRESS = {"enabled": False, "total": 0, "current": 0, "external_updates": False}


def configure_bitsmoe_load_progress(total_experts: int, enabled: bool = True, external_updates: bool = False) -> None:
    finalize_bitsmoe_load_progress()
    if enabled and int(total_experts) > 0:
        _PROGRESS.update(enabled=True, total=int(total_experts), current=0, external_updates=bool(external_updates))


def advance_bitsmoe_load_progress(step: int = 1, source: str = "internal") -> None:
    if not _PROGRESS["enabled"] or int(step) <= 0:
        return
    if source == "internal" and _PROGRESS["external_updates"]:
        return
    total = _PROGRESS["total"]
    cur = min(total, _PROGRESS["current"] + int(step))
    _PROGRESS["current"] = cur
    if cur == total or cur % max(1, total // 20) == 0:
        print(f"BitsMoE packed expert load: {cur}/{total}", flush=True)


def finalize_bitsmoe_load_progress() -> None:
    _PROGRESS.update(enabled=False, total=0, current=0, external_updates=False)


def _activation(name: str):
    table = {"silu": F.silu, "swish": F.silu, "gelu": F.gelu, "relu": F.relu}
    if name in table:
        return table[name]
    from transformers.activations import ACT2FN
    return ACT2FN[name]


class BitsMoE_BaseMoeMLP(nn.Module):
    _MTYPE_TO_TAG = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}
    _RUNTIME_BUFFER_DTYPES = {
        "payload_buffer": torch.uint32,
        "rank_idx_buffer": torch.int32,
        "tile_meta_buffer": torch.int32,
        "slab_meta_buffer": torch.int32,
        "scale_buffer": torch.float16,
        "s_buffer": torch.float16,
        "segments": torch.int32,
        "original_indices": torch.int32,
        "groupsize": torch.int16,
        "original_rank": torch.int32,
    }
    _SCALARS = ("groupsize", "original_rank")
    _CAST = ("payload_buffer", "rank_idx_buffer", "tile_meta_buffer", "slab_meta_buffer", "scale_buffer", "s_buffer")

    @classmethod
    def _runtime_buffer_leaf_keys(cls):
        return tuple(f"{tag}_{name}" for tag in cls._MTYPE_TO_TAG.values() for name in cls._RUNTIME_BUFFER_DTYPES)

    def __init__(self, config, intermediate_size: Optional[int] = None,
                 packed_state: Optional[Dict[str, torch.Tensor]] = None, packed_prefix: Optional[str] = None,
                 packed_device: torch.device = torch.device("cpu"), defer_runtime_buffer_init: bool = False):
        super().__init__()
        self.config = config
        self.hidden_size = int(config.hidden_size)
        self.intermediate_size = int(intermediate_size if intermediate_size is not None else config.intermediate_size)
        self.act_fn = _activation(config.hidden_act)
        self.is_bitsmoe_packed = False
        self.skip_expert = True
        self.runtime_meta: Dict[str, Dict[str, Any]] = {}
        self._load_progress_marked = False
        self._defer_runtime_buffer_init = bool(defer_runtime_buffer_init)
        if not self._defer_runtime_buffer_init:
            self._init_runtime_buffers()
        if packed_state is not None:
            if packed_prefix is None:
                raise ValueError("packed_prefix must be provided when packed_state is provided")
            self.load_runtime_packed_from_state(state_dict=packed_state, prefix=packed_prefix, device=packed_device)

    def _init_runtime_buffers(self) -> None:
        for key in self._runtime_buffer_leaf_keys():
            name = key.split("_", 1)[1]
            dtype = self._RUNTIME_BUFFER_DTYPES[name]
            init = torch.tensor(0, dtype=dtype) if name in self._SCALARS else torch.empty(0, dtype=dtype)
            self.register_buffer(key, init, persistent=True)

    @staticmethod
    def _scalar_tensor_to_int(t: torch.Tensor, name: str) -> int:
        if t.numel() != 1:
            raise ValueError(f"{name} must be scalar, got shape {tuple(t.shape)}")
        return int(t.detach().to(device="cpu", dtype=torch.int64).reshape(()))

    def _register_or_replace_buffer(self, name: str, tensor: torch.Tensor) -> None:
        if name in self._buffers:
            self._buffers[name] = tensor
        else:
            self.register_buffer(name, tensor, persistent=True)

    def _source_keys(self, state_dict, prefix: str, mtype: str) -> Optional[Dict[str, str]]:
        """Maps each of the ten buffer names to the state-dict key that holds it, or None."""
        tag = self._MTYPE_TO_TAG[mtype]
        fld = "u" if mtype in ("gate_proj", "up_proj") else "vh"
        packer_keys = {n: (f"{prefix}.{mtype}.{fld}.{n}" if n in ("payload_buffer", "rank_idx_buffer",
                                                                 "tile_meta_buffer", "slab_meta_buffer", "scale_buffer")
                           else f"{prefix}.{mtype}.{n}") for n in self._RUNTIME_BUFFER_DTYPES}
        if all(k in state_dict for k in packer_keys.values()):
            return packer_keys
        module_keys = {n: f"{prefix}.{tag}_{n}" for n in self._RUNTIME_BUFFER_DTYPES}
        required = [module_keys[n] for n in self._RUNTIME_BUFFER_DTYPES if n not in self._SCALARS]
        if all(k in state_dict for k in required):
            return module_keys
        return None

    def _load_one_mtype(self, state_dict, prefix: str, mtype: str, device: torch.device) -> bool:
        keys = self._source_keys(state_dict, prefix, mtype)
        if keys is None:
            return False
        tag = self._MTYPE_TO_TAG[mtype]
        loaded: Dict[str, torch.Tensor] = {}
        for name in self._RUNTIME_BUFFER_DTYPES:
            if name in self._SCALARS:
                continue
            t = state_dict[keys[name]].detach().to(device=device, non_blocking=True).contiguous()
            if name in self._CAST:
                t = t.to(self._RUNTIME_BUFFER_DTYPES[name])
            loaded[name] = t
        original_rank = (self._scalar_tensor_to_int(state_dict[keys["original_rank"]], keys["original_rank"])
                         if keys["original_rank"] in state_dict else int(loaded["original_indices"].numel()))
        groupsize = (self._scalar_tensor_to_int(state_dict[keys["groupsize"]], keys["groupsize"])
                     if keys["groupsize"] in state_dict else 128)
        for name, t in loaded.items():
            self._register_or_replace_buffer(f"{tag}_{name}", t)
        self._register_or_replace_buffer(f"{tag}_groupsize", torch.tensor(groupsize, dtype=torch.int16, device=device))
        self._register_or_replace_buffer(f"{tag}_original_rank",
                                         torch.tensor(original_rank, dtype=torch.int32, device=device))

        def rows(t: torch.Tensor) -> List[tuple]:
            return [tuple(int(v) for v in r) for r in t.to(dtype=torch.int64, device="cpu").tolist()]

        self.runtime_meta[mtype] = {
            "groupsize": groupsize,
            "original_rank": original_rank,
            "slab_meta_rows": rows(loaded["slab_meta_buffer"]),
            "tile_meta_rows": rows(loaded["tile_meta_buffer"]),
            "segments": rows(loaded["segments"]),
            "packed_field": "u" if mtype in ("gate_proj", "up_proj") else "vh",
        }
        return True

    def load_runtime_packed_from_state(self, state_dict: Dict[str, torch.Tensor], prefix: str,
                                       device: torch.device = torch.device("cpu")) -> bool:
        ok = True
        for mtype in ("gate_proj", "up_proj", "down_proj"):
            ok = self._load_one_mtype(state_dict, prefix, mtype, device=device) and ok
        self.is_bitsmoe_packed = ok
        self.skip_expert = not ok
        return ok

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        assign = bool(local_metadata.get("assign_to_params_buffers", False))
        consumed = []
        # packer key schema (<prefix><mtype>.{u|vh}.payload_buffer ...): bind the tensors matrix by matrix
        base = prefix[:-1] if prefix.endswith(".") else prefix
        for mtype in self._MTYPE_TO_TAG:
            keys = self._source_keys(state_dict, base, mtype)
            if keys is None or keys["payload_buffer"] == f"{base}.{self._MTYPE_TO_TAG[mtype]}_payload_buffer":
                continue
            dev = state_dict[keys["payload_buffer"]].device
            if self._load_one_mtype(state_dict, base, mtype, device=dev):
                for k in keys.values():
                    if k in state_dict:
                        consumed.append(k)
        for leaf in self._runtime_buffer_leaf_keys():
            t = state_dict.get(f"{prefix}{leaf}", None)
            if not isinstance(t, torch.Tensor):
                continue
            consumed.append(f"{prefix}{leaf}")
            cur = getattr(self, leaf, None)
            if isinstance(cur, torch.Tensor) and cur.shape == t.shape and cur.dtype == t.dtype and not assign:
                cur.copy_(t)
                continue
            self._register_or_replace_buffer(leaf, t.detach() if assign else t.detach().clone())
        if consumed and not self._load_progress_marked:
            self._load_progress_marked = True
            advance_bitsmoe_load_progress(1, source="internal")
        for k in consumed:
            state_dict.pop(k, None)
        # buffers bound above are no longer "missing" for the generic loader
        own = set(self._runtime_buffer_leaf_keys())
        before = len(missing_keys)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
        bound = {f"{prefix}{leaf}" for leaf in own if f"{prefix}{leaf}" in consumed}
        missing_keys[before:] = [k for k in missing_keys[before:] if k not in bound]
        self.is_bitsmoe_packed = all(
            isinstance(getattr(self, f"{tag}_payload_buffer", None), torch.Tensor)
            and getattr(self, f"{tag}_payload_buffer").numel() > 0 for tag in self._MTYPE_TO_TAG.values())
        self.skip_expert = not self.is_bitsmoe_packed

    def load_quantized_weight_from_state(self, state_dict: Dict[str, torch.Tensor], orig_prefix: str) -> bool:
        return self.load_runtime_packed_from_state(state_dict=state_dict, prefix=orig_prefix)

    def forward(self, x: torch.Tensor, h_gate_proj: Optional[torch.Tensor] = None,
                h_up_proj: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError(
            "BitsMoE_BaseMoeMLP forward is intentionally not implemented in this stage. "
            "This module currently only stores packed payload/metadata.")
