"""Model patcher: turns the MoE blocks of a Hugging Face causal LM into BitsMoE blocks.

Same job and the same entry points as ``bitsmoe.models.auto.bitsmoe_auto_patch``
(bitsmoe/models/auto/bitsmoe_auto_patch.py: ``_patch_bitsmoe_inplace`` :432-508, the patched
``AutoModelForCausalLM.from_pretrained(..., bitsmoe=, bitsmoe_model_type=)`` :611-695,
``ensure_auto_patch_installed`` :698-708, the runtime preparation :385-429 and its environment flags), but written
against the module layout of transformers 5.x, where the routed experts of a block are ONE fused module
(``mlp.experts.gate_up_proj [E, 2I, H]``, ``mlp.experts.down_proj [E, H, I]``) and the router is a ``*TopKRouter`` with a
bare ``weight`` instead of an ``nn.Linear``; the reference iterates ``source_moe.experts`` as a list of per-expert modules
(:105-111), which no longer exists.  Per-expert list layouts (transformers 4.x, DeepSeek remote code) are handled too.

What the patcher does per decoder layer that has routed experts:
  * the router becomes a bias-free ``nn.Linear`` sharing the router's ``weight`` (state-dict key ``...gate.weight`` is
    unchanged); a DeepSeek ``MoEGate`` (returns top-k itself) is kept as it is;
  * every routed expert becomes a packed ``BitsMoE_*MLP`` whose thirty buffers are bound from the checkpoint (either
    key schema), except the "super" experts of the reference's table (:42-46), which stay dense modules cut out of the
    fused tensors;
  * shared experts and their gates are carried over;
  * the block is a ``BitsMoE_*SparseMoeBlock`` of this package; with fused-expert models it returns the hidden states
    only, as the 5.x decoder layer expects (``return_router_logits = False``).
"""
from __future__ import annotations

import copy
import os
from types import SimpleNamespace
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from bitsmoe_b200.models.base_block import BitsMoE_BaseSparseMoeBlock
from bitsmoe_b200.models.deepseekv2.bitsmoe_block import BitsMoE_DeepSeekSparseMoeBlock
from bitsmoe_b200.models.deepseekv2.bitsmoe_mlp import BitsMoE_DeepSeekMLP
from bitsmoe_b200.models.qwen3moe.bitsmoe_block import BitsMoE_Qwen3MoeSparseMoeBlock
from bitsmoe_b200.models.qwen3moe.bitsmoe_mlp import BitsMoE_Qwen3MoeMLP
from bitsmoe_b200.models.qwen3next.bitsmoe_block import BitsMoE_Qwen3NextSparseMoeBlock
from bitsmoe_b200.models.qwen3next.bitsmoe_mlp import BitsMoE_Qwen3NextMLP

# un-quantised ("super") experts per layer of the released checkpoints (bitsmoe_auto_patch.py:42-46)
_SUPER_EXPERTS_BY_MODEL: Dict[str, Dict[int, List[int]]] = {
    "qwen3moe": {1: [68], 2: [92], 3: [82]},
    "deepseekv2": {2: [54], 3: [38]},
    "qwen3next": {10: [288, 401], 21: [251], 25: [381], 26: [264], 35: [38, 69, 303]},
}
_BLOCK_BY_MODEL = {"qwen3moe": BitsMoE_Qwen3MoeSparseMoeBlock, "deepseekv2": BitsMoE_DeepSeekSparseMoeBlock,
                   "qwen3next": BitsMoE_Qwen3NextSparseMoeBlock}
_MLP_BY_MODEL = {"qwen3moe": BitsMoE_Qwen3MoeMLP, "deepseekv2": BitsMoE_DeepSeekMLP, "qwen3next": BitsMoE_Qwen3NextMLP}


class _DenseExpert(nn.Module):
    """One un-quantised expert cut out of a fused experts module (gate_up_proj [E, 2I, H], down_proj [E, H, I])."""

    def __init__(self, gate_up: torch.Tensor, down: torch.Tensor):
        super().__init__()
        inter, hidden = gate_up.shape[0] // 2, gate_up.shape[1]
        self.gate_proj = nn.Linear(hidden, inter, bias=False, device=gate_up.device, dtype=gate_up.dtype)
        self.up_proj = nn.Linear(hidden, inter, bias=False, device=gate_up.device, dtype=gate_up.dtype)
        self.down_proj = nn.Linear(inter, hidden, bias=False, device=gate_up.device, dtype=gate_up.dtype)
        if not gate_up.is_meta:
            with torch.no_grad():
                self.gate_proj.weight.copy_(gate_up[:inter])
                self.up_proj.weight.copy_(gate_up[inter:])
                self.down_proj.weight.copy_(down)

    def forward(self, x):
        return self.down_proj(nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


def _moe_attr(layer) -> Optional[str]:
    for name in ("mlp", "block_sparse_moe"):
        blk = getattr(layer, name, None)
        if blk is not None and hasattr(blk, "experts") and hasattr(blk, "gate"):
            return name
    return None


def _num_experts(source_moe, config) -> int:
    ex = source_moe.experts
    if isinstance(ex, (nn.ModuleList, list, tuple)):
        return len(ex)
    for obj, name in ((ex, "num_experts"), (source_moe, "num_experts"), (config, "num_experts"), (config, "n_routed_experts")):
        v = getattr(obj, name, None)
        if v is not None:
            return int(v)
    raise RuntimeError("cannot tell how many routed experts the source block has")


def _expert_intermediate(source_moe, config) -> int:
    ex = source_moe.experts
    gu = getattr(ex, "gate_up_proj", None)
    if isinstance(gu, torch.Tensor):
        return int(gu.shape[1] // 2)
    if isinstance(ex, (nn.ModuleList, list, tuple)):
        for m in ex:
            w = getattr(getattr(m, "gate_proj", None), "weight", None)
            if isinstance(w, torch.Tensor):
                return int(w.shape[0])
    for name in ("moe_intermediate_size", "intermediate_size"):
        v = getattr(config, name, None)
        if v is not None:
            return int(v)
    raise RuntimeError("failed to infer the experts' intermediate size")


def _router_as_linear(gate) -> nn.Module:
    """A bias-free Linear that shares the router's weight (the block computes logits itself and selects on the GPU)."""
    if isinstance(gate, nn.Linear):
        return gate
    w = getattr(gate, "weight", None)
    if isinstance(w, torch.Tensor) and w.dim() == 2 and not hasattr(gate, "topk_method"):
        lin = nn.Linear(w.shape[1], w.shape[0], bias=False, device="meta")
        lin.weight = w if isinstance(w, nn.Parameter) else nn.Parameter(w, requires_grad=False)
        return lin
    return gate          # a gate that selects by itself (DeepSeek MoEGate): used as it is


def _dense_expert_from(source_moe, idx: int) -> nn.Module:
    ex = source_moe.experts
    if isinstance(ex, (nn.ModuleList, list, tuple)):
        if ex[idx] is not None:
            return copy.deepcopy(ex[idx])
    elif isinstance(getattr(ex, "gate_up_proj", None), torch.Tensor):
        return _DenseExpert(ex.gate_up_proj[idx].detach(), ex.down_proj[idx].detach())
    shared = getattr(source_moe, "shared_expert", None)
    if shared is None:
        raise RuntimeError("Cannot build dense super expert: no source expert template and no shared_expert fallback.")
    return copy.deepcopy(shared)


def patch_bitsmoe_inplace(model, bitsmoe_model_type: str, packed_state: Optional[Dict[str, torch.Tensor]] = None,
                          super_experts_by_layer: Optional[Dict[int, List[int]]] = None) -> int:
    """Rewrites every MoE block of ``model.model.layers`` in place; returns the number of packed experts.

    ``packed_state``: a checkpoint state dict; when given the experts' buffers are bound from it right away (keys
    ``<layer prefix>.<moe attr>.experts.<e>.…``), otherwise the experts are created empty and a later
    ``load_state_dict`` fills them (both key schemas are understood by ``BitsMoE_BaseMoeMLP``)."""
    if bitsmoe_model_type not in _BLOCK_BY_MODEL:
        raise ValueError(f"Unsupported bitsmoe_model_type={bitsmoe_model_type}. Supported={list(_BLOCK_BY_MODEL.keys())}")
    if not hasattr(model, "model") or not hasattr(model.model, "layers"):
        raise ValueError("BitsMoE model patch requires model.model.layers")
    block_cls, mlp_cls = _BLOCK_BY_MODEL[bitsmoe_model_type], _MLP_BY_MODEL[bitsmoe_model_type]
    super_map = _SUPER_EXPERTS_BY_MODEL.get(bitsmoe_model_type, {}) if super_experts_by_layer is None else super_experts_by_layer
    defer = bitsmoe_model_type == "qwen3next"
    total = 0
    for layer_idx, layer in enumerate(model.model.layers):
        attr = _moe_attr(layer)
        if attr is None:
            continue
        source = getattr(layer, attr)
        n_exp = _num_experts(source, model.config)
        inter = _expert_intermediate(source, model.config)
        fused = not isinstance(source.experts, (nn.ModuleList, list, tuple))
        supers = sorted({int(e) for e in super_map.get(layer_idx, []) if 0 <= int(e) < n_exp})
        shim = SimpleNamespace(gate=_router_as_linear(source.gate), experts=[None] * n_exp)
        for name in ("shared_expert", "shared_expert_gate", "shared_experts", "ep_size", "experts_per_rank", "ep_rank"):
            if hasattr(source, name):
                setattr(shim, name, getattr(source, name))
        block = block_cls(config=model.config, layer_idx=layer_idx, source_block=shim, super_experts=supers,
                          copy_source_experts=False)
        block.gate = shim.gate                      # the block deep-copies its source's gate; keep the shared weight
        prefix = f"model.layers.{layer_idx}.{attr}.experts"
        for e in range(n_exp):
            if e in supers:
                block.set_expert(e, _dense_expert_from(source, e), packed=False)
                continue
            kw = dict(config=model.config, intermediate_size=inter)
            if packed_state is not None:
                kw.update(packed_state=packed_state, packed_prefix=f"{prefix}.{e}")
            elif defer:
                kw.update(defer_runtime_buffer_init=True)
            block.set_expert(e, mlp_cls(**kw), packed=True)
            total += 1
        if packed_state is not None:
            basis = [packed_state.get(f"model.layers.{layer_idx}.{attr}.{k}") for k in block._SHARED_BASIS_BUFFER_KEYS]
            if all(isinstance(b, torch.Tensor) for b in basis):
                for k, b in zip(block._SHARED_BASIS_BUFFER_KEYS, basis):
                    setattr(block, k, b.detach().to(torch.float16))
                block._invalidate_runtime_cache()
        if fused:
            block.return_router_logits = False      # the 5.x decoder layer takes the hidden states only
        setattr(layer, attr, block)
    setattr(model, "_bitsmoe_packed_expert_total", int(total))
    return total


def prepare_bitsmoe_runtime(model, warmup: Optional[bool] = None) -> int:
    """Builds every block's runtime cache (pointer tables, arena) ahead of the first forward, as
    ``_maybe_prepare_bitsmoe_runtime`` does (bitsmoe_auto_patch.py:385-429); honours BITSMOE_PREPARE_RUNTIME=0 and
    BITSMOE_PREPARE_WARMUP.  Returns the number of blocks prepared; failures of single blocks are re-raised."""
    if os.environ.get("BITSMOE_PREPARE_RUNTIME", "1").lower() in ("0", "false", "no"):
        return 0
    if warmup is None:
        warmup = os.environ.get("BITSMOE_PREPARE_WARMUP", "1").lower() not in ("0", "false", "no")
    n = 0
    for module in model.modules():
        if isinstance(module, BitsMoE_BaseSparseMoeBlock) and module._runtime_device().type == "cuda":
            module.prepare_runtime_fastpath(warmup=warmup)
            n += 1
    return n


def _rematerialize_nonpersistent_buffers(model) -> None:
    """Buffers a checkpoint does not hold (rotary tables and the like) were created on the meta device with the rest of
    the model: rebuild them by constructing a fresh instance of the owning module from its config."""
    for module in model.modules():
        meta = [n for n, b in module.named_buffers(recurse=False) if b.is_meta and n in module._non_persistent_buffers_set]
        if not meta:
            continue
        cfg = getattr(module, "config", None)
        if cfg is None:
            raise RuntimeError(f"cannot rebuild the non-persistent buffers {meta} of {type(module).__name__}")
        fresh = type(module)(cfg)
        for n in meta:
            module._buffers[n] = getattr(fresh, n)


def build_patched_model(config, bitsmoe_model_type: str, state_dict: Optional[Dict[str, torch.Tensor]] = None,
                        device: Optional[torch.device] = None, dtype: torch.dtype = torch.float16,
                        super_experts_by_layer: Optional[Dict[int, List[int]]] = None):
    """``AutoModelForCausalLM.from_config`` + patch + (optionally) ``load_state_dict(assign=True)``: the dense routed
    experts of the stock model are never materialised (the model is created on the meta device and only what the
    checkpoint holds becomes real)."""
    from transformers import AutoModelForCausalLM
    with torch.device("meta"):
        model = AutoModelForCausalLM.from_config(config, dtype=dtype)
    patch_bitsmoe_inplace(model, bitsmoe_model_type, super_experts_by_layer=super_experts_by_layer)
    if state_dict is not None:
        missing, unexpected = model.load_state_dict(state_dict, strict=False, assign=True)
        _rematerialize_nonpersistent_buffers(model)
        still_meta = [n for n, p in list(model.named_parameters()) + list(model.named_buffers()) if p.is_meta]
        if still_meta:
            raise RuntimeError(f"{len(still_meta)} tensors have no value after loading, e.g. {still_meta[:4]}")
        model._bitsmoe_missing_keys, model._bitsmoe_unexpected_keys = list(missing), list(unexpected)
    if device is not None:
        model.to(device)
        prepare_bitsmoe_runtime(model)
    return model


_INSTALLED = False


def ensure_auto_patch_installed() -> None:
    """``AutoModelForCausalLM.from_pretrained(path, bitsmoe=True, bitsmoe_model_type="qwen3moe" | …)`` builds the patched
    model from ``path``'s config and its single-file checkpoint (``pytorch_model.bin``, as the reference's
    ``save_sharded_checkpoint`` writes it, bitsmoe/quant/packer.py:752-771); without ``bitsmoe`` the call is untouched."""
    global _INSTALLED
    if _INSTALLED:
        return
    from transformers import AutoConfig, AutoModelForCausalLM
    stock = AutoModelForCausalLM.from_pretrained.__func__

    def from_pretrained(cls, pretrained_model_name_or_path, *args, bitsmoe=None, bitsmoe_model_type=None, **kwargs):
        config = kwargs.get("config") or AutoConfig.from_pretrained(pretrained_model_name_or_path,
                                                                    trust_remote_code=kwargs.get("trust_remote_code", False))
        want = bitsmoe if bitsmoe is not None else getattr(config, "bitsmoe", None)
        mtype = bitsmoe_model_type or getattr(config, "bitsmoe_model_type", None)
        if not want:
            return stock(cls, pretrained_model_name_or_path, *args, **kwargs)
        if mtype is None:
            raise ValueError("bitsmoe=True needs bitsmoe_model_type (qwen3moe, qwen3next or deepseekv2)")
        path = os.path.join(str(pretrained_model_name_or_path), "pytorch_model.bin")
        state = torch.load(path, map_location="cpu", weights_only=True)
        device = kwargs.get("device_map")
        device = torch.device(device) if isinstance(device, (str, torch.device)) and str(device) not in ("auto",) else None
        return build_patched_model(config, mtype, state, device=device, dtype=kwargs.get("torch_dtype", kwargs.get("dtype", torch.float16)))

    AutoModelForCausalLM.from_pretrained = classmethod(from_pretrained)
    _INSTALLED = True
