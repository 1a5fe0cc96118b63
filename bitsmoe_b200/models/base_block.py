"""Base sparse-MoE block over packed experts, backed by the sm_100a library.

Keeps the module interface of ``bitsmoe.models.base_block.BitsMoE_BaseSparseMoeBlock``
(bitsmoe/models/base_block.py:9-446): the three persistent fp16 shared-basis buffers,
``set_shared_basis`` / ``set_expert`` / ``set_super_expert_projected_weights`` /
``prepare_runtime_fastpath``, the lazily built runtime cache with its ``_*_static`` tuples and
``_packed_global_to_local`` map, ``_build_packed_routing``, ``_run_super_experts``,
``_packed_forward_cuda`` / ``_packed_forward_grouped`` at the reference's op boundary.

What differs is where the work happens: the cache also owns a ``PackedLayer`` (device pointer
tables built once per block), routing is built by one kernel without a device->host sync, and
``_fused_forward`` runs route -> basis -> experts -> down basis (+ residual) on one stream.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from bitsmoe_b200.algorithms import _HAS_MLP_FORWARD_CUDA, mlp_forward_cuda

_FIELDS = ("payload", "rank_idx", "tile_meta", "slab_meta", "scale", "s")
_TAGS = ("gate", "up", "down")


class BitsMoE_BaseSparseMoeBlock(nn.Module):
    _SHARED_BASIS_BUFFER_KEYS = ("shared_vh_gate_proj", "shared_vh_up_proj", "shared_u_down")

    def _init_bitsmoe_common_state(self, super_experts: Optional[List[int]] = None,
                                   track_super_projected_weights: bool = False) -> None:
        self.super_experts = sorted(set(int(x) for x in (super_experts or [])))
        self._super_expert_set = set(self.super_experts)
        self.packed_expert_mask = [False for _ in range(len(self.experts))]
        if track_super_projected_weights:
            self.super_projected_weights: Dict[int, Dict[str, torch.Tensor]] = {}
        for key in self._SHARED_BASIS_BUFFER_KEYS:
            self.register_buffer(key, torch.empty(0, dtype=torch.float16), persistent=True)
        self._super_expert_items: List[Tuple[int, nn.Module]] = []
        self._packed_expert_count = 0
        self._packed_intermediate_size = 0
        self._packed_global_to_local: Optional[torch.Tensor] = None
        self._packed_layer = None
        for tag in _TAGS:
            for f in _FIELDS:
                setattr(self, f"_{tag}_{f}_static", ())
        self._invalidate_runtime_cache()

    # ---- configuration ----------------------------------------------------------------------------
    def _runtime_device(self) -> torch.device:
        gate = getattr(self, "gate", None)
        weight = getattr(gate, "weight", None)
        if isinstance(weight, torch.Tensor):
            return weight.device
        return next(gate.parameters()).device

    def _set_buffer(self, name: str, tensor: torch.Tensor) -> None:
        setattr(self, name, tensor.detach().to(device=self._runtime_device(), dtype=torch.float16,
                                               non_blocking=True).contiguous())

    def set_shared_basis(self, gate_vh: torch.Tensor, up_vh: torch.Tensor, down_u: torch.Tensor) -> None:
        self._set_buffer("shared_vh_gate_proj", gate_vh)
        self._set_buffer("shared_vh_up_proj", up_vh)
        self._set_buffer("shared_u_down", down_u)
        self._invalidate_runtime_cache()

    def set_expert(self, expert_idx: int, expert_module: nn.Module, packed: bool) -> None:
        idx = int(expert_idx)
        self.experts[idx] = expert_module
        self.packed_expert_mask[idx] = bool(packed)
        self._invalidate_runtime_cache()

    def set_super_expert_projected_weights(self, expert_idx: int, gate_us: torch.Tensor, up_us: torch.Tensor,
                                           down_svh: torch.Tensor) -> None:
        if not hasattr(self, "super_projected_weights"):
            self.super_projected_weights = {}
        self.super_projected_weights[int(expert_idx)] = {
            "gate_us": gate_us.detach().to(dtype=torch.float16).contiguous(),
            "up_us": up_us.detach().to(dtype=torch.float16).contiguous(),
            "down_svh": down_svh.detach().to(dtype=torch.float16).contiguous(),
        }

    def _resize_basis_for(self, state_dict, prefix: str, assign: bool) -> None:
        for key in self._SHARED_BASIS_BUFFER_KEYS:
            t = state_dict.get(f"{prefix}{key}", None)
            if not isinstance(t, torch.Tensor):
                continue
            cur = getattr(self, key, None)
            if isinstance(cur, torch.Tensor) and cur.shape == t.shape and cur.dtype == t.dtype:
                continue
            setattr(self, key, t.detach() if assign else torch.empty_like(t))

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        self._resize_basis_for(state_dict, prefix, bool(local_metadata.get("assign_to_params_buffers", False)))
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
        self._invalidate_runtime_cache()

    def _act_type(self) -> int:
        hidden_act = str(getattr(self.config, "hidden_act", "silu")).lower()
        if hidden_act != "silu":
            raise RuntimeError(f"Unsupported hidden_act for packed CUDA path: {hidden_act}")
        return 0

    # ---- runtime cache ----------------------------------------------------------------------------
    def _invalidate_runtime_cache(self) -> None:
        self._runtime_cache_ready = False
        self._runtime_cache_device: Optional[torch.device] = None
        self._runtime_warmed = False
        self._cached_token_count = -1
        self._cached_flat_token_ids: Optional[torch.Tensor] = None
        layer = getattr(self, "_packed_layer", None)
        if layer is not None:
            layer.close()
        self._packed_layer = None

    def _ensure_runtime_cache(self, device: torch.device) -> None:
        if self._runtime_cache_ready and self._runtime_cache_device == device:
            return
        super_items, packed_items = [], []
        for idx, module in enumerate(self.experts):
            if module is None:
                continue
            if idx in self._super_expert_set:
                super_items.append((idx, module))
            elif getattr(module, "is_bitsmoe_packed", False):
                packed_items.append((idx, module))
            else:
                raise RuntimeError(
                    f"Layer {self.layer_idx} expert {idx} is active but not packed. "
                    "BitsMoE forward expects non-super routed experts to use packed kernel.")
        self._super_expert_items = super_items
        self._packed_expert_count = len(packed_items)
        self._packed_intermediate_size = int(packed_items[0][1].intermediate_size) if packed_items else 0
        g2l = torch.full((self.num_experts,), -1, dtype=torch.int32)
        for local, (idx, _) in enumerate(packed_items):
            g2l[idx] = local
        self._packed_global_to_local = g2l.to(device)
        self._identity_map = self._packed_expert_count == self.num_experts and not super_items
        modules = [m for _, m in packed_items]
        for tag in _TAGS:
            for f in _FIELDS:
                setattr(self, f"_{tag}_{f}_static", tuple(getattr(m, f"{tag}_{f}_buffer") for m in modules))
        self._packed_layer = None
        if modules and device.type == "cuda" and _HAS_MLP_FORWARD_CUDA:
            from bitsmoe_b200.layer import PackedLayer
            self._act_type()
            self._packed_layer = PackedLayer.from_expert_modules(
                modules, self._packed_intermediate_size,
                int(self.shared_u_down.shape[1]) if self.shared_u_down.numel() else int(self.shared_vh_gate_proj.shape[0]),
                self.shared_vh_gate_proj, self.shared_vh_up_proj, self.shared_u_down, device=device)
        self._runtime_cache_ready = True
        self._runtime_cache_device = device
        self._runtime_warmed = False

    def _get_flat_token_ids(self, token_count: int, device: torch.device) -> torch.Tensor:
        ids = self._cached_flat_token_ids
        if ids is None or self._cached_token_count != token_count or ids.device != device:
            ids = torch.arange(token_count, dtype=torch.long, device=device).repeat_interleave(self.top_k)
            self._cached_flat_token_ids, self._cached_token_count = ids, token_count
        return ids

    # ---- routing / experts at the reference's internal boundaries -----------------------------------
    def _build_packed_routing(self, flat_selected_experts: torch.Tensor, flat_token_ids: torch.Tensor,
                              flat_route_weights_fp32: torch.Tensor):
        """-> (token_indices int32, expert_offsets int32 [E'+1], route_flat fp32) or None when the block has no
        packed experts.  Built by one kernel; the arrays keep their full length T*k and entries past
        expert_offsets[-1] are unspecified (the op walks expert_offsets)."""
        if self._packed_expert_count <= 0 or self._packed_global_to_local is None:
            return None
        from bitsmoe_b200.layer import route_build
        k = self.top_k
        tok, off, rw, _, _ = route_build(flat_selected_experts.reshape(-1, k), flat_route_weights_fp32.reshape(-1, k),
                                         self._packed_expert_count,
                                         None if self._identity_map else self._packed_global_to_local)
        return tok, off, rw

    def _run_super_experts(self, hidden_states, final_hidden_states, flat_selected_experts, flat_token_ids,
                           flat_route_weights_hidden) -> None:
        for expert_idx, module in self._super_expert_items:
            rows = (flat_selected_experts == expert_idx).nonzero(as_tuple=True)[0]
            if rows.numel() == 0:
                continue
            token_ids = flat_token_ids[rows]
            out = module(hidden_states.index_select(0, token_ids)) * flat_route_weights_hidden[rows].unsqueeze(-1)
            final_hidden_states.index_add_(0, token_ids, out.to(hidden_states.dtype))

    def prepare_runtime_fastpath(self, warmup: bool = True) -> None:
        device = self._runtime_device()
        self._ensure_runtime_cache(device)
        if warmup:
            self._warmup_runtime_once(device)

    def _warmup_runtime_once(self, device: torch.device) -> None:
        if self._runtime_warmed or device.type != "cuda" or self._packed_layer is None:
            return
        if self.shared_vh_gate_proj.numel() == 0 or self.shared_vh_up_proj.numel() == 0:
            return
        x = torch.zeros((1, int(self.shared_vh_gate_proj.shape[1])), dtype=torch.float16, device=device)
        logits = torch.zeros((1, self.num_experts), dtype=torch.float32, device=device)
        with torch.no_grad():
            self._fused_forward(x, logits=logits)
        torch.cuda.synchronize(device)
        self._runtime_warmed = True

    def _packed_forward_cuda(self, h_gate_proj, h_up_proj, token_indices, expert_offsets_t, route_flat,
                             token_count: int) -> torch.Tensor:
        rank_out = int(self.shared_u_down.shape[1])
        if int(self._packed_intermediate_size) <= 0:
            raise RuntimeError(f"Layer {self.layer_idx} has no packed experts for CUDA path.")
        args = [getattr(self, f"_{tag}_{f}_static") for tag in _TAGS for f in _FIELDS]
        rank_accum = mlp_forward_cuda.moe_packed_forward(h_gate_proj, h_up_proj, token_indices, expert_offsets_t,
                                                         route_flat, *args, rank_out,
                                                         int(self._packed_intermediate_size), self._act_type())
        if rank_accum.shape[0] != token_count or rank_accum.shape[1] != rank_out:
            raise RuntimeError(f"Invalid rank_accum shape from CUDA kernel: got {tuple(rank_accum.shape)}, "
                               f"expected ({token_count}, {rank_out})")
        return torch.matmul(rank_accum.to(self.shared_u_down.dtype), self.shared_u_down.T)

    def _packed_forward_grouped(self, h_gate_proj, h_up_proj, token_indices, expert_offsets_t, route_flat,
                                token_count: int) -> torch.Tensor:
        if self.shared_u_down.numel() == 0:
            raise RuntimeError(f"Layer {self.layer_idx} missing shared_u_down for packed routed experts.")
        if not (_HAS_MLP_FORWARD_CUDA and mlp_forward_cuda is not None and h_gate_proj.is_cuda and h_up_proj.is_cuda):
            raise RuntimeError("Packed routed experts require CUDA mlp_forward extension; "
                               "python fallback is intentionally disabled.")
        return self._packed_forward_cuda(h_gate_proj, h_up_proj, token_indices, expert_offsets_t, route_flat, token_count)

    # ---- dense modules of the block on the library's kernels --------------------------------------------
    @staticmethod
    def _plain_linear(m) -> bool:
        return isinstance(m, nn.Linear) and m.bias is None

    def _library_gate_logits(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """x @ gate.weight.T by the library when the gate is a bias-free Linear on the GPU (inference), else None."""
        gate = getattr(self, "gate", None)
        if not (x.is_cuda and self._plain_linear(gate) and not torch.is_grad_enabled()):
            return None
        from bitsmoe_b200.layer import gate_logits
        return gate_logits(x, gate.weight)

    def _library_dense_mlp(self, x: torch.Tensor, mlp, token_gate=None) -> Optional[torch.Tensor]:
        """SwiGLU MLP ``mlp`` (gate_proj / up_proj / down_proj, bias-free, SiLU) by the library, scaled per token by
        sigmoid(token_gate(x)) when a one-output bias-free Linear is given; None when the module is of another kind."""
        parts = [getattr(mlp, n, None) for n in ("gate_proj", "up_proj", "down_proj")]
        if not (x.is_cuda and all(self._plain_linear(p) for p in parts) and not torch.is_grad_enabled()):
            return None
        if token_gate is not None and not (self._plain_linear(token_gate) and token_gate.weight.shape[0] == 1):
            return None
        if parts[0].weight.shape[0] % 2:
            return None
        from bitsmoe_b200.layer import dense_mlp
        return dense_mlp(x, parts[0].weight, parts[1].weight, parts[2].weight,
                         None if token_gate is None else token_gate.weight)

    # ---- fused path -----------------------------------------------------------------------------------
    def _require_fused(self, x: torch.Tensor):
        if self.shared_vh_gate_proj.numel() == 0 or self.shared_vh_up_proj.numel() == 0:
            raise RuntimeError(f"Layer {self.layer_idx} missing shared_vh basis for packed routed experts.")
        if self.shared_u_down.numel() == 0:
            raise RuntimeError(f"Layer {self.layer_idx} missing shared_u_down for packed routed experts.")
        if self._packed_layer is None or not x.is_cuda:
            raise RuntimeError("Packed routed experts require CUDA mlp_forward extension; "
                               "python fallback is intentionally disabled.")
        return self._packed_layer

    def _fused_forward(self, x: torch.Tensor, logits: Optional[torch.Tensor] = None,
                       topk: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                       residual: Optional[torch.Tensor] = None, round_weights: bool = True) -> torch.Tensor:
        """x [T,H]; either router ``logits`` [T,E] (softmax/top-k run on the device) or a precomputed
        ``topk = (idx [T,k], weights [T,k])``.  Returns y [T,H] = packed experts (+ residual)."""
        layer = self._require_fused(x)
        g2l = None if self._identity_map else self._packed_global_to_local
        if topk is None:
            return layer.forward(x, logits, self.top_k, getattr(self, "norm_topk_prob", True),
                                 x.dtype if round_weights else None, residual=residual, global_to_local=g2l)
        from bitsmoe_b200.layer import route_build
        idx, w = topk
        tok, off, rw, _, _ = route_build(idx, w, self._packed_expert_count, g2l)
        hg, hu = layer.basis_project(x)
        acc = layer.experts_forward(hg, hu, tok, off, rw)
        return layer.combine_down_basis(acc, x.dtype, residual=residual)
