"""Qwen3-MoE block (interface of bitsmoe/models/qwen3moe/bitsmoe_block.py:10-98)."""
from __future__ import annotations

import copy
from typing import List, Optional

import torch
import torch.nn as nn

from bitsmoe_b200.models.base_block import BitsMoE_BaseSparseMoeBlock


class BitsMoE_Qwen3MoeSparseMoeBlock(BitsMoE_BaseSparseMoeBlock):
    _TRACK_SUPER = True

    def __init__(self, config, layer_idx: int, source_block: Optional[nn.Module] = None,
                 super_experts: Optional[List[int]] = None, copy_source_experts: bool = True):
        super().__init__()
        self.config = config
        self.layer_idx = int(layer_idx)
        self.num_experts = int(getattr(config, "num_experts", 0))
        self.top_k = int(getattr(config, "num_experts_per_tok", 0))
        self.norm_topk_prob = bool(getattr(config, "norm_topk_prob", True))
        if source_block is None:
            raise ValueError(f"source_block is required for {type(self).__name__}")
        self.gate = copy.deepcopy(source_block.gate)
        self._adopt_experts(source_block, copy_source_experts)
        self._adopt_extras(source_block)
        self._init_bitsmoe_common_state(super_experts=super_experts, track_super_projected_weights=self._TRACK_SUPER)

    def _adopt_experts(self, source_block, copy_source_experts: bool) -> None:
        # experts are filled in by the caller through set_expert
        self.experts = nn.ModuleList([None] * len(source_block.experts))

    def _adopt_extras(self, source_block) -> None:
        pass

    def _shared_contribution(self, hidden_states: torch.Tensor) -> Optional[torch.Tensor]:
        return None

    def forward(self, hidden_states: torch.Tensor):
        batch, seq, hidden = hidden_states.shape
        x = hidden_states.reshape(-1, hidden)
        self._ensure_runtime_cache(x.device)
        router_logits = self._library_gate_logits(x)
        if router_logits is None:
            router_logits = self.gate(x)
        residual = self._shared_contribution(x)
        if self._super_expert_items:
            # dense (unquantised) experts need the selection on the torch side as well
            from bitsmoe_b200.layer import route_topk
            idx, w = route_topk(router_logits, self.top_k, self.norm_topk_prob, x.dtype)
            dense = torch.zeros_like(x)
            self._run_super_experts(x, dense, idx.reshape(-1).long(), self._get_flat_token_ids(x.shape[0], x.device),
                                    w.reshape(-1).to(x.dtype))
            residual = dense if residual is None else residual + dense
            y = self._fused_forward(x, topk=(idx, w), residual=residual)
        else:
            y = self._fused_forward(x, logits=router_logits, residual=residual)
        y = y.reshape(batch, seq, hidden)
        # (hidden, router_logits) as the reference returns; hidden only where the surrounding decoder layer expects
        # that (fused-expert models of transformers 5.x: the patcher clears the flag)
        return (y, router_logits) if getattr(self, "return_router_logits", True) else y
