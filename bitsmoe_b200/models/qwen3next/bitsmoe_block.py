"""Qwen3-Next block: Qwen3-MoE routing plus one sigmoid-gated dense shared expert
(interface of bitsmoe/models/qwen3next/bitsmoe_block.py:10-150)."""
from __future__ import annotations

import copy
from typing import Optional

import torch
import torch.nn as nn

from bitsmoe_b200.models.base_block import BitsMoE_BaseSparseMoeBlock
from bitsmoe_b200.models.qwen3moe.bitsmoe_block import BitsMoE_Qwen3MoeSparseMoeBlock


class BitsMoE_Qwen3NextSparseMoeBlock(BitsMoE_Qwen3MoeSparseMoeBlock):
    _TRACK_SUPER = False

    def _adopt_experts(self, source_block, copy_source_experts: bool) -> None:
        if copy_source_experts:
            self.experts = nn.ModuleList([copy.deepcopy(e) for e in source_block.experts])
        else:
            self.experts = nn.ModuleList([None] * len(source_block.experts))

    def _adopt_extras(self, source_block) -> None:
        if hasattr(source_block, "shared_expert"):
            self.shared_expert = copy.deepcopy(source_block.shared_expert)
        if hasattr(source_block, "shared_expert_gate"):
            self.shared_expert_gate = copy.deepcopy(source_block.shared_expert_gate)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        # assign-aware: bind checkpoint basis tensors directly instead of allocating placeholders
        self._resize_basis_for(state_dict, prefix, bool(local_metadata.get("assign_to_params_buffers", False)))
        nn.Module._load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                                        unexpected_keys, error_msgs)
        self._invalidate_runtime_cache()

    def _shared_contribution(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        if hasattr(self, "shared_expert") and hasattr(self, "shared_expert_gate"):
            y = self._library_dense_mlp(x, self.shared_expert, self.shared_expert_gate)
            if y is not None:
                return y
            return torch.sigmoid(self.shared_expert_gate(x)) * self.shared_expert(x)
        return None
