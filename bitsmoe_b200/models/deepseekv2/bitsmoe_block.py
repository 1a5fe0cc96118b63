"""DeepSeek-V2 block: third-party gate module returning (topk_idx, topk_weight, aux_loss), dense
shared experts added to the output (interface of bitsmoe/models/deepseekv2/bitsmoe_block.py:10-127)."""
from __future__ import annotations

import copy
from typing import List, Optional

import torch
import torch.nn as nn

from bitsmoe_b200.models.base_block import BitsMoE_BaseSparseMoeBlock


class AddAuxiliaryLoss(torch.autograd.Function):
    """Identity on x that routes a unit gradient into the auxiliary loss (training only)."""

    @staticmethod
    def forward(ctx, x, loss):
        assert loss.numel() == 1
        ctx.dtype = loss.dtype
        ctx.required_aux_loss = loss.requires_grad
        return x

    @staticmethod
    def backward(ctx, grad_output):
        grad_loss = torch.ones(1, dtype=ctx.dtype, device=grad_output.device) if ctx.required_aux_loss else None
        return grad_output, grad_loss


class BitsMoE_DeepSeekSparseMoeBlock(BitsMoE_BaseSparseMoeBlock):
    def __init__(self, config, layer_idx: int, source_block: Optional[nn.Module] = None,
                 super_experts: Optional[List[int]] = None, copy_source_experts: bool = True):
        super().__init__()
        self.config = config
        self.layer_idx = int(layer_idx)
        self.num_experts_per_tok = int(getattr(config, "num_experts_per_tok", 0))
        self.top_k = self.num_experts_per_tok
        if source_block is None:
            raise ValueError("source_block is required for BitsMoE_DeepSeekSparseMoeBlock")
        self.gate = copy.deepcopy(source_block.gate)
        if copy_source_experts:
            self.experts = nn.ModuleList([copy.deepcopy(e) if e is not None else None for e in source_block.experts])
        else:
            self.experts = nn.ModuleList([None] * len(source_block.experts))
        self.num_experts = len(self.experts)
        if hasattr(source_block, "shared_experts"):
            self.shared_experts = copy.deepcopy(source_block.shared_experts)
        for name in ("ep_size", "experts_per_rank", "ep_rank"):
            if hasattr(source_block, name):
                setattr(self, name, int(getattr(source_block, name)))
        self._init_bitsmoe_common_state(super_experts=super_experts, track_super_projected_weights=True)

    def forward(self, hidden_states: torch.Tensor):
        orig_shape = hidden_states.shape
        topk_idx, topk_weight, aux_loss = self.gate(hidden_states)
        x = hidden_states.reshape(-1, orig_shape[-1])
        self._ensure_runtime_cache(x.device)
        idx = topk_idx.reshape(-1, topk_idx.shape[-1])
        w = topk_weight.reshape(-1, topk_weight.shape[-1]).to(torch.float32)   # not rounded through x.dtype
        residual = None
        if getattr(self.config, "n_shared_experts", None) is not None and hasattr(self, "shared_experts"):
            residual = self._library_dense_mlp(x, self.shared_experts)
            if residual is None:
                residual = self.shared_experts(hidden_states).reshape(-1, orig_shape[-1])
        if self._super_expert_items:
            dense = torch.zeros_like(x)
            self._run_super_experts(x, dense, idx.reshape(-1).long(), self._get_flat_token_ids(x.shape[0], x.device),
                                    w.reshape(-1).to(x.dtype))
            residual = dense if residual is None else residual + dense
        y = self._fused_forward(x, topk=(idx, w), residual=residual).reshape(*orig_shape)
        if self.training and aux_loss is not None:
            y = AddAuxiliaryLoss.apply(y, aux_loss)
        return y
