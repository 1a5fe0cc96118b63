"""Forward algebra of a BitsMoE block on the CPU (torch).  Test infrastructure.

Restates, as dequantise-then-matmul:
  router            bitsmoe/models/qwen3moe/bitsmoe_block.py:45-51, :66-68
                    (softmax fp32 -> top-k -> optional renorm -> round through the
                    activation dtype); the DeepSeek block does not round
                    (bitsmoe/models/deepseekv2/bitsmoe_block.py:79-80)
  routing build     bitsmoe/models/base_block.py:258-289 (expert-contiguous
                    permutation, offsets); the reference sorts with an unstable
                    argsort, this oracle defines the order inside an expert as
                    ascending flat (token, slot) index
  packed forward    bitsmoe/algorithms/cpp/mlp_forward.cu:722-750 (A = h*s,
                    B = q*scale), :1478-1501 (z = silu(g)*u), :2036-2066
                    (rank_accum[token, logical rank] += acc * s * route weight)
  down basis        bitsmoe/models/base_block.py:414 (rank_accum.half() @ U_down.T)

Two flavours: ``mode="fp32"`` keeps every operand in fp32 (accumulating in
fp64); ``mode="faithful"`` rounds h*s, q*scale and z to fp16 before the
products as the reference tensor-core kernels do.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from . import packer


def router(logits: torch.Tensor, top_k: int, norm_topk_prob: bool = True,
           weight_dtype: Optional[torch.dtype] = torch.float16) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (topk_idx int64 [T,k], topk_w fp32 [T,k]); ties go to the lower expert id."""
    p = F.softmax(logits, dim=1, dtype=torch.float32)
    vals, idx = torch.sort(p, dim=-1, descending=True, stable=True)
    w, idx = vals[:, :top_k].contiguous(), idx[:, :top_k].contiguous()
    if norm_topk_prob:
        w = w / w.sum(dim=-1, keepdim=True)
    if weight_dtype is not None:
        w = w.to(weight_dtype)
    return idx, w.to(torch.float32)


def build_routing(topk_idx: torch.Tensor, topk_w: torch.Tensor, num_local: int,
                  global_to_local: Optional[torch.Tensor] = None):
    """-> token_indices int32 [A'], expert_offsets int32 [num_local+1], route_flat fp32 [A']."""
    T, k = topk_idx.shape
    flat_e = topk_idx.reshape(-1).long()
    if global_to_local is not None:
        flat_e = global_to_local.long()[flat_e]
    flat_t = torch.arange(T).repeat_interleave(k)
    flat_w = topk_w.reshape(-1).to(torch.float32)
    keep = flat_e >= 0
    flat_e, flat_t, flat_w = flat_e[keep], flat_t[keep], flat_w[keep]
    order = torch.sort(flat_e, stable=True).indices
    counts = torch.bincount(flat_e, minlength=num_local)
    offsets = torch.zeros(num_local + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    return flat_t[order].to(torch.int32), offsets, flat_w[order]


def canonical_routing(token_indices, expert_offsets, route_flat):
    """Sort every expert segment by (token, weight) so that an unstable sort on the
    other side compares equal."""
    tok = np.asarray(token_indices).copy()
    w = np.asarray(route_flat).copy()
    off = np.asarray(expert_offsets)
    for e in range(len(off) - 1):
        a, b = int(off[e]), int(off[e + 1])
        o = np.lexsort((w[a:b], tok[a:b]))
        tok[a:b], w[a:b] = tok[a:b][o], w[a:b][o]
    return tok, w


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


class DecodedExpert:
    """Dequantised view of one expert's three matrices (from the ten buffers each)."""

    def __init__(self, gate: Dict, up: Dict, down: Dict, intermediate: int):
        self.parts = {}
        for name, buf in (("gate", gate), ("up", up), ("down", down)):
            d = packer.decode_matrix(buf, intermediate)
            self.parts[name] = {
                "w": torch.from_numpy(d["w"]),
                "rank_idx": torch.from_numpy(d["rank_idx"]).long(),
                "s": torch.from_numpy(d["s"]),
            }


def packed_forward(h_gate: torch.Tensor, h_up: torch.Tensor, token_indices: torch.Tensor,
                   expert_offsets: torch.Tensor, route_weights: torch.Tensor,
                   experts: Sequence[DecodedExpert], rank_out: int, mode: str = "fp32") -> torch.Tensor:
    """The op contract of ``moe_packed_forward``: returns rank_accum fp32 [T, rank_out]."""
    T = h_gate.shape[0]
    acc_t = torch.float64 if mode == "fp32" else torch.float32
    out = torch.zeros((T, rank_out), dtype=acc_t)
    hg, hu = h_gate.to(torch.float32), h_up.to(torch.float32)
    off = expert_offsets.tolist()
    for e in range(len(experts)):
        a0, a1 = off[e], off[e + 1]
        if a1 <= a0:
            continue
        ex = experts[e]
        tok = token_indices[a0:a1].long()
        rw = route_weights[a0:a1].to(torch.float32)

        def proj(h, part):
            a = h[tok][:, part["rank_idx"]] * part["s"]
            w = part["w"]
            if mode == "faithful":
                a, w = a.to(torch.float16).float(), w.to(torch.float16).float()
            return (a.to(acc_t) @ w.to(acc_t)).to(torch.float32)

        g = proj(hg, ex.parts["gate"])
        u = proj(hu, ex.parts["up"])
        z = silu(g) * u
        d = ex.parts["down"]
        wd = d["w"]
        if mode == "faithful":
            z, wd = z.to(torch.float16).float(), wd.to(torch.float16).float()
        acc = (z.to(acc_t) @ wd.to(acc_t).T).to(torch.float32)
        contrib = acc * d["s"] * rw[:, None]
        valid = d["rank_idx"] < rank_out
        idx = d["rank_idx"][valid]
        out.index_put_((tok[:, None].expand(-1, idx.numel()), idx[None, :].expand(tok.numel(), -1)),
                       contrib[:, valid].to(acc_t), accumulate=True)
    return out.to(torch.float32)


def basis_project(x: torch.Tensor, vh: torch.Tensor) -> torch.Tensor:
    """h = x @ Vh.T rounded to fp16 (qwen3moe/bitsmoe_block.py:63-64)."""
    return (x.to(torch.float64) @ vh.to(torch.float64).T).to(torch.float16)


def down_basis(rank_accum: torch.Tensor, u_down: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """y = fp16(rank_accum) @ U_down.T (base_block.py:414)."""
    y = rank_accum.to(torch.float16).to(torch.float64) @ u_down.to(torch.float64).T
    return y.to(out_dtype)


def dense_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """SwiGLU MLP of a shared expert, fp64 accumulate, result in fp32."""
    xd = x.to(torch.float64)
    g = xd @ w_gate.to(torch.float64).T
    u = xd @ w_up.to(torch.float64).T
    return ((silu(g) * u) @ w_down.to(torch.float64).T).to(torch.float32)


def layer_forward(x: torch.Tensor, logits: torch.Tensor, vh_gate: torch.Tensor, vh_up: torch.Tensor,
                  u_down: torch.Tensor, experts: Sequence[DecodedExpert], top_k: int,
                  norm_topk_prob: bool = True, weight_dtype: Optional[torch.dtype] = torch.float16,
                  mode: str = "fp32", shared: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    """Whole block for one batch of tokens ``x [T,H]`` given router logits ``[T,E]``."""
    idx, w = router(logits, top_k, norm_topk_prob, weight_dtype)
    tok, off, rw = build_routing(idx, w, len(experts))
    hg, hu = basis_project(x, vh_gate), basis_project(x, vh_up)
    acc = packed_forward(hg, hu, tok, off, rw, experts, u_down.shape[1], mode=mode)
    y = down_basis(acc, u_down, torch.float32)
    if shared is not None:
        sh = dense_mlp(x, shared["gate"], shared["up"], shared["down"])
        if "gate_logit_w" in shared:
            sh = torch.sigmoid(x.to(torch.float64) @ shared["gate_logit_w"].to(torch.float64).T).float() * sh
        y = y + sh
    return {"y": y.to(x.dtype), "y_fp32": y, "rank_accum": acc, "topk_idx": idx, "topk_w": w,
            "token_indices": tok, "expert_offsets": off, "route_flat": rw, "h_gate": hg, "h_up": hu}
