"""Seeded synthetic BitsMoE layers of the benchmark shapes (stand-ins for real checkpoints).

Every routed expert matrix is a rank-major factor ~ N(0, 0.02) with a positive descending S,
rows get a bit width drawn i.i.d. from the configured distribution and are then ordered so
that wider rows come first in logical rank order (as an energy-guided allocation would), and
the result is quantised and packed into exactly the buffers the reference's checkpoints hold
(bitsmoe/quant/packer.py:711-724).  On a GPU each slab is quantised, bit-plane packed and reordered by one
launch of the library's fused kernel; on the host quantisation and bit-slicing run batched over all experts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .quant import packer

MTYPES = (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj"))


@dataclass(frozen=True)
class LayerConfig:
    name: str
    hidden: int
    num_experts: int
    intermediate: int
    top_k: int
    rank: int = 256
    bit_probs: Tuple[Tuple[int, float], ...] = ((2, 0.8), (3, 0.15), (4, 0.05))
    norm_topk_prob: bool = True
    shared_intermediate: int = 0        # width of the dense shared expert (0 = none)
    shared_gated: bool = False          # sigmoid(x . w) gate on the shared expert (Qwen3-Next)
    round_route_weights: bool = True    # Qwen blocks round weights through the activation dtype


QWEN3_30B = LayerConfig("qwen3-30b-a3b", 2048, 128, 768, 8)
QWEN3_NEXT_80B = LayerConfig("qwen3-next-80b-a3b", 2048, 512, 512, 10,
                             bit_probs=((2, 0.75), (3, 0.2), (4, 0.05)), shared_intermediate=512, shared_gated=True)
DEEPSEEK_V2_LITE = LayerConfig("deepseek-v2-lite", 2048, 64, 1408, 6, bit_probs=((2, 1.0),), norm_topk_prob=False,
                               shared_intermediate=2816, round_route_weights=False)
PRESETS = {c.name: c for c in (QWEN3_30B, QWEN3_NEXT_80B, DEEPSEEK_V2_LITE)}


def tiny(name: str = "tiny", hidden: int = 256, num_experts: int = 8, intermediate: int = 160, top_k: int = 2,
         rank: int = 80, **kw) -> LayerConfig:
    return LayerConfig(name, hidden, num_experts, intermediate, top_k, rank, **kw)


@dataclass
class SynthLayer:
    cfg: LayerConfig
    tables: Dict[str, Dict[str, List[torch.Tensor]]]      # tag -> field -> per-expert tensors
    vh_gate: torch.Tensor
    vh_up: torch.Tensor
    u_down: torch.Tensor
    shared: Optional[Dict[str, torch.Tensor]] = None
    extras: Dict[str, List[Dict[str, torch.Tensor]]] = field(default_factory=dict)  # tag -> per-expert full buffers

    def expert_state_dict(self, e: int, prefix: str) -> Dict[str, torch.Tensor]:
        """Checkpoint keys of expert ``e`` in the packer's schema (bitsmoe/models/base_mlp.py:192-206)."""
        out = {}
        for tag, mtype in MTYPES:
            fld = "vh" if tag == "down" else "u"
            buf = self.extras[tag][e]
            for k in packer.RUNTIME_KEYS:
                out[f"{prefix}.{mtype}.{fld}.{k}"] = buf[k]
            for k in ("s_buffer", "segments", "original_indices", "original_rank", "groupsize"):
                out[f"{prefix}.{mtype}.{k}"] = buf[k]
        return out


def draw_bits(cfg: LayerConfig, gen: torch.Generator, device) -> torch.Tensor:
    widths = torch.tensor([b for b, _ in cfg.bit_probs], device=device)
    probs = torch.tensor([p for _, p in cfg.bit_probs], device=device, dtype=torch.float32)
    pick = torch.multinomial(probs.expand(cfg.num_experts, -1), cfg.rank, replacement=True, generator=gen)
    return torch.sort(widths[pick], dim=1, descending=True).values  # [E, rank], wide rows first


def make_layer(cfg: LayerConfig, seed: int = 42, device="cpu", keep_full: bool = False) -> SynthLayer:
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    E, r, I, H = cfg.num_experts, cfg.rank, cfg.intermediate, cfg.hidden
    tiles = (I + packer.N_TILE - 1) // packer.N_TILE

    def normal(*shape, std=0.02):
        return torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * std

    vh_gate, vh_up = normal(r, H).half(), normal(r, H).half()
    u_down = normal(H, r).half()
    tables = {tag: {f: [] for f in ("payload", "rank_idx", "tile_meta", "slab_meta", "scale", "s")} for tag, _ in MTYPES}
    extras = {tag: [] for tag, _ in MTYPES}
    for tag, _ in MTYPES:
        R = normal(E, r, I)
        S = torch.sort(torch.randn(E, r, generator=gen, device=device).abs() + 0.05, dim=1, descending=True).values
        bits = draw_bits(cfg, gen, device)
        # On a GPU every slab goes through the library's fused quantise + pack + reorder kernel; on the host the rows
        # are quantised and bit-sliced in one batch per width and the slabs assembled from that.
        pre = None
        if device.type != "cuda":
            pre = {}
            for b in sorted({b for b, _ in cfg.bit_probs}):
                q, sc = packer.quantize_rows(R.view(E * r, I), b)
                pre[b] = (packer.codes_to_planes(q, b).view(E, r, tiles, packer.MICROS_PER_TILE, b), sc.view(E, r, tiles))
        bits_cpu = bits.cpu()
        for e in range(E):
            row_bits = bits_cpu[e]
            segs, start = [], 0
            while start < r:
                end = start
                while end < r and int(row_bits[end]) == int(row_bits[start]):
                    end += 1
                segs.append((int(row_bits[start]), (start, end)))
                start = end
            buf = packer.pack_rank_major(R[e], S[e], segs,
                                         precomputed=None if pre is None else {b: (pre[b][0][e], pre[b][1][e]) for b in pre})
            for f in tables[tag]:
                tables[tag][f].append(buf[f + "_buffer"])
            if keep_full:
                buf = dict(buf)
                buf["_rank_major"], buf["_s"], buf["_segments"] = R[e].clone(), S[e].clone(), segs
                extras[tag].append(buf)
    shared = None
    if cfg.shared_intermediate:
        shared = {"gate": normal(cfg.shared_intermediate, H).half(), "up": normal(cfg.shared_intermediate, H).half(),
                  "down": normal(H, cfg.shared_intermediate).half()}
        if cfg.shared_gated:
            shared["gate_logit_w"] = normal(1, H).half()
    return SynthLayer(cfg, tables, vh_gate, vh_up, u_down, shared, extras)


def router_logits(cfg: LayerConfig, tokens: int, seed: int = 0, zipf_s: float = 0.0, device="cpu") -> torch.Tensor:
    """fp32 N(0,1) logits; ``zipf_s`` > 0 adds log p_e of a Zipf(s) law over the expert index."""
    gen = torch.Generator(device=torch.device(device)).manual_seed(seed)
    logits = torch.randn(tokens, cfg.num_experts, generator=gen, device=device, dtype=torch.float32)
    if zipf_s > 0:
        p = 1.0 / torch.arange(1, cfg.num_experts + 1, device=device, dtype=torch.float32) ** zipf_s
        logits = logits + torch.log(p / p.sum())
    return logits


def activations(cfg: LayerConfig, tokens: int, seed: int = 1, dtype=torch.bfloat16, device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=torch.device(device)).manual_seed(seed)
    return torch.randn(tokens, cfg.hidden, generator=gen, device=device, dtype=torch.float32).to(dtype)


def to_packed_layer(layer: SynthLayer, device=None):
    from .layer import PackedLayer
    dev = torch.device(device) if device is not None else layer.vh_gate.device
    t = {tag: {f: [x.to(dev) for x in v] for f, v in fields.items()} for tag, fields in layer.tables.items()}
    return PackedLayer(t["gate"], t["up"], t["down"], layer.cfg.intermediate, layer.cfg.rank,
                       layer.vh_gate.to(dev), layer.vh_up.to(dev), layer.u_down.to(dev), device=dev)
