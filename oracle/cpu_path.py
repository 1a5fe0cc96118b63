"""Dequantise-then-matmul forward of one layer on the host cores (torch CPU).  Test
infrastructure and the timed CPU baseline.

The reference has no CPU forward (bitsmoe/models/base_block.py:428-438 disables it); this is the
pure-PyTorch path its semantics imply: decode every routed expert's codes through the meta
tables (bitsmoe/quant/packer.py:79-101), W = q * scale (bitsmoe/quant/quantizer.py:116-128),
then the block algebra of bitsmoe/models/qwen3moe/bitsmoe_block.py:39-98 and
bitsmoe/models/base_block.py:409-414 in fp32.  Decoding is vectorised per slab (numpy) so that
the timing reflects arithmetic, not interpreter overhead; it is checked against the loop decoder
of oracle.packer in the tests.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import forward as oforward
from .packer import K_STAGE, MICROS_PER_TILE, N_MICRO, N_TILE, words_per_row

_LANES = np.arange(N_MICRO, dtype=np.uint32)


def dequant_matrix(buf: Dict[str, np.ndarray], dim: int) -> Dict[str, np.ndarray]:
    """fp32 W [stored rows, dim] with W = q * scale, plus rank_idx and S."""
    slab_meta = np.asarray(buf["slab_meta_buffer"]).astype(np.int64).reshape(-1, 4)
    tile_meta = np.asarray(buf["tile_meta_buffer"]).astype(np.int64).reshape(-1, 3)
    payload = np.asarray(buf["payload_buffer"])
    scale = np.asarray(buf["scale_buffer"])
    n_rows = int(slab_meta[:, 1].sum()) if slab_meta.size else 0
    w = np.zeros((n_rows, dim), dtype=np.float32)
    for i in range(slab_meta.shape[0]):
        bits, k, rank_off, tile_off = (int(v) for v in slab_meta[i])
        tile_end = int(slab_meta[i + 1, 3]) if i + 1 < slab_meta.shape[0] else tile_meta.shape[0]
        tiles = tile_end - tile_off
        if tiles <= 0:
            continue
        wpr = words_per_row(bits)
        wpt = k * MICROS_PER_TILE * wpr
        p0 = int(tile_meta[tile_off, 0])
        s0 = int(tile_meta[tile_off, 1])
        contiguous = all(int(tile_meta[tile_off + t, 0]) == p0 + t * wpt and int(tile_meta[tile_off + t, 1]) == s0 + t * k
                         for t in range(tiles))
        if not contiguous:
            raise ValueError("tiles of a slab are expected back to back")
        per_tile = payload[p0:p0 + tiles * wpt].reshape(tiles, wpt)
        words = np.empty((k, tiles, MICROS_PER_TILE, wpr), dtype=np.uint32)
        full = (k // K_STAGE) * K_STAGE
        split = full * MICROS_PER_TILE * wpr
        if full:
            words[:full] = per_tile[:, :split].reshape(tiles, full // K_STAGE, MICROS_PER_TILE, K_STAGE, wpr).transpose(
                1, 3, 0, 2, 4).reshape(full, tiles, MICROS_PER_TILE, wpr)
        if k > full:
            words[full:] = per_tile[:, split:].reshape(tiles, MICROS_PER_TILE, k - full, wpr).transpose(2, 0, 1, 3)
        if bits == 16:
            lo = (words & np.uint32(0xFFFF)).astype(np.uint16)
            hi = (words >> np.uint32(16)).astype(np.uint16)
            vals = np.stack((lo, hi), axis=-1).reshape(k, tiles * N_TILE).view(np.float16).astype(np.float32)
        else:
            u = np.zeros((k, tiles, MICROS_PER_TILE, N_MICRO), dtype=np.int32)
            for p in range(bits):
                u |= (((words[..., p, None] >> _LANES) & np.uint32(1)).astype(np.int32) << p)
            q = (2 * u - 1) if bits == 1 else (u - (1 << (bits - 1)))
            sc = scale[s0:s0 + tiles * k].reshape(tiles, k).astype(np.float32).T   # [k, tiles]
            vals = (q.reshape(k, tiles, N_TILE).astype(np.float32) * sc[:, :, None]).reshape(k, tiles * N_TILE)
        n_cols = min(dim, tiles * N_TILE)
        w[rank_off:rank_off + k, :n_cols] = vals[:, :n_cols]
    return {"w": w, "rank_idx": np.asarray(buf["rank_idx_buffer"]).astype(np.int64)[:n_rows],
            "s": np.asarray(buf["s_buffer"]).astype(np.float32)[:n_rows]}


class CpuLayer:
    """Holds one layer's packed buffers on the host and runs the fp32 forward, dequantising the experts
    that receive tokens on every call."""

    def __init__(self, experts: Sequence[Dict[str, Dict[str, np.ndarray]]], vh_gate: torch.Tensor, vh_up: torch.Tensor,
                 u_down: torch.Tensor, intermediate: int, top_k: int, norm_topk_prob: bool = True,
                 weight_dtype: Optional[torch.dtype] = torch.float16):
        self.experts = experts          # [{"gate": buf, "up": buf, "down": buf}]
        self.vh_gate, self.vh_up, self.u_down = vh_gate.float(), vh_up.float(), u_down.float()
        self.intermediate, self.top_k = intermediate, top_k
        self.norm_topk_prob, self.weight_dtype = norm_topk_prob, weight_dtype

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        idx, w = oforward.router(logits, self.top_k, self.norm_topk_prob, self.weight_dtype)
        tok, off, rw = oforward.build_routing(idx, w, len(self.experts))
        xf = x.float()
        hg = (xf @ self.vh_gate.T).half().float()
        hu = (xf @ self.vh_up.T).half().float()
        rank_out = self.u_down.shape[1]
        acc = torch.zeros((x.shape[0], rank_out), dtype=torch.float32)
        offs = off.tolist()
        for e, ex in enumerate(self.experts):
            a0, a1 = offs[e], offs[e + 1]
            if a1 <= a0:
                continue
            t = tok[a0:a1].long()
            parts = {k: dequant_matrix(ex[k], self.intermediate) for k in ("gate", "up", "down")}
            g = (hg[t][:, parts["gate"]["rank_idx"]] * torch.from_numpy(parts["gate"]["s"])) @ torch.from_numpy(parts["gate"]["w"])
            u = (hu[t][:, parts["up"]["rank_idx"]] * torch.from_numpy(parts["up"]["s"])) @ torch.from_numpy(parts["up"]["w"])
            z = torch.nn.functional.silu(g) * u
            d = z @ torch.from_numpy(parts["down"]["w"]).T
            d = d * torch.from_numpy(parts["down"]["s"]) * rw[a0:a1, None]
            ridx = torch.from_numpy(parts["down"]["rank_idx"])
            keep = ridx < rank_out
            acc.index_put_((t[:, None].expand(-1, int(keep.sum())), ridx[keep][None, :].expand(t.numel(), -1)),
                           d[:, keep], accumulate=True)
        return (acc.half().float() @ self.u_down.T).to(x.dtype)
