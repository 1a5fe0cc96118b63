"""Symmetric scale-only quantiser (torch, CPU).  Test infrastructure.

Restates bitsmoe/quant/quantizer.py:30-84 (``quantize_symmetric``) and
:116-128 (``dequantize_symmetric``).  Codes are signed integers in
[-2^(b-1), 2^(b-1)-1]; there is no stored zero point.

  b in {2,3,4}: scale starts at mean|x| and is refined ``iters`` times with
                q = clamp(round(x/scale)), scale = <x,q>/(<q,q>+eps)
  b == 1      : q = sign(x) with sign(0) = +1, scale = mean|x|
  otherwise   : scale = max|x| / qmax
``round`` is round-half-to-even (torch.round).
"""
from __future__ import annotations

import torch


def quantize_symmetric(x: torch.Tensor, bits: int = 8, dim: int = 0, eps: float = 1e-8,
                       iters: int = 50):
    if bits <= 0:
        raise ValueError(f"bits must be in (0, 8], got {bits}")
    if x.numel() == 0:
        return x.to(torch.int8), torch.tensor(1.0)
    if bits == 1:
        scale = x.abs().mean(dim=dim, keepdim=True).clamp(min=eps)
        sgn = torch.sign(x)
        sgn = torch.where(sgn == 0, torch.ones_like(sgn), sgn)
        return sgn.to(torch.int8), scale.squeeze(dim)
    qmax = 2 ** (bits - 1) - 1
    qmin = -qmax - 1
    if bits in (2, 3, 4):
        scale = x.abs().mean(dim=dim, keepdim=True).clamp(min=eps)
        q = None
        for _ in range(iters):
            q = (x / scale).round().clamp(qmin, qmax)
            num = (x * q).mean(dim=dim, keepdim=True)
            den = (q * q).mean(dim=dim, keepdim=True)
            scale = (num / (den + eps)).clamp(min=eps)
        return q.to(torch.int8), scale.squeeze(dim)
    scale = (x.abs().amax(dim=dim, keepdim=True) / qmax).clamp(min=eps)
    q = (x / scale).round().clamp(qmin, qmax).to(torch.int8)
    return q, scale.squeeze(dim)


def dequantize_symmetric(q: torch.Tensor, scale: torch.Tensor, dim: int = 0) -> torch.Tensor:
    return (q.to(torch.float32) * scale.to(torch.float32).unsqueeze(dim)).to(torch.float16)
