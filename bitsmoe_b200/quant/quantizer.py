"""Symmetric scale-only quantisation of expert factors (host-side, any torch device).

Same contract as ``bitsmoe.quant.quantizer`` (bitsmoe/quant/quantizer.py:17-128):
``quantize_symmetric`` returns signed int8 codes in [-2^(b-1), 2^(b-1)-1] and one scale per
channel; 2/3/4-bit scales are refined by alternating least squares, wider codes use absmax,
1-bit is sign with a mean-|x| scale.  ``pack_quantized`` / ``unpack_quantized`` go through
the CUDA bit-plane codec.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .bitpack import BitPack

_REFINED = (2, 3, 4)


def pack_quantized(W_q: Tensor, bits: int):
    return BitPack.pack(W_q, bits)


def unpack_quantized(W_q: Tensor, bits: int, original_size: int):
    return BitPack.unpack(W_q, bits, original_size)


def _code_range(bits: int):
    hi = (1 << (bits - 1)) - 1
    return -hi - 1, hi


def quantize_symmetric(x: Tensor, bits: int = 8, dim: int = 0, eps: float = 1e-8, iters: int = 50):
    if bits <= 0:
        raise ValueError(f"bits must be in (0, 8], got {bits}")
    if x.numel() == 0:
        return x.to(torch.int8), torch.tensor(1.0, device=x.device)
    mean_abs = x.abs().mean(dim=dim, keepdim=True).clamp(min=eps)
    if bits == 1:
        codes = torch.where(x < 0, -torch.ones_like(x), torch.ones_like(x))
        return codes.to(torch.int8), mean_abs.squeeze(dim)
    lo, hi = _code_range(bits)
    if bits in _REFINED:
        scale = mean_abs
        codes = None
        for _ in range(iters):
            codes = torch.clamp(torch.round(x / scale), lo, hi)
            xq = (x * codes).mean(dim=dim, keepdim=True)
            qq = (codes * codes).mean(dim=dim, keepdim=True)
            scale = (xq / (qq + eps)).clamp(min=eps)
        return codes.to(torch.int8), scale.squeeze(dim)
    scale = (x.abs().amax(dim=dim, keepdim=True) / hi).clamp(min=eps)
    codes = torch.clamp(torch.round(x / scale), lo, hi).to(torch.int8)
    return codes, scale.squeeze(dim)


def dequantize_symmetric(x_quant: Tensor, scale: Tensor, dim: int = 0) -> Tensor:
    return (x_quant.to(torch.float32) * scale.to(torch.float32).unsqueeze(dim)).to(torch.float16)
