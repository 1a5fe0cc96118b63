"""uint32 bit-plane packing of int8 codes on the GPU.

Mirrors ``bitsmoe.quant.bitpack.BitPack`` (bitsmoe/quant/bitpack/__init__.py:19-134): same
class, same ``pack`` / ``unpack`` signatures, CUDA tensors only.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch
from torch import Tensor

from bitsmoe_b200 import capi


class BitPack:
    BIT_OFFSETS: Dict[int, int] = {1: 1, 2: 2, 3: 4, 4: 8, 6: 32, 8: 128}

    @staticmethod
    def _check_bits(bits: int) -> None:
        if bits not in BitPack.BIT_OFFSETS:
            raise ValueError(f"Unsupported bit width: {bits}")

    @staticmethod
    def pack(W_q: Tensor, bits: int) -> Tuple[Tensor, int]:
        """int8 [rows, cols] -> (uint32 [rows, ceil(cols/32)*bits], cols)."""
        BitPack._check_bits(bits)
        if W_q.dim() != 2:
            raise ValueError(f"BitPack.pack expects 2D tensor, got shape={tuple(W_q.shape)}")
        if W_q.dtype != torch.int8:
            raise TypeError(f"BitPack.pack only supports int8 input, got {W_q.dtype}")
        if not W_q.is_cuda:
            raise ValueError("BitPack.pack requires CUDA tensor input")
        W_q = W_q.contiguous()
        rows, cols = W_q.shape
        groups = (cols + 31) // 32
        out = torch.empty((rows, groups * bits), dtype=torch.uint32, device=W_q.device)
        with torch.cuda.device(W_q.device):
            capi.check(capi.lib().bm_pack_bitplanes_i8(W_q.data_ptr(), out.data_ptr(), rows, cols, bits,
                                                       capi.stream_ptr(W_q.device)))
        return out, cols

    @staticmethod
    def unpack(W_q: Tensor, bits: int, original_size: int) -> Tensor:
        """uint32 [rows, groups*bits] -> int8 [rows, original_size]."""
        BitPack._check_bits(bits)
        if W_q.dim() != 2:
            raise ValueError(f"BitPack.unpack expects 2D tensor, got shape={tuple(W_q.shape)}")
        if W_q.dtype != torch.uint32:
            raise TypeError(f"BitPack.unpack expects uint32 packed tensor, got {W_q.dtype}")
        if not W_q.is_cuda:
            raise ValueError("BitPack.unpack requires CUDA tensor input")
        if original_size < 0:
            raise ValueError(f"original_size must be non-negative, got {original_size}")
        W_q = W_q.contiguous()
        rows, width = W_q.shape
        if width % bits:
            raise ValueError(f"packed width {width} is not a multiple of bits={bits}")
        groups = width // bits
        if original_size > groups * 32:
            raise ValueError(f"original_size={original_size} exceeds unpacked width={groups * 32}")
        out = torch.empty((rows, groups * 32), dtype=torch.int8, device=W_q.device)
        with torch.cuda.device(W_q.device):
            capi.check(capi.lib().bm_unpack_bitplanes_i8(W_q.data_ptr(), out.data_ptr(), rows, groups, bits,
                                                         capi.stream_ptr(W_q.device)))
        return out[:, :original_size].contiguous()


__all__ = ["BitPack"]
