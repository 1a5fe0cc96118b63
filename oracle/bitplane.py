"""Bit-plane packing of signed low-bit codes (numpy).  Test infrastructure.

Follows bitsmoe/quant/bitpack/bitpack_cuda_kernel.cu:81-121 (pack) and
:157-196 (unpack): a row of ``cols`` int8 codes is cut into groups of 32
columns; each group becomes ``bits`` consecutive uint32 words, word ``p``
holding bit ``p`` of the unsigned code ``u = q + offset`` of column
``group*32 + lane`` at bit position ``lane``.  Offsets are
bitsmoe/quant/bitpack/__init__.py:22; the 1-bit case stores ``(q + 1) >> 1``
and decodes ``2u - 1`` (bitpack_cuda_kernel.cu:106-107, :188-189).
"""
from __future__ import annotations

import numpy as np

BIT_OFFSETS = {1: 1, 2: 2, 3: 4, 4: 8, 6: 32, 8: 128}
SUPPORTED_BITS = (1, 2, 3, 4, 6, 8)


def _check_bits(bits: int) -> None:
    if bits not in BIT_OFFSETS:
        raise ValueError(f"Unsupported bit width: {bits}")


def to_unsigned(q: np.ndarray, bits: int) -> np.ndarray:
    _check_bits(bits)
    q16 = q.astype(np.int16)
    if bits == 1:
        return ((q16 + 1) >> 1).astype(np.uint8)
    return (q16 + BIT_OFFSETS[bits]).astype(np.uint8)


def to_signed(u: np.ndarray, bits: int) -> np.ndarray:
    _check_bits(bits)
    u16 = u.astype(np.int16)
    if bits == 1:
        return ((u16 << 1) - 1).astype(np.int8)
    return (u16 - BIT_OFFSETS[bits]).astype(np.int8)


def pack_bitplanes_i8(q: np.ndarray, bits: int) -> np.ndarray:
    """int8 [rows, cols] -> uint32 [rows, ceil(cols/32) * bits]."""
    _check_bits(bits)
    if q.ndim != 2 or q.dtype != np.int8:
        raise ValueError("expects a 2-D int8 array")
    rows, cols = q.shape
    groups = (cols + 31) // 32
    u = np.zeros((rows, groups * 32), dtype=np.uint8)
    u[:, :cols] = to_unsigned(q, bits)
    u = u.reshape(rows, groups, 32).astype(np.uint64)
    lanes = np.arange(32, dtype=np.uint64)
    out = np.empty((rows, groups, bits), dtype=np.uint32)
    for p in range(bits):
        bit = (u >> np.uint64(p)) & np.uint64(1)
        out[:, :, p] = (bit << lanes).sum(axis=2).astype(np.uint32)
    return out.reshape(rows, groups * bits)


def unpack_bitplanes_i8(words: np.ndarray, bits: int) -> np.ndarray:
    """uint32 [rows, groups * bits] -> int8 [rows, groups * 32]."""
    _check_bits(bits)
    if words.ndim != 2 or words.dtype != np.uint32:
        raise ValueError("expects a 2-D uint32 array")
    rows, width = words.shape
    if width % bits:
        raise ValueError("row width is not a multiple of the bit width")
    groups = width // bits
    w = words.reshape(rows, groups, bits).astype(np.uint64)
    lanes = np.arange(32, dtype=np.uint64)
    u = np.zeros((rows, groups, 32), dtype=np.uint64)
    for p in range(bits):
        u |= ((w[:, :, p, None] >> lanes) & np.uint64(1)) << np.uint64(p)
    return to_signed(u.reshape(rows, groups * 32).astype(np.uint8), bits)
