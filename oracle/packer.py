"""Runtime buffer layout of one packed expert matrix (numpy + torch CPU).  Test infrastructure.

Restates, with explicit loops, what bitsmoe/quant/packer.py:517-724
(``pack_single_weight``) emits for one rank-major matrix ``[rank, dim]`` and
what the kernels decode (bitsmoe/algorithms/cpp/mlp_forward.cu:203-275):

  rows are bucketed by bit width, buckets in descending width, ranges inside a
  bucket by ascending start (packer.py:566-589); rows given 0 bits are dropped
  (packer.py:616-617); each bucket is cut into slabs of <= 64 rows
  (K_SLAB, packer.py:13, :636-640);
  payload order  [slab][tile of 128 cols][stage of 16 rows][micro of 32 cols]
                 [row][plane word]                  (packer.py:527-541, :169-207)
  one fp16 scale per (tile, row), stored [slab][tile][row]      (packer.py:261-263)
  tile_meta row = [payload word offset, scale offset, valid cols] (packer.py:671-680)
  slab_meta row = [bits, rows, rank_idx offset, tile_meta offset] (packer.py:643)
  16-"bit" slabs hold raw fp16, two per word, low half = even column, scale 1
                                                                (packer.py:309-374)
"""
from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from . import bitplane
from .quantize import quantize_symmetric

K_SLAB = 64
N_TILE = 128
K_STAGE = 16
N_MICRO = 32
MICROS_PER_TILE = N_TILE // N_MICRO
SUPPORTED_BITS = (1, 2, 3, 4, 6, 8, 16)

Segments = Sequence[Tuple[int, Tuple[int, int]]]


def words_per_row(bits: int) -> int:
    if bits == 16:
        return 16
    if bits in bitplane.BIT_OFFSETS:
        return bits
    raise ValueError(f"Unsupported bits={bits}")


def _stage_micro_order(per_row: np.ndarray) -> np.ndarray:
    """[rows, micro, words] -> flat [stage][micro][row][word] (packer.py:169-207)."""
    rows = per_row.shape[0]
    parts = []
    for r0 in range(0, rows, K_STAGE):
        parts.append(np.ascontiguousarray(per_row[r0:r0 + K_STAGE].transpose(1, 0, 2)).reshape(-1))
    return np.concatenate(parts) if parts else np.empty((0,), np.uint32)


def pack_tile_lowbit(tile_q: np.ndarray, bits: int) -> np.ndarray:
    """int8 [rows, 128] (padded with code 0) -> payload words of one tile."""
    rows = tile_q.shape[0]
    planes = bitplane.pack_bitplanes_i8(np.ascontiguousarray(tile_q), bits)
    return _stage_micro_order(planes.reshape(rows, MICROS_PER_TILE, bits))


def pack_tile_fp16(tile_h: np.ndarray) -> np.ndarray:
    """float16 [rows, 128] -> payload words of one raw-fp16 tile."""
    rows = tile_h.shape[0]
    u16 = np.ascontiguousarray(tile_h).view(np.uint16).astype(np.uint32)
    words = u16[:, 0::2] | (u16[:, 1::2] << np.uint32(16))
    return _stage_micro_order(words.reshape(rows, MICROS_PER_TILE, 16))


def unpack_tile(payload_tile: np.ndarray, bits: int, rows: int) -> np.ndarray:
    """Inverse of pack_tile_*: returns int8 codes or float16 values [rows, 128]."""
    wpr = words_per_row(bits)
    out = np.empty((rows, N_TILE), dtype=np.float16 if bits == 16 else np.int8)
    ptr = 0
    for r0 in range(0, rows, K_STAGE):
        n = min(K_STAGE, rows - r0)
        for micro in range(MICROS_PER_TILE):
            chunk = payload_tile[ptr:ptr + n * wpr].reshape(n, wpr)
            ptr += n * wpr
            c0 = micro * N_MICRO
            if bits == 16:
                u16 = np.empty((n, N_MICRO), dtype=np.uint16)
                u16[:, 0::2] = (chunk & np.uint32(0xFFFF)).astype(np.uint16)
                u16[:, 1::2] = (chunk >> np.uint32(16)).astype(np.uint16)
                out[r0:r0 + n, c0:c0 + N_MICRO] = u16.view(np.float16)
            else:
                out[r0:r0 + n, c0:c0 + N_MICRO] = bitplane.unpack_bitplanes_i8(
                    np.ascontiguousarray(chunk), bits)
    if ptr != payload_tile.size:
        raise RuntimeError("tile payload size does not match its meta")
    return out


def bucket_rows(segments: Segments, rank: int) -> List[Tuple[int, np.ndarray]]:
    """[(bits, logical row indices)] in the order slabs are emitted."""
    groups: Dict[int, List[Tuple[int, int]]] = defaultdict(list)
    seen = np.zeros(rank, dtype=bool)
    for bits, (s, e) in segments:
        bits, s, e = int(bits), int(s), int(e)
        if bits not in SUPPORTED_BITS and bits != 0:
            raise ValueError(f"Unsupported bits={bits}")
        if not (0 <= s <= e <= rank):
            raise ValueError(f"Invalid segment range (s={s}, e={e}) for rank={rank}")
        if e == s:
            continue
        if seen[s:e].any():
            raise ValueError(f"Overlapping segments in range [{s}, {e})")
        seen[s:e] = True
        groups[bits].append((s, e))
    out = []
    for bits in sorted(groups, reverse=True):
        if bits == 0:
            continue
        idx = np.concatenate([np.arange(s, e, dtype=np.int32) for s, e in sorted(groups[bits])])
        if idx.size:
            out.append((bits, idx))
    return out


def pack_matrix(rank_major: torch.Tensor, s_vec: torch.Tensor, segments: Segments,
                groupsize: int = N_TILE) -> Dict[str, np.ndarray]:
    """Quantise + pack one rank-major matrix into the ten runtime buffers."""
    if groupsize != N_TILE:
        raise ValueError(f"runtime layout requires groupsize == {N_TILE}")
    rank, dim = rank_major.shape
    if rank != s_vec.numel():
        raise ValueError("rank mismatch between matrix and S")
    if dim <= 0 or dim % N_MICRO:
        raise ValueError(f"dim={dim} must be a positive multiple of {N_MICRO}")
    n_tiles = (dim + N_TILE - 1) // N_TILE
    full_tiles = dim // N_TILE
    rem = dim - full_tiles * N_TILE

    payload: List[np.ndarray] = []
    scales: List[np.ndarray] = []
    rank_idx: List[np.ndarray] = []
    s_out: List[np.ndarray] = []
    slab_meta: List[List[int]] = []
    tile_meta: List[List[int]] = []
    seg_meta: List[List[int]] = []
    pay_off = sc_off = ri_off = cursor = 0

    for bits, idx in bucket_rows(segments, rank):
        seg_meta.append([bits, cursor, cursor + idx.size])
        cursor += idx.size
        rows_all = rank_major.index_select(0, torch.from_numpy(idx).long())
        s_all = s_vec.index_select(0, torch.from_numpy(idx).long())
        for r0 in range(0, idx.size, K_SLAB):
            r1 = min(idx.size, r0 + K_SLAB)
            k_slab = r1 - r0
            slab = rows_all[r0:r1]
            slab_meta.append([bits, k_slab, ri_off, len(tile_meta)])
            rank_idx.append(idx[r0:r1].copy())
            ri_off += k_slab
            s_out.append(s_all[r0:r1].to(torch.float16).numpy())
            wpt = k_slab * MICROS_PER_TILE * words_per_row(bits)
            tiles_payload: List[np.ndarray] = []
            tiles_scale: List[np.ndarray] = []
            if bits == 16:
                h = slab.to(torch.float16).numpy()
                for t in range(n_tiles):
                    tile = np.zeros((k_slab, N_TILE), dtype=np.float16)
                    c0 = t * N_TILE
                    n_valid = min(N_TILE, dim - c0)
                    tile[:, :n_valid] = h[:, c0:c0 + n_valid]
                    tiles_payload.append(pack_tile_fp16(tile))
                    tiles_scale.append(np.ones((k_slab,), dtype=np.float16))
            else:
                slab32 = slab.to(torch.float32)
                if full_tiles:
                    full = slab32[:, :full_tiles * N_TILE].contiguous().view(k_slab, full_tiles, N_TILE)
                    q_full, sc_full = quantize_symmetric(full, bits=bits, dim=2)
                    q_np = q_full.numpy()
                    sc_np = sc_full.to(torch.float16).numpy()
                    for t in range(full_tiles):
                        tiles_payload.append(pack_tile_lowbit(q_np[:, t, :], bits))
                        tiles_scale.append(np.ascontiguousarray(sc_np[:, t]))
                if rem:
                    tail = slab32[:, full_tiles * N_TILE:].contiguous()
                    q_tail, sc_tail = quantize_symmetric(tail, bits=bits, dim=1)
                    q_pad = np.zeros((k_slab, N_TILE), dtype=np.int8)
                    q_pad[:, :rem] = q_tail.numpy()
                    tiles_payload.append(pack_tile_lowbit(q_pad, bits))
                    tiles_scale.append(sc_tail.to(torch.float16).numpy().reshape(-1))
            for t in range(n_tiles):
                if tiles_payload[t].size != wpt:
                    raise RuntimeError("payload width mismatch")
                tile_meta.append([pay_off + t * wpt, sc_off + t * k_slab, min(N_TILE, dim - t * N_TILE)])
            payload.extend(tiles_payload)
            scales.extend(tiles_scale)
            pay_off += n_tiles * wpt
            sc_off += n_tiles * k_slab

    def cat(parts, dtype):
        return np.concatenate(parts).astype(dtype) if parts else np.empty((0,), dtype=dtype)

    ridx = cat(rank_idx, np.int32)
    return {
        "payload_buffer": cat(payload, np.uint32),
        "rank_idx_buffer": ridx,
        "tile_meta_buffer": np.asarray(tile_meta, dtype=np.int32).reshape(-1, 3),
        "slab_meta_buffer": np.asarray(slab_meta, dtype=np.int32).reshape(-1, 4),
        "scale_buffer": cat(scales, np.float16),
        "s_buffer": cat(s_out, np.float16),
        "segments": np.asarray(seg_meta, dtype=np.int32).reshape(-1, 3),
        "original_indices": ridx.copy(),
        "original_rank": np.asarray(rank, dtype=np.int32),
        "groupsize": np.asarray(groupsize, dtype=np.int16),
    }


def decode_matrix(buf: Dict[str, np.ndarray], dim: int) -> Dict[str, np.ndarray]:
    """Walk slab_meta / tile_meta exactly as the kernels do and return, per
    stored (local) row: integer codes, fp32 scales per tile, bit width, the
    logical rank it maps to, its S value, and the dequantised fp32 row
    ``w = q * scale`` (raw fp16 value for 16-"bit" rows;
    bitsmoe/quant/quantizer.py:116-128, mlp_forward.cu:756-764)."""
    slab_meta = np.asarray(buf["slab_meta_buffer"]).astype(np.int64).reshape(-1, 4)
    tile_meta = np.asarray(buf["tile_meta_buffer"]).astype(np.int64).reshape(-1, 3)
    payload = np.asarray(buf["payload_buffer"]).astype(np.uint32)
    scale = np.asarray(buf["scale_buffer"]).astype(np.float16)
    n_rows = int(slab_meta[:, 1].sum()) if slab_meta.size else 0
    n_tiles = (dim + N_TILE - 1) // N_TILE
    codes = np.zeros((n_rows, dim), dtype=np.int8)
    w = np.zeros((n_rows, dim), dtype=np.float32)
    sc = np.ones((n_rows, n_tiles), dtype=np.float32)
    bits_row = np.zeros((n_rows,), dtype=np.int32)
    for i in range(slab_meta.shape[0]):
        bits, k_slab, rank_off, tile_off = (int(v) for v in slab_meta[i])
        tile_end = int(slab_meta[i + 1, 3]) if i + 1 < slab_meta.shape[0] else tile_meta.shape[0]
        wpt = k_slab * MICROS_PER_TILE * words_per_row(bits)
        bits_row[rank_off:rank_off + k_slab] = bits
        for t in range(tile_off, tile_end):
            pack_off, scale_off, n_valid = (int(v) for v in tile_meta[t])
            tl = t - tile_off
            c0 = tl * N_TILE
            tile = unpack_tile(payload[pack_off:pack_off + wpt], bits, k_slab)[:, :n_valid]
            if bits == 16:
                w[rank_off:rank_off + k_slab, c0:c0 + n_valid] = tile.astype(np.float32)
            else:
                s_t = scale[scale_off:scale_off + k_slab].astype(np.float32)
                codes[rank_off:rank_off + k_slab, c0:c0 + n_valid] = tile
                sc[rank_off:rank_off + k_slab, tl] = s_t
                w[rank_off:rank_off + k_slab, c0:c0 + n_valid] = tile.astype(np.float32) * s_t[:, None]
    return {
        "codes": codes,
        "scales": sc,
        "bits": bits_row,
        "rank_idx": np.asarray(buf["rank_idx_buffer"]).astype(np.int32)[:n_rows],
        "s": np.asarray(buf["s_buffer"]).astype(np.float16).astype(np.float32)[:n_rows],
        "w": w,
    }


def validate_layout(rank_major: torch.Tensor, buf: Dict[str, np.ndarray]) -> None:
    """The reference's only known-answer check, restated (packer.py:377-460):
    decoding the payload through the meta tables must reproduce a fresh
    per-tile quantisation of the same rows bit-exactly; scales within 1e-3."""
    dim = rank_major.shape[1]
    dec = decode_matrix(buf, dim)
    n_tiles = (dim + N_TILE - 1) // N_TILE
    rows = rank_major.index_select(0, torch.from_numpy(dec["rank_idx"]).long())
    for r in range(rows.shape[0]):
        bits = int(dec["bits"][r])
        for t in range(n_tiles):
            c0, c1 = t * N_TILE, min(dim, (t + 1) * N_TILE)
            if bits == 16:
                ref = rows[r, c0:c1].to(torch.float16).to(torch.float32).numpy()
                if not np.array_equal(dec["w"][r, c0:c1], ref):
                    raise AssertionError(f"fp16 row {r} tile {t} differs")
                continue
            q_ref, s_ref = quantize_symmetric(rows[r:r + 1, c0:c1].to(torch.float32), bits=bits, dim=1)
            if not np.array_equal(dec["codes"][r, c0:c1], q_ref.numpy()[0]):
                raise AssertionError(f"codes differ (row {r}, tile {t}, bits {bits})")
            if not np.allclose(dec["scales"][r, t], float(s_ref), atol=1e-3, rtol=1e-3):
                raise AssertionError(f"scale differs (row {r}, tile {t}, bits {bits})")


def expert_bytes(buf: Dict[str, np.ndarray]) -> int:
    """Bytes the forward path reads for one matrix, exactly as stored."""
    keys = ("payload_buffer", "scale_buffer", "s_buffer", "rank_idx_buffer",
            "tile_meta_buffer", "slab_meta_buffer")
    return int(sum(np.asarray(buf[k]).nbytes for k in keys))
