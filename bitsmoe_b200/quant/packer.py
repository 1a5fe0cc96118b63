"""Offline packer: one expert factor -> the ten runtime buffers of the checkpoint schema.

Keeps the interface of ``bitsmoe.quant.packer`` (bitsmoe/quant/packer.py): ``pack_single_weight``
(:517) writes the same state-dict keys, ``validate_runtime_layout`` (:377) performs the same
self-check.  The implementation is vectorised per slab over all tiles with plain torch integer
ops, so it runs on whatever device holds the factors (a GPU when there is one).

Layout reminder (payload): [bit bucket, wide first][slab <= 64 rows][tile 128 cols]
[stage 16 rows][micro 32 cols][row][plane word]; scales fp16 [slab][tile][row].
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from .quantizer import quantize_symmetric

K_SLAB = 64
N_TILE = 128
K_STAGE = 16
N_MICRO = 32
MICROS_PER_TILE = N_TILE // N_MICRO
_SUPPORTED_BITS = {1, 2, 3, 4, 6, 8, 16}
_BIT_OFFSETS = {1: 1, 2: 2, 3: 4, 4: 8, 6: 32, 8: 128}

RUNTIME_KEYS = ("payload_buffer", "rank_idx_buffer", "tile_meta_buffer", "slab_meta_buffer", "scale_buffer")


def _words_per_row(bits: int) -> int:
    if bits == 16:
        return 16
    if bits in _BIT_OFFSETS:
        return bits
    raise ValueError(f"Unsupported bits={bits}")


def codes_to_planes(q: Tensor, bits: int) -> Tensor:
    """int8 codes [..., 32*g] -> int64 plane words [..., g, bits] (values < 2^32)."""
    if bits == 1:
        u = (q.to(torch.int64) + 1) >> 1
    else:
        u = q.to(torch.int64) + _BIT_OFFSETS[bits]
    u = u.reshape(*q.shape[:-1], q.shape[-1] // N_MICRO, N_MICRO)
    lanes = torch.arange(N_MICRO, device=q.device, dtype=torch.int64)
    planes = [(((u >> p) & 1) << lanes).sum(dim=-1) for p in range(bits)]
    return torch.stack(planes, dim=-1)


def planes_to_codes(words: Tensor, bits: int) -> Tensor:
    """int64 plane words [..., g, bits] -> int8 codes [..., 32*g]."""
    lanes = torch.arange(N_MICRO, device=words.device, dtype=torch.int64)
    u = torch.zeros(*words.shape[:-1], N_MICRO, dtype=torch.int64, device=words.device)
    for p in range(bits):
        u |= ((words[..., p, None] >> lanes) & 1) << p
    q = (u * 2 - 1) if bits == 1 else (u - _BIT_OFFSETS[bits])
    return q.reshape(*words.shape[:-2], -1).to(torch.int8)


def fp16_to_words(h: Tensor) -> Tensor:
    """fp16 [..., 32*g] -> int64 words [..., g, 16]; low half = even column."""
    u = h.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
    u = u.reshape(*h.shape[:-1], h.shape[-1] // N_MICRO, N_MICRO)
    return u[..., 0::2] | (u[..., 1::2] << 16)


def words_to_fp16(words: Tensor) -> Tensor:
    lo = (words & 0xFFFF).to(torch.int32)
    hi = ((words >> 16) & 0xFFFF).to(torch.int32)
    u = torch.stack((lo, hi), dim=-1).reshape(*words.shape[:-2], -1)
    u = torch.where(u >= 0x8000, u - 0x10000, u).to(torch.int16)
    return u.view(torch.float16)


def slab_words_to_payload(words: Tensor) -> Tensor:
    """[rows, tiles, micro, wpr] -> flat [tile][stage][micro][row][word]."""
    rows, tiles, micros, wpr = words.shape
    full = (rows // K_STAGE) * K_STAGE
    parts = []
    if full:
        head = words[:full].reshape(full // K_STAGE, K_STAGE, tiles, micros, wpr).permute(2, 0, 3, 1, 4)
        parts.append(head.reshape(tiles, -1))
    if rows > full:
        parts.append(words[full:].permute(1, 2, 0, 3).reshape(tiles, -1))
    return torch.cat(parts, dim=1).reshape(-1)


def payload_to_slab_words(payload: Tensor, rows: int, tiles: int, wpr: int) -> Tensor:
    """Inverse of slab_words_to_payload for tiles of equal size."""
    per_tile = payload.reshape(tiles, rows * MICROS_PER_TILE * wpr)
    full = (rows // K_STAGE) * K_STAGE
    out = torch.empty((rows, tiles, MICROS_PER_TILE, wpr), dtype=payload.dtype, device=payload.device)
    split = full * MICROS_PER_TILE * wpr
    if full:
        head = per_tile[:, :split].reshape(tiles, full // K_STAGE, MICROS_PER_TILE, K_STAGE, wpr)
        out[:full] = head.permute(1, 3, 0, 2, 4).reshape(full, tiles, MICROS_PER_TILE, wpr)
    if rows > full:
        tail = per_tile[:, split:].reshape(tiles, MICROS_PER_TILE, rows - full, wpr)
        out[full:] = tail.permute(2, 0, 1, 3)
    return out


def quantize_rows(rows: Tensor, bits: int) -> Tuple[Tensor, Tensor]:
    """fp32 [n, dim] -> (int8 codes [n, tiles*128] zero-padded, fp32 scales [n, tiles]), one group per
    (row, 128-column tile); a ragged last tile is quantised on its valid columns only."""
    n, dim = rows.shape
    full_tiles, rem = divmod(dim, N_TILE)
    tiles = full_tiles + (1 if rem else 0)
    q = torch.zeros((n, tiles, N_TILE), dtype=torch.int8, device=rows.device)
    sc = torch.ones((n, tiles), dtype=torch.float32, device=rows.device)
    if full_tiles:
        body = rows[:, :full_tiles * N_TILE].contiguous().view(n, full_tiles, N_TILE)
        q[:, :full_tiles], sc[:, :full_tiles] = quantize_symmetric(body, bits=bits, dim=2)
    if rem:
        qt, st = quantize_symmetric(rows[:, full_tiles * N_TILE:].contiguous(), bits=bits, dim=1)
        q[:, full_tiles, :rem] = qt
        sc[:, full_tiles] = st
    return q.view(n, tiles * N_TILE), sc


def bucket_segments(segments: Sequence[Tuple[int, Tuple[int, int]]], rank: int) -> List[Tuple[int, Tensor]]:
    """Rows per bit width, widest bucket first, ranges by ascending start; 0-bit rows are dropped."""
    taken = torch.zeros(rank, dtype=torch.bool)
    by_bits: Dict[int, List[Tuple[int, int]]] = {}
    for bits, (s, e) in segments:
        bits, s, e = int(bits), int(s), int(e)
        if bits not in _SUPPORTED_BITS and bits != 0:
            raise ValueError(f"Unsupported bits={bits}")
        if not (0 <= s <= e <= rank):
            raise ValueError(f"Invalid segment range (s={s}, e={e}) for rank={rank}")
        if s == e:
            continue
        if bool(taken[s:e].any()):
            raise ValueError(f"Overlapping segments in range [{s}, {e})")
        taken[s:e] = True
        by_bits.setdefault(bits, []).append((s, e))
    out = []
    for bits in sorted(by_bits, reverse=True):
        if bits == 0:
            continue
        idx = torch.cat([torch.arange(s, e, dtype=torch.int32) for s, e in sorted(by_bits[bits])])
        out.append((bits, idx))
    return out


def quantize_pack_slab(rows: Tensor, bits: int, want_codes: bool = False):
    """One slab (<= 64 fp32 rows of one width, on a CUDA device) -> (payload uint32 words in the runtime layout, fp16
    scales [tiles, k][, int8 codes [k, tiles*128]]) by the library's fused kernel: quantise, bit-plane pack, reorder."""
    from .. import capi
    if not rows.is_cuda:
        raise ValueError("quantize_pack_slab requires CUDA tensors")
    rows = rows.to(torch.float32)
    if rows.stride(-1) != 1:
        rows = rows.contiguous()
    k, dim = rows.shape
    tiles = (dim + N_TILE - 1) // N_TILE
    payload = torch.empty(tiles * k * MICROS_PER_TILE * bits, dtype=torch.int32, device=rows.device)
    scale = torch.empty((tiles, k), dtype=torch.float16, device=rows.device)
    codes = torch.empty((k, tiles * N_TILE), dtype=torch.int8, device=rows.device) if want_codes else None
    with torch.cuda.device(rows.device):
        capi.check(capi.lib().bm_quantize_pack_slab(rows.data_ptr(), rows.stride(0) if k > 1 else dim, k, dim, bits,
                                                    payload.data_ptr(), scale.data_ptr(), capi.ptr(codes),
                                                    capi.stream_ptr(rows.device)))
    return (payload, scale, codes) if want_codes else (payload, scale)


def pack_rank_major(rank_major: Tensor, s_vec: Tensor, segments, groupsize: int = N_TILE,
                    precomputed: Optional[Dict[int, Tuple[Tensor, Tensor]]] = None,
                    fused: Optional[bool] = None) -> Dict[str, Tensor]:
    """Quantise + pack a rank-major factor [rank, dim].  ``precomputed[bits] = (plane words
    [rank, tiles, 4, bits], scales [rank, tiles])`` lets a caller that quantised and bit-sliced many
    experts in one batch skip both steps.  Buffers stay on the factor's device."""
    if groupsize != N_TILE:
        raise ValueError(f"Current runtime layout requires groupsize == N_TILE ({N_TILE}), got {groupsize}")
    rank, dim = rank_major.shape
    if rank != int(s_vec.numel()):
        raise ValueError(f"rank mismatch: matrix rank={rank}, S={int(s_vec.numel())}")
    if dim <= 0:
        raise ValueError("dim must be positive")
    if dim % N_MICRO:
        raise ValueError(f"dim={dim} must be divisible by microtile width {N_MICRO}")
    dev = rank_major.device
    if fused is None:
        fused = dev.type == "cuda" and precomputed is None
    tiles = (dim + N_TILE - 1) // N_TILE
    payload, scales, ridx, s_parts = [], [], [], []
    slab_rows, tile_rows, seg_rows = [], [], []
    pay_off = sc_off = ri_off = cursor = 0
    for bits, idx in bucket_segments(segments, rank):
        seg_rows.append([bits, cursor, cursor + idx.numel()])
        cursor += idx.numel()
        sel = idx.to(device=dev, dtype=torch.long)
        rows = rank_major.index_select(0, sel)
        s_rows = s_vec.index_select(0, sel).to(torch.float16)
        wpr = _words_per_row(bits)
        for r0 in range(0, idx.numel(), K_SLAB):
            r1 = min(idx.numel(), r0 + K_SLAB)
            k = r1 - r0
            slab_rows.append([bits, k, ri_off, len(tile_rows)])
            ridx.append(idx[r0:r1])
            s_parts.append(s_rows[r0:r1])
            if bits == 16:
                padded = torch.zeros((k, tiles * N_TILE), dtype=torch.float16, device=dev)
                padded[:, :dim] = rows[r0:r1].to(torch.float16)
                words = fp16_to_words(padded).view(k, tiles, MICROS_PER_TILE, 16)
                sc = torch.ones((k, tiles), dtype=torch.float16, device=dev)
            elif fused:
                # quantise + bit-plane pack + reorder in one kernel, straight into the runtime layout
                pay, sc_t = quantize_pack_slab(rows[r0:r1], bits)
                payload.append(pay.to(torch.int64) & 0xFFFFFFFF)
                scales.append(sc_t.reshape(-1))
                wpt = k * MICROS_PER_TILE * wpr
                for t in range(tiles):
                    tile_rows.append([pay_off + t * wpt, sc_off + t * k, min(N_TILE, dim - t * N_TILE)])
                pay_off += tiles * wpt
                sc_off += tiles * k
                ri_off += k
                continue
            else:
                if precomputed is not None:
                    w_all, sc_all = precomputed[bits]
                    words, sc = w_all.index_select(0, sel[r0:r1]), sc_all.index_select(0, sel[r0:r1])
                else:
                    q, sc = quantize_rows(rows[r0:r1].to(torch.float32), bits)
                    words = codes_to_planes(q, bits).view(k, tiles, MICROS_PER_TILE, bits)
                sc = sc.to(torch.float16)
            payload.append(slab_words_to_payload(words))
            scales.append(sc.transpose(0, 1).reshape(-1))
            wpt = k * MICROS_PER_TILE * wpr
            for t in range(tiles):
                tile_rows.append([pay_off + t * wpt, sc_off + t * k, min(N_TILE, dim - t * N_TILE)])
            pay_off += tiles * wpt
            sc_off += tiles * k
            ri_off += k

    def cat(parts, dtype, device=None):
        return torch.cat(parts).to(dtype) if parts else torch.empty((0,), dtype=dtype, device=device)

    rank_idx = cat(ridx, torch.int32)
    pay64 = torch.cat(payload) if payload else torch.empty((0,), dtype=torch.int64, device=dev)
    return {
        "payload_buffer": pay64.to(torch.uint32),
        "rank_idx_buffer": rank_idx,
        "tile_meta_buffer": torch.tensor(tile_rows, dtype=torch.int32).reshape(-1, 3),
        "slab_meta_buffer": torch.tensor(slab_rows, dtype=torch.int32).reshape(-1, 4),
        "scale_buffer": cat(scales, torch.float16, dev),
        "s_buffer": cat(s_parts, torch.float16, dev),
        "segments": torch.tensor(seg_rows, dtype=torch.int32).reshape(-1, 3),
        "original_indices": rank_idx.clone(),
        "original_rank": torch.tensor(rank, dtype=torch.int32),
        "groupsize": torch.tensor(groupsize, dtype=torch.int16),
    }


def unpack_rank_major(buf: Dict[str, Tensor], dim: int) -> Dict[str, Tensor]:
    """Decode the runtime buffers: per stored row the int8 codes, per-tile scales, width, and the
    dequantised fp32 row (raw fp16 rows pass through)."""
    slab_meta = buf["slab_meta_buffer"].to("cpu", torch.int64).reshape(-1, 4)
    tile_meta = buf["tile_meta_buffer"].to("cpu", torch.int64).reshape(-1, 3)
    payload = buf["payload_buffer"].cpu().to(torch.int64) & 0xFFFFFFFF
    scale = buf["scale_buffer"].cpu().to(torch.float16)
    n_rows = int(slab_meta[:, 1].sum()) if slab_meta.numel() else 0
    tiles = (dim + N_TILE - 1) // N_TILE
    codes = torch.zeros((n_rows, tiles * N_TILE), dtype=torch.int8)
    w = torch.zeros((n_rows, tiles * N_TILE), dtype=torch.float32)
    sc = torch.ones((n_rows, tiles), dtype=torch.float32)
    bits_row = torch.zeros((n_rows,), dtype=torch.int32)
    for i in range(slab_meta.shape[0]):
        bits, k, rank_off, tile_off = (int(v) for v in slab_meta[i])
        tile_end = int(slab_meta[i + 1, 3]) if i + 1 < slab_meta.shape[0] else tile_meta.shape[0]
        wpr = _words_per_row(bits)
        wpt = k * MICROS_PER_TILE * wpr
        bits_row[rank_off:rank_off + k] = bits
        for t in range(tile_off, tile_end):
            po, so, _ = (int(v) for v in tile_meta[t])
            tl = t - tile_off
            words = payload_to_slab_words(payload[po:po + wpt], k, 1, wpr)[:, 0]
            cols = slice(tl * N_TILE, (tl + 1) * N_TILE)
            if bits == 16:
                w[rank_off:rank_off + k, cols] = words_to_fp16(words).to(torch.float32)
            else:
                q = planes_to_codes(words, bits)
                s_t = scale[so:so + k].to(torch.float32)
                codes[rank_off:rank_off + k, cols] = q
                sc[rank_off:rank_off + k, tl] = s_t
                w[rank_off:rank_off + k, cols] = q.to(torch.float32) * s_t[:, None]
    return {"codes": codes[:, :dim], "w": w[:, :dim], "scales": sc, "bits": bits_row}


def validate_runtime_layout(rank_major_ref: Tensor, slab_meta_buffer: Tensor, tile_meta_buffer: Tensor,
                            rank_idx_buffer: Tensor, payload_buffer: Tensor, scale_buffer: Tensor,
                            groupsize: int = N_TILE, atol: float = 0.0, rtol: float = 0.0) -> None:
    """Decode payload/meta and compare with a direct per-tile quantisation of the same rows:
    codes must be identical, scales within 1e-3, raw-fp16 rows within (atol, rtol)."""
    if groupsize != N_TILE:
        raise ValueError(f"Validation currently expects groupsize={N_TILE}, got {groupsize}")
    dim = rank_major_ref.shape[1]
    dec = unpack_rank_major({"slab_meta_buffer": slab_meta_buffer, "tile_meta_buffer": tile_meta_buffer,
                             "payload_buffer": payload_buffer, "scale_buffer": scale_buffer}, dim)
    n = dec["codes"].shape[0]
    ref_rows = rank_major_ref.detach().cpu().index_select(0, rank_idx_buffer.cpu().long()[:n])
    for bits in sorted(set(dec["bits"].tolist())):
        rows = (dec["bits"] == bits).nonzero().flatten()
        ref = ref_rows.index_select(0, rows)
        if bits == 16:
            got = dec["w"].index_select(0, rows)
            if not torch.allclose(got, ref.to(torch.float16).to(torch.float32), atol=atol, rtol=rtol):
                raise AssertionError("fp16 payload validation failed")
            continue
        q_ref, s_ref = quantize_rows(ref.to(torch.float32), bits)
        if not torch.equal(dec["codes"].index_select(0, rows), q_ref[:, :dim]):
            raise AssertionError(f"low-bit payload validation failed (bits={bits})")
        if not torch.allclose(dec["scales"].index_select(0, rows), s_ref, atol=1e-3, rtol=1e-3):
            raise AssertionError(f"scale validation failed (bits={bits})")


def _rank_major_and_s(moe_dict, layer_idx: int, expert_idx: int, mtype: str, device):
    entry = moe_dict[layer_idx][expert_idx][mtype]
    if not isinstance(entry, tuple) or len(entry) != 2:
        raise ValueError(f"Expected tuple(matrix, S) for {mtype}, got type={type(entry)}")
    matrix, s_vec = entry
    if s_vec.dim() != 1:
        raise ValueError(f"S must be 1-D, got shape={tuple(s_vec.shape)}")
    if matrix.dim() != 2:
        raise ValueError(f"factor must be 2-D, got shape={tuple(matrix.shape)}")
    rank = int(s_vec.numel())
    if mtype in ("gate_proj", "up_proj"):
        if matrix.shape[0] != rank:
            raise ValueError(f"U_rank_dim shape mismatch: rank={rank}, tensor shape={tuple(matrix.shape)}")
        return matrix.to(device).contiguous(), s_vec.to(device).contiguous(), "u"
    if mtype == "down_proj":
        if matrix.shape[1] != rank:
            raise ValueError(f"Vh_dim_rank shape mismatch: rank={rank}, tensor shape={tuple(matrix.shape)}")
        return matrix.to(device).t().contiguous(), s_vec.to(device).contiguous(), "vh"
    raise ValueError(f"Unsupported mtype: {mtype}")


def pack_single_weight(moe_dict, segments, state_dict: Dict[str, Tensor], layer_idx: int, expert_idx: int,
                       mtype: str, groupsize: int = N_TILE, validate_layout: bool = False):
    """Quantise + pack one expert matrix and write the checkpoint keys
    ``quantized.layer{L}.expert{E}.{mtype}.{u|vh}.{payload,rank_idx,tile_meta,slab_meta,scale}_buffer``,
    ``….s_buffer``, ``….segments``, ``….original_indices``, ``….original_rank``, ``….groupsize``."""
    if groupsize != N_TILE:
        raise ValueError(f"Current runtime layout requires groupsize == N_TILE ({N_TILE}), got {groupsize}")
    device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    t0 = time.perf_counter()
    rank_major, s_vec, field = _rank_major_and_s(moe_dict, layer_idx, expert_idx, mtype, device)
    buf = pack_rank_major(rank_major, s_vec, segments, groupsize)
    prefix = f"quantized.layer{layer_idx}.expert{expert_idx}.{mtype}"
    for key in RUNTIME_KEYS:
        state_dict[f"{prefix}.{field}.{key}"] = buf[key].cpu()
    for key in ("s_buffer", "segments", "original_indices", "original_rank", "groupsize"):
        state_dict[f"{prefix}.{key}"] = buf[key].cpu()
    if validate_layout and buf["payload_buffer"].numel() > 0:
        validate_runtime_layout(rank_major, buf["slab_meta_buffer"], buf["tile_meta_buffer"], buf["rank_idx_buffer"],
                                buf["payload_buffer"], buf["scale_buffer"], groupsize)
    total = time.perf_counter() - t0
    return {"total_s": total, "quantize_s": 0.0, "pack_s": total}
