"""Shared fixtures: synthetic layers handed to both the CUDA path and the CPU oracle."""
from __future__ import annotations

import glob
import importlib.util
import os
from typing import Dict, List

import numpy as np
import torch

from bitsmoe_b200 import synth
from bitsmoe_b200.quant import packer as ppacker
from oracle import forward as oforward

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RTOL, ATOL = 2e-2, 1e-2   # layer-output tolerance of the benchmark specification


def to_numpy_buf(buf: Dict[str, torch.Tensor]) -> Dict[str, np.ndarray]:
    out = {}
    for k, v in buf.items():
        if not isinstance(v, torch.Tensor):
            continue
        v = v.detach().cpu()
        out[k] = v.to(torch.int64).numpy().astype(np.uint32) if v.dtype == torch.uint32 else v.numpy()
    return out


def table_entry(layer: synth.SynthLayer, tag: str, e: int) -> Dict[str, np.ndarray]:
    t = layer.tables[tag]
    return to_numpy_buf({f + "_buffer": t[f][e] for f in t})


def decoded_experts(layer: synth.SynthLayer) -> List[oforward.DecodedExpert]:
    I = layer.cfg.intermediate
    return [oforward.DecodedExpert(table_entry(layer, "gate", e), table_entry(layer, "up", e),
                                   table_entry(layer, "down", e), I) for e in range(layer.cfg.num_experts)]


def mixed_everything_layer(seed: int = 7, num_experts: int = 6, rank: int = 90, intermediate: int = 160,
                           hidden: int = 128) -> synth.SynthLayer:
    """Small layer that exercises every stored width (16, 8, 6, 4, 3, 2, 1), dropped 0-bit rows, tail slabs
    (rows not a multiple of 16) and a ragged last tile (intermediate = 128 + 32)."""
    g = torch.Generator().manual_seed(seed)
    cfg = synth.LayerConfig("mixed", hidden, num_experts, intermediate, 2, rank)
    tables = {tag: {f: [] for f in ("payload", "rank_idx", "tile_meta", "slab_meta", "scale", "s")} for tag, _ in synth.MTYPES}
    extras = {tag: [] for tag, _ in synth.MTYPES}
    cuts = [(16, 5), (8, 9), (6, 7), (4, 13), (3, 17), (0, 4), (2, 30), (1, 5)]
    for tag, _ in synth.MTYPES:
        for e in range(num_experts):
            R = torch.randn(rank, intermediate, generator=g) * 0.02
            S = torch.rand(rank, generator=g) + 0.25
            segs, start = [], 0
            order = cuts[e % len(cuts):] + cuts[:e % len(cuts)]
            for bits, n in order:
                n = min(n, rank - start)
                if n > 0:
                    segs.append((bits, (start, start + n)))
                    start += n
            buf = ppacker.pack_rank_major(R, S, segs)
            for f in tables[tag]:
                tables[tag][f].append(buf[f + "_buffer"])
            extras[tag].append(dict(buf, _rank_major=R, _s=S, _segments=segs))
    vh_gate = (torch.randn(rank, hidden, generator=g) * 0.05).half()
    vh_up = (torch.randn(rank, hidden, generator=g) * 0.05).half()
    u_down = (torch.randn(hidden, rank, generator=g) * 0.05).half()
    return synth.SynthLayer(cfg, tables, vh_gate, vh_up, u_down, None, extras)


def load_reference_ext(name: str):
    """The reference's own extension compiled for sm_100a (oracle/build_ref.py), or None."""
    hits = glob.glob(os.path.join(ROOT, "oracle", "_ref", name + "*.so"))
    if not hits:
        return None
    spec = importlib.util.spec_from_file_location(name, hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def ref_args(layer: synth.SynthLayer, device) -> list:
    """The 18 buffer lists of moe_packed_forward in the reference's argument order."""
    out = []
    for tag in ("gate", "up", "down"):
        for f in ("payload", "rank_idx", "tile_meta", "slab_meta", "scale", "s"):
            out.append([t.to(device) for t in layer.tables[tag][f]])
    return out


def assert_close(got: torch.Tensor, want: torch.Tensor, rtol: float = RTOL, atol: float = ATOL, what: str = "",
                 rel_max: float = 2e-2, rel_l2: float = 1e-2, outlier_frac: float = 0.0) -> None:
    """Element-wise ``|err| <= atol + rtol*|want|`` AND two bounds relative to the size of the expected signal:
    ``max|err| <= rel_max * max|want|`` and ``||err||_2 <= rel_l2 * ||want||_2``.  The synthetic layers produce
    outputs of order 1e-3 .. 1e-2, far below the absolute tolerance of the specification, so the element-wise test
    alone would accept an all-zero result; the relative bounds are what makes a wrong kernel fail.
    ``outlier_frac`` (only for comparisons against a reference that is itself noisy) lets that fraction of the
    elements (at least two) violate the element-wise and peak bounds; the L2 bound always covers every element."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert bool(torch.isfinite(got).all()), f"{what}: non-finite values"
    if want.numel() == 0:
        return
    err = (got - want).abs()
    peak = float(want.abs().max())
    allowed = max(2, int(outlier_frac * want.numel())) if outlier_frac > 0 else 0
    bad = err > atol + rtol * want.abs()
    assert int(bad.sum()) <= allowed, (f"{what}: {int(bad.sum())}/{bad.numel()} outside rtol={rtol} atol={atol}; "
                                       f"max abs err {float(err.max()):.4g}, max |want| {peak:.4g}")
    if peak == 0.0:
        assert float(err.max()) == 0.0, f"{what}: expected exact zeros, max |got| {float(got.abs().max()):.4g}"
        return
    over = int((err > rel_max * peak).sum())
    assert over <= allowed, (f"{what}: {over} elements with abs err > {rel_max} * max|want| ({peak:.4g}); "
                             f"max abs err {float(err.max()):.4g}")
    l2 = float(torch.linalg.vector_norm(got - want)) / float(torch.linalg.vector_norm(want))
    assert l2 <= rel_l2, f"{what}: relative L2 error {l2:.4g} > {rel_l2}"


def assert_detects_damage(got: torch.Tensor, want: torch.Tensor, what: str = "", **tol) -> None:
    """The check used on ``got`` must reject a halved result and a result with one row's signal removed: proof
    that the tolerance can see a wrong kernel at this shape and scale."""
    import pytest
    with pytest.raises(AssertionError):
        assert_close(got * 0.5, want, what=what + " (halved)", **tol)
    with pytest.raises(AssertionError):
        assert_close(torch.zeros_like(got), want, what=what + " (zeroed)", **tol)


class LazyDecodedExperts:
    """Sequence of DecodedExpert that dequantises an expert only when the oracle touches it (large layers)."""

    def __init__(self, layer: synth.SynthLayer):
        self.layer, self._cache = layer, {}

    def __len__(self):
        return self.layer.cfg.num_experts

    def __getitem__(self, e):
        if e not in self._cache:
            I = self.layer.cfg.intermediate
            self._cache[e] = oforward.DecodedExpert(table_entry(self.layer, "gate", e), table_entry(self.layer, "up", e),
                                                    table_entry(self.layer, "down", e), I)
        return self._cache[e]

    def __iter__(self):
        return (self[e] for e in range(len(self)))
