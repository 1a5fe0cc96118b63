"""Generate tests/golden/*.npz from the reference's own Python.  Run in a container
that has the reference tree; the fixtures it writes are committed, the tree is
not needed afterwards.

    python tests/golden/make_golden.py [--reference <BitsMoE checkout>]

What is taken from the reference (imported, executed on the CPU, unmodified):
  bitsmoe.quant.quantizer.quantize_symmetric
  bitsmoe.quant.packer._reorder_packed_rows_to_runtime_layout
  bitsmoe.quant.packer._pack_lowbit_slab_payload_and_scale
  bitsmoe.quant.packer._pack_fp16_slab_payload_and_scale
  bitsmoe.quant.packer._pack_lowbit_tile_payload / _unpack_lowbit_tile_payload
  bitsmoe.quant.packer.validate_runtime_layout

The reference's bit-plane primitive is a CUDA extension
(bitsmoe/quant/_bitpack_cuda) that cannot run without a GPU; for these fixtures
it is replaced by oracle.bitplane, and the package ``__init__`` (which
monkey-patches transformers) is bypassed.  The primitive itself is pinned
separately, on the GPU, against the compiled reference extension.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import bitplane, packer as opacker  # noqa: E402


def import_reference(ref_root: str):
    pkg_dir = os.path.join(ref_root, "bitsmoe")
    for name, sub in (("bitsmoe", ""), ("bitsmoe.quant", "quant"), ("bitsmoe.utils", "utils")):
        m = types.ModuleType(name)
        m.__path__ = [os.path.join(pkg_dir, sub)]
        m.__file__ = os.path.join(pkg_dir, sub, "__init__.py")
        sys.modules[name] = m
    stub = types.ModuleType("bitsmoe.quant._bitpack_cuda")

    def mk_pack(bits):
        return lambda t: torch.from_numpy(
            bitplane.pack_bitplanes_i8(t.numpy(), bits).astype(np.int64)).to(torch.uint32)

    def mk_unpack(bits):
        return lambda t: torch.from_numpy(
            bitplane.unpack_bitplanes_i8(t.to(torch.int64).numpy().astype(np.uint32), bits))

    for b in bitplane.SUPPORTED_BITS:
        setattr(stub, f"pack_int8_{b}bit", mk_pack(b))
        setattr(stub, f"unpack_int8_{b}bit", mk_unpack(b))
    sys.modules["bitsmoe.quant._bitpack_cuda"] = stub
    import bitsmoe.quant.bitpack as bp
    bp.BitPack._check_pack_input = staticmethod(lambda t: t.contiguous())
    bp.BitPack._check_unpack_input = staticmethod(lambda t: t.contiguous())
    import bitsmoe.quant.packer as rpacker
    import bitsmoe.quant.quantizer as rquant
    return rquant, rpacker


def u32(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.int64).numpy().astype(np.uint32)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a BitsMoE source tree")
    a = ap.parse_args()
    rquant, rpacker = import_reference(a.reference)
    g = torch.Generator().manual_seed(42)
    out = {}

    # 1. quantize_symmetric known answers, every supported width.
    x3 = torch.randn(7, 3, 128, generator=g) * 0.02
    xt = torch.randn(7, 96, generator=g) * 0.02
    out["quant_x_full"] = x3.numpy()
    out["quant_x_tail"] = xt.numpy()
    for b in (1, 2, 3, 4, 6, 8):
        q, s = rquant.quantize_symmetric(x3, bits=b, dim=2)
        out[f"quant_q_full_b{b}"] = q.numpy()
        out[f"quant_s_full_b{b}"] = s.numpy()
        q, s = rquant.quantize_symmetric(xt, bits=b, dim=1)
        out[f"quant_q_tail_b{b}"] = q.numpy()
        out[f"quant_s_tail_b{b}"] = s.numpy()

    # 2. stage/micro reorder, including tail slabs.
    for k_slab, wpr in ((64, 2), (16, 3), (13, 4), (37, 2)):
        src = torch.arange(2 * k_slab * 4 * wpr, dtype=torch.int64).view(2, k_slab, 4, wpr)
        out[f"reorder_k{k_slab}_w{wpr}"] = rpacker._reorder_packed_rows_to_runtime_layout(
            src, k_slab, wpr).numpy()

    # 3. slab packer: payload + scales for low-bit and raw-fp16 slabs.
    for k_slab, dim, b in ((13, 160, 4), (64, 256, 2), (38, 384, 3), (5, 96, 8), (16, 128, 1), (9, 224, 6)):
        slab = torch.randn(k_slab, dim, generator=g) * 0.02
        pay, sc = rpacker._pack_lowbit_slab_payload_and_scale(slab, b)
        out[f"slab_x_k{k_slab}_d{dim}_b{b}"] = slab.numpy()
        out[f"slab_payload_k{k_slab}_d{dim}_b{b}"] = u32(pay)
        out[f"slab_scale_k{k_slab}_d{dim}_b{b}"] = sc.numpy()
    slab = torch.randn(21, 160, generator=g) * 0.02
    pay, sc = rpacker._pack_fp16_slab_payload_and_scale(slab)
    out["slab16_x"] = slab.numpy()
    out["slab16_payload"] = u32(pay)
    out["slab16_scale"] = sc.numpy()

    # 4. per-tile payload round trip through the reference's tile codec.
    tq = torch.randint(-4, 4, (37, 96), generator=g, dtype=torch.int8)
    tp = rpacker._pack_lowbit_tile_payload(tq, 3)
    out["tile_q"] = tq.numpy()
    out["tile_payload_b3"] = u32(tp)
    out["tile_decoded_b3"] = rpacker._unpack_lowbit_tile_payload(tp, 3, 37, torch.device("cpu")).numpy()

    # 5. whole-matrix buffers from the oracle packer, accepted by the reference's validator.
    rank, dim = 150, 416
    mat = torch.randn(rank, dim, generator=g) * 0.02
    svec = torch.rand(rank, generator=g) + 0.5
    segments = [(4, (0, 13)), (3, (13, 51)), (2, (51, 120)), (0, (120, 126)), (16, (126, 131)),
                (8, (131, 140)), (2, (140, 150))]
    buf = opacker.pack_matrix(mat, svec, segments)
    rpacker.validate_runtime_layout(
        rank_major_ref=mat,
        slab_meta_buffer=torch.from_numpy(buf["slab_meta_buffer"]),
        tile_meta_buffer=torch.from_numpy(buf["tile_meta_buffer"]),
        rank_idx_buffer=torch.from_numpy(buf["rank_idx_buffer"]),
        payload_buffer=torch.from_numpy(buf["payload_buffer"].astype(np.int64)).to(torch.uint32),
        scale_buffer=torch.from_numpy(buf["scale_buffer"]),
    )
    out["matrix_x"] = mat.numpy()
    out["matrix_s"] = svec.numpy()
    out["matrix_in_segments"] = np.asarray([[b, s, e] for b, (s, e) in segments], dtype=np.int32)
    out["matrix_reference_validator_passed"] = np.asarray(1, dtype=np.int8)
    for k, v in buf.items():
        out[f"matrix_{k}"] = v

    path = os.path.join(HERE, "format_golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
