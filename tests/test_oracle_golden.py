"""The CPU oracle against fixtures produced by the reference's own Python
(tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import bitplane, packer, quantize

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "format_golden.npz"))


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 6, 8])
def test_quantize_symmetric_known_answers(bits):
    for tag, dim in (("full", 2), ("tail", 1)):
        x = torch.from_numpy(G[f"quant_x_{tag}"])
        q, s = quantize.quantize_symmetric(x, bits=bits, dim=dim)
        assert np.array_equal(q.numpy(), G[f"quant_q_{tag}_b{bits}"])
        assert np.array_equal(s.numpy(), G[f"quant_s_{tag}_b{bits}"])


@pytest.mark.parametrize("k_slab,wpr", [(64, 2), (16, 3), (13, 4), (37, 2)])
def test_stage_micro_reorder(k_slab, wpr):
    src = np.arange(2 * k_slab * 4 * wpr, dtype=np.int64).reshape(2, k_slab, 4, wpr)
    want = G[f"reorder_k{k_slab}_w{wpr}"]
    for t in range(2):
        got = packer._stage_micro_order(src[t])
        assert np.array_equal(got, want[t])


@pytest.mark.parametrize("k_slab,dim,bits", [(13, 160, 4), (64, 256, 2), (38, 384, 3), (5, 96, 8),
                                             (16, 128, 1), (9, 224, 6)])
def test_slab_payload_and_scale(k_slab, dim, bits):
    x = torch.from_numpy(G[f"slab_x_k{k_slab}_d{dim}_b{bits}"])
    buf = packer.pack_matrix(x, torch.ones(k_slab), [(bits, (0, k_slab))])
    assert np.array_equal(buf["payload_buffer"], G[f"slab_payload_k{k_slab}_d{dim}_b{bits}"].reshape(-1))
    assert np.array_equal(buf["scale_buffer"], G[f"slab_scale_k{k_slab}_d{dim}_b{bits}"])


def test_fp16_slab():
    x = torch.from_numpy(G["slab16_x"])
    buf = packer.pack_matrix(x, torch.ones(x.shape[0]), [(16, (0, x.shape[0]))])
    assert np.array_equal(buf["payload_buffer"], G["slab16_payload"].reshape(-1))
    assert np.array_equal(buf["scale_buffer"], G["slab16_scale"])
    dec = packer.decode_matrix(buf, x.shape[1])
    assert np.array_equal(dec["w"], x.to(torch.float16).float().numpy())


def test_tile_codec():
    q = np.zeros((37, 128), dtype=np.int8)
    q[:, :96] = G["tile_q"]
    pay = packer.pack_tile_lowbit(q, 3)
    assert np.array_equal(pay, G["tile_payload_b3"])
    assert np.array_equal(packer.unpack_tile(G["tile_payload_b3"], 3, 37), G["tile_decoded_b3"])


def test_whole_matrix_buffers_and_validator():
    assert int(G["matrix_reference_validator_passed"]) == 1
    x, s = torch.from_numpy(G["matrix_x"]), torch.from_numpy(G["matrix_s"])
    segs = [(int(b), (int(a), int(e))) for b, a, e in G["matrix_in_segments"]]
    buf = packer.pack_matrix(x, s, segs)
    for k, v in buf.items():
        assert np.array_equal(v, G[f"matrix_{k}"]), k
    packer.validate_layout(x, buf)
    dec = packer.decode_matrix(buf, x.shape[1])
    # rows given 0 bits are dropped; slabs come in descending width
    assert dec["rank_idx"].size == 150 - 6
    assert list(buf["slab_meta_buffer"][:, 0]) == sorted(buf["slab_meta_buffer"][:, 0], reverse=True)


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 6, 8])
def test_bitplane_roundtrip(bits):
    rng = np.random.default_rng(bits)
    lo, hi = (-(2 ** (bits - 1)), 2 ** (bits - 1)) if bits > 1 else (0, 2)
    q = rng.integers(lo, hi, size=(5, 96)).astype(np.int8)
    if bits == 1:
        q = (q * 2 - 1).astype(np.int8)
    w = bitplane.pack_bitplanes_i8(q, bits)
    assert w.shape == (5, 3 * bits)
    assert np.array_equal(bitplane.unpack_bitplanes_i8(w, bits), q)
    # word p, bit l  ==  bit p of the unsigned code at column group*32 + l
    u = bitplane.to_unsigned(q, bits)
    assert ((int(w[2, 1 * bits + (bits - 1)]) >> 7) & 1) == ((int(u[2, 32 + 7]) >> (bits - 1)) & 1)
