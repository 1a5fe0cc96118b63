"""CPU tests: generator vs oracle packer, oracle self-consistency, C-ABI surface, module API."""
import ctypes
import os
import re
from types import SimpleNamespace as NS

import numpy as np
import pytest
import torch

from bitsmoe_b200 import capi, synth
from bitsmoe_b200.quant import packer as ppacker
from oracle import forward as oforward
from oracle import packer as opacker
from tests import helpers

ROOT = helpers.ROOT


def test_generator_matches_oracle_packer():
    layer = synth.make_layer(synth.tiny(rank=150), seed=5, keep_full=True)
    for tag in ("gate", "up", "down"):
        for e in (0, 3, 7):
            full = layer.extras[tag][e]
            want = opacker.pack_matrix(full["_rank_major"], full["_s"], full["_segments"])
            got = helpers.to_numpy_buf(full)
            for k, v in want.items():
                assert np.array_equal(got[k], v), (tag, e, k)
            opacker.validate_layout(full["_rank_major"], got)


def test_product_packer_all_widths_match_oracle():
    layer = helpers.mixed_everything_layer()
    for tag in ("gate", "down"):
        for e in range(layer.cfg.num_experts):
            full = layer.extras[tag][e]
            want = opacker.pack_matrix(full["_rank_major"], full["_s"], full["_segments"])
            got = helpers.to_numpy_buf(full)
            for k, v in want.items():
                assert np.array_equal(got[k], v), (tag, e, k)
            dec = ppacker.unpack_rank_major(full, layer.cfg.intermediate)
            ref = opacker.decode_matrix(got, layer.cfg.intermediate)
            assert np.array_equal(dec["codes"].numpy(), ref["codes"])
            assert np.array_equal(dec["w"].numpy(), ref["w"])
            ppacker.validate_runtime_layout(full["_rank_major"], full["slab_meta_buffer"], full["tile_meta_buffer"],
                                            full["rank_idx_buffer"], full["payload_buffer"], full["scale_buffer"])


def test_pack_single_weight_writes_checkpoint_schema():
    g = torch.Generator().manual_seed(0)
    gate = (torch.randn(40, 96, generator=g) * 0.02, torch.rand(40, generator=g))
    down = (torch.randn(96, 40, generator=g) * 0.02, torch.rand(40, generator=g))
    sd = {}
    segs = [(4, (0, 8)), (2, (8, 40))]
    ppacker.pack_single_weight({0: {3: {"gate_proj": gate}}}, segs, sd, 0, 3, "gate_proj", validate_layout=True)
    ppacker.pack_single_weight({0: {3: {"down_proj": down}}}, segs, sd, 0, 3, "down_proj", validate_layout=True)
    p = "quantized.layer0.expert3"
    for k in ("payload_buffer", "rank_idx_buffer", "tile_meta_buffer", "slab_meta_buffer", "scale_buffer"):
        assert f"{p}.gate_proj.u.{k}" in sd and f"{p}.down_proj.vh.{k}" in sd
    for k in ("s_buffer", "segments", "original_indices", "original_rank", "groupsize"):
        assert f"{p}.gate_proj.{k}" in sd
    assert sd[f"{p}.gate_proj.u.payload_buffer"].dtype == torch.uint32
    assert int(sd[f"{p}.down_proj.original_rank"]) == 40
    with pytest.raises(ValueError):
        ppacker.pack_single_weight({0: {3: {"gate_proj": gate}}}, [(5, (0, 40))], sd, 0, 3, "gate_proj")
    with pytest.raises(ValueError):
        ppacker.pack_single_weight({0: {3: {"gate_proj": gate}}}, [(2, (0, 30)), (3, (20, 40))], sd, 0, 3, "gate_proj")


def test_oracle_forward_flavours_agree():
    layer = helpers.mixed_everything_layer()
    experts = helpers.decoded_experts(layer)
    cfg = layer.cfg
    x = synth.activations(cfg, 9, seed=2)
    logits = synth.router_logits(cfg, 9, seed=3)
    a = oforward.layer_forward(x, logits, layer.vh_gate, layer.vh_up, layer.u_down, experts, cfg.top_k, mode="fp32")
    b = oforward.layer_forward(x, logits, layer.vh_gate, layer.vh_up, layer.u_down, experts, cfg.top_k, mode="faithful")
    helpers.assert_close(b["y_fp32"], a["y_fp32"], what="faithful vs fp32 oracle")
    assert a["expert_offsets"][-1] == 9 * cfg.top_k
    # expert-contiguous, token-ascending inside each expert
    off = a["expert_offsets"].tolist()
    for e in range(cfg.num_experts):
        seg = a["token_indices"][off[e]:off[e + 1]].tolist()
        assert seg == sorted(seg)


def test_router_tie_break_and_rounding():
    logits = torch.zeros(2, 8)
    logits[1, 5] = 1.0
    idx, w = oforward.router(logits, 3, True, torch.float16)
    assert idx[0].tolist() == [0, 1, 2] and idx[1].tolist() == [5, 0, 1]
    assert torch.equal(w, w.half().float())
    idx2, w2 = oforward.router(logits, 3, False, None)
    assert abs(float(w2[0].sum()) - 3 / 8) < 1e-6


def test_c_abi_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "bitsmoe_b200.h")).read()
    declared = set(re.findall(r"\b(bm_[a-z0-9_]+)\s*\(", header))
    assert declared == set(capi.exported_symbols())
    if not os.path.exists(capi.LIB_PATH):
        pytest.skip("library not built")
    handle = ctypes.CDLL(capi.LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), name
    assert capi.lib().bm_abi_version() == 2
    assert capi.lib().bm_status_string(5) == b"device wait timed out"


def _qwen_config(cfg: synth.LayerConfig):
    return NS(hidden_size=cfg.hidden, intermediate_size=cfg.intermediate, moe_intermediate_size=cfg.intermediate,
              num_experts=cfg.num_experts, num_experts_per_tok=cfg.top_k, norm_topk_prob=True, hidden_act="silu")


def test_expert_module_loads_both_key_schemas():
    from bitsmoe_b200.models.qwen3moe.bitsmoe_mlp import BitsMoE_Qwen3MoeMLP
    layer = synth.make_layer(synth.tiny(), seed=1, keep_full=True)
    conf = _qwen_config(layer.cfg)
    sd = layer.expert_state_dict(2, "quantized.layer0.expert2")
    m = BitsMoE_Qwen3MoeMLP(conf, layer.cfg.intermediate, packed_state=sd, packed_prefix="quantized.layer0.expert2")
    assert m.is_bitsmoe_packed and not m.skip_expert
    assert m.gate_payload_buffer.dtype == torch.uint32 and m.down_s_buffer.dtype == torch.float16
    assert m.runtime_meta["down_proj"]["packed_field"] == "vh"
    assert len(list(m.buffers())) == 30
    # materialised module schema, through nn.Module.load_state_dict on a fresh module
    m2 = BitsMoE_Qwen3MoeMLP(conf, layer.cfg.intermediate)
    assert not m2.is_bitsmoe_packed
    m2.load_state_dict(m.state_dict())
    assert m2.is_bitsmoe_packed
    for k, v in m.state_dict().items():
        assert torch.equal(m2.state_dict()[k], v), k
    m3 = BitsMoE_Qwen3MoeMLP(conf, layer.cfg.intermediate)
    assert m3.load_runtime_packed_from_state({f"p.{k}": v for k, v in m.state_dict().items()}, "p")
    assert torch.equal(m3.up_scale_buffer, m.up_scale_buffer)
    with pytest.raises(NotImplementedError):
        m(torch.zeros(1, layer.cfg.hidden))
    assert not BitsMoE_Qwen3MoeMLP(conf, 160).load_runtime_packed_from_state({}, "missing")


def test_block_api_and_errors_without_gpu():
    from bitsmoe_b200.models.qwen3moe.bitsmoe_block import BitsMoE_Qwen3MoeSparseMoeBlock
    from bitsmoe_b200.models.qwen3moe.bitsmoe_mlp import BitsMoE_Qwen3MoeMLP
    layer = synth.make_layer(synth.tiny(), seed=1, keep_full=True)
    cfg = layer.cfg
    conf = _qwen_config(cfg)
    src = NS(gate=torch.nn.Linear(cfg.hidden, cfg.num_experts, bias=False).half(), experts=[None] * cfg.num_experts)
    with pytest.raises(ValueError):
        BitsMoE_Qwen3MoeSparseMoeBlock(conf, 0, None)
    blk = BitsMoE_Qwen3MoeSparseMoeBlock(conf, 0, src, super_experts=None, copy_source_experts=False)
    assert blk.shared_vh_gate_proj.numel() == 0 and blk.shared_vh_gate_proj.dtype == torch.float16
    for e in range(cfg.num_experts):
        m = BitsMoE_Qwen3MoeMLP(conf, cfg.intermediate, packed_state=layer.expert_state_dict(e, f"x.{e}"),
                                packed_prefix=f"x.{e}")
        blk.set_expert(e, m, packed=True)
    blk.set_shared_basis(layer.vh_gate, layer.vh_up, layer.u_down)
    assert all(blk.packed_expert_mask)
    blk._ensure_runtime_cache(torch.device("cpu"))
    assert blk._packed_expert_count == cfg.num_experts and len(blk._gate_payload_static) == cfg.num_experts
    assert blk._packed_global_to_local.tolist() == list(range(cfg.num_experts))
    # no CPU fallback: forward on CPU tensors must fail loudly
    with pytest.raises(RuntimeError, match="python fallback is intentionally disabled"):
        blk(torch.zeros(1, 2, cfg.hidden, dtype=torch.float16))
    # state dict round trip resizes the basis buffers
    blk2 = BitsMoE_Qwen3MoeSparseMoeBlock(conf, 0, src, copy_source_experts=False)
    for e in range(cfg.num_experts):
        blk2.set_expert(e, BitsMoE_Qwen3MoeMLP(conf, cfg.intermediate), packed=True)
    blk2.load_state_dict(blk.state_dict())
    assert torch.equal(blk2.shared_u_down, blk.shared_u_down)
    assert blk2.experts[3].is_bitsmoe_packed
    conf_bad = _qwen_config(cfg)
    conf_bad.hidden_act = "gelu"
    blk.config = conf_bad
    with pytest.raises(RuntimeError, match="Unsupported hidden_act"):
        blk._act_type()


def test_op_argument_checks_match_reference_messages():
    from bitsmoe_b200.algorithms import _mlp_forward as op
    z = torch.zeros
    lists = [[] for _ in range(18)]
    with pytest.raises(RuntimeError, match="h_gate must be 2D"):
        op.moe_packed_forward(z(4), z(1, 4), z(0), z(1), z(0), *lists, 4, 128, 0)
    with pytest.raises(RuntimeError, match="h_gate must be CUDA tensor"):
        op.moe_packed_forward(z(1, 4), z(1, 4), z(0, dtype=torch.int32), z(1, dtype=torch.int32), z(0), *lists, 4, 128, 0)
