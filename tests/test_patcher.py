"""The model patcher against transformers' current (fused-experts) Qwen3-MoE layout: structure and checkpoint loading on
the CPU, a forward of the patched model on the GPU."""
import pytest
import torch

from bitsmoe_b200 import synth
from bitsmoe_b200.models.auto import build_patched_model, patch_bitsmoe_inplace
from bitsmoe_b200.models.base_block import BitsMoE_BaseSparseMoeBlock
from oracle import forward as oforward
from tests import helpers

transformers = pytest.importorskip("transformers")

HID, NEXP, INTER, TOPK, RANK, LAYERS = 64, 8, 128, 2, 32, 2
SUPER = {1: [3]}


def _config():
    return transformers.Qwen3MoeConfig(
        vocab_size=128, hidden_size=HID, intermediate_size=128, moe_intermediate_size=INTER, num_hidden_layers=LAYERS,
        num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_experts=NEXP, num_experts_per_tok=TOPK,
        max_position_embeddings=64, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True, hidden_act="silu")


def _checkpoint(cfg, super_map=SUPER):
    """A BitsMoE checkpoint for the tiny model: the stock model's dense tensors (attention, norms, embeddings, router),
    plus per MoE layer the three basis buffers and every expert's packed buffers in the packer's key schema; expert 3
    of layer 1 stays dense ("super") under the default ``super_map``."""
    torch.manual_seed(0)
    stock = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    state = {k: v.clone() for k, v in stock.state_dict().items() if ".mlp.experts." not in k}
    layers = []
    lcfg = synth.LayerConfig("tiny-hf", HID, NEXP, INTER, TOPK, rank=RANK)
    for li in range(LAYERS):
        layer = synth.make_layer(lcfg, seed=50 + li, keep_full=True)
        layers.append(layer)
        pre = f"model.layers.{li}.mlp"
        state[f"{pre}.shared_vh_gate_proj"], state[f"{pre}.shared_vh_up_proj"] = layer.vh_gate, layer.vh_up
        state[f"{pre}.shared_u_down"] = layer.u_down
        for e in range(NEXP):
            if e in super_map.get(li, []):
                gu, dn = stock.model.layers[li].mlp.experts.gate_up_proj[e], stock.model.layers[li].mlp.experts.down_proj[e]
                state[f"{pre}.experts.{e}.gate_proj.weight"] = gu[:INTER].detach().clone()
                state[f"{pre}.experts.{e}.up_proj.weight"] = gu[INTER:].detach().clone()
                state[f"{pre}.experts.{e}.down_proj.weight"] = dn.detach().clone()
            else:
                state.update(layer.expert_state_dict(e, f"{pre}.experts.{e}"))
    return stock, state, layers


def test_patcher_rewrites_fused_expert_blocks_and_loads_the_checkpoint():
    cfg = _config()
    stock, state, _ = _checkpoint(cfg)
    model = build_patched_model(cfg, "qwen3moe", state, super_experts_by_layer=SUPER)
    assert model._bitsmoe_packed_expert_total == LAYERS * NEXP - 1
    assert not [n for n, p in list(model.named_parameters()) + list(model.named_buffers()) if p.is_meta]
    for li, layer in enumerate(model.model.layers):
        blk = layer.mlp
        assert isinstance(blk, BitsMoE_BaseSparseMoeBlock) and blk.return_router_logits is False
        assert isinstance(blk.gate, torch.nn.Linear) and blk.gate.bias is None
        assert torch.equal(blk.gate.weight, stock.model.layers[li].mlp.gate.weight)
        assert tuple(blk.shared_vh_gate_proj.shape) == (RANK, HID) and blk.shared_u_down.dtype == torch.float16
        for e, m in enumerate(blk.experts):
            if e in SUPER.get(li, []):
                assert not blk.packed_expert_mask[e] and tuple(m.gate_proj.weight.shape) == (INTER, HID)
            else:
                assert blk.packed_expert_mask[e] and m.is_bitsmoe_packed
                assert m.gate_payload_buffer.dtype == torch.uint32 and m.gate_payload_buffer.numel() > 0
    # no dense routed-expert tensors survive in the patched model
    assert not [k for k in model.state_dict() if k.endswith("gate_up_proj")]
    # in-place form on a real (non-meta) model, buffers bound straight from the state dict
    stock2 = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    n = patch_bitsmoe_inplace(stock2, "qwen3moe", packed_state=state, super_experts_by_layer=SUPER)
    assert n == LAYERS * NEXP - 1 and stock2.model.layers[0].mlp.experts[0].is_bitsmoe_packed
    assert stock2.model.layers[0].mlp.shared_vh_up_proj.numel() == RANK * HID
    with pytest.raises(ValueError, match="Unsupported bitsmoe_model_type"):
        patch_bitsmoe_inplace(stock2, "mixtral")


def _oracle_block(x2, logits, layer, dense):
    """The block's output on the CPU: packed experts through the oracle; an expert listed in ``dense`` (id -> its three
    matrices) acts as a plain MLP on its tokens instead."""
    idx, w = oforward.router(logits, TOPK, True, torch.float16)
    w_packed = w.clone()
    for e in dense:
        w_packed[idx == e] = 0.0
    tok, off, rw = oforward.build_routing(idx, w_packed, NEXP)
    hg, hu = oforward.basis_project(x2, layer.vh_gate), oforward.basis_project(x2, layer.vh_up)
    acc = oforward.packed_forward(hg, hu, tok, off, rw, helpers.decoded_experts(layer), layer.u_down.shape[1])
    y = oforward.down_basis(acc, layer.u_down, torch.float32)
    for e, (wg, wu, wd) in dense.items():
        rows, slots = (idx == e).nonzero(as_tuple=True)
        if rows.numel():
            y[rows] += w[rows, slots].float()[:, None] * oforward.dense_mlp(x2[rows], wg, wu, wd).float()
    return y


@pytest.mark.gpu
@pytest.mark.parametrize("super_map", [{}, SUPER], ids=["all-packed", "one-dense-expert"])
def test_patched_model_runs_and_its_blocks_match_the_oracle(super_map):
    cfg = _config()
    _, state, layers = _checkpoint(cfg, super_map)
    dev = torch.device("cuda", 0)
    model = build_patched_model(cfg, "qwen3moe", state, device=dev, super_experts_by_layer=super_map)
    model.eval()
    seen = {}
    hooks = [model.model.layers[li].mlp.register_forward_hook(lambda mod, inp, out, li=li: seen.__setitem__(li, (inp[0].detach(), out.detach())))
             for li in range(LAYERS)]
    ids = torch.randint(0, 128, (2, 9), generator=torch.Generator().manual_seed(3)).to(dev)
    with torch.no_grad():
        out = model(input_ids=ids)
    for h in hooks:
        h.remove()
    assert tuple(out.logits.shape) == (2, 9, 128) and bool(torch.isfinite(out.logits.float()).all())
    for li in range(LAYERS):
        x, y = seen[li]
        x2 = x.reshape(-1, HID).cpu()
        blk = model.model.layers[li].mlp
        logits = (x2.double() @ blk.gate.weight.detach().cpu().double().T).to(torch.float16)
        dense = {e: tuple(state[f"model.layers.{li}.mlp.experts.{e}.{m}.weight"] for m in ("gate_proj", "up_proj", "down_proj"))
                 for e in super_map.get(li, [])}
        want = _oracle_block(x2, logits.float(), layers[li], dense)
        helpers.assert_close(y.reshape(-1, HID), want, what=f"patched model, MoE block of layer {li}")
        helpers.assert_detects_damage(y.reshape(-1, HID), want)
