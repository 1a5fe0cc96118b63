"""GPU: the drop-in block modules end to end against the CPU oracle."""
from types import SimpleNamespace as NS

import pytest
import torch
import torch.nn as nn

from bitsmoe_b200 import synth
from oracle import forward as oforward
from tests import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class DenseMLP(nn.Module):
    def __init__(self, hidden, inter, w=None):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)
        if w is not None:
            self.gate_proj.weight.data, self.up_proj.weight.data, self.down_proj.weight.data = w["gate"], w["up"], w["down"]

    def forward(self, x):
        return self.down_proj(nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


def _conf(cfg, **kw):
    return NS(hidden_size=cfg.hidden, intermediate_size=cfg.intermediate, num_experts=cfg.num_experts,
              num_experts_per_tok=cfg.top_k, norm_topk_prob=cfg.norm_topk_prob, hidden_act="silu", **kw)


def _fill(blk, mlp_cls, conf, layer, skip=()):
    for e in range(layer.cfg.num_experts):
        if e in skip:
            continue
        m = mlp_cls(conf, layer.cfg.intermediate, packed_state=layer.expert_state_dict(e, f"p.{e}"), packed_prefix=f"p.{e}")
        blk.set_expert(e, m, packed=True)
    blk.set_shared_basis(layer.vh_gate, layer.vh_up, layer.u_down)


def test_qwen3moe_block_matches_oracle_with_and_without_super_expert():
    from bitsmoe_b200.models.qwen3moe.bitsmoe_block import BitsMoE_Qwen3MoeSparseMoeBlock
    from bitsmoe_b200.models.qwen3moe.bitsmoe_mlp import BitsMoE_Qwen3MoeMLP
    cfg = synth.tiny(hidden=256, num_experts=8, intermediate=256, top_k=2, rank=64)
    layer = synth.make_layer(cfg, seed=9, keep_full=True)
    experts = helpers.decoded_experts(layer)
    conf = _conf(cfg)
    gate = nn.Linear(cfg.hidden, cfg.num_experts, bias=False).half()
    src = NS(gate=gate, experts=[None] * cfg.num_experts)
    blk = BitsMoE_Qwen3MoeSparseMoeBlock(conf, 3, src, copy_source_experts=False).to(DEV)
    _fill(blk, BitsMoE_Qwen3MoeMLP, conf, layer)
    blk.prepare_runtime_fastpath(warmup=True)
    x = synth.activations(cfg, 12, seed=1, dtype=torch.float16).reshape(3, 4, cfg.hidden)
    y, logits = blk(x.to(DEV))
    assert tuple(y.shape) == (3, 4, cfg.hidden) and tuple(logits.shape) == (12, cfg.num_experts)
    o = oforward.layer_forward(x.reshape(12, -1), logits.float().cpu(), layer.vh_gate, layer.vh_up, layer.u_down, experts,
                               cfg.top_k, True, torch.float16)
    helpers.assert_close(y.reshape(12, -1), o["y_fp32"], what="Qwen3-MoE block")

    # expert 2 becomes an unquantised "super" expert: it runs as a dense module and leaves the packed set
    dense = DenseMLP(cfg.hidden, cfg.intermediate).half().to(DEV)
    blk2 = BitsMoE_Qwen3MoeSparseMoeBlock(conf, 3, src, super_experts=[2], copy_source_experts=False).to(DEV)
    _fill(blk2, BitsMoE_Qwen3MoeMLP, conf, layer, skip=(2,))
    blk2.set_expert(2, dense, packed=False)
    y2, _ = blk2(x.to(DEV))
    idx, w = oforward.router(logits.float().cpu(), cfg.top_k, True, torch.float16)
    g2l = torch.tensor([0, 1, -1, 2, 3, 4, 5, 6], dtype=torch.int32)
    tok, off, rw = oforward.build_routing(idx, w, 7, g2l)
    hg, hu = oforward.basis_project(x.reshape(12, -1), layer.vh_gate), oforward.basis_project(x.reshape(12, -1), layer.vh_up)
    acc = oforward.packed_forward(hg, hu, tok, off, rw, [experts[i] for i in (0, 1, 3, 4, 5, 6, 7)], cfg.rank)
    want = oforward.down_basis(acc, layer.u_down, torch.float32)
    dw = {k: getattr(dense, k + "_proj").weight.detach().cpu() for k in ("gate", "up", "down")}
    d = oforward.dense_mlp(x.reshape(12, -1), dw["gate"], dw["up"], dw["down"])
    sel = (idx == 2)
    want = want + d * (w * sel).sum(-1, keepdim=True)
    helpers.assert_close(y2.reshape(12, -1), want, what="Qwen3-MoE block with a super expert")


def test_qwen3next_block_adds_gated_shared_expert():
    from bitsmoe_b200.models.qwen3next.bitsmoe_block import BitsMoE_Qwen3NextSparseMoeBlock
    from bitsmoe_b200.models.qwen3next.bitsmoe_mlp import BitsMoE_Qwen3NextMLP
    cfg = synth.tiny(hidden=256, num_experts=16, intermediate=128, top_k=4, rank=48, shared_intermediate=128,
                     shared_gated=True)
    layer = synth.make_layer(cfg, seed=10, keep_full=True)
    experts = helpers.decoded_experts(layer)
    conf = _conf(cfg)
    src = NS(gate=nn.Linear(cfg.hidden, cfg.num_experts, bias=False).half(), experts=[None] * cfg.num_experts,
             shared_expert=DenseMLP(cfg.hidden, cfg.shared_intermediate, layer.shared).half(),
             shared_expert_gate=nn.Linear(cfg.hidden, 1, bias=False).half())
    src.shared_expert_gate.weight.data = layer.shared["gate_logit_w"]
    blk = BitsMoE_Qwen3NextSparseMoeBlock(conf, 0, src, copy_source_experts=False).to(DEV)
    _fill(blk, BitsMoE_Qwen3NextMLP, conf, layer)
    x = synth.activations(cfg, 10, seed=2, dtype=torch.bfloat16).reshape(1, 10, cfg.hidden)
    blk = blk.to(torch.bfloat16)
    y, logits = blk(x.to(DEV))
    o = oforward.layer_forward(x.reshape(10, -1), logits.float().cpu(), layer.vh_gate, layer.vh_up, layer.u_down, experts,
                               cfg.top_k, True, torch.bfloat16, shared=layer.shared)
    helpers.assert_close(y.reshape(10, -1), o["y_fp32"], what="Qwen3-Next block")


class StubMoEGate(nn.Module):
    """softmax -> top-k, no renormalisation (DeepSeek-V2-Lite defaults)."""

    def __init__(self, hidden, experts, k):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(experts, hidden) * 0.05)
        self.k = k

    def forward(self, h):
        x = h.reshape(-1, h.shape[-1])
        p = torch.softmax(nn.functional.linear(x.float(), self.weight.float()), dim=-1)
        w, idx = torch.topk(p, self.k, dim=-1, sorted=False)
        return idx, w, None


def test_deepseek_block_adds_shared_experts():
    from bitsmoe_b200.models.deepseekv2.bitsmoe_block import BitsMoE_DeepSeekSparseMoeBlock
    from bitsmoe_b200.models.deepseekv2.bitsmoe_mlp import BitsMoE_DeepSeekMLP
    cfg = synth.tiny(hidden=256, num_experts=8, intermediate=160, top_k=3, rank=40, bit_probs=((2, 1.0),),
                     norm_topk_prob=False, shared_intermediate=320)
    layer = synth.make_layer(cfg, seed=12, keep_full=True)
    experts = helpers.decoded_experts(layer)
    conf = _conf(cfg, n_shared_experts=2)
    src = NS(gate=StubMoEGate(cfg.hidden, cfg.num_experts, cfg.top_k), experts=[None] * cfg.num_experts,
             shared_experts=DenseMLP(cfg.hidden, cfg.shared_intermediate, layer.shared).half(), ep_size=1,
             experts_per_rank=cfg.num_experts, ep_rank=0)
    blk = BitsMoE_DeepSeekSparseMoeBlock(conf, 1, src, copy_source_experts=False).to(DEV).eval()
    _fill(blk, BitsMoE_DeepSeekMLP, conf, layer)
    x = synth.activations(cfg, 6, seed=3, dtype=torch.float16).reshape(2, 3, cfg.hidden)
    y = blk(x.to(DEV))
    assert tuple(y.shape) == (2, 3, cfg.hidden)
    idx, w, _ = blk.gate(x.to(DEV))
    tok, off, rw = oforward.build_routing(idx.cpu(), w.cpu(), cfg.num_experts)
    xf = x.reshape(6, -1)
    acc = oforward.packed_forward(oforward.basis_project(xf, layer.vh_gate), oforward.basis_project(xf, layer.vh_up), tok,
                                  off, rw, experts, cfg.rank)
    want = oforward.down_basis(acc, layer.u_down, torch.float32) + oforward.dense_mlp(
        xf, layer.shared["gate"], layer.shared["up"], layer.shared["down"])
    helpers.assert_close(y.reshape(6, -1), want, what="DeepSeek block")
