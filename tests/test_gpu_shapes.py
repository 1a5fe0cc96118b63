"""GPU: the three benchmark layer shapes at small token counts, every experts path against the CPU oracle."""
import pytest
import torch

from bitsmoe_b200 import capi, synth
from oracle import forward as oforward
from tests import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module", params=["deepseek-v2-lite", "qwen3-next-80b-a3b", "qwen3-30b-a3b"])
def shaped(request):
    cfg = synth.PRESETS[request.param]
    layer = synth.make_layer(cfg, seed=17, device=DEV)
    return layer, synth.to_packed_layer(layer, DEV), helpers.LazyDecodedExperts(layer)


@pytest.mark.parametrize("T", [1, 6])
def test_full_shapes_layer_forward(shaped, T):
    layer, packed, experts = shaped
    cfg = layer.cfg
    x = synth.activations(cfg, T, seed=5)
    logits = synth.router_logits(cfg, T, seed=6)
    wdt = torch.bfloat16 if cfg.round_route_weights else None
    o = oforward.layer_forward(x, logits, layer.vh_gate.cpu(), layer.vh_up.cpu(), layer.u_down.cpu(), experts, cfg.top_k,
                               cfg.norm_topk_prob, wdt)
    assert packed.has_fast_layout
    for path in (capi.PATH_DECODE, capi.PATH_TENSOR, capi.PATH_GENERIC):
        y = packed.forward(x.to(DEV), logits.to(DEV), cfg.top_k, cfg.norm_topk_prob, wdt, path=path)
        packed.check_status()
        helpers.assert_close(y, o["y_fp32"], what=f"{cfg.name} T={T} path={path}")
    # bytes one expert costs the forward path, as the reference stores them
    per_expert = packed.expert_bytes(0)
    want = {"qwen3-30b-a3b": 180768, "qwen3-next-80b-a3b": 124570, "deepseek-v2-lite": 293616}[cfg.name]
    assert abs(per_expert - want) / want < 0.05
