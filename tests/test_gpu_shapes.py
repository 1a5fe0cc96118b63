"""GPU: the three benchmark layer shapes (64 x 1408, 512 x 512 and 128 x 768 experts), every experts path, at the
token counts the benchmark quotes: layer outputs against the CPU oracle, and rank_accum of the decode and tensor paths
against the generic path, the reference's own recompiled kernels and the fp32 oracle on sampled tokens."""
import pytest
import torch

from bitsmoe_b200 import capi, synth
from bitsmoe_b200.layer import route_build, route_topk
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


def _routed_problem(layer, packed, T, seed, zipf_s=0.0):
    """x, logits -> (h_gate, h_up, token_indices, expert_offsets, route_flat) on the device, plus the top-k on the host.
    Routing and projection come from the library's own kernels (pinned bit-exactly / at 2e-3 elsewhere), so that the
    three implementations of the packed-expert stage below see identical inputs."""
    cfg = layer.cfg
    x = synth.activations(cfg, T, seed=seed).to(DEV)
    logits = synth.router_logits(cfg, T, seed=seed + 1, zipf_s=zipf_s).to(DEV)
    wdt = torch.float16 if cfg.round_route_weights else None
    idx, w = route_topk(logits, cfg.top_k, cfg.norm_topk_prob, wdt)
    tok, off, rw, _, counts = route_build(idx, w, cfg.num_experts)
    n = int(counts.cpu()[0])
    hg, hu = packed.basis_project(x)
    return (hg.contiguous(), hu.contiguous(), tok[:n].contiguous(), off, rw[:n].contiguous()), idx.cpu().long(), w.cpu()


def _oracle_rows(layer, experts, args, idx, w, tokens):
    """fp32 oracle rank_accum rows of a few tokens (only the experts those tokens use are dequantised)."""
    hg, hu = args[0].cpu(), args[1].cpu()
    sel = torch.tensor(tokens)
    tok, off, rw = oforward.build_routing(idx[sel], w[sel], layer.cfg.num_experts)
    return oforward.packed_forward(hg[sel], hu[sel], tok, off, rw, experts, layer.cfg.rank, mode="fp32")


def _reference_rank_accum(layer, args):
    ref = helpers.load_reference_ext("_mlp_forward_cuda")
    if ref is None:
        return None
    lists = helpers.ref_args(layer, DEV)
    return lambda: ref.moe_packed_forward(*args, *lists, layer.cfg.rank, layer.cfg.intermediate, 0)


def _check_stage(layer, packed, experts, args, idx, w, path, tag, rtol, atol):
    T = args[0].shape[0]
    got = packed.experts_forward(*args, path=path)
    packed.check_status()
    gen = packed.experts_forward(*args, path=capi.PATH_GENERIC)
    helpers.assert_close(got, gen, rtol=rtol, atol=atol, what=f"{tag}: fast path vs generic path")
    helpers.assert_detects_damage(got, gen, rtol=rtol, atol=atol, what=tag)
    # a dropped expert must be visible: zero the route weights of the busiest expert's assignments
    off = args[3].cpu()
    e = int((off[1:] - off[:-1]).argmax())
    rw = args[4].clone()
    rw[int(off[e]):int(off[e + 1])] = 0
    dropped = packed.experts_forward(args[0], args[1], args[2], args[3], rw, path=path)
    with pytest.raises(AssertionError):
        helpers.assert_close(dropped, gen, rtol=rtol, atol=atol, what=f"{tag}: expert {e} dropped")
    tokens = sorted({0, T // 2, T - 1})
    want = _oracle_rows(layer, experts, args, idx, w, tokens)
    helpers.assert_close(got[tokens], want, rtol=rtol, atol=atol, what=f"{tag}: fast path vs fp32 oracle (sampled tokens)")
    run_ref = _reference_rank_accum(layer, args)
    if run_ref is not None:
        # The recompiled reference kernels are not run-to-run stable on this GPU on their tensor-core path (32 tokens
        # and more): single calls return whole token rows off by up to 30 % of the peak, in different rows from call
        # to call, while most calls agree with the fp32 oracle to 4e-4 relative L2.  The element-wise median of five
        # calls is the reference value.  Both sides round their operands to fp16 in different places: element-wise the
        # specification's tolerance (rtol 2e-2 / atol 1e-2); what makes the comparison sharp are assert_close's
        # bounds relative to the peak (2e-2) and in L2 (1e-2); even the median keeps single wrong elements at 8192
        # tokens, so one element in a thousand may miss the element-wise and peak bounds (never the L2 bound).
        outs = []
        for _ in range(5):
            outs.append(run_ref().float().clone())
            torch.cuda.synchronize()
        ref_out = torch.stack(outs).median(dim=0).values
        helpers.assert_close(got, ref_out, outlier_frac=1e-3,
                             what=f"{tag}: fast path vs the reference's kernels (median of five calls)")


@pytest.mark.parametrize("T", [1, 8, 32, 64])
def test_full_shapes_decode_rank_accum(shaped, T):
    layer, packed, experts = shaped
    args, idx, w = _routed_problem(layer, packed, T, seed=700 + T)
    _check_stage(layer, packed, experts, args, idx, w, capi.PATH_DECODE, f"{layer.cfg.name} decode T={T}", 5e-3, 1e-4)


def test_full_shapes_prefill_rank_accum_zipf(shaped):
    layer, packed, experts = shaped
    args, idx, w = _routed_problem(layer, packed, 8192, seed=900, zipf_s=1.1)
    _check_stage(layer, packed, experts, args, idx, w, capi.PATH_TENSOR, f"{layer.cfg.name} prefill T=8192 Zipf", 1e-2, 3e-4)
    # and the path the dispatcher picks by itself at this size is the tensor path
    auto = packed.experts_forward(*args, path=capi.PATH_AUTO)
    tc = packed.experts_forward(*args, path=capi.PATH_TENSOR)
    helpers.assert_close(auto, tc, rtol=1e-3, atol=1e-5, what="AUTO vs tensor path at 8192 tokens")
