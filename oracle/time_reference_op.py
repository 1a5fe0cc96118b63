"""Times the reference's own CUDA op (oracle/_ref, recompiled for sm_100a by oracle/build_ref.py) at the op boundary,
beside this build's packed-experts stage on the same prepared inputs.  Test infrastructure, one GPU:

    python oracle/time_reference_op.py            # TOKENS=1,8,32,64,2048 LAYERS=6 by default
"""
import sys, os, json, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from bitsmoe_b200 import synth, capi
from bitsmoe_b200.layer import route_build, route_topk
from tests import helpers
dev = "cuda:0"
cfg = synth.QWEN3_30B
L = int(os.environ.get("LAYERS", "6"))
ref = helpers.load_reference_ext("_mlp_forward_cuda")
layers = [synth.make_layer(cfg, seed=42 + i, device=dev) for i in range(L)]
packed = [synth.to_packed_layer(l, dev) for l in layers]
refargs = [helpers.ref_args(l, dev) for l in layers]
res = {}
for T in [int(t) for t in os.environ.get("TOKENS", "1,8,32,64,2048").split(",")]:
    prep = []
    for i in range(L):
        x = synth.activations(cfg, T, seed=7 + i, device=dev)
        lg = synth.router_logits(cfg, T, seed=9 + i, device=dev, zipf_s=1.1 if T > 1000 else 0.0)
        idx, w = route_topk(lg, cfg.top_k, True, torch.bfloat16)
        tok, off, rw, _, _ = route_build(idx, w, cfg.num_experts)
        hg, hu = packed[i].basis_project(x)
        prep.append((hg, hu, tok, off, rw))
    def run(fn, n):
        for i in range(3): fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n): fn(i)
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / n
    n = 50 if T <= 64 else 5
    ours = run(lambda i: packed[i % L].experts_forward(*prep[i % L]), n)
    theirs = run(lambda i: ref.moe_packed_forward(*prep[i % L], *refargs[i % L], cfg.rank, cfg.intermediate, 0), n) if ref else None
    res[T] = {"ours_ms": ours, "reference_kernels_ms": theirs}
    print(T, res[T], flush=True)
print(json.dumps(res))
