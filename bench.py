"""MoE-layer tokens/s on synthetic Qwen3-30B-A3B-shaped layers (decode headline, prefill beside it).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one forward of one packed MoE layer over one batch of tokens: route -> basis
projections -> packed experts -> down basis.  The timed loop rotates over `--layers` distinct
weight sets (more than two L2s of packed bytes) so every step streams its experts from HBM.
Rank 0 prints one JSON line.  `--impl reference` times the CPU dequantise-then-matmul path on
the host cores instead (the reference ships no CPU forward; see oracle/cpu_path.py).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "moe_layer_decode_tokens_per_s"
UNIT = "tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=64, help="decode batch of the headline number")
    ap.add_argument("--layers", type=int, default=12, help="distinct weight sets rotated through")
    ap.add_argument("--prefill-tokens", type=int, default=8192)
    ap.add_argument("--no-extras", action="store_true", help="headline only (skip other batch sizes / prefill / cpu)")
    ap.add_argument("--path", type=int, default=0, help="experts path: 0 auto, 1 generic, 2 decode, 3 tensor")
    ap.add_argument("--parallel", default="dp", choices=["dp", "ep"],
                    help="with --gpus N > 1: dp = every rank runs the whole layer on its own tokens (weights replicated, "
                         "no data-path collective); ep = experts sharded over the ranks, rank-space exchange over NCCL")
    ap.add_argument("--probe", default=None, choices=["experts", "forward"],
                    help="no timing: run the packed-experts stage or the whole layer forward --steps times over --layers "
                         "rotating weight sets with --tokens tokens (Zipf(1.1) routing above 256 tokens) and exit; the "
                         "target of profiler captures")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def dist_env(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ------------------------------------------------------------------------------------------- CPU arm
def cpu_layer_from(layer, top_k, weight_dtype):
    import numpy as np
    from oracle import cpu_path

    def host(t):
        t = t.detach().cpu()
        return t.to(torch.int64).numpy().astype(np.uint32) if t.dtype == torch.uint32 else t.numpy()

    E = layer.cfg.num_experts
    experts = [{tag: {f + "_buffer": host(layer.tables[tag][f][e]) for f in layer.tables[tag]} for tag in ("gate", "up", "down")}
               for e in range(E)]
    return cpu_path.CpuLayer(experts, layer.vh_gate.cpu(), layer.vh_up.cpu(), layer.u_down.cpu(), layer.cfg.intermediate,
                             top_k, layer.cfg.norm_topk_prob, weight_dtype)


def time_cpu(layer, tokens, steps, warmup):
    from bitsmoe_b200 import synth
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cl = cpu_layer_from(layer, layer.cfg.top_k, torch.bfloat16)
    x = synth.activations(layer.cfg, tokens, seed=1)
    logits = synth.router_logits(layer.cfg, tokens, seed=2)
    for _ in range(warmup):
        cl.forward(x, logits)
    t0 = time.perf_counter()
    for _ in range(steps):
        cl.forward(x, logits)
    dt = (time.perf_counter() - t0) / steps
    return tokens / dt, dt, cores


def workload_name(tokens):
    return (f"qwen3-30b-a3b moe layer decode, {tokens} tokens per GPU, mixed 2/3/4-bit (0.8/0.15/0.05), "
            "rank-256 shared basis, top-8 of 128 experts")


def reference_arm(args):
    rank, world, _ = dist_env(args)
    if rank != 0:
        return
    from bitsmoe_b200 import synth
    cfg = synth.QWEN3_30B
    layer = synth.make_layer(cfg, seed=42, device="cpu")
    steps = max(1, min(args.steps, 20))
    warm = max(1, min(args.warmup, 2))
    tps, dt, cores = time_cpu(layer, args.tokens, steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.tokens), "tokens_per_gpu": args.tokens,
                   "sample": "one layer on the host cores of rank 0; the GPU arm's step on the same shapes"},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{steps} forwards of one layer, {args.tokens} tokens, dequantise-then-matmul fp32"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- GPU arm
def timed(fn, steps, stream_sync, use_graph=True, repeats_out=None):
    """CUDA-event time, in ms, of `steps` calls of fn(i).  The calls are captured once into a CUDA graph
    (the launch sequence of all `steps` steps), replayed once untimed and then once inside the timed region, so the
    number reflects the device and not the Python interpreter; every launch of the eager sequence is a
    node of the graph."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if not use_graph:
        stream_sync()
        start.record()
        for i in range(steps):
            fn(i)
        stop.record()
        stream_sync()
        return start.elapsed_time(stop)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(steps):
                fn(i)
    torch.cuda.current_stream().wait_stream(side)
    stream_sync()
    graph.replay()      # untimed: the first launch of an instantiated graph also uploads it to the device
    stream_sync()
    start.record()
    graph.replay()
    stop.record()
    stream_sync()
    first = start.elapsed_time(stop)
    if repeats_out is not None:
        # further replays of the same graph, each timed on its own: spread of the measurement
        for _ in range(repeats_out[0]):
            start.record()
            graph.replay()
            stop.record()
            stream_sync()
            repeats_out[1].append(start.elapsed_time(stop))
    return first


def active_expert_bytes(packed, offsets_cpu):
    n = 0
    act = 0
    for e in range(packed.num_experts):
        if offsets_cpu[e + 1] > offsets_cpu[e]:
            n += packed.expert_bytes(e)
            act += 1
    return n, act


def probe(args):
    """Small fixed workload for profiler captures (one GPU): see --probe."""
    from bitsmoe_b200 import synth
    from bitsmoe_b200.layer import route_build, route_topk
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = synth.QWEN3_30B
    T, L = args.tokens, args.layers
    layers = [synth.to_packed_layer(synth.make_layer(cfg, seed=42 + i, device=dev), dev) for i in range(L)]
    zipf = 1.1 if T > 256 else None
    prep = []
    for i in range(L):
        x = synth.activations(cfg, T, seed=7 + i, device=dev)
        lg = synth.router_logits(cfg, T, seed=9 + i, device=dev) if zipf is None else \
            synth.router_logits(cfg, T, seed=9 + i, zipf_s=zipf, device=dev)
        idx, w = route_topk(lg, cfg.top_k, True, torch.bfloat16)
        tok, off, rw, _, _ = route_build(idx, w, cfg.num_experts)
        hg, hu = layers[i].basis_project(x)
        prep.append((x, lg, hg, hu, tok, off, rw))
    torch.cuda.synchronize(dev)
    for it in range(args.steps):
        i = it % L
        if args.probe == "experts":
            layers[i].experts_forward(*prep[i][2:], path=args.path)
        else:
            layers[i].forward(prep[i][0], prep[i][1], cfg.top_k, True, torch.bfloat16, path=args.path)
    torch.cuda.synchronize(dev)
    layers[0].check_status()
    print(json.dumps({"probe": args.probe, "tokens": T, "layers": L, "steps": args.steps}), flush=True)


def gpu_arm(args):
    from bitsmoe_b200 import capi, synth
    from bitsmoe_b200.layer import route_build, route_topk
    rank, world, local = dist_env(args)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    cfg = synth.QWEN3_30B
    pk = peaks()
    L = args.layers
    use_ep = world > 1 and args.parallel == "ep"
    if world > 1:
        from bitsmoe_b200 import ep

        class _EpAdapter:
            """Gives an expert-parallel layer the call signature the step functions use."""

            def __init__(self, lyr):
                self.epl = ep.ExpertParallelPackedLayer(lyr.tables, lyr.vh_gate, lyr.vh_up, lyr.u_down, cfg.intermediate, cfg.rank,
                                                        cfg.num_experts, cfg.top_k, device=dev)
                self.num_experts = cfg.num_experts // world
                self.packed = self.epl.packed

            def forward(self, x, logits, top_k, renorm, wdt, out=None, path=0):
                y = self.epl.forward(x, logits, wdt, uniform=True)
                if out is not None:
                    out.copy_(y)
                return y

    if use_ep:
        # every rank generates the same weight sets (same seeds) and keeps only its experts
        layers = [_EpAdapter(synth.make_layer(cfg, seed=42 + i, device=dev)) for i in range(L)]
    else:
        layers = [synth.to_packed_layer(synth.make_layer(cfg, seed=42 + i, device=dev), dev) for i in range(L)]
    sync = lambda: torch.cuda.synchronize(dev)

    def barrier():
        sync()
        if world > 1:
            torch.distributed.barrier()
            sync()

    def decode_case(T, steps, warmup, want_roofline):
        # every rank draws its own tokens
        xs = [synth.activations(cfg, T, seed=7 + i + 1000 * rank, device=dev) for i in range(L)]
        lg = [synth.router_logits(cfg, T, seed=9 + i + 1000 * rank, device=dev) for i in range(L)]
        ys = [torch.empty_like(xs[0]) for _ in range(L)]
        step = lambda i: layers[i % L].forward(xs[i % L], lg[i % L], cfg.top_k, True, torch.bfloat16, out=ys[i % L], path=args.path)
        for i in range(max(warmup, 3)):
            step(i)
        barrier()
        reps = (8, [])
        ms = timed(step, steps, sync, use_graph=True, repeats_out=reps if want_roofline else None)
        out = {"tokens": T, "ms_per_step": ms / steps, "tokens_per_s": T * steps / (ms * 1e-3)}
        if reps[1]:
            r = sorted(x / steps for x in reps[1])
            out["ms_per_step_replays"] = {"n": len(r), "p10": r[max(0, int(0.1 * len(r)) )], "p50": r[len(r) // 2], "p90": r[min(len(r) - 1, int(0.9 * len(r)))]}
        if want_roofline and use_ep:
            out.update(experts_kernel_ms=None, experts_bytes=None, active_experts=None)
        elif want_roofline:
            # dominant kernel alone: the packed-experts stage on prepared routing, same rotation
            prep = []
            for i in range(L):
                idx, w = route_topk(lg[i], cfg.top_k, True, torch.bfloat16)
                tok, off, rw, _, _ = route_build(idx, w, cfg.num_experts)
                hg, hu = layers[i].basis_project(xs[i])
                prep.append((hg, hu, tok, off, rw))
            est = lambda i: layers[i % L].experts_forward(*prep[i % L], path=args.path)
            for i in range(3):
                est(i)
            ems = timed(est, steps, sync) / steps
            byts = 0
            act = 0
            for i in range(L):
                b, a = active_expert_bytes(layers[i], prep[i][3].cpu().tolist())
                byts += b
                act += a
            byts = byts / L + T * cfg.rank * 2 * 2 + T * cfg.top_k * 8 + (cfg.num_experts + 1) * 4 + T * cfg.rank * 4
            out["experts_kernel_ms"] = ems
            out["experts_bytes"] = byts
            out["active_experts"] = act / L
        return out

    def e2e_case(T, steps, warmup):
        """Host buffers in, host buffer out, every step: the step's inputs are copied from pinned memory and its
        result is copied back inside the timed region.  The copies run on their own streams, so that uploads and
        downloads overlap other steps' kernels as a serving loop would arrange them; steps are handed from stream
        to stream in groups of GROUP (two groups of device buffer sets), because every cross-stream edge of the
        CUDA graph costs a few microseconds.  The whole pipeline is one CUDA graph."""
        GROUP = int(os.environ.get("BM_E2E_GROUP", "4"))
        NB = 2 * GROUP
        hx = [synth.activations(cfg, T, seed=70 + i + 1000 * rank).pin_memory() for i in range(4)]
        hl = [synth.router_logits(cfg, T, seed=90 + i + 1000 * rank).pin_memory() for i in range(4)]
        hy = [torch.empty((T, cfg.hidden), dtype=torch.bfloat16).pin_memory() for _ in range(NB)]
        dx = [torch.empty((T, cfg.hidden), dtype=torch.bfloat16, device=dev) for _ in range(NB)]
        dl = [torch.empty((T, cfg.num_experts), dtype=torch.float32, device=dev) for _ in range(NB)]
        dy = [torch.empty_like(dx[0]) for _ in range(NB)]
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def pipeline(n):
            comp = torch.cuda.current_stream(dev)
            ngroups = (n + GROUP - 1) // GROUP
            ev_c, ev_out = [None] * ngroups, [None] * ngroups
            s_in.wait_stream(comp)
            s_out.wait_stream(comp)
            for gidx in range(ngroups):
                lo, hi = gidx * GROUP, min(n, (gidx + 1) * GROUP)
                with torch.cuda.stream(s_in):
                    if gidx >= 2:
                        s_in.wait_event(ev_c[gidx - 2])       # the kernels that read these buffer sets are done
                    for i in range(lo, hi):
                        dx[i % NB].copy_(hx[i % 4], non_blocking=True)
                        dl[i % NB].copy_(hl[i % 4], non_blocking=True)
                    ev_in = torch.cuda.Event()
                    ev_in.record(s_in)
                comp.wait_event(ev_in)
                if gidx >= 2:
                    comp.wait_event(ev_out[gidx - 2])         # the previous results in these buffer sets have left
                for i in range(lo, hi):
                    layers[i % L].forward(dx[i % NB], dl[i % NB], cfg.top_k, True, torch.bfloat16, out=dy[i % NB], path=args.path)
                ev_c[gidx] = torch.cuda.Event()
                ev_c[gidx].record(comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_c[gidx])
                    for i in range(lo, hi):
                        hy[i % NB].copy_(dy[i % NB], non_blocking=True)
                    ev_out[gidx] = torch.cuda.Event()
                    ev_out[gidx].record(s_out)
            comp.wait_stream(s_in)
            comp.wait_stream(s_out)

        pipeline(max(warmup, 3))
        barrier()
        ms = timed(lambda _i: pipeline(steps), 1, sync, use_graph=True)
        return {"value": T * steps / (ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": dx[0].numel() * 2 + dl[0].numel() * 4,
                "d2h_bytes_per_step": dy[0].numel() * 2,
                "overlap": f"uploads and downloads on their own streams, handed over in groups of {GROUP} steps, {NB} device "
                           "buffer sets, one CUDA graph"}

    with ClockSampler(local) as clk:
        head = decode_case(args.tokens, args.steps, args.warmup, True)
        e2e = e2e_case(args.tokens, args.steps, args.warmup)
    clocks = clk.summary()

    extra = {}
    if not args.no_extras and world == 1:
        for T in (1, 8, 32):
            extra[f"decode_{T}"] = decode_case(T, args.steps, args.warmup, True)
        try:
            Tp = args.prefill_tokens
            xs = synth.activations(cfg, Tp, seed=3, device=dev)
            lg = synth.router_logits(cfg, Tp, seed=4, zipf_s=1.1, device=dev)
            yo = torch.empty_like(xs)
            pstep = lambda i: layers[i % L].forward(xs, lg, cfg.top_k, True, torch.bfloat16, out=yo, path=args.path)
            for i in range(2):
                pstep(i)
            n = max(2, min(args.steps, 5))
            pms = timed(pstep, n, sync) / n
            flops = Tp * cfg.top_k * 3 * 2 * cfg.rank * cfg.intermediate + Tp * 3 * 2 * cfg.hidden * cfg.rank
            extra[f"prefill_{Tp}"] = {"tokens": Tp, "ms_per_step": pms, "tokens_per_s": Tp / (pms * 1e-3),
                                      "tflops": flops / (pms * 1e-3) / 1e12,
                                      "frac_of_bf16_peak": flops / (pms * 1e-3) / 1e12 / pk["bf16_tflops"], "router": "zipf 1.1"}
        except Exception as ex:  # keep the headline if the large case fails
            extra["prefill_error"] = repr(ex)

    if world > 1 and not use_ep and not args.no_extras:
        # the same layer expert-parallel (experts sharded over the ranks, rank-space exchange over NCCL): both steps
        # in CUDA graphs (fixed-size all_gather / reduce_scatter exchange); max over ranks
        import torch.distributed as dist
        try:
            ep_layers = [_EpAdapter(synth.make_layer(cfg, seed=42 + i, device=dev)) for i in range(min(L, 4))]
            Le = len(ep_layers)
            T = args.tokens
            xs = [synth.activations(cfg, T, seed=7 + i + 1000 * rank, device=dev) for i in range(Le)]
            lg = [synth.router_logits(cfg, T, seed=9 + i + 1000 * rank, device=dev) for i in range(Le)]
            estep = lambda i: ep_layers[i % Le].forward(xs[i % Le], lg[i % Le], cfg.top_k, True, torch.bfloat16)
            for i in range(3):
                estep(i)
            barrier()
            n = min(args.steps, 50)
            ems = timed(estep, n, sync, use_graph=True) / n
            Tp = args.prefill_tokens
            xp = synth.activations(cfg, Tp, seed=3 + 1000 * rank, device=dev)
            lp = synth.router_logits(cfg, Tp, seed=4 + 1000 * rank, device=dev)     # N(0,1): near-uniform expert load
            pstep = lambda i: ep_layers[i % Le].forward(xp, lp, cfg.top_k, True, torch.bfloat16)
            for i in range(2):
                pstep(i)
            barrier()
            pms = timed(pstep, 3, sync, use_graph=True) / 3
            t = torch.tensor([ems, pms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            extra["ep_decode"] = {"tokens_per_gpu": T, "ms_per_step": float(t[0]), "tokens_per_s": world * T / (float(t[0]) * 1e-3)}
            extra["ep_prefill"] = {"tokens_per_gpu": Tp, "ms_per_step": float(t[1]), "tokens_per_s": world * Tp / (float(t[1]) * 1e-3),
                                   "router": "N(0,1) logits"}
            del ep_layers
        except Exception as ex:
            extra["ep_error"] = repr(ex)

    value = head["tokens_per_s"]
    ms_step = head["ms_per_step"]
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms_step, e2e["value"]], device=dev, dtype=torch.float64)
        mx = t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        mn = t.clone()
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        ms_step = float(mx[0])
        value = world * args.tokens / (ms_step * 1e-3)
        e2e["value"] = float(mn[1]) * world
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    if rank != 0:
        return
    achieved = head["experts_bytes"] / (head["experts_kernel_ms"] * 1e-3) / 1e9 if not use_ep else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": workload_name(args.tokens),
                   "tokens_per_gpu": args.tokens, "layers_rotated": L,
                   "l2": f"inputs larger than L2: {L} distinct weight sets of ~23 MB rotate through the timed loop",
                   "launch": "all timed steps captured in one CUDA graph, replayed once inside the CUDA-event bracket",
                   "parallelism": "1 GPU" if world == 1 else
                   (f"ep{world}: experts sharded over {world} GPUs, rank-space all_gather dispatch / reduce_scatter combine (NCCL), captured in the same CUDA graph"
                    if use_ep else
                    f"dp{world}: every GPU runs the whole layer on its own {args.tokens} tokens, weights replicated, no data-path collective")},
        "e2e": e2e, "gpu_launches": 5 * args.steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": (achieved / pk["hbm_gbs"]) if achieved else None,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch at this workload, from the ncu capture
                     # summarised in profiles/experts_decode_kernel_qwen3-30b_64tok.md
                     "traffic": 25056512 if (args.tokens == 64 and args.path == 0 and achieved) else None,
                     "peak_source": pk["source"],
                     "kernel": "packed experts stage", "kernel_ms": head["experts_kernel_ms"],
                     "algorithmic_bytes": head["experts_bytes"], "active_experts": head["active_experts"]},
        "extra": extra,
    }
    if "ms_per_step_replays" in head:
        line["ms_per_step_replays"] = head["ms_per_step_replays"]
    if not args.no_extras and world == 1:
        cpu_layer = synth.make_layer(cfg, seed=42, device=dev)
        cpu_layer.tables = {t: {f: [x.cpu() for x in v] for f, v in fl.items()} for t, fl in cpu_layer.tables.items()}
        tps, dt, cores = time_cpu(cpu_layer, args.tokens, 3, 1)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"3 forwards of one layer, {args.tokens} tokens, dequantise-then-matmul fp32 "
                                          f"({dt * 1e3:.0f} ms each)"}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        reference_arm(a)
    elif a.probe:
        probe(a)
    else:
        gpu_arm(a)
