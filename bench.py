"""MoE-layer tokens/s on synthetic layers of the benchmark shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload auto|decode|ep]

Two workloads, both "one step = one forward of one packed MoE layer over one batch of tokens":

  decode  Qwen3-30B-A3B layer shape (128 experts of 768, top-8, rank-256 shared basis, mixed 2/3/4 bits), 64 tokens:
          route -> basis projections -> packed experts -> down basis.  The timed loop rotates over --layers distinct
          weight sets (more than two L2s of packed bytes), so every step streams its experts from HBM.  1 / 8 / 32
          tokens and the 8192-token Zipf prefill of the same layer are reported beside it.
  ep      Qwen3-Next-80B-A3B layer shape (512 experts of 512, top-10, gated shared expert), 16384 tokens in total,
          expert-parallel over the N GPUs (strong scaling: the batch is split over the ranks, experts are sharded,
          rank-space rows are exchanged through peer memory).  N = 1 is the same layer and batch on one GPU.

  stack   (explicit only) 48 Qwen3-30B-A3B-shaped decoder layers: bf16 torch attention (32 query / 4 KV heads of 128, 2048
          tokens in the KV cache) and RMSNorm around this library's MoE block (router Linear included), one decode step of
          64 sequences, expert-parallel over the N GPUs; end-to-end tokens/s.

--workload auto (the default) picks `ep` when the process is one of several ranks or when several GPUs are visible
(the run is then one point of a 1/2/4/8-GPU series, which has to be one workload), else `decode`.
Rank 0 prints one JSON line.  `--impl reference` times the CPU dequantise-then-matmul path of the same workload on
the host cores instead (the reference ships no CPU forward; oracle/cpu_path.py restates it).
"""
from __future__ import annotations

import argparse
import glob
import importlib.util
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

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
# DRAM bytes (read + write) of one launch of the packed-experts kernel at the decode headline (64 tokens, Qwen3-30B-A3B
# shape), from a profiler capture; valid only for the arena layout version it was captured with.
DECODE_KERNEL_DRAM_BYTES = {3: 25089792}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "decode", "ep", "stack"])
    ap.add_argument("--stack-layers", type=int, default=48, help="stack workload: decoder layers")
    ap.add_argument("--stack-batch", type=int, default=64, help="stack workload: sequences decoded per step, over all GPUs")
    ap.add_argument("--stack-context", type=int, default=2048, help="stack workload: tokens already in the KV cache")
    ap.add_argument("--tokens", type=int, default=64, help="decode batch of the headline number")
    ap.add_argument("--layers", type=int, default=12, help="distinct weight sets rotated through (decode workload)")
    ap.add_argument("--prefill-tokens", type=int, default=8192)
    ap.add_argument("--ep-tokens", type=int, default=16384, help="tokens of one step of the ep workload, over all GPUs")
    ap.add_argument("--ep-layers", type=int, default=4, help="distinct weight sets rotated through (ep workload)")
    ap.add_argument("--waves", type=int, default=1,
                    help="ep workload: waves per step and rank (2: the exchange of one runs beside the compute of the other; "
                         "measured no faster than 1 at the default sizes)")
    ap.add_argument("--no-extras", action="store_true", help="headline only (skip other batch sizes / prefill / cpu / reference kernels)")
    ap.add_argument("--path", type=int, default=0, help="experts path: 0 auto, 1 generic, 2 decode, 3 tensor")
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


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def pick_workload(args, world):
    if args.workload != "auto":
        return args.workload
    visible = torch.cuda.device_count() if torch.cuda.is_available() else 1
    return "ep" if (world > 1 or args.gpus > 1 or visible > 1) else "decode"


def decode_workload_name(tokens):
    return (f"qwen3-30b-a3b moe layer decode, {tokens} tokens per GPU, mixed 2/3/4-bit (0.8/0.15/0.05), "
            "rank-256 shared basis, top-8 of 128 experts")


def ep_workload_name(tokens):
    return (f"qwen3-next-80b-a3b moe layer prefill, {tokens} tokens in total, mixed 2/3/4-bit (0.75/0.2/0.05), rank-256 shared "
            "basis, top-10 of 512 experts + gated shared expert, expert-parallel")


def config_for(workload, args, world):
    """The `config` object of the JSON line: identical for the GPU arm and the reference arm of one workload."""
    if workload == "decode":
        return {"workload": decode_workload_name(args.tokens), "tokens_per_gpu": args.tokens, "layers_rotated": args.layers,
                "l2": f"inputs larger than L2: {args.layers} distinct weight sets of ~23 MB rotate through the timed loop",
                "launch": "all timed steps captured in one CUDA graph, replayed once inside the CUDA-event bracket",
                "parallelism": "1 GPU" if world == 1 else
                f"dp{world}: every GPU runs the whole layer on its own {args.tokens} tokens, weights replicated, no data-path collective"}
    per = 512 // world
    return {"workload": ep_workload_name(args.ep_tokens), "tokens_total": args.ep_tokens, "tokens_per_gpu": args.ep_tokens // world,
            "waves": args.waves, "layers_rotated": args.ep_layers,
            "l2": f"inputs larger than L2: every step reads {args.ep_tokens // world} fresh token rows per GPU and rotates over "
                  f"{args.ep_layers} weight sets",
            "launch": "all timed steps captured in one CUDA graph per rank, replayed once inside the CUDA-event bracket, max over ranks",
            "parallelism": "1 GPU (all 512 experts local)" if world == 1 else
            f"ep{world}: {per} experts per GPU, tokens split over the GPUs, rank-space rows pushed to the owners of each token's "
            "experts and partial rows pulled back through peer memory (NVLink), bounded barriers between the stages"}


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


def cpu_shared_expert(x, shared):
    """Dense shared expert(s) on the host cores, fp32 (gated by sigmoid(x . w) where the layer has a gate)."""
    xf = x.float()
    y = (torch.nn.functional.silu(xf @ shared["gate"].float().T) * (xf @ shared["up"].float().T)) @ shared["down"].float().T
    if "gate_logit_w" in shared:
        y = torch.sigmoid(xf @ shared["gate_logit_w"].float().T) * y
    return y


def time_cpu(layer, tokens, steps, warmup):
    """tokens/s of the dequantise-then-matmul forward of `layer` on all host cores (dense shared expert included)."""
    from bitsmoe_b200 import synth
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = layer.cfg
    cl = cpu_layer_from(layer, cfg.top_k, torch.bfloat16 if cfg.round_route_weights else None)
    shared = None if layer.shared is None else {k: v.cpu() for k, v in layer.shared.items()}
    x = synth.activations(cfg, tokens, seed=1)
    logits = synth.router_logits(cfg, tokens, seed=2)

    def step():
        y = cl.forward(x, logits)
        if shared is not None:
            y = y.float() + cpu_shared_expert(x, shared)
        return y

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return tokens / dt, dt, cores


def reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from bitsmoe_b200 import synth
    workload = pick_workload(args, world)
    if workload == "decode":
        cfg, tokens, name = synth.QWEN3_30B, args.tokens, decode_workload_name(args.tokens)
        sample = f"forwards of one layer, {tokens} tokens, dequantise-then-matmul fp32"
        scaling = "weak"
    else:
        # a bounded sample of the 16384-token step: 64 of its tokens through the same layer
        cfg, tokens, name = synth.QWEN3_NEXT_80B, 64, ep_workload_name(args.ep_tokens)
        sample = (f"forwards of one layer on a 64-token sample of the {args.ep_tokens}-token step, dequantise-then-matmul "
                  "fp32, dense shared expert included")
        scaling = "strong"
    layer = synth.make_layer(cfg, seed=42, device="cpu")
    # honour --steps / --warmup; one CPU step takes 0.3 .. 1 s, so the defaults stay within minutes
    steps, warm = max(1, args.steps), max(0, args.warmup)
    t_probe = time.perf_counter()
    tps, dt, cores = time_cpu(layer, tokens, 1, 1)
    budget = 240.0 - (time.perf_counter() - t_probe)
    if (steps + warm) * dt > budget:          # never more than ~4 minutes of CPU work, whatever was asked for
        scale = budget / ((steps + warm) * dt)
        steps, warm = max(1, int(steps * scale)), max(0, int(warm * scale))
    tps, dt, cores = time_cpu(layer, tokens, steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "steps_asked": args.steps, "warmup_asked": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_for(workload, args, max(world, args.gpus)),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": f"{steps} {sample}"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- GPU helpers
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


def load_reference_kernels():
    """The reference's own extension recompiled for sm_100a (oracle/_ref, built by oracle/build_ref.py), or None."""
    hits = glob.glob(os.path.join(ROOT, "oracle", "_ref", "_mlp_forward_cuda*.so"))
    if not hits:
        return None
    spec = importlib.util.spec_from_file_location("_mlp_forward_cuda", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


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


def init_dist(dev, world):
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")     # plain peer traffic: no multicast objects on this pool
        dist.init_process_group("nccl", device_id=dev)


# ------------------------------------------------------------------------------------------- decode workload
def decode_arm(args):
    from bitsmoe_b200 import capi, synth
    from bitsmoe_b200.layer import route_build, route_topk
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    init_dist(dev, world)
    cfg = synth.QWEN3_30B
    pk = peaks()
    lib = capi.lib()
    L = args.layers
    layers = [synth.to_packed_layer(synth.make_layer(cfg, seed=42 + i, device=dev), dev) for i in range(L)]
    sync = lambda: torch.cuda.synchronize(dev)

    def barrier():
        sync()
        if world > 1:
            torch.distributed.barrier()
            sync()

    def experts_stage(T, steps, zipf=0.0, n_layers=L):
        """The packed-experts stage alone on prepared routing, same rotation: its time, algorithmic bytes and flops."""
        prep = []
        for i in range(n_layers):
            x = synth.activations(cfg, T, seed=7 + i + 1000 * rank, device=dev)
            lg = synth.router_logits(cfg, T, seed=9 + i + 1000 * rank, zipf_s=zipf, device=dev)
            idx, w = route_topk(lg, cfg.top_k, True, torch.bfloat16)
            tok, off, rw, _, _ = route_build(idx, w, cfg.num_experts)
            hg, hu = layers[i].basis_project(x)
            prep.append((hg, hu, tok, off, rw))
        est = lambda i: layers[i % n_layers].experts_forward(*prep[i % n_layers], path=args.path)
        for i in range(3):
            est(i)
        ems = timed(est, steps, sync) / steps
        byts, act = 0, 0
        for i in range(n_layers):
            b, a = active_expert_bytes(layers[i], prep[i][3].cpu().tolist())
            byts += b
            act += a
        byts = byts / n_layers + T * cfg.rank * 2 * 2 + T * cfg.top_k * 8 + (cfg.num_experts + 1) * 4 + T * cfg.rank * 4
        return ems, byts, act / n_layers, prep

    def hbm_roofline(ems, byts, act, traffic=None):
        achieved = byts / (ems * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                "traffic": traffic, "peak_source": pk["source"], "kernel": "packed experts stage (rank_accum clear + experts_decode_kernel)",
                "kernel_ms": ems, "algorithmic_bytes": byts, "active_experts": act}

    def decode_case(T, steps, warmup, spread):
        # every rank draws its own tokens
        xs = [synth.activations(cfg, T, seed=7 + i + 1000 * rank, device=dev) for i in range(L)]
        lg = [synth.router_logits(cfg, T, seed=9 + i + 1000 * rank, device=dev) for i in range(L)]
        ys = [torch.empty_like(xs[0]) for _ in range(L)]
        step = lambda i: layers[i % L].forward(xs[i % L], lg[i % L], cfg.top_k, True, torch.bfloat16, out=ys[i % L], path=args.path)
        for i in range(max(warmup, 3)):
            step(i)
        barrier()
        reps = (8, [])
        n0 = int(lib.bm_launch_count())
        ms = timed(step, steps, sync, use_graph=True, repeats_out=reps if spread else None)
        launches = int(lib.bm_launch_count()) - n0       # launches recorded into the graph = launches of one replay
        out = {"tokens": T, "ms_per_step": ms / steps, "tokens_per_s": T * steps / (ms * 1e-3), "gpu_launches": launches}
        if reps[1]:
            r = sorted(x / steps for x in reps[1])
            out["ms_per_step_replays"] = {"n": len(r), "p10": r[max(0, int(0.1 * len(r)))], "p50": r[len(r) // 2],
                                          "p90": r[min(len(r) - 1, int(0.9 * len(r)))]}
        ems, byts, act, _ = experts_stage(T, steps)
        traffic = DECODE_KERNEL_DRAM_BYTES.get(int(lib.bm_arena_layout_version())) if (T == 64 and args.path == 0) else None
        out["roofline"] = hbm_roofline(ems, byts, act, traffic)
        return out

    def e2e_case(T, steps, warmup):
        """Host buffers in, host buffer out, every step: the step's inputs are copied from pinned memory and its
        result is copied back inside the timed region.  The copies run on their own streams, so that uploads and
        downloads overlap other steps' kernels as a serving loop would arrange them; steps are handed from stream
        to stream in groups of GROUP (two groups of device buffer sets), because every cross-stream edge of the
        CUDA graph costs a few microseconds.  The whole pipeline is one CUDA graph."""
        GROUP = 4
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
            extra[f"decode_{T}"] = decode_case(T, args.steps, args.warmup, False)
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
            flops_experts = Tp * cfg.top_k * 3 * 2 * cfg.rank * cfg.intermediate
            flops = flops_experts + Tp * 3 * 2 * cfg.hidden * cfg.rank
            kms, _, _, _ = experts_stage(Tp, n, zipf=1.1, n_layers=min(L, 4))
            extra[f"prefill_{Tp}"] = {
                "tokens": Tp, "ms_per_step": pms, "tokens_per_s": Tp / (pms * 1e-3), "tflops": flops / (pms * 1e-3) / 1e12,
                "frac_of_bf16_peak": flops / (pms * 1e-3) / 1e12 / pk["bf16_tflops"], "router": "zipf 1.1",
                "roofline": {"bound": "tensor", "achieved": flops_experts / (kms * 1e-3) / 1e12, "peak": pk["bf16_tflops"],
                             "unit": "TFLOP/s", "frac": flops_experts / (kms * 1e-3) / 1e12 / pk["bf16_tflops"], "traffic": None,
                             "peak_source": pk["source"], "kernel": "packed experts stage (rank_accum clear + experts_tc_kernel)",
                             "kernel_ms": kms, "algorithmic_flops": flops_experts}}
        except Exception as ex:  # keep the headline if the large case fails
            extra["prefill_error"] = repr(ex)
        # the same step with the router Linear inside it (x @ W_gate^T by the library instead of ready-made logits)
        try:
            from bitsmoe_b200.layer import gate_logits
            T = args.tokens
            gw = [(torch.randn(cfg.num_experts, cfg.hidden, device=dev) * 0.02).half() for _ in range(L)]
            xs = [synth.activations(cfg, T, seed=7 + i, device=dev) for i in range(L)]
            ys = [torch.empty_like(xs[0]) for _ in range(L)]
            gstep = lambda i: layers[i % L].forward(xs[i % L], gate_logits(xs[i % L], gw[i % L]), cfg.top_k, True, torch.bfloat16,
                                                    out=ys[i % L], path=args.path)
            for i in range(3):
                gstep(i)
            gms = timed(gstep, args.steps, sync) / args.steps
            extra[f"decode_{T}_with_router_linear"] = {"tokens": T, "ms_per_step": gms, "tokens_per_s": T / (gms * 1e-3),
                                                       "note": "router logits computed inside the step (bm_gate_logits), then the same five launches"}
        except Exception as ex:
            extra["router_linear_error"] = repr(ex)
        # the kernels to beat: the reference's own CUDA op, recompiled for sm_100a, at the op boundary on the same inputs
        try:
            ref = load_reference_kernels()
            if ref is None:
                extra["reference_cuda"] = {"unavailable": "oracle/_ref holds no recompiled reference extension"}
            else:
                lyr = synth.make_layer(cfg, seed=42, device=dev)
                lists = []
                for tag in ("gate", "up", "down"):
                    for f in ("payload", "rank_idx", "tile_meta", "slab_meta", "scale", "s"):
                        lists.append([t.to(dev) for t in lyr.tables[tag][f]])
                rows = {}
                for T in (1, 8, 32, 64, 2048):
                    _, _, _, prep = experts_stage(T, 2, zipf=1.1 if T > 256 else 0.0, n_layers=1)
                    hg, hu, tok, off, rw = prep[0]
                    call = lambda _i: ref.moe_packed_forward(hg, hu, tok, off, rw, *lists, cfg.rank, cfg.intermediate, 0)
                    for i in range(3):
                        call(i)
                    n = 20 if T <= 64 else 5
                    rms = timed(call, n, sync, use_graph=False) / n      # the reference op synchronises: no graph
                    oms = timed(lambda i: layers[0].experts_forward(hg, hu, tok, off, rw, path=args.path), n, sync, use_graph=False) / n
                    rows[str(T)] = {"reference_op_ms": rms, "this_op_ms": oms, "timing": "eager launches, CUDA events, same inputs"}
                extra["reference_cuda"] = rows
        except Exception as ex:
            extra["reference_cuda"] = {"error": repr(ex)}

    value, ms_step = head["tokens_per_s"], head["ms_per_step"]
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms_step, e2e["value"]], device=dev, dtype=torch.float64)
        mx, mn = t.clone(), t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        ms_step = float(mx[0])
        value = world * args.tokens / (ms_step * 1e-3)
        e2e["value"] = float(mn[1]) * world
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": config_for("decode", args, world),
        "e2e": e2e, "gpu_launches": head["gpu_launches"], "clocks": clocks, "roofline": head["roofline"], "extra": extra,
    }
    if "ms_per_step_replays" in head:
        line["ms_per_step_replays"] = head["ms_per_step_replays"]
    if not args.no_extras and world == 1:
        cpu_layer = synth.make_layer(cfg, seed=42, device="cpu")
        tps, dt, cores = time_cpu(cpu_layer, args.tokens, 3, 1)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"3 forwards of one layer, {args.tokens} tokens, dequantise-then-matmul fp32 "
                                          f"({dt * 1e3:.0f} ms each)"}
        # the CPU-runnable configuration of the specification: DeepSeek-V2-Lite shape, uniform 2-bit, 64 tokens,
        # two shared experts (a dense MLP of width 2816), through the same dequantise-then-matmul path
        ds = synth.make_layer(synth.DEEPSEEK_V2_LITE, seed=42, device="cpu")
        tps, dt, cores = time_cpu(ds, 64, 3, 1)
        line["extra"]["cpu_baseline_deepseek_v2_lite"] = {
            "value": tps, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"3 forwards of one deepseek-v2-lite-shaped layer (64 experts of 1408, top-6, 2-bit, shared experts), "
                      f"64 tokens ({dt * 1e3:.0f} ms each)"}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- ep workload
def ep_arm(args):
    """Strong scaling of one Qwen3-Next-80B-A3B-shaped layer over the ranks: see the module docstring."""
    from bitsmoe_b200 import capi, ep, synth
    from bitsmoe_b200.layer import PackedLayer, dense_mlp
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    init_dist(dev, world)
    import torch.distributed as dist
    cfg = synth.QWEN3_NEXT_80B
    pk = peaks()
    lib = capi.lib()
    total = args.ep_tokens
    if total % (world * args.waves):
        raise SystemExit(f"--ep-tokens {total} must be a multiple of gpus * waves = {world * args.waves}")
    T_loc = total // world
    L = args.ep_layers
    sync = lambda: torch.cuda.synchronize(dev)

    def barrier():
        sync()
        if world > 1:
            dist.barrier()
            sync()

    # every rank generates the same weight sets (same seeds) and keeps only its experts
    synth_layers = [synth.make_layer(cfg, seed=42 + i, device=dev) for i in range(L)]
    shared = [{k: v.to(dev, torch.float16) for k, v in s.shared.items()} for s in synth_layers]

    def local_layer(s):
        t = ep.shard_tables(s.tables, rank, world)
        return PackedLayer(t["gate"], t["up"], t["down"], cfg.intermediate, cfg.rank, s.vh_gate, s.vh_up, s.u_down, device=dev)

    packed = [local_layer(s) for s in synth_layers]
    sym = [ep.SymmetricExpertParallel(p, cfg.num_experts, cfg.top_k, T_loc // args.waves, cfg.norm_topk_prob) for p in packed] \
        if world > 1 else None

    def shared_expert(x, sh):
        """sigmoid(x . w_g) * MLP(x) of the gated shared expert on this library's dense kernels (bm_dense_mlp_forward:
        fp16 weights, tcgen05 GEMMs), added as the residual."""
        return dense_mlp(x, sh["gate"], sh["up"], sh["down"], sh["gate_logit_w"])

    xs = [synth.activations(cfg, T_loc, seed=7 + i + 1000 * rank, device=dev) for i in range(L)]
    lg = [synth.router_logits(cfg, T_loc, seed=9 + i + 1000 * rank, device=dev) for i in range(L)]
    ys = [torch.empty_like(xs[0]) for _ in range(L)]

    def step(i, with_shared=True):
        j = i % L
        if world == 1:
            res = shared_expert(xs[j], shared[j]) if with_shared else None
            packed[j].forward(xs[j], lg[j], cfg.top_k, cfg.norm_topk_prob, torch.bfloat16, residual=res, out=ys[j], path=args.path)
        else:
            # the shared expert runs on a side stream beside the exchange
            fn = (lambda xw: shared_expert(xw, shared[j])) if with_shared else None
            sym[j].forward(xs[j], lg[j], torch.bfloat16, out=ys[j], overlap=args.waves > 1, residual_fn=fn)
        return ys[j]

    # on-box parity of the expert-parallel step: rank 0 runs its own tokens through the whole layer on one GPU
    parity = None
    if world > 1:
        # (routed experts only: the dense shared expert is two orders of magnitude larger and would hide them)
        y_ep = step(0, with_shared=False).float().clone()
        sync()
        if rank == 0:
            full = synth.to_packed_layer(synth_layers[0], dev)
            y_one = full.forward(xs[0], lg[0], cfg.top_k, cfg.norm_topk_prob, torch.bfloat16).float()
            sync()
            err = (y_ep - y_one)
            parity = {"max_abs_err": float(err.abs().max()), "max_abs_ref": float(y_one.abs().max()),
                      "rel_l2": float(err.norm() / y_one.norm()), "tokens_checked": T_loc,
                      "against": "the routed experts of the same layer with all 512 experts on one GPU, same tokens of rank 0"}
            parity["ok"] = bool(parity["max_abs_err"] <= 2e-2 * parity["max_abs_ref"] and parity["rel_l2"] <= 1e-2)
            del full
        barrier()

    steps, warm = max(1, args.steps), max(3, args.warmup)
    with ClockSampler(local) as clk:
        for i in range(warm):
            step(i)
        barrier()
        n0 = int(lib.bm_launch_count())
        # all timed steps in one CUDA graph per rank (the barriers between the ranks are kernels of the graph)
        ms = timed(step, steps, sync, use_graph=True) / steps
        launches = int(lib.bm_launch_count()) - n0
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # end to end: the step's inputs come from pinned host memory and its result goes back, every step
        hx = [x.cpu().pin_memory() for x in xs[:2]]
        hl = [l.cpu().pin_memory() for l in lg[:2]]
        hy = torch.empty(xs[0].shape, dtype=xs[0].dtype).pin_memory()

        def e2e_step(i):
            xs[i % L].copy_(hx[i % 2], non_blocking=True)
            lg[i % L].copy_(hl[i % 2], non_blocking=True)
            hy.copy_(step(i), non_blocking=True)

        for i in range(2):
            e2e_step(i)
        barrier()
        start.record()
        n_e2e = max(1, min(steps, 20))
        for i in range(n_e2e):
            e2e_step(i)
        stop.record()
        sync()
        ms_e2e = start.elapsed_time(stop) / n_e2e
    clocks = clk.summary()
    for p in packed:
        p.check_status()
    nv = None
    if world > 1:
        idx, _ = packed[0].route_topk(lg[0][: T_loc // args.waves], cfg.top_k, cfg.norm_topk_prob, torch.bfloat16)
        push, pull = sym[0].nvlink_bytes_per_wave(idx)
        nv = {"pushed_per_rank_per_step": push * args.waves, "pulled_per_rank_per_step": pull * args.waves,
              "estimate": "rows once per (token, destination rank): 2r fp16 out, r_out fp32 back, top-k ids and weights to every rank"}
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    flops_experts = total * cfg.top_k * 3 * 2 * cfg.rank * cfg.intermediate
    flops = flops_experts + total * 3 * 2 * cfg.hidden * cfg.rank + total * 3 * 2 * cfg.hidden * cfg.shared_intermediate
    tf_per_gpu = flops / (ms * 1e-3) / 1e12 / world
    line = {
        "metric": METRIC, "value": total / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": config_for("ep", args, world),
        "e2e": {"value": total / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": xs[0].numel() * 2 + lg[0].numel() * 4,
                "d2h_bytes_per_step": xs[0].numel() * 2, "overlap": "copies on the compute stream (per rank)"},
        "gpu_launches": launches, "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": tf_per_gpu, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": tf_per_gpu / pk["bf16_tflops_sustained"], "traffic": None, "peak_source": pk["source"] + " (sustained)",
                     "kernel": "whole step per GPU (algorithmic flops of routed experts + basis products + shared expert)",
                     "kernel_ms": ms, "algorithmic_flops": flops},
        "extra": {"ep_parity": parity, "nvlink_bytes": nv},
    }
    if world == 1 and not args.no_extras:
        cpu_layer = synth.make_layer(cfg, seed=42, device="cpu")
        tps, dt, cores = time_cpu(cpu_layer, 64, 3, 1)
        line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"3 forwards of one layer on a 64-token sample of the step, dequantise-then-matmul fp32 "
                                          f"({dt * 1e3:.0f} ms each)"}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- stack workload
def stack_arm(args):
    """One decode step of a 48-layer stack (BASELINE.json configs[4]): per layer RMSNorm -> attention over a 2048-token
    KV cache (bf16 torch: library GEMMs and scaled_dot_product_attention) -> RMSNorm -> this library's MoE block
    (router Linear, routing, packed experts, down basis), expert-parallel over the ranks.  Weights are seeded random."""
    from bitsmoe_b200 import capi, ep, synth
    from bitsmoe_b200.layer import PackedLayer, gate_logits
    import torch.nn.functional as F
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    init_dist(dev, world)
    cfg = synth.QWEN3_30B
    NL, B, CTX = args.stack_layers, args.stack_batch, args.stack_context
    if B % world:
        raise SystemExit(f"--stack-batch {B} must be a multiple of the number of GPUs")
    Bl = B // world
    H, NH, NKV, HD = cfg.hidden, 32, 4, 128
    sync = lambda: torch.cuda.synchronize(dev)
    g = torch.Generator(device=dev).manual_seed(1234)          # replicated weights: the same seed on every rank
    rnd = lambda *shape, std=0.02: (torch.randn(*shape, generator=g, device=dev) * std).to(torch.bfloat16)
    layers = []
    t_build = time.perf_counter()
    for li in range(NL):
        s = synth.make_layer(cfg, seed=42 + li, device=dev)
        if world > 1:
            t = ep.shard_tables(s.tables, rank, world)
            pk = PackedLayer(t["gate"], t["up"], t["down"], cfg.intermediate, cfg.rank, s.vh_gate, s.vh_up, s.u_down, device=dev)
            moe = ep.SymmetricExpertParallel(pk, cfg.num_experts, cfg.top_k, Bl, cfg.norm_topk_prob)
        else:
            pk = synth.to_packed_layer(s, dev)
            moe = None
        layers.append(dict(
            pk=pk, moe=moe, wq=rnd(NH * HD, H), wk=rnd(NKV * HD, H), wv=rnd(NKV * HD, H), wo=rnd(H, NH * HD),
            gate=rnd(cfg.num_experts, H).half(), n1=torch.ones(H, device=dev, dtype=torch.bfloat16),
            n2=torch.ones(H, device=dev, dtype=torch.bfloat16),
            kc=rnd(Bl, NKV, CTX + 1, HD, std=1.0), vc=rnd(Bl, NKV, CTX + 1, HD, std=1.0)))
        del s
    t_build = time.perf_counter() - t_build
    x0 = torch.randn(Bl, H, generator=g, device=dev).to(torch.bfloat16)
    out = torch.empty_like(x0)

    def step(_i=0):
        x = x0
        for ly in layers:
            h = F.rms_norm(x, (H,), ly["n1"], 1e-6)
            q = (h @ ly["wq"].T).view(Bl, NH, 1, HD)
            ly["kc"][:, :, CTX] = (h @ ly["wk"].T).view(Bl, NKV, HD)
            ly["vc"][:, :, CTX] = (h @ ly["wv"].T).view(Bl, NKV, HD)
            a = F.scaled_dot_product_attention(q, ly["kc"], ly["vc"], enable_gqa=True)
            x = x + a.reshape(Bl, NH * HD) @ ly["wo"].T
            h = F.rms_norm(x, (H,), ly["n2"], 1e-6)
            logits = gate_logits(h, ly["gate"])
            if ly["moe"] is None:
                x = ly["pk"].forward(h, logits, cfg.top_k, cfg.norm_topk_prob, torch.bfloat16, residual=x)
            else:
                x = ly["moe"].forward(h, logits, torch.bfloat16, residual=x, overlap=False)
        out.copy_(x)

    for _ in range(3):
        step()
    sync()
    if world > 1:
        torch.distributed.barrier()
    steps = max(1, min(args.steps, 50))
    with ClockSampler(local) as clk:
        n0 = int(capi.lib().bm_launch_count())
        ms = timed(step, steps, sync, use_graph=True) / steps
        launches = int(capi.lib().bm_launch_count()) - n0
    clocks = clk.summary()
    for ly in layers:
        ly["pk"].check_status()
    finite = bool(torch.isfinite(out.float()).all())
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t[0])
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    if rank != 0:
        return
    print(json.dumps({
        "metric": "stack_decode_tokens_per_s", "value": B / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": 3,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 attention, f16 experts",
        "data": "synthetic",
        "config": {"workload": f"{NL} qwen3-30b-a3b-shaped decoder layers, one decode step of {B} sequences, {CTX}-token KV cache, "
                               f"expert-parallel over {world} GPU(s)", "batch_per_gpu": Bl,
                   "launch": "the whole step captured in one CUDA graph per rank", "attention": "torch bf16 (library kernels)"},
        "gpu_launches": launches, "clocks": clocks, "extra": {"output_finite": finite, "layer_build_s": t_build}}), flush=True)


if __name__ == "__main__":
    a = parse()
    _, _world, _ = dist_env()
    if a.impl == "reference":
        reference_arm(a)
    elif a.probe:
        probe(a)
    elif pick_workload(a, _world) == "stack":
        stack_arm(a)
    elif pick_workload(a, _world) == "ep":
        ep_arm(a)
    else:
        decode_arm(a)
