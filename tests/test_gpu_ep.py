"""GPU: expert-parallel layers against the single-GPU layer (needs >= 2 GPUs; skipped otherwise): the peer-memory
exchange (rows pushed once per (token, destination rank), partial rows pulled by the home rank) and the two
exchanges over NCCL collectives.  Every comparison is relative to the size of the signal."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from bitsmoe_b200 import ep, synth
        cfg = synth.LayerConfig("ep-test", 1024, 16, 256, 4, rank=64)
        layer = synth.make_layer(cfg, seed=31, device=dev)          # identical weights on all ranks (same seed)
        full = synth.to_packed_layer(layer, dev)
        epl = ep.ExpertParallelPackedLayer(layer.tables, layer.vh_gate, layer.vh_up, layer.u_down, cfg.intermediate,
                                           cfg.rank, cfg.num_experts, cfg.top_k, device=dev)
        import sys
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        from tests import helpers
        # 48 tokens everywhere: gathered fixed-size exchange; 300 + 8*rank tokens: ragged all-to-all exchange
        for T in (48, 300 + 8 * rank):
            x = synth.activations(cfg, T, seed=300 + rank, device=dev)
            logits = synth.router_logits(cfg, T, seed=400 + rank, device=dev)
            y_ep = epl.forward(x, logits, torch.bfloat16)
            y_one = full.forward(x, logits, cfg.top_k, True, torch.bfloat16)
            torch.cuda.synchronize()
            helpers.assert_close(y_ep, y_one, what=f"rank {rank}: NCCL exchange, {T} tokens")
            helpers.assert_detects_damage(y_ep, y_one)
        # peer-memory exchange: two waves of 256 tokens per rank (tensor path over the gathered rows), then decode-sized waves
        for wave, n_waves in ((256, 2), (32, 3)):
            sym = ep.SymmetricExpertParallel(epl.packed, cfg.num_experts, cfg.top_k, wave, group=None)
            T = wave * n_waves
            x = synth.activations(cfg, T, seed=500 + rank, device=dev)
            logits = synth.router_logits(cfg, T, seed=600 + rank, zipf_s=1.1 if wave == 256 else 0.0, device=dev)
            res = (torch.randn(T, cfg.hidden, device=dev) * 0.01).to(torch.bfloat16)
            y_one = full.forward(x, logits, cfg.top_k, True, torch.bfloat16, residual=res)
            for overlap in (False, True):
                y_ep = sym.forward(x, logits, torch.bfloat16, residual=res, overlap=overlap)
                torch.cuda.synchronize()
                epl.packed.check_status()
                helpers.assert_close(y_ep, y_one, what=f"rank {rank}: peer-memory exchange, waves of {wave}, overlap={overlap}")
                helpers.assert_detects_damage(y_ep - res.float(), y_one.float() - res.float())
            # a dense part handed in as residual_fn runs on the side stream beside the exchange and joins before the
            # down basis: same result as the same function computed up front (several GEMMs, so that a missing join shows)
            gw = torch.Generator(device="cpu").manual_seed(77)
            wa = (torch.randn(cfg.hidden, cfg.hidden, generator=gw) * 0.02).to(dev, torch.bfloat16)
            dense = lambda xw: (((xw @ wa) @ wa) @ wa) * 0.05
            y_one_fn = full.forward(x, logits, cfg.top_k, True, torch.bfloat16, residual=dense(x))
            for overlap in (False, True):
                y_ep = sym.forward(x, logits, torch.bfloat16, overlap=overlap, residual_fn=dense)
                torch.cuda.synchronize()
                epl.packed.check_status()
                helpers.assert_close(y_ep, y_one_fn, what=f"rank {rank}: residual_fn on the side stream, waves of {wave}, overlap={overlap}")
            # the combine at rank_accum level: pulled sum == single-GPU rank_accum of the same tokens (last wave)
            idx, w = full.route_topk(logits[-wave:], cfg.top_k, True, torch.bfloat16)
            from bitsmoe_b200.layer import route_build
            tok, off, rw, _, cnt = route_build(idx, w, cfg.num_experts)
            n = int(cnt.cpu()[0])
            hg, hu = full.basis_project(x[-wave:])
            want = full.experts_forward(hg, hu, tok[:n].contiguous(), off, rw[:n].contiguous())
            helpers.assert_close(sym._scratch[(n_waves - 1) % 2]["acc"], want, rtol=1e-2, atol=3e-4,
                                 what=f"rank {rank}: pulled rank_accum, waves of {wave}")
            push, pull = sym.nvlink_bytes_per_wave(idx)
            assert 0 < push <= (world - 1) * wave * (2 * cfg.rank * 2 + cfg.top_k * 8)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_expert_parallel_layer_matches_single_gpu():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for rank in range(world):
        assert ret.get(rank) == "ok", rank
