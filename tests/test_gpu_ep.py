"""GPU: expert-parallel layer over NCCL against the single-GPU layer (needs >= 2 GPUs; skipped otherwise)."""
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
        worst, mag = 0.0, 0.0
        # 48 tokens everywhere: gathered fixed-size exchange; 300 + 8*rank tokens: ragged all-to-all exchange
        for T in (48, 300 + 8 * rank):
            x = synth.activations(cfg, T, seed=300 + rank, device=dev)
            logits = synth.router_logits(cfg, T, seed=400 + rank, device=dev)
            y_ep = epl.forward(x, logits, torch.bfloat16)
            y_one = full.forward(x, logits, cfg.top_k, True, torch.bfloat16)
            torch.cuda.synchronize()
            worst = max(worst, float((y_ep.float() - y_one.float()).abs().max()))
            mag = max(mag, float(y_one.float().abs().max()))
        ret[rank] = worst, mag
    finally:
        dist.destroy_process_group()


def test_expert_parallel_layer_matches_single_gpu():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for rank in range(world):
        err, mag = ret[rank]
        assert err <= 1e-2 + 2e-2 * mag, (rank, err, mag)
