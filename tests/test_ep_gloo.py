"""Expert-parallel bookkeeping on CPU: world_size 2 and 4 over gloo, compute stages served by the oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bitsmoe_b200 import ep, synth
from oracle import forward as oforward
from tests import helpers


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, T_per_rank: int, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        cfg = synth.tiny(hidden=128, num_experts=8, intermediate=128, top_k=3, rank=32)
        layer = synth.make_layer(cfg, seed=21)                      # same weights on every rank
        experts = helpers.decoded_experts(layer)
        per = cfg.num_experts // world
        local = experts[rank * per:(rank + 1) * per]

        def experts_fn(hg, hu, tok, off, rw):
            return oforward.packed_forward(hg, hu, tok, off, rw, local, cfg.rank)

        # every rank owns different tokens; rank 1's batch is smaller to exercise ragged splits
        T = T_per_rank - (3 if rank == 1 else 0)
        x = synth.activations(cfg, T, seed=100 + rank)
        logits = synth.router_logits(cfg, T, seed=200 + rank, zipf_s=0.8)
        idx, w = oforward.router(logits, cfg.top_k, True, torch.float16)
        hg, hu = oforward.basis_project(x, layer.vh_gate), oforward.basis_project(x, layer.vh_up)
        epl = ep.ExpertParallelLayer(cfg.num_experts, cfg.top_k, experts_fn)
        acc = epl.forward_rank_space(hg, hu, idx, w, cfg.rank)
        # single-rank answer for the same tokens
        tok, off, rw = oforward.build_routing(idx, w, cfg.num_experts)
        want = oforward.packed_forward(hg, hu, tok, off, rw, experts, cfg.rank)
        err = float((acc - want).abs().max())
        # each (token, destination) pair is sent once: never more rows than assignments, never more than T*world
        plan = epl.last_plan
        ok_rows = sum(plan.send_row_splits) <= min(T * cfg.top_k, T * world)
        ret[rank] = (err, ok_rows, sum(plan.send_row_splits), T * cfg.top_k)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_matches_single_rank(world):
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 11, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        err, ok_rows, rows, assigns = ret[rank]
        assert err < 1e-5, (rank, err)
        assert ok_rows, (rank, rows, assigns)


def test_dispatch_plan_dedups_token_destination_pairs():
    idx = torch.tensor([[0, 1, 5], [4, 6, 7], [2, 3, 0]])      # 8 experts over 2 ranks: ranks {0,0,1}, {1,1,1}, {0,0,0}
    w = torch.full((3, 3), 1 / 3)
    row_token, row_splits, a_exp, a_row, a_w, a_splits = ep.build_dispatch(idx, w, 2, 4)
    assert row_splits.tolist() == [2, 2]                        # tokens {0,2} -> rank 0, tokens {0,1} -> rank 1
    assert row_token.tolist() == [0, 2, 0, 1]
    assert a_splits.tolist() == [5, 4]
    assert a_exp.tolist() == [0, 1, 2, 3, 0, 1, 0, 2, 3]
    assert a_row.tolist() == [0, 0, 1, 1, 1, 0, 1, 1, 1]


def _gather_worker(rank: int, world: int, port: int, T: int, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        cfg = synth.tiny(hidden=128, num_experts=8, intermediate=128, top_k=3, rank=32)
        layer = synth.make_layer(cfg, seed=21)
        experts = helpers.decoded_experts(layer)
        per = cfg.num_experts // world
        local = experts[rank * per:(rank + 1) * per]

        def route_build_fn(idx, w, g2l):
            return oforward.build_routing(idx.long(), w, per, g2l)

        def experts_fn(hg, hu, tok, off, rw):
            n = hu.shape[0]                                   # the up view is T rows shorter
            return oforward.packed_forward(hg[:n], hu, tok, off, rw, local, cfg.rank)

        x = synth.activations(cfg, T, seed=100 + rank)
        logits = synth.router_logits(cfg, T, seed=200 + rank, zipf_s=0.8)
        idx, w = oforward.router(logits, cfg.top_k, True, torch.float16)
        hg, hu = oforward.basis_project(x, layer.vh_gate), oforward.basis_project(x, layer.vh_up)
        gep = ep.GatherExpertParallel(cfg.num_experts, cfg.top_k, route_build_fn, experts_fn)
        acc = gep.forward_rank_space(torch.stack((hg, hu)), idx.to(torch.int32), w, cfg.rank)
        tok, off, rw = oforward.build_routing(idx, w, cfg.num_experts)
        want = oforward.packed_forward(hg, hu, tok, off, rw, experts, cfg.rank)
        ret[rank] = float((acc - want).abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gather_expert_parallel_matches_single_rank(world):
    ret = mp.Manager().dict()
    mp.spawn(_gather_worker, args=(world, _free_port(), 9, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        assert ret[rank] < 1e-5, (rank, ret[rank])
