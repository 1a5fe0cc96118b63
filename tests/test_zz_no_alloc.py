"""GPU: the routing build that brings its own scratch.

bm_route_build_static is for hosts that have no way to give the library a workspace -- a serving loop that
keeps cudaMalloc off its hot path, or a plug-in that is only handed input and output pointers.  It must give
exactly what bm_route_build gives with a caller workspace, call after call, although every call reuses the
same built-in table (which still holds the previous call's counts on entry)."""
import ctypes as C

import pytest
import torch

from bitsmoe_b200 import capi
from bitsmoe_b200.layer import route_build

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _static_build(idx, w, num_local, tile_rows=128):
    lib = capi.lib()
    T, k = idx.shape
    max_tiles = int(lib.bm_route_max_tiles(T, k, num_local, tile_rows))
    tok = torch.full((T * k,), -7, dtype=torch.int32, device=DEV)
    off = torch.empty((num_local + 1,), dtype=torch.int32, device=DEV)
    rw = torch.full((T * k,), -7.0, dtype=torch.float32, device=DEV)
    tiles = torch.empty((max_tiles, 3), dtype=torch.int32, device=DEV)
    counts = torch.empty((2,), dtype=torch.int32, device=DEV)
    with torch.cuda.device(DEV):
        status = lib.bm_route_build_static(idx.data_ptr(), w.data_ptr(), None, num_local, T, k, num_local, tile_rows, tok.data_ptr(),
                                           off.data_ptr(), rw.data_ptr(), tiles.data_ptr(), counts.data_ptr(),
                                           capi.stream_ptr(torch.device(DEV)))
    return status, (tok, off, rw, tiles, counts)


def _problem(T, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g) - torch.log(torch.arange(1, E + 1, dtype=torch.float32)) * 0.7
    w, idx = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    return idx.to(torch.int32).to(DEV).contiguous(), w.to(DEV).contiguous()


def test_static_route_build_matches_workspace_version_twice_in_a_row():
    # two different multi-block problems back to back: the second starts from the first one's leftovers
    for T, E, k, seed in ((3000, 128, 8, 1), (1500, 512, 10, 2), (3000, 128, 8, 1)):
        idx, w = _problem(T, E, k, seed)
        want = route_build(idx, w, E)
        status, got = _static_build(idx, w, E)
        assert status == capi.BM_OK, capi.lib().bm_last_error()
        n, n_tiles = (int(v) for v in want[4].cpu())
        assert got[4].cpu().tolist() == [n, n_tiles]
        assert torch.equal(got[1], want[1])                     # expert_offsets
        assert torch.equal(got[0][:n], want[0][:n])             # token_indices
        assert torch.equal(got[2][:n], want[2][:n])             # route_flat
        assert torch.equal(got[3][:n_tiles], want[3][:n_tiles])  # tile table
    # a single-block problem needs no scratch at all and takes the same entry point
    idx, w = _problem(17, 64, 6, 3)
    want = route_build(idx, w, 64)
    status, got = _static_build(idx, w, 64)
    assert status == capi.BM_OK and torch.equal(got[1], want[1]) and torch.equal(got[0], want[0])


def test_static_route_build_rejects_what_does_not_fit():
    lib = capi.lib()
    cap = int(lib.bm_route_build_static_capacity())
    assert cap == 1 << 20
    T, E, k = 40000, 1024, 8            # 313 blocks * 1024 experts * 4 bytes > 1 MiB
    assert int(lib.bm_route_build_workspace_bytes(T, k, E)) > cap
    idx = torch.zeros((T, k), dtype=torch.int32, device=DEV)
    w = torch.zeros((T, k), dtype=torch.float32, device=DEV)
    status, _ = _static_build(idx, w, E)
    assert status == 4                   # BM_ERR_WORKSPACE
    assert b"built-in array holds" in lib.bm_last_error()
