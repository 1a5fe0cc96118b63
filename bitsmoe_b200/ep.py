"""Expert parallelism for one packed MoE layer: one process per GPU, experts sharded, tokens data-parallel.

The reference has no distributed code (its only multi-GPU mechanism is HF ``device_map`` placement,
bitsmoe/evaluation/ppl_eval.py:321-327); this module adds the exchange that sharding the experts of
bitsmoe/models/base_block.py needs.  Rank g owns experts ``[g*E/G, (g+1)*E/G)``; the shared basis, the
router and the dense shared expert are replicated.  Because the routed experts act in *rank space*,
what crosses NVLink is small:

  dispatch  one row ``[h_gate | h_up]`` (2r fp16 values) per (token, destination rank) pair -- not per
            assignment and not the hidden vector -- plus, per assignment, (local expert id, row, weight)
  combine   one partial ``rank_accum`` row (r_out fp32 values) per (token, destination rank) pair, summed
            at the token's home rank before the single down-basis product

Both exchanges are ``all_to_all_single`` calls (NCCL over NVLink/NVSwitch on GPUs, gloo in the CPU tests).
The compute stages are injected, so the same bookkeeping runs against the CUDA library or a CPU oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    """Bookkeeping of one dispatch, kept for the combine step."""
    send_row_token: torch.Tensor      # [rows_sent] home token of every (token, destination) row, grouped by destination
    send_row_splits: List[int]        # rows sent to each rank
    recv_row_splits: List[int]        # rows received from each rank
    recv_assign_splits: List[int]


def expert_owner(expert_ids: torch.Tensor, experts_per_rank: int) -> torch.Tensor:
    return torch.div(expert_ids, experts_per_rank, rounding_mode="floor")


def build_dispatch(topk_idx: torch.Tensor, topk_w: torch.Tensor, world: int, experts_per_rank: int):
    """From the routing of the local tokens: rows and assignments to send, grouped by destination rank.

    Returns (row_token [R], row_splits [G], assign_expert_local [A], assign_row [A], assign_w [A], assign_splits [G]);
    ``assign_row`` indexes the rows sent to the same destination (0-based inside that destination's block)."""
    T, k = topk_idx.shape
    dev = topk_idx.device
    dest = expert_owner(topk_idx.long(), experts_per_rank)                       # [T, k]
    pair = torch.zeros((T, world), dtype=torch.bool, device=dev)
    pair.scatter_(1, dest, True)                                                 # token t talks to rank d
    pair_t = pair.t().contiguous()                                               # [G, T]
    row_splits = pair_t.sum(dim=1)
    row_token = pair_t.nonzero(as_tuple=False)[:, 1]                             # ascending tokens inside every destination
    # position of token t inside destination d's row block
    pos_in_block = torch.cumsum(pair_t.to(torch.int64), dim=1) - 1               # [G, T]
    flat_dest = dest.reshape(-1)
    flat_tok = torch.arange(T, device=dev).repeat_interleave(k)
    order = torch.sort(flat_dest, stable=True).indices                           # assignments grouped by destination
    a_dest = flat_dest[order]
    a_tok = flat_tok[order]
    assign_expert_local = (topk_idx.reshape(-1).long()[order] - a_dest * experts_per_rank).to(torch.int32)
    assign_row = pos_in_block[a_dest, a_tok].to(torch.int32)
    assign_w = topk_w.reshape(-1)[order].to(torch.float32)
    assign_splits = torch.bincount(a_dest, minlength=world)
    return row_token, row_splits, assign_expert_local, assign_row, assign_w, assign_splits


def _a2a(t: torch.Tensor, out_splits: List[int], in_splits: List[int], group) -> torch.Tensor:
    out = t.new_empty((sum(out_splits),) + tuple(t.shape[1:]))
    dist.all_to_all_single(out, t.contiguous(), out_splits, in_splits, group=group)
    return out


class ExpertParallelLayer:
    """``experts_fn(h_gate [R,r], h_up [R,r], token_indices [A] int32, expert_offsets [E_local+1] int32,
    route_w [A] fp32) -> rank_accum [R, r_out] fp32`` is the op contract of ``moe_packed_forward`` applied to
    the rows this rank received; ``sort_fn(expert_local [A], num_local) -> (order, expert_offsets)`` groups
    the received assignments by local expert (stable)."""

    def __init__(self, num_experts: int, top_k: int, experts_fn: Callable, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not shard over {self.world} ranks")
        self.experts_per_rank = num_experts // self.world
        self.top_k = top_k
        self.experts_fn = experts_fn

    def local_expert_range(self) -> Tuple[int, int]:
        return self.rank * self.experts_per_rank, (self.rank + 1) * self.experts_per_rank

    def forward_rank_space(self, h_gate: torch.Tensor, h_up: torch.Tensor, topk_idx: torch.Tensor,
                           topk_w: torch.Tensor, rank_out: int) -> torch.Tensor:
        """h_gate / h_up [T, r] fp16 of the local tokens and their routing -> rank_accum [T, rank_out] fp32."""
        T, r = h_gate.shape
        G = self.world
        row_token, row_splits, a_exp, a_row, a_w, a_splits = build_dispatch(topk_idx, topk_w, G, self.experts_per_rank)
        # 1. sizes (one small exchange; the only host synchronisation of the layer)
        sizes = torch.stack((row_splits, a_splits), dim=1).to(torch.int64)           # [G, 2]
        recv_sizes = torch.empty_like(sizes)
        dist.all_to_all_single(recv_sizes, sizes, group=self.group)
        send_rows, send_assign = [int(v) for v in row_splits.tolist()], [int(v) for v in a_splits.tolist()]
        rs = recv_sizes.tolist()
        recv_rows, recv_assign = [int(v[0]) for v in rs], [int(v[1]) for v in rs]
        # 2. dispatch: rank-space rows once per (token, destination), assignment records
        rows = torch.cat((h_gate.index_select(0, row_token), h_up.index_select(0, row_token)), dim=1)   # [R_send, 2r]
        rows_in = _a2a(rows, recv_rows, send_rows, self.group)
        meta = torch.stack((a_exp, a_row), dim=1)
        meta_in = _a2a(meta, recv_assign, send_assign, self.group)
        w_in = _a2a(a_w, recv_assign, send_assign, self.group)
        # rows of source s start at base[s] in the received buffer
        base = torch.zeros(G, dtype=torch.int64, device=h_gate.device)
        if G > 1:
            base[1:] = torch.cumsum(torch.tensor(recv_rows[:-1], device=h_gate.device), 0)
        src_of_assign = torch.repeat_interleave(torch.arange(G, device=h_gate.device),
                                                torch.tensor(recv_assign, device=h_gate.device))
        row_global = meta_in[:, 1].long() + base[src_of_assign]
        # 3. group the received assignments by local expert (stable) and run the packed experts on them
        order = torch.sort(meta_in[:, 0].long(), stable=True).indices
        counts = torch.bincount(meta_in[:, 0].long(), minlength=self.experts_per_rank)
        offsets = torch.zeros(self.experts_per_rank + 1, dtype=torch.int32, device=h_gate.device)
        offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
        hg_in, hu_in = rows_in[:, :r].contiguous(), rows_in[:, r:].contiguous()
        if rows_in.shape[0] > 0:
            partial = self.experts_fn(hg_in, hu_in, row_global[order].to(torch.int32).contiguous(), offsets,
                                      w_in[order].contiguous())
        else:
            partial = torch.zeros((0, rank_out), dtype=torch.float32, device=h_gate.device)
        # 4. combine: partial rows travel back and are summed at the home rank
        back = _a2a(partial, send_rows, recv_rows, self.group)                     # same order as `rows`
        acc = torch.zeros((T, rank_out), dtype=torch.float32, device=h_gate.device)
        acc.index_add_(0, row_token, back)
        self.last_plan = DispatchPlan(row_token, send_rows, recv_rows, recv_assign)
        return acc


def shard_tables(tables, rank: int, world: int):
    """Per-expert buffer lists of a whole layer -> the slice this rank owns."""
    out = {}
    for tag, fields in tables.items():
        n = len(next(iter(fields.values())))
        per = n // world
        out[tag] = {f: v[rank * per:(rank + 1) * per] for f, v in fields.items()}
    return out


class ExpertParallelPackedLayer:
    """GPU layer: this rank's slice of the experts as a ``PackedLayer`` plus the replicated basis; the
    exchanges run over ``group`` (NCCL)."""

    def __init__(self, tables, vh_gate, vh_up, u_down, intermediate_size: int, rank_out: int, num_experts: int,
                 top_k: int, norm_topk_prob: bool = True, device=None, group=None):
        from .layer import PackedLayer
        self.group = group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        local = shard_tables(tables, rank, world)
        self.packed = PackedLayer(local["gate"], local["up"], local["down"], intermediate_size, rank_out, vh_gate, vh_up,
                                  u_down, device=device)
        self.rank_out = rank_out
        self.top_k, self.norm_topk_prob = top_k, norm_topk_prob
        self.ep = ExpertParallelLayer(num_experts, top_k, self.packed.experts_forward, group)
        from .layer import route_build

        def build(idx, w, g2l):
            tok, off, rw, _, _ = route_build(idx, w, num_experts // world, g2l)
            return tok, off, rw

        self.gather_ep = GatherExpertParallel(num_experts, top_k, build, self.packed.experts_forward, group,
                                              device=self.packed.device)
        self.gather_max_tokens = 256
        # with `uniform=True` (the caller guarantees one token count on all ranks) the gather exchange is used up to
        # this many tokens per rank; it moves G*T rows per rank but needs no host read and no sorting
        self.gather_max_tokens_uniform = 131072 // world

    def forward(self, x: torch.Tensor, logits: torch.Tensor, weight_dtype=torch.float16,
                residual: Optional[torch.Tensor] = None, uniform: bool = False) -> torch.Tensor:
        from .layer import route_topk
        idx, w = route_topk(logits, self.top_k, self.norm_topk_prob, weight_dtype)
        if x.shape[0] <= (self.gather_max_tokens_uniform if uniform else self.gather_max_tokens):
            # decode-sized batch: fixed-size exchanges, nothing read back to the host (CUDA-graph capturable);
            # every rank must take this branch together, i.e. use the same token count per rank
            pair = torch.empty((2, x.shape[0], self.packed.rank_in), dtype=torch.float16, device=x.device)
            self.packed.basis_project(x, out=pair)
            acc = self.gather_ep.forward_rank_space(pair, idx, w, self.rank_out)
            return self.packed.combine_down_basis(acc, x.dtype, residual=residual)
        hg, hu = self.packed.basis_project(x)
        acc = self.ep.forward_rank_space(hg, hu, idx, w, self.rank_out)
        return self.packed.combine_down_basis(acc, x.dtype, residual=residual)


# ---------------------------------------------------------------------------------------------------------
# Small batches (decode): fixed-size exchanges, no host synchronisation, CUDA-graph capturable.
#
# With T tokens per rank and T small, sending every rank-space row to every rank costs G*T*2r*2 bytes per
# rank (512 KB at G=8, T=64, r=256) -- less than a microsecond of NVLink time -- and removes all
# data-dependent sizes: one all_gather of [h_gate | h_up], one all_gather of the top-k (ids, weights), the
# routing build over all G*T tokens with a map that keeps only this rank's experts, the packed experts on
# the gathered rows, and one reduce_scatter of the partial rank_accum rows back to the tokens' home ranks.
# ---------------------------------------------------------------------------------------------------------
def _gather(x: torch.Tensor, group) -> torch.Tensor:
    """[...] on every rank -> [G, ...]."""
    world = dist.get_world_size(group)
    out = x.new_empty((world,) + tuple(x.shape))
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out.view(-1), x.contiguous().view(-1), group=group)
    else:
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        out = torch.stack(parts)
    return out


def _reduce_scatter_rows(x: torch.Tensor, group) -> torch.Tensor:
    """[G, T, c] partial sums on every rank -> [T, c]: the slice of this rank, summed over ranks."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if dist.get_backend(group) == "nccl":
        out = x.new_empty(tuple(x.shape[1:]))
        dist.reduce_scatter_tensor(out.view(-1), x.contiguous().view(-1), group=group)
        return out
    y = x.clone()
    dist.all_reduce(y, group=group)
    return y[rank].contiguous()


class GatherExpertParallel:
    """``route_build_fn(topk_idx [N,k] int32, topk_w [N,k] fp32, global_to_local int32 [E]) -> (token_indices,
    expert_offsets, route_flat)`` over the gathered tokens; ``experts_fn`` as in ExpertParallelLayer with the
    gathered rows laid out as [G, 2, T, r] (gate block, up block per source rank)."""

    def __init__(self, num_experts: int, top_k: int, route_build_fn: Callable, experts_fn: Callable, group=None,
                 device="cpu"):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not shard over {self.world} ranks")
        self.per = num_experts // self.world
        self.top_k = top_k
        self.route_build_fn, self.experts_fn = route_build_fn, experts_fn
        g2l = torch.full((num_experts,), -1, dtype=torch.int32)
        g2l[self.rank * self.per:(self.rank + 1) * self.per] = torch.arange(self.per, dtype=torch.int32)
        self.g2l = g2l.to(device)

    def forward_rank_space(self, h_pair: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                           rank_out: int) -> torch.Tensor:
        """h_pair [2, T, r] fp16 (gate rows, up rows of the local tokens), topk_idx int32 [T,k], topk_w fp32 [T,k]
        -> rank_accum [T, rank_out] fp32 of the local tokens, summed over all ranks' experts."""
        _, T, r = h_pair.shape
        G, k = self.world, self.top_k
        h_all = _gather(h_pair, self.group)                                   # [G, 2, T, r]
        routing = torch.stack((topk_idx.to(torch.int32), topk_w.to(torch.float32).view(torch.int32)))   # [2, T, k]
        r_all = _gather(routing, self.group)                                  # [G, 2, T, k]
        idx_all = r_all[:, 0].reshape(G * T, k).contiguous()
        w_all = r_all[:, 1].reshape(G * T, k).contiguous().view(torch.float32)
        tok, off, rw = self.route_build_fn(idx_all, w_all, self.g2l)
        # token u = s*T + t of the gathered batch lives at row s*2T + t of the gate block view and the same row
        # of the up block view (which starts T rows later)
        tok_v = (torch.div(tok, T, rounding_mode="floor") * (2 * T) + tok % T).to(torch.int32)
        flat = h_all.view(G * 2 * T, r)
        part = self.experts_fn(flat, flat[T:], tok_v, off, rw)                # one row per row of `flat` (or T fewer)
        if part.shape[0] == G * 2 * T:
            mine = part.view(G, 2, T, rank_out)[:, 0].contiguous()            # [G, T, rank_out]: the gate-block rows
        else:
            full = torch.zeros((G * 2 * T, rank_out), dtype=torch.float32, device=h_pair.device)
            full[: part.shape[0]] = part
            mine = full.view(G, 2, T, rank_out)[:, 0].contiguous()
        return _reduce_scatter_rows(mine, self.group)


# ---------------------------------------------------------------------------------------------------------
# Prefill-sized batches on one NVLink box: exchange through peer memory, no collective library on the data
# path, no data-dependent sizes, no host synchronisation.
#
# Every rank maps one receive area of every other rank (torch's symmetric memory: one allocation per rank,
# exchanged once at construction).  A wave of T tokens per rank then runs, stream-ordered on every rank:
#
#   top-k and basis projection write into the rank's own slice of its area
#   bm_ep_push        rows to the ranks that own one of the token's experts (once per (token, destination)),
#                     top-k of every token to every rank
#   barrier
#   routing build over all G*T tokens with a map that keeps this rank's experts, packed experts straight
#   out of the receive area into the partial rank_accum of the wave
#   barrier
#   bm_ep_pull_reduce the token's home rank adds the partial rows of the ranks that contributed, ascending
#   down basis (+ residual)
#
# Two waves alternate between two areas (and two streams) so that one wave's exchange can run beside the
# other's expert kernel.
# ---------------------------------------------------------------------------------------------------------
class SymmetricExpertParallel:
    """Expert-parallel forward of one packed layer over the ranks of ``group`` (all on one NVLink domain).

    ``packed`` is this rank's ``PackedLayer`` (its slice of the experts plus the replicated basis),
    ``wave_tokens`` the number of tokens per rank and wave (the same on every rank)."""

    AREAS = 2

    def __init__(self, packed, num_experts: int, top_k: int, wave_tokens: int, norm_topk_prob: bool = True,
                 group=None):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm
        from . import capi
        self._C, self._capi = C, capi
        self.packed, self.group = packed, group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not shard over {self.world} ranks")
        self.per = num_experts // self.world
        if packed.num_experts != self.per:
            raise ValueError(f"this rank's layer holds {packed.num_experts} experts, expected {self.per}")
        self.top_k, self.norm_topk_prob, self.T = top_k, norm_topk_prob, int(wave_tokens)
        dev = packed.device
        G, T, k, r, r_out = self.world, self.T, top_k, packed.rank_in, packed.rank_out
        align = lambda n: (n + 255) // 256 * 256
        self.h_bytes = align(2 * G * T * r * 2)
        self.r_bytes = align(2 * G * T * k * 4)
        self.p_bytes = align(G * T * r_out * 4)
        self.area_bytes = self.h_bytes + self.r_bytes + self.p_bytes
        flag_bytes = align(int(capi.lib().bm_ep_flag_bytes()))
        self.buf = symm.empty(self.AREAS * self.area_bytes + flag_bytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.hdl = symm.rendezvous(self.buf, self.group)
        ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        Arr = C.c_void_p * G
        self._tabs = []
        for a in range(self.AREAS):
            base = [p + a * self.area_bytes for p in ptrs]
            self._tabs.append((Arr(*base), Arr(*[b + self.h_bytes for b in base]),
                               Arr(*[b + self.h_bytes + self.r_bytes for b in base])))
        self._flags = Arr(*[p + self.AREAS * self.area_bytes for p in ptrs])
        self.barrier_limit_ms = 5000
        g2l = torch.full((num_experts,), -1, dtype=torch.int32)
        g2l[self.rank * self.per:(self.rank + 1) * self.per] = torch.arange(self.per, dtype=torch.int32)
        self.g2l = g2l.to(dev)
        # per-area scratch of the routing build over the G*T tokens of a wave, and of the combine
        lib = capi.lib()
        A = G * T * k
        self._ws_bytes = int(lib.bm_route_build_workspace_bytes(G * T, k, self.per))
        self._scratch = []
        for _ in range(self.AREAS):
            self._scratch.append(dict(
                tok=torch.empty(A, dtype=torch.int32, device=dev), off=torch.empty(self.per + 1, dtype=torch.int32, device=dev),
                rw=torch.empty(A, dtype=torch.float32, device=dev),
                ws=torch.empty(max(self._ws_bytes, 256), dtype=torch.uint8, device=dev),
                acc=torch.empty((T, r_out), dtype=torch.float32, device=dev)))
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(self.AREAS)]
        self._side = [torch.cuda.Stream(device=dev) for _ in range(self.AREAS)]
        torch.cuda.synchronize(dev)          # the zeroed flag area is in place before any peer signals into it
        dist.barrier(group=self.group)

    # views into this rank's own area ------------------------------------------------------------------
    def _own(self, area: int):
        G, T, k, r = self.world, self.T, self.top_k, self.packed.rank_in
        base = area * self.area_bytes
        h = self.buf[base: base + 2 * G * T * r * 2].view(torch.float16).view(2, G, T, r)
        rt = self.buf[base + self.h_bytes: base + self.h_bytes + 2 * G * T * k * 4].view(torch.int32).view(2, G, T, k)
        part = self.buf[base + self.h_bytes + self.r_bytes: base + self.h_bytes + self.r_bytes + G * T * self.packed.rank_out * 4]
        return h, rt, part.view(torch.float32).view(G * T, self.packed.rank_out)

    def nvlink_bytes_per_wave(self, topk_idx: torch.Tensor) -> Tuple[int, int]:
        """(bytes this rank pushes, bytes it pulls) for the given routing of its tokens -- bookkeeping for reports."""
        dest = expert_owner(topk_idx.long(), self.per)
        pair = torch.zeros((topk_idx.shape[0], self.world), dtype=torch.bool, device=topk_idx.device)
        pair.scatter_(1, dest, True)
        pair[:, self.rank] = False
        rows = int(pair.sum())
        push = rows * 2 * self.packed.rank_in * 2 + topk_idx.shape[0] * self.top_k * 8 * (self.world - 1)
        return push, rows * self.packed.rank_out * 4

    def forward_wave(self, x: torch.Tensor, logits: torch.Tensor, weight_dtype, out: torch.Tensor,
                     residual: Optional[torch.Tensor] = None, area: int = 0, residual_fn=None) -> torch.Tensor:
        """One wave on the current stream: x [T, H], logits [T, E] of this rank's tokens -> out [T, H].

        ``residual_fn(x) -> [T, H]`` (e.g. a dense shared expert) runs on a side stream beside the exchange and the
        barriers, where the GPU is mostly idle (it starts once the basis projection is queued); the wave waits for it
        only before the final down-basis product."""
        capi, lib, pk = self._capi, self._capi.lib(), self.packed
        G, T, k, r, r_out = self.world, self.T, self.top_k, pk.rank_in, pk.rank_out
        if x.shape[0] != T:
            raise ValueError(f"a wave holds {T} tokens per rank, got {x.shape[0]}")
        h, rt, part = self._own(area)
        sc = self._scratch[area]
        h_tab, r_tab, p_tab = self._tabs[area]
        st = capi.stream_ptr(pk.device)
        x, logits = x.contiguous(), logits.contiguous()
        with torch.cuda.device(pk.device):
            idx_mine, w_mine = rt[0, self.rank], rt[1, self.rank]
            capi.check(lib.bm_route_topk(logits.data_ptr(), capi.dtype_code(logits.dtype), T, logits.shape[1], k,
                                         int(bool(self.norm_topk_prob)), capi.round_code(weight_dtype), idx_mine.data_ptr(),
                                         w_mine.data_ptr(), st))
            capi.check(lib.bm_basis_project(pk._handle, x.data_ptr(), capi.dtype_code(x.dtype), T, h[0, self.rank].data_ptr(),
                                            h[1, self.rank].data_ptr(), st))
            if residual_fn is not None:
                # forked here, after the projection: the side stream's GEMMs then run beside the push, the barrier and
                # the routing build, which leave most SMs idle, instead of competing with the projection
                main, side = torch.cuda.current_stream(pk.device), self._side[area]
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    residual = residual_fn(x)
                    residual.record_stream(main)
            capi.check(lib.bm_ep_push(h_tab, r_tab, G, self.rank, T, r, k, self.per, st))
            capi.check(lib.bm_ep_barrier(pk._handle, self._flags, G, self.rank, 2 * area, self.barrier_limit_ms, st))
            capi.check(lib.bm_route_build(rt[0].data_ptr(), rt[1].data_ptr(), self.g2l.data_ptr(), self.g2l.numel(), G * T, k,
                                          self.per, 128, sc["tok"].data_ptr(), sc["off"].data_ptr(), sc["rw"].data_ptr(), None,
                                          None, sc["ws"].data_ptr(), sc["ws"].numel(), st))
            need = int(lib.bm_experts_workspace_bytes(pk._handle, G * T, G * T * k, capi.PATH_AUTO))
            if need and (sc.get("xws") is None or sc["xws"].numel() < need):
                sc["xws"] = torch.empty(need, dtype=torch.uint8, device=pk.device)      # deterministic mode only
            capi.check(lib.bm_experts_forward(pk._handle, h[0].data_ptr(), h[1].data_ptr(), sc["tok"].data_ptr(),
                                              sc["off"].data_ptr(), sc["rw"].data_ptr(), G * T, G * T * k, part.data_ptr(),
                                              capi.PATH_AUTO, capi.ptr(sc.get("xws")) if need else None, need, st))
            capi.check(lib.bm_ep_barrier(pk._handle, self._flags, G, self.rank, 2 * area + 1, self.barrier_limit_ms, st))
            capi.check(lib.bm_ep_pull_reduce(p_tab, idx_mine.data_ptr(), G, self.rank, T, r_out, k, self.per,
                                             sc["acc"].data_ptr(), st))
            if residual_fn is not None:
                with torch.cuda.stream(side):
                    residual = residual.to(x.dtype).contiguous()
                main.wait_stream(side)
            elif residual is not None:
                residual = residual.to(x.dtype).contiguous()
            capi.check(lib.bm_combine_down_basis(pk._handle, sc["acc"].data_ptr(), T, capi.ptr(residual), out.data_ptr(),
                                                 capi.dtype_code(out.dtype), st))
        return out

    def forward(self, x: torch.Tensor, logits: torch.Tensor, weight_dtype=torch.float16,
                residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                overlap: bool = True, residual_fn=None) -> torch.Tensor:
        """x [n*T, H] -> y [n*T, H] in n waves of T tokens; with ``overlap`` consecutive waves alternate between two
        streams (and two receive areas), so one wave's exchange runs beside the other's expert kernel.
        ``residual_fn``: see ``forward_wave`` (called once per wave with that wave's rows of ``x``)."""
        T = self.T
        if x.shape[0] % T:
            raise ValueError(f"{x.shape[0]} tokens are not a whole number of waves of {T}")
        n = x.shape[0] // T
        y = out if out is not None else torch.empty_like(x)
        cur = torch.cuda.current_stream(self.packed.device)
        if not overlap or n == 1:
            for w in range(n):
                s = slice(w * T, (w + 1) * T)
                self.forward_wave(x[s], logits[s], weight_dtype, y[s], None if residual is None else residual[s], area=w % self.AREAS,
                                  residual_fn=residual_fn)
            return y
        for st in self.streams:
            st.wait_stream(cur)
        for w in range(n):
            s = slice(w * T, (w + 1) * T)
            with torch.cuda.stream(self.streams[w % self.AREAS]):
                self.forward_wave(x[s], logits[s], weight_dtype, y[s], None if residual is None else residual[s], area=w % self.AREAS,
                                  residual_fn=residual_fn)
        for st in self.streams:
            cur.wait_stream(st)
        return y
