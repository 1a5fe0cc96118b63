"""Device-side state of one packed MoE layer and the calls into the CUDA library.

``PackedLayer`` takes the buffers exactly as the reference's expert modules hold them
(bitsmoe/models/base_mlp.py:96-102: payload, rank_idx, tile_meta, slab_meta, scale, s per
matrix per expert) plus the three shared-basis matrices (bitsmoe/models/base_block.py:27-29),
hands their device pointers to ``bm_layer_create`` once, and then runs the stages of the
forward path.  It replaces the process-global pointer-table cache of
bitsmoe/algorithms/cpp/mlp_forward.cu:2464-2503 with state owned by the block.
All device memory (arena, workspaces, outputs) comes from torch's allocator.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import capi

MATRIX_FIELDS = ("payload", "rank_idx", "tile_meta", "slab_meta", "scale", "s")
TILE_ROWS = 128


def _as(t: torch.Tensor, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    if t.dtype != dtype or t.device != device or not t.is_contiguous():
        t = t.to(device=device, dtype=dtype).contiguous()
    return t


class PackedLayer:
    def __init__(self, gate: Dict[str, Sequence[torch.Tensor]], up: Dict[str, Sequence[torch.Tensor]],
                 down: Dict[str, Sequence[torch.Tensor]], intermediate_size: int, rank_out: int,
                 vh_gate: Optional[torch.Tensor] = None, vh_up: Optional[torch.Tensor] = None,
                 u_down: Optional[torch.Tensor] = None, rank_in: Optional[int] = None,
                 act_type: int = 0, device: Optional[torch.device] = None):
        self._handle = None
        n = len(gate["payload"])
        if device is None:
            device = (vh_gate.device if vh_gate is not None else
                      (gate["payload"][0].device if n else torch.device("cuda", torch.cuda.current_device())))
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("Packed routed experts require CUDA mlp_forward extension; "
                               "python fallback is intentionally disabled.")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.num_experts = n
        self.intermediate_size = int(intermediate_size)
        self.rank_out = int(rank_out)
        dtypes = {"payload": torch.uint32, "rank_idx": torch.int32, "tile_meta": torch.int32,
                  "slab_meta": torch.int32, "scale": torch.float16, "s": torch.float16}
        self._keep = []
        tables = []
        for name, bufs in (("gate", gate), ("up", up), ("down", down)):
            for f in MATRIX_FIELDS:
                if len(bufs[f]) != n:
                    raise RuntimeError(f"{name}_{f} size mismatch, expected {n}, got {len(bufs[f])}")
            arr = (capi.Matrix * max(n, 1))()
            for e in range(n):
                t = {f: _as(bufs[f][e], dtypes[f], device) for f in MATRIX_FIELDS}
                self._keep.append(t)
                m = arr[e]
                m.payload, m.payload_words = t["payload"].data_ptr(), t["payload"].numel()
                m.rank_idx, m.n_rows = t["rank_idx"].data_ptr(), t["rank_idx"].numel()
                m.tile_meta, m.n_tile_rows = t["tile_meta"].data_ptr(), t["tile_meta"].numel() // 3
                m.slab_meta, m.n_slabs = t["slab_meta"].data_ptr(), t["slab_meta"].numel() // 4
                m.scale, m.n_scales = t["scale"].data_ptr(), t["scale"].numel()
                m.s = t["s"].data_ptr()
                if t["s"].numel() < t["rank_idx"].numel():
                    raise RuntimeError(f"{name}_s of expert {e} is shorter than its rank_idx")
            tables.append(arr)
        self._tables = tables
        basis = []
        for b in (vh_gate, vh_up, u_down):
            basis.append(None if b is None or b.numel() == 0 else _as(b.detach(), torch.float16, device))
        self.vh_gate, self.vh_up, self.u_down = basis
        if rank_in is None:
            rank_in = int(self.vh_gate.shape[0]) if self.vh_gate is not None else self.rank_out
        self.rank_in = int(rank_in)
        self.hidden = int(self.vh_gate.shape[1]) if self.vh_gate is not None else (
            int(self.u_down.shape[0]) if self.u_down is not None else 0)
        if self.u_down is not None and int(self.u_down.shape[1]) != self.rank_out:
            raise RuntimeError(f"shared_u_down has {int(self.u_down.shape[1])} columns, rank_out is {self.rank_out}")
        d = capi.LayerDesc()
        d.num_experts, d.hidden, d.intermediate = n, self.hidden, self.intermediate_size
        d.rank_in, d.rank_out, d.act_type = self.rank_in, self.rank_out, int(act_type)
        d.gate, d.up, d.down = tables[0], tables[1], tables[2]
        d.vh_gate, d.vh_up, d.u_down = capi.ptr(self.vh_gate), capi.ptr(self.vh_up), capi.ptr(self.u_down)
        self._desc = d
        lib = capi.lib()
        with torch.cuda.device(device):
            need = C.c_size_t(0)
            capi.check(lib.bm_layer_plan(C.byref(d), C.byref(need)))
            self._arena = torch.empty(max(int(need.value), 256), dtype=torch.uint8, device=device)
            h = C.c_void_p()
            capi.check(lib.bm_layer_create(C.byref(d), self._arena.data_ptr(), self._arena.numel(),
                                           capi.stream_ptr(device), C.byref(h)))
        self._handle = h
        self._ws: Dict[Tuple[int, int], torch.Tensor] = {}

    # -- construction helpers -------------------------------------------------------------------------
    @classmethod
    def from_expert_modules(cls, experts, intermediate_size, rank_out, vh_gate=None, vh_up=None, u_down=None,
                            act_type: int = 0, device=None) -> "PackedLayer":
        """``experts``: modules carrying ``{gate,up,down}_{payload,rank_idx,tile_meta,slab_meta,scale,s}_buffer``."""
        def tab(tag):
            return {f: [getattr(m, f"{tag}_{f}_buffer") for m in experts] for f in MATRIX_FIELDS}
        return cls(tab("gate"), tab("up"), tab("down"), intermediate_size, rank_out, vh_gate, vh_up, u_down,
                   act_type=act_type, device=device)

    def close(self) -> None:
        if getattr(self, "_handle", None) is not None:
            capi.lib().bm_layer_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- stages ---------------------------------------------------------------------------------------
    def expert_bytes(self, e: int) -> int:
        return int(capi.lib().bm_layer_expert_bytes(self._handle, e))

    @property
    def has_fast_layout(self) -> bool:
        return bool(capi.lib().bm_layer_has_fast_layout(self._handle))

    def set_deterministic(self, on: bool = True) -> None:
        """Packed-expert kernels add into rank_accum through 64-bit fixed-point atomics: bit-identical results from run
        to run (the reference's fp32 atomics, bitsmoe/algorithms/cpp/mlp_forward.cu:2062, depend on arrival order)."""
        capi.check(capi.lib().bm_layer_set_option(self._handle, 1, int(bool(on))))
        self._ws.clear()

    def set_decode_ctas_per_sm(self, n: int = 0) -> None:
        capi.check(capi.lib().bm_layer_set_option(self._handle, 0, int(n)))

    def check_status(self) -> None:
        """Synchronises and raises if a kernel of this layer gave up a bounded device-side wait."""
        with torch.cuda.device(self.device):
            capi.check(capi.lib().bm_layer_status(self._handle, capi.stream_ptr(self.device)))

    def decode_codes(self, e: int, which: int, source: int = 0) -> torch.Tensor:
        """int8 codes [stored rows, intermediate]; source 0 = reference buffers, 1 = repacked arena."""
        n_rows = self._keep[which * self.num_experts + e]["rank_idx"].numel()
        out = torch.empty((n_rows, self.intermediate_size), dtype=torch.int8, device=self.device)
        with torch.cuda.device(self.device):
            capi.check(capi.lib().bm_layer_decode_codes(self._handle, e, which, source, out.data_ptr(),
                                                        capi.stream_ptr(self.device)))
        return out

    def route_topk(self, logits: torch.Tensor, top_k: int, norm_topk_prob: bool, weight_dtype) -> Tuple[torch.Tensor, torch.Tensor]:
        return route_topk(logits, top_k, norm_topk_prob, weight_dtype)

    def basis_project(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """h_gate, h_up [T, r] fp16; ``out`` may be a preallocated [2, T, r] fp16 tensor that receives both."""
        x = x.contiguous()
        T = x.shape[0]
        if out is None:
            out = torch.empty((2, T, self.rank_in), dtype=torch.float16, device=self.device)
        hg, hu = out[0], out[1]
        with torch.cuda.device(self.device):
            capi.check(capi.lib().bm_basis_project(self._handle, x.data_ptr(), capi.dtype_code(x.dtype), T,
                                                   hg.data_ptr(), hu.data_ptr(), capi.stream_ptr(self.device)))
        return hg, hu

    def experts_forward(self, h_gate, h_up, token_indices, expert_offsets, route_weights,
                        path: int = capi.PATH_AUTO) -> torch.Tensor:
        T = h_gate.shape[0]
        A = token_indices.numel()
        out = torch.empty((T, self.rank_out), dtype=torch.float32, device=self.device)
        lib = capi.lib()
        with torch.cuda.device(self.device):
            need = int(lib.bm_experts_workspace_bytes(self._handle, T, A, path))
            ws = torch.empty(max(need, 1), dtype=torch.uint8, device=self.device) if need else None
            capi.check(lib.bm_experts_forward(self._handle, h_gate.data_ptr(), h_up.data_ptr(), token_indices.data_ptr(),
                                              expert_offsets.data_ptr(), route_weights.data_ptr(), T, A, out.data_ptr(),
                                              path, capi.ptr(ws), need, capi.stream_ptr(self.device)))
        return out

    def combine_down_basis(self, rank_accum: torch.Tensor, out_dtype: torch.dtype,
                           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        T = rank_accum.shape[0]
        y = torch.empty((T, self.hidden), dtype=out_dtype, device=self.device)
        if residual is not None:
            residual = residual.to(out_dtype).contiguous()
        with torch.cuda.device(self.device):
            capi.check(capi.lib().bm_combine_down_basis(self._handle, rank_accum.data_ptr(), T, capi.ptr(residual),
                                                        y.data_ptr(), capi.dtype_code(out_dtype),
                                                        capi.stream_ptr(self.device)))
        return y

    def workspace(self, T: int, k: int) -> torch.Tensor:
        key = (T, k)
        ws = self._ws.get(key)
        if ws is None:
            need = int(capi.lib().bm_layer_workspace_bytes(self._handle, T, k))
            ws = torch.empty(max(need, 256), dtype=torch.uint8, device=self.device)
            if len(self._ws) > 8:
                self._ws.clear()
            self._ws[key] = ws
        return ws

    def forward(self, x: torch.Tensor, logits: torch.Tensor, top_k: int, norm_topk_prob: bool = True,
                weight_dtype=torch.float16, residual: Optional[torch.Tensor] = None,
                global_to_local: Optional[torch.Tensor] = None, path: int = capi.PATH_AUTO,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [T, H] (fp16 / bf16), logits [T, E_routed] -> y [T, H] in x's dtype.  One stream, no host sync."""
        x = x.contiguous()
        logits = logits.contiguous()
        T = x.shape[0]
        y = out if out is not None else torch.empty_like(x)
        if residual is not None:
            residual = residual.to(x.dtype).contiguous()
        ws = self.workspace(T, top_k)
        with torch.cuda.device(self.device):
            capi.check(capi.lib().bm_layer_forward(
                self._handle, x.data_ptr(), capi.dtype_code(x.dtype), logits.data_ptr(), capi.dtype_code(logits.dtype),
                T, logits.shape[1], top_k, int(bool(norm_topk_prob)), capi.round_code(weight_dtype),
                capi.ptr(global_to_local), capi.ptr(residual), y.data_ptr(), path, ws.data_ptr(), ws.numel(),
                capi.stream_ptr(self.device)))
        return y


def route_topk(logits: torch.Tensor, top_k: int, norm_topk_prob: bool = True, weight_dtype=torch.float16):
    """softmax -> top-k -> renorm -> rounding; returns (int32 [T,k], fp32 [T,k])."""
    if not logits.is_cuda:
        raise RuntimeError("route_topk requires a CUDA tensor; there is no CPU path")
    logits = logits.contiguous()
    T, E = logits.shape
    idx = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device):
        capi.check(capi.lib().bm_route_topk(logits.data_ptr(), capi.dtype_code(logits.dtype), T, E, top_k,
                                            int(bool(norm_topk_prob)), capi.round_code(weight_dtype), idx.data_ptr(),
                                            w.data_ptr(), capi.stream_ptr(logits.device)))
    return idx, w


def route_build(topk_idx: torch.Tensor, topk_w: torch.Tensor, num_local: int,
                global_to_local: Optional[torch.Tensor] = None, tile_rows: int = TILE_ROWS):
    """-> token_indices int32 [T*k], expert_offsets int32 [num_local+1], route_flat fp32 [T*k],
    tile_table int32 [max_tiles, 3], counts int32 [2] = (assignments kept, tiles).  Entries of
    token_indices / route_flat past counts[0] are unspecified."""
    if not topk_idx.is_cuda:
        raise RuntimeError("route_build requires CUDA tensors; there is no CPU path")
    dev = topk_idx.device
    topk_idx = topk_idx.to(torch.int32).contiguous()
    topk_w = topk_w.to(torch.float32).contiguous()
    T, k = topk_idx.shape
    lib = capi.lib()
    max_tiles = int(lib.bm_route_max_tiles(T, k, num_local, tile_rows))
    tok = torch.empty((T * k,), dtype=torch.int32, device=dev)
    off = torch.empty((num_local + 1,), dtype=torch.int32, device=dev)
    rw = torch.empty((T * k,), dtype=torch.float32, device=dev)
    tiles = torch.empty((max_tiles, 3), dtype=torch.int32, device=dev)
    counts = torch.empty((2,), dtype=torch.int32, device=dev)
    need = int(lib.bm_route_build_workspace_bytes(T, k, num_local))
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=dev) if need else None
    num_routed = num_local
    if global_to_local is not None:
        global_to_local = global_to_local.to(device=dev, dtype=torch.int32).contiguous()
        num_routed = global_to_local.numel()
    with torch.cuda.device(dev):
        capi.check(lib.bm_route_build(topk_idx.data_ptr(), topk_w.data_ptr(), capi.ptr(global_to_local), num_routed, T, k, num_local,
                                      tile_rows, tok.data_ptr(), off.data_ptr(), rw.data_ptr(), tiles.data_ptr(),
                                      counts.data_ptr(), capi.ptr(ws), need, capi.stream_ptr(dev)))
    return tok, off, rw, tiles, counts


def gate_logits(x: torch.Tensor, gate_weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Router logits x @ gate_weight.T on the library's kernels: x [T, H] (fp16 / bf16 / fp32), gate_weight fp16 [E, H]
    -> [T, E] in ``out_dtype`` (default: x's dtype, as ``self.gate(hidden_states)`` gives in the reference)."""
    if not x.is_cuda:
        raise RuntimeError("gate_logits requires CUDA tensors; there is no CPU path")
    x = x.contiguous()
    w = _as(gate_weight.detach(), torch.float16, x.device)
    out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        capi.check(capi.lib().bm_gate_logits(x.data_ptr(), capi.dtype_code(x.dtype), w.data_ptr(), x.shape[0], w.shape[0],
                                             w.shape[1], out.data_ptr(), capi.dtype_code(out.dtype), capi.stream_ptr(x.device)))
    return out


def dense_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
              token_gate_weight: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dense SwiGLU MLP of a shared expert on the library's kernels: (silu(x Wg^T) * (x Wu^T)) Wd^T, scaled per token by
    sigmoid(x . token_gate_weight) when that is given, plus ``residual``.  Weights fp16; result in x's dtype."""
    if not x.is_cuda:
        raise RuntimeError("dense_mlp requires CUDA tensors; there is no CPU path")
    x = x.contiguous()
    dev = x.device
    wg, wu, wd = (_as(w.detach(), torch.float16, dev) for w in (w_gate, w_up, w_down))
    tg = None if token_gate_weight is None else _as(token_gate_weight.detach().reshape(-1), torch.float16, dev)
    T, H, I = x.shape[0], x.shape[1], wg.shape[0]
    y = torch.empty_like(x)
    if residual is not None:
        residual = residual.to(x.dtype).contiguous()
    lib = capi.lib()
    need = int(lib.bm_dense_mlp_workspace_bytes(T, I))
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        capi.check(lib.bm_dense_mlp_forward(x.data_ptr(), capi.dtype_code(x.dtype), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(),
                                            capi.ptr(tg), T, H, I, capi.ptr(residual), y.data_ptr(), capi.dtype_code(y.dtype),
                                            ws.data_ptr(), ws.numel(), capi.stream_ptr(dev)))
    return y
