"""Expert-parallel dispatch / combine.

Two routing disciplines:

* ``dispatch_with_capacity`` / ``combine_with_layout`` reproduce the reference's semantics
  (crates/rmlx-distributed/src/moe_exchange.rs:519-581,724-807,1102-1195,2288-2330): expert ``e`` lives
  on rank ``e // (E / world)``, each expert accepts ``ceil(tokens * k / E * capacity_factor)`` rows
  per source rank, rows beyond that are dropped (route index -1) and counted as overflow, and the
  dispatched buffer is laid out ``[local_expert][src_rank * capacity + cursor][hidden]``.
* ``EpExchange`` is the capacity-free form this framework uses: (token, slot) pairs are sorted by
  destination expert, per-destination counts are exchanged first, rows travel in one all-to-all,
  and the receiver gets rows grouped by local expert with prefix offsets (nothing is ever
  dropped). On GPUs the fused kernels of ``csrc/comm/ep_dispatch.cu`` do the same thing by
  writing rows straight into the peers' slabs; this class is the library-collective path (NCCL or
  gloo) and the oracle for it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Tuple

import torch

from .group import Group


@dataclass
class DispatchLayout:
    """What combine needs to undo a dispatch."""
    order: torch.Tensor            # [T*k] pair index (token*k + slot) in send order
    send_counts: List[int]         # rows sent to each rank
    recv_counts: List[int]         # rows received from each rank
    recv_expert: torch.Tensor      # [R] local expert id of every received row (grouped order)
    recv_perm: torch.Tensor        # [R] position in arrival order of each grouped row
    offsets: torch.Tensor          # [E_local + 1] prefix offsets of the grouped rows
    num_tokens: int
    top_k: int


def fp8_quant_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[n, d] -> (E4M3 codes as uint8 [n, d], fp32 scale [n]): scale = max|row| / 448, the wire
    format of the reference's FP8 exchange (crates/rmlx-distributed/src/fp8_exchange.rs:85-160).
    bf16 rows on a GPU go through this package's kernel, everything else through torch."""
    n, d = x.shape
    if x.is_cuda and x.dtype == torch.bfloat16 and n > 0:
        from .. import _lib
        q = torch.empty(n, d, dtype=torch.uint8, device=x.device)
        scale = torch.empty(n, dtype=torch.float32, device=x.device)
        xc = x.contiguous()
        _lib.check(_lib.cuda().rmlx_fp8_quant_rows(xc.data_ptr(), q.data_ptr(), scale.data_ptr(), n, d,
                                                   _lib.stream_ptr()), "fp8_quant_rows")
        return q, scale
    xf = x.float()
    amax = xf.abs().amax(-1, keepdim=True) if n else xf.new_zeros(0, 1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    return (xf / scale).to(torch.float8_e4m3fn).view(torch.uint8), scale.squeeze(-1)


def fp8_dequant_rows(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    n, d = q.shape
    if q.is_cuda and dtype == torch.bfloat16 and n > 0:
        from .. import _lib
        out = torch.empty(n, d, dtype=torch.bfloat16, device=q.device)
        _lib.check(_lib.cuda().rmlx_fp8_dequant_rows(q.contiguous().data_ptr(), scale.contiguous().data_ptr(),
                                                     out.data_ptr(), n, d, _lib.stream_ptr()), "fp8_dequant_rows")
        return out
    return (q.view(torch.float8_e4m3fn).float() * scale[:, None]).to(dtype)


class EpExchange:
    """``payload="fp8"``: rows cross the wire as E4M3 codes plus one fp32 scale per row (d + 4
    bytes instead of 2 d), in both directions; ``wire_bytes`` counts what was sent either way."""

    def __init__(self, group: Group, num_experts: int, payload: str = "bf16"):
        if payload not in ("bf16", "fp8"):
            raise ValueError("payload is 'bf16' (rows as they are) or 'fp8'")
        self.payload = payload
        self.wire_bytes = 0
        self.group = group
        self.world, self.rank = group.world_size, group.local_rank
        if num_experts % self.world:
            raise ValueError("num_experts must divide by the expert-parallel size")
        self.E, self.e_local = num_experts, num_experts // self.world

    def dispatch(self, x: torch.Tensor, idx: torch.Tensor) -> Tuple[torch.Tensor, DispatchLayout]:
        """x [T, D], idx [T, k] (global expert ids). Returns rows grouped by local expert."""
        t, k = idx.shape
        flat = idx.reshape(-1).long()
        order = torch.argsort(flat, stable=True)            # by expert => by destination rank
        dest = flat[order] // self.e_local
        send_counts = torch.bincount(dest, minlength=self.world).tolist()
        rows = x[order // k]
        meta = (flat[order] % self.e_local).to(torch.int64)
        recv_counts = self.group.all_to_all(
            torch.tensor(send_counts, dtype=torch.int64, device=x.device)).tolist() \
            if self.world > 1 else list(send_counts)
        got = self._rows_all_to_all(rows, send_counts, recv_counts)
        got_e = self.group.all_to_all(meta, send_counts, recv_counts)
        perm = torch.argsort(got_e, stable=True)             # group by local expert
        counts = torch.bincount(got_e, minlength=self.e_local)
        offsets = torch.zeros(self.e_local + 1, dtype=torch.int64, device=x.device)
        offsets[1:] = torch.cumsum(counts, 0)
        layout = DispatchLayout(order, send_counts, recv_counts, got_e[perm], perm, offsets, t, k)
        return got[perm], layout

    def _rows_all_to_all(self, rows: torch.Tensor, send_counts: List[int], recv_counts: List[int]) -> torch.Tensor:
        if self.payload == "bf16":
            self.wire_bytes += rows.numel() * rows.element_size()
            return self.group.all_to_all(rows, send_counts, recv_counts)
        q, scale = fp8_quant_rows(rows)
        self.wire_bytes += q.numel() + 4 * scale.numel()
        got_q = self.group.all_to_all(q, send_counts, recv_counts)
        got_s = self.group.all_to_all(scale, send_counts, recv_counts)
        return fp8_dequant_rows(got_q, got_s, rows.dtype)

    def combine(self, y: torch.Tensor, wts: torch.Tensor, layout: DispatchLayout) -> torch.Tensor:
        """y: expert outputs for the grouped rows. Returns sum_k w[t,k] * y(t,k) as fp32 [T, D]."""
        arrival = torch.empty_like(y)
        arrival[layout.recv_perm] = y                        # back to arrival order
        back = self._rows_all_to_all(arrival, layout.recv_counts, layout.send_counts)
        out = torch.zeros(layout.num_tokens, y.shape[-1], dtype=torch.float32, device=y.device)
        pair = layout.order
        w = wts.reshape(-1)[pair].float()
        out.index_add_(0, pair // layout.top_k, back.float() * w[:, None])
        return out


# ------------------------------------------------------------------------------------------------
# Reference-compatible capacity-limited routing (single process view of one rank's send side)
# ------------------------------------------------------------------------------------------------
def expert_capacity(num_tokens: int, top_k: int, num_experts: int, capacity_factor: float) -> int:
    return max(1, math.ceil(num_tokens * top_k / num_experts * capacity_factor))


def dispatch_with_capacity(x: torch.Tensor, idx: torch.Tensor, num_experts: int, world: int,
                           src_rank: int, capacity_factor: float = 1.0):
    """Returns (buffers, route_indices, overflow): ``buffers[r]`` is what goes to rank r, shaped
    [E_local, capacity, D] (this source's stripe of the destination layout); ``route_indices``
    [T, k] holds the slot ``local_expert * world*capacity + src_rank*capacity + cursor`` or -1."""
    t, k = idx.shape
    e_local = num_experts // world
    cap = expert_capacity(t, k, num_experts, capacity_factor)
    bufs = [torch.zeros(e_local, cap, x.shape[1], dtype=x.dtype) for _ in range(world)]
    cursors = [0] * num_experts
    route = torch.full((t, k), -1, dtype=torch.int64)
    overflow = 0
    for ti in range(t):
        for s in range(k):
            e = int(idx[ti, s])
            c = cursors[e]
            if c >= cap:
                overflow += 1
                continue
            cursors[e] = c + 1
            r, le = e // e_local, e % e_local
            bufs[r][le, c] = x[ti]
            route[ti, s] = le * world * cap + src_rank * cap + c
    return bufs, route, overflow


def combine_with_layout(expert_out: List[torch.Tensor], idx: torch.Tensor, wts: torch.Tensor,
                        route: torch.Tensor, num_experts: int, world: int, src_rank: int,
                        capacity: int) -> torch.Tensor:
    """expert_out[r]: [E_local, world*capacity, D] results held by rank r. Dropped pairs add 0."""
    t, k = idx.shape
    e_local = num_experts // world
    d = expert_out[0].shape[-1]
    out = torch.zeros(t, d, dtype=torch.float32)
    for ti in range(t):
        for s in range(k):
            slot = int(route[ti, s])
            if slot < 0:
                continue
            e = int(idx[ti, s])
            r = e // e_local
            le, pos = slot // (world * capacity), slot % (world * capacity)
            out[ti] += float(wts[ti, s]) * expert_out[r][le, pos].float()
    return out


class GuardedCapacityRouter:
    """Capacity-limited routing with the overflow guard in the loop, as the reference wires it
    (crates/rmlx-distributed/src/moe_exchange.rs:556-576 with sparse_guard.rs:80-129): every
    dispatch reports its dropped pairs to a ``SparseGuard``; when the windowed overflow ratio
    crosses the guard's first threshold the capacity factor grows (x1.5, bounded), past the second
    the router stops dropping (capacity = every pair, the dense fallback), and a window below both
    puts the configured factor back. The capacity-free exchange of this framework never drops;
    this class is for callers that want the reference's fixed-shape buffers."""

    def __init__(self, num_experts: int, world: int, src_rank: int, capacity_factor: float = 1.0,
                 guard=None, max_factor: float = 8.0):
        from .moe_policy import SparseGuard
        if num_experts % world:
            raise ValueError("num_experts must divide by the expert-parallel size")
        self.E, self.world, self.src_rank = num_experts, world, src_rank
        self.base_factor = self.factor = float(capacity_factor)
        self.max_factor = float(max_factor)
        self.guard = guard or SparseGuard()
        self.dense = False
        self.total_overflow = 0
        self.increases = self.dense_fallbacks = self.resets = 0

    def capacity(self, num_tokens: int, top_k: int) -> int:
        if self.dense:
            return num_tokens * top_k                    # room for every pair on one expert
        return expert_capacity(num_tokens, top_k, self.E, self.factor)

    def dispatch(self, x: torch.Tensor, idx: torch.Tensor):
        """(buffers, route_indices, overflow, capacity) of this step; then the guard's verdict on
        the step adjusts the capacity of the next ones."""
        from .moe_policy import GuardAction
        t, k = idx.shape
        cap = self.capacity(t, k)
        factor = cap * self.E / max(1, t * k)            # the factor that yields exactly this capacity
        bufs, route, overflow = dispatch_with_capacity(x, idx, self.E, self.world, self.src_rank, factor)
        assert bufs[0].shape[1] == cap
        self.total_overflow += overflow
        action = self.guard.record_step(overflow, t * k)
        if action is GuardAction.INCREASE_CAPACITY and not self.dense:
            self.factor = min(self.max_factor, self.factor * 1.5)
            self.increases += 1
        elif action is GuardAction.DENSE_FALLBACK:
            if not self.dense:
                self.dense_fallbacks += 1
            self.dense = True
        elif action is GuardAction.RESET:
            self.factor, self.dense = self.base_factor, False
            self.resets += 1
        return bufs, route, overflow, cap

    def combine(self, expert_out: List[torch.Tensor], idx: torch.Tensor, wts: torch.Tensor,
                route: torch.Tensor, capacity: int) -> torch.Tensor:
        return combine_with_layout(expert_out, idx, wts, route, self.E, self.world, self.src_rank, capacity)
