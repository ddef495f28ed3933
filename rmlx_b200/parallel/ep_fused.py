"""Expert-parallel dispatch / combine by this package's peer-memory kernels
(csrc/comm/ep_dispatch.cu), and the expert-parallel MoE block built on them: router -> dispatch
(rows land grouped by local expert in this rank's slab) -> grouped tensor-core expert FFN on the
slab -> combine (rows return to their source, weighted sum + residual there).

``parallel.ep.EpExchange`` is the same exchange on library collectives (NCCL / gloo): the oracle and
the baseline. Reference counterpart: ``MoeDispatchExchange`` / ``MoeCombineExchange``
(crates/rmlx-distributed/src/moe_exchange.rs:519-581, 1102-1195, 2288-2330).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import _lib
from ..ops import decode as D
from ..ops.gemm import GemmStatus
from ..ops.grouped import grouped_expert_ffn
from ..ops.weights import LinearWeight
from .comm import SymmetricRegion
from .tp_gemm import _RawCuda, _align

_lib.register_cuda_sigs({
    "rmlx_ep_ctl_words": ("ii", "i"),
    "rmlx_ep_dispatch": ("ppppiipippiiiiippipp", "i"),
    "rmlx_ep_combine": ("ppppiipppppipiiiiipp", "i"),
})


class FusedEpExchange:
    """Peer-mapped slabs for up to ``max_tokens`` local tokens x ``top_k`` and ``capacity_rows``
    inbound rows per rank (default: twice the number of local pairs, at least 1024)."""

    def __init__(self, max_tokens: int, hidden: int, top_k: int, num_experts: int,
                 capacity_rows: Optional[int] = None, group=None, device=None, blocks: int = 128):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        if num_experts % self.world:
            raise ValueError("num_experts must divide by the expert-parallel size")
        self.E, self.e_local = num_experts, num_experts // self.world
        self.D, self.k, self.max_tokens = hidden, top_k, max_tokens
        self.max_pairs = max_tokens * top_k
        self.capacity = capacity_rows or max(1024, 2 * self.max_pairs)
        self.blocks = blocks
        words = int(_lib.cuda().rmlx_ep_ctl_words(self.world, self.E))
        ctl_bytes = _align(words * 4)
        self.off_ctl, self.off_ctl2 = 0, ctl_bytes
        self.off_meta = 2 * ctl_bytes
        self.off_slab = self.off_meta + _align(self.capacity * 4)
        self.off_ret = self.off_slab + _align(self.capacity * hidden * 2)
        total = self.off_ret + _align(self.max_pairs * hidden * 2)
        self.region = SymmetricRegion(total, group)
        rg = self.region
        self._ctl, self._slab = rg.peer_array(self.off_ctl), rg.peer_array(self.off_slab)
        self._meta, self._ret = rg.peer_array(self.off_meta), rg.peer_array(self.off_ret)
        self.slab = torch.as_tensor(_RawCuda(rg.local + self.off_slab, self.capacity * hidden * 2),
                                    device=self.device).view(torch.bfloat16).view(self.capacity, hidden)
        self.recv_offsets = torch.zeros(self.e_local + 1, dtype=torch.int32, device=self.device)
        self.recv_rows = torch.zeros(1, dtype=torch.int32, device=self.device)

    def _blocks_for(self, tokens: int) -> int:
        """Few blocks for few rows (ranks publish one arrival each, so grids may differ per rank)."""
        return max(8, min(self.blocks, (tokens * self.k + 15) // 16))

    def dispatch(self, x: torch.Tensor, idx: torch.Tensor, counts: torch.Tensor
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
        """x [T, D] bf16, idx [T, k] int32 (global expert ids), counts [E] int32 (the router's).
        Returns (slab, offsets): inbound rows grouped by local expert, offsets int32 [E_local+1]."""
        t, k = idx.shape
        assert t <= self.max_tokens and k == self.k and x.shape[1] == self.D and x.stride(1) == 1
        assert idx.dtype == torch.int32 and counts.dtype == torch.int32 and idx.is_contiguous()
        rc = _lib.cuda().rmlx_ep_dispatch(
            self._ctl, self._slab, self._meta, self._ret, self.rank, self.world, x.data_ptr(),
            x.stride(0), idx.data_ptr(), counts.data_ptr(), t, k, self.D, self.E, self.capacity,
            self.recv_offsets.data_ptr(), self.recv_rows.data_ptr(), self._blocks_for(t),
            GemmStatus.get(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ep_dispatch")
        return self.slab, self.recv_offsets

    def combine(self, y: torch.Tensor, wts: torch.Tensor, num_tokens: int,
                residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """y: expert outputs in slab order [>= rows, D] bf16; wts [T, k] fp32. -> [T, D] bf16."""
        assert y.dtype == torch.bfloat16 and y.stride(1) == 1 and y.stride(0) == self.D
        assert wts.dtype == torch.float32 and wts.is_contiguous()
        if out is None:
            out = torch.empty(num_tokens, self.D, dtype=torch.bfloat16, device=self.device)
        rc = _lib.cuda().rmlx_ep_combine(
            self._ctl, self._slab, self._meta, self._ret, self.rank, self.world,
            ctypes.c_void_p(self.region.local + self.off_ctl2), y.data_ptr(), self.recv_rows.data_ptr(),
            wts.data_ptr(), _lib.ptr(residual), 0 if residual is None else residual.stride(0),
            out.data_ptr(), out.stride(0), num_tokens, self.k, self.D, self._blocks_for(num_tokens),
            GemmStatus.get(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ep_combine")
        return out

    def status(self) -> int:
        return int(GemmStatus.get(self.device).item())

    def close(self) -> None:
        self.slab = None
        self.region.close()


class FusedEpMoe:
    """Expert-parallel MoE feed-forward over one rank's local experts."""

    def __init__(self, exchange: FusedEpExchange, gate_up: LinearWeight, down: LinearWeight):
        assert gate_up.experts == exchange.e_local
        self.ex, self.gate_up, self.down = exchange, gate_up, down
        from ..runtime.graph import GraphCache
        self.graphs = GraphCache(max_entries=16)
        self._static = {}

    @torch.no_grad()
    def forward(self, x: torch.Tensor, router_w: torch.Tensor, top_k: int,
                expert_bias: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [T, D] bf16 (already normalised); router_w [E, D]. Returns [T, D] bf16 (+ residual)."""
        logits = x.float() @ router_w.float().t()
        idx, wts, counts, _ = D.topk_route(logits, top_k, expert_bias)
        slab, offsets = self.ex.dispatch(x, idx, counts)
        rows = int(self.ex.capacity)            # the grouped kernel only touches rows below offsets[-1]
        y = grouped_expert_ffn(slab[:rows], offsets, self.gate_up, self.down)
        return self.ex.combine(y, wts, x.shape[0], residual)

    @torch.no_grad()
    def forward_captured(self, x: torch.Tensor, router_w: torch.Tensor, top_k: int,
                         expert_bias: Optional[torch.Tensor] = None,
                         residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``forward`` as ONE CUDA-graph replay per token count: router, dispatch, grouped expert
        FFN and combine are captured together (the exchange keeps its epochs on the device, so a
        replay needs nothing from the host), which removes the launches and allocations from
        Python between the phases. Collective: every rank calls it with the same token count, the
        first call per count captures (one eager warm-up run, then the capture). The result is a
        buffer owned by the graph, valid until the next call with the same token count.
        Counterpart of the reference's asynchronous exchange-and-compute chain
        (crates/rmlx-nn/src/moe.rs:786-1008)."""
        t = x.shape[0]
        key = (t, top_k, residual is not None)
        st = self._static.get(key)
        if st is None:
            # everything the graph reads lives in buffers the graph's owner keeps: activations and
            # residual are copied in per call; the router matrix and the bias are kept by reference
            # when the caller passes the same tensors again (model parameters) and copied otherwise
            st = {"x": torch.empty_like(x), "res": None if residual is None else torch.empty_like(residual),
                  "out": torch.empty(t, self.ex.D, dtype=torch.bfloat16, device=x.device),
                  "router": router_w, "bias": expert_bias}
            self._static[key] = st

        def body():
            st["out"].copy_(self.forward(st["x"], st["router"], top_k, st["bias"], st["res"]))

        st["x"].copy_(x)
        if residual is not None:
            st["res"].copy_(residual)
        if router_w is not st["router"]:
            st["router"].copy_(router_w)
        if expert_bias is not None and expert_bias is not st["bias"]:
            st["bias"].copy_(expert_bias)
        self.graphs.get_or_capture(key, body, warmup=1, device=x.device).replay()
        return st["out"]
