"""Overlap schedules for the MoE block: shared-expert overlap (SBO) and token-batch overlap (TBO).

SBO runs the always-on shared expert on a side stream while the routed path (route -> exchange ->
grouped experts -> combine) runs on the main stream; TBO splits the tokens into two micro-batches
so that one half's expert compute overlaps the other half's exchange. Streams are chained with
events and the host waits once at the end, as in crates/rmlx-nn/src/moe_pipeline.rs:45-500 (GpuEvent
chains, one CPU wait). On CPU tensors the same schedule runs sequentially, which makes the results
checkable against ``MoeLayer.forward`` bit for bit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..reference import ops as ref
from .moe import MoeLayer


@dataclass
class OverlapStats:
    micro_batches: int = 1
    used_side_stream: bool = False
    shared_tokens: int = 0
    routed_tokens: int = 0


class MoePipeline:
    def __init__(self, layer: MoeLayer, side_stream: Optional["torch.cuda.Stream"] = None):
        self.layer = layer
        self._side = side_stream
        self.stats = OverlapStats()

    def _side_stream(self, x: torch.Tensor):
        if not x.is_cuda:
            return None
        if self._side is None:
            self._side = torch.cuda.Stream(x.device)
        return self._side

    def _shared(self, x: torch.Tensor) -> torch.Tensor:
        gu, dn = self.layer.shared
        a = ref.swiglu(x @ gu.dequantized().to(x.dtype).t())
        return (a @ dn.dequantized().to(x.dtype).t()).float()

    def _routed(self, x: torch.Tensor) -> torch.Tensor:
        shared, self.layer.shared = self.layer.shared, None
        try:
            return self.layer.forward(x).float()
        finally:
            self.layer.shared = shared

    # ------------------------------------------------------------------ SBO
    def forward_sbo(self, x: torch.Tensor) -> torch.Tensor:
        """Shared expert on the side stream, routed experts on the current stream, one join."""
        if self.layer.shared is None:
            return self.layer.forward(x)
        side = self._side_stream(x)
        self.stats = OverlapStats(1, side is not None, x.shape[0], x.shape[0])
        if side is None:
            return (self._routed(x) + self._shared(x)).to(x.dtype)
        main = torch.cuda.current_stream(x.device)
        side.wait_stream(main)                    # x is ready
        with torch.cuda.stream(side):
            s = self._shared(x)
        r = self._routed(x)
        main.wait_stream(side)                    # join: the sum needs both
        s.record_stream(main)
        return (r + s).to(x.dtype)

    # ------------------------------------------------------------------ TBO
    def forward_tbo(self, x: torch.Tensor, micro_batches: int = 2) -> torch.Tensor:
        """Token micro-batches alternate between the two streams, so that one micro-batch's
        exchange overlaps the other's expert compute. Rows are independent, so the result equals
        the un-split forward."""
        t = x.shape[0]
        n = max(1, min(micro_batches, t))
        bounds = [t * i // n for i in range(n + 1)]
        side = self._side_stream(x)
        self.stats = OverlapStats(n, side is not None and n > 1, t if self.layer.shared else 0, t)
        outs = []
        if side is None or n == 1:
            for i in range(n):
                outs.append(self.layer.forward(x[bounds[i]:bounds[i + 1]]))
            return torch.cat(outs, 0)
        main = torch.cuda.current_stream(x.device)
        side.wait_stream(main)
        for i in range(n):
            chunk = x[bounds[i]:bounds[i + 1]]
            if i % 2 == 0:
                outs.append(self.layer.forward(chunk))
            else:
                with torch.cuda.stream(side):
                    o = self.layer.forward(chunk)
                o.record_stream(main)
                outs.append(o)
        main.wait_stream(side)
        return torch.cat(outs, 0)
