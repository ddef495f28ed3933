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
    """The two streams come from a ``StreamManager``; every piece of work is submitted with the
    tensors it reads and writes, and the manager's hazard tracker inserts the event waits (so
    ``RMLX_DEBUG_SERIALIZE=1`` serialises the schedule without touching this code)."""

    def __init__(self, layer: MoeLayer, streams=None):
        self.layer = layer
        self._streams = streams
        self.stats = OverlapStats()

    def _manager(self, x: torch.Tensor):
        if not x.is_cuda:
            return None
        if self._streams is None:
            from ..runtime.streams import StreamManager
            self._streams = StreamManager(x.device)
        return self._streams

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
        sm = self._manager(x)
        self.stats = OverlapStats(1, sm is not None, x.shape[0], x.shape[0])
        if sm is None:
            return (self._routed(x) + self._shared(x)).to(x.dtype)
        from ..runtime.streams import STREAM_COPY, STREAM_DEFAULT
        _, x = sm.submit(STREAM_DEFAULT, lambda: x, writes=[x])          # x is produced on the main stream
        _, s = sm.submit(STREAM_COPY, lambda: self._shared(x), reads=[x])
        _, r = sm.submit(STREAM_DEFAULT, lambda: self._routed(x), reads=[x])
        s.record_stream(sm.get(STREAM_DEFAULT))
        # the sum reads what the side stream wrote: the tracker makes the main stream wait for it
        _, out = sm.submit(STREAM_DEFAULT, lambda: (r + s).to(x.dtype), reads=[r, s])
        sm.reap()
        return out

    # ------------------------------------------------------------------ TBO
    def forward_tbo(self, x: torch.Tensor, micro_batches: int = 2) -> torch.Tensor:
        """Token micro-batches alternate between the two streams, so that one micro-batch's
        exchange overlaps the other's expert compute. Rows are independent, so the result equals
        the un-split forward."""
        t = x.shape[0]
        n = max(1, min(micro_batches, t))
        bounds = [t * i // n for i in range(n + 1)]
        sm = self._manager(x)
        self.stats = OverlapStats(n, sm is not None and n > 1, t if self.layer.shared else 0, t)
        outs = []
        if sm is None or n == 1:
            for i in range(n):
                outs.append(self.layer.forward(x[bounds[i]:bounds[i + 1]]))
            return torch.cat(outs, 0)
        from ..runtime.streams import STREAM_COPY, STREAM_DEFAULT
        _, x = sm.submit(STREAM_DEFAULT, lambda: x, writes=[x])
        for i in range(n):
            chunk = x[bounds[i]:bounds[i + 1]]
            name = STREAM_DEFAULT if i % 2 == 0 else STREAM_COPY
            _, o = sm.submit(name, lambda c=chunk: self.layer.forward(c), reads=[chunk])
            if name != STREAM_DEFAULT:
                o.record_stream(sm.get(STREAM_DEFAULT))
            outs.append(o)
        _, out = sm.submit(STREAM_DEFAULT, lambda: torch.cat(outs, 0), reads=outs)
        sm.reap()
        return out
