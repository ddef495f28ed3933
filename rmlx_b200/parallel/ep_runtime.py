"""One object that owns what an expert-parallel step needs besides the kernels: the exchange
(fused or library), a slab ring for staged payloads, the credit window per (peer, tag), the progress
tracker for pending asynchronous work, the stream manager and the MoE metrics. The shape of the
reference's ``EpRuntimeContext`` (crates/rmlx-distributed/src/ep_runtime.rs: transport +
ProgressEngine + SharedBufferPool + CreditManager + compute/transfer events, RAII
``AcquiredBuffer``); the GPU-doorbell proxy it boots has no counterpart, because here the GPU writes
to its peers directly."""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Iterator, Optional

import torch

from ..utils.metrics import MoeMetrics
from .health import ProgressTracker
from .slab_ring import CreditManager, SlabRing, SlabRingConfig


@dataclass
class AcquiredBuffer:
    """A slab held for writing; handed back to the ring by the context manager that produced it."""
    index: int
    tensor: torch.Tensor


@dataclass
class EpRuntimeContext:
    rank: int = 0
    world: int = 1
    exchange: object = None                      # FusedEpExchange, EpExchange or None (single rank)
    ring: SlabRing = field(default_factory=lambda: SlabRing(SlabRingConfig(depth=3, slab_bytes=1 << 16)))
    credits: CreditManager = field(default_factory=CreditManager)
    progress: ProgressTracker = field(default_factory=ProgressTracker)
    streams: object = None                       # runtime.streams.StreamManager on CUDA
    metrics: Optional[MoeMetrics] = None

    @contextmanager
    def staged(self, peer: int, tag: int, timeout_s: float = 5.0, stream=None) -> Iterator[AcquiredBuffer]:
        """Credit + slab for one outgoing message: the body fills ``buf.tensor`` (queues the work
        that does); on exit the slab is published and the credit stays taken until ``delivered``."""
        self.credits.acquire(peer, tag, timeout_s, poll=self.progress.poll)
        try:
            i = self.ring.acquire_for_write(timeout_s)
        except Exception:
            self.credits.release(peer, tag)
            raise
        try:
            yield AcquiredBuffer(i, self.ring.slab(i))
        except Exception:
            # nothing was published: give the slot and the credit back
            self.ring.state[i] = SlabRing.FREE
            self.ring.head = i
            self.credits.release(peer, tag)
            raise
        self.ring.produce(i, stream)

    def delivered(self, peer: int, tag: int, timeout_s: float = 5.0) -> torch.Tensor:
        """Consumer side of ``staged``: the next published slab, after its producer's work finished;
        returns a copy-free view valid until ``done``."""
        self._reading = self.ring.consume(timeout_s)
        self._reading_key = (peer, tag)
        return self.ring.slab(self._reading)

    def done(self) -> None:
        self.ring.release(self._reading)
        self.credits.release(*self._reading_key)

    def healthy(self) -> bool:
        return not self.progress.health_warning
