"""Ring of pre-allocated exchange buffers with producer / consumer positions and bounded waits.

Shape of the reference's ``SlabRing`` (crates/rmlx-distributed/src/slab_ring.rs:48-460: depth 3 x
4 MiB, ``acquire_for_write(_timeout)``, ``produce``, ``consume(timeout)``, ``release``,
back-pressure counters). Slots here are slices of one device (or symmetric) allocation; readiness
is a CUDA event per slot, polled with a deadline, so a stalled producer or consumer surfaces as a
timeout on the host instead of a hang."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional

import torch

from ..runtime.streams import GpuEvent, WaitTimeout


@dataclass
class SlabRingConfig:
    depth: int = 3
    slab_bytes: int = 4 << 20

    def validate(self) -> "SlabRingConfig":
        if self.depth < 2 or self.slab_bytes <= 0:
            raise ValueError("slab ring needs depth >= 2 and a positive slab size")
        return self


class SlabRing:
    FREE, WRITING, READY, READING = range(4)

    def __init__(self, cfg: Optional[SlabRingConfig] = None, device="cpu"):
        self.cfg = (cfg or SlabRingConfig()).validate()
        self.buf = torch.empty(self.cfg.depth, self.cfg.slab_bytes, dtype=torch.uint8, device=device)
        self.state = [self.FREE] * self.cfg.depth
        self.events: List[GpuEvent] = [GpuEvent() for _ in range(self.cfg.depth)]
        self.head = 0           # next slot to write
        self.tail = 0           # next slot to read
        self.backpressure_events = 0
        self.produced = 0
        self.consumed = 0

    def slab(self, i: int) -> torch.Tensor:
        return self.buf[i]

    def acquire_for_write(self, timeout_s: float = 0.0) -> int:
        """Index of a free slot; waits up to ``timeout_s`` for the consumer to release one."""
        deadline = time.monotonic() + timeout_s
        while self.state[self.head] != self.FREE:
            self.backpressure_events += 1
            if time.monotonic() >= deadline:
                raise WaitTimeout("slab ring full: consumer has not released a slot")
            time.sleep(0.0001)
        i = self.head
        self.state[i] = self.WRITING
        self.head = (self.head + 1) % self.cfg.depth
        return i

    def produce(self, i: int, stream=None) -> None:
        """The writer's work on slot i is queued; record its completion."""
        assert self.state[i] == self.WRITING
        self.events[i].record(stream)
        self.state[i] = self.READY
        self.produced += 1

    def consume(self, timeout_s: float = 5.0) -> int:
        """Next ready slot in order, after its producer's work completed on the device."""
        i = self.tail
        deadline = time.monotonic() + timeout_s
        while self.state[i] != self.READY:
            if time.monotonic() >= deadline:
                raise WaitTimeout("slab ring empty: producer has not published a slot")
            time.sleep(0.0001)
        self.events[i].cpu_wait(max(0.0, deadline - time.monotonic()) + 1e-3)
        self.state[i] = self.READING
        self.tail = (self.tail + 1) % self.cfg.depth
        return i

    def release(self, i: int) -> None:
        assert self.state[i] == self.READING
        self.state[i] = self.FREE
        self.consumed += 1


class CreditManager:
    """Per-(peer, tag) window of receive credits: a sender may only have ``window`` messages of one
    kind in flight towards one peer, which is what guarantees that the receiver's slots (slabs of a
    ring, slots of a symmetric receive area) are free when the data lands. The reference pre-posts
    receive work requests for the same purpose (crates/rmlx-distributed/src/credit_manager.rs); on
    NVLink the credit is the receiver's slot itself and is returned when the consumer releases it."""

    def __init__(self, window: int = 2):
        if window < 1:
            raise ValueError("window must be >= 1")
        self.window = window
        self._in_flight = {}
        self.stalls = 0

    def available(self, peer: int, tag: int) -> int:
        return self.window - self._in_flight.get((peer, tag), 0)

    def try_acquire(self, peer: int, tag: int) -> bool:
        k = (peer, tag)
        if self._in_flight.get(k, 0) >= self.window:
            self.stalls += 1
            return False
        self._in_flight[k] = self._in_flight.get(k, 0) + 1
        return True

    def acquire(self, peer: int, tag: int, timeout_s: float = 5.0, poll=None, interval_s: float = 0.0005) -> None:
        """Wait (bounded) for a credit; ``poll`` is called between attempts to make progress on
        whatever returns credits (e.g. ``ProgressTracker.poll``)."""
        deadline = time.monotonic() + timeout_s
        while not self.try_acquire(peer, tag):
            if time.monotonic() >= deadline:
                raise WaitTimeout(f"no credit for peer {peer} tag {tag} within {timeout_s} s")
            if poll is not None:
                poll()
            time.sleep(interval_s)

    def release(self, peer: int, tag: int) -> None:
        k = (peer, tag)
        if self._in_flight.get(k, 0) <= 0:
            raise ValueError(f"credit for peer {peer} tag {tag} released twice")
        self._in_flight[k] -= 1
