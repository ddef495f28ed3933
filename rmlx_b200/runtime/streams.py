"""Streams, events and fences with bounded host waits.

``GpuEvent`` wraps a CUDA event with a monotonically increasing signal counter; ``cpu_wait`` polls
``query()`` with spin -> yield -> sleep back-off until a deadline or a cancel flag, and never
blocks without a bound (crates/rmlx-metal/src/event.rs:15-117). ``GpuFence`` orders two streams
(crates/rmlx-metal/src/fence.rs:24-130). ``StreamManager`` owns the named streams
default / compute / copy and the cross-stream synchronisation helpers
(crates/rmlx-metal/src/stream.rs:56-330). On a machine without a GPU the classes run in a host
emulation (work is considered complete immediately) so the control logic stays testable.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, Optional

import torch

STREAM_DEFAULT, STREAM_COMPUTE, STREAM_COPY = "default", "compute", "copy"


class WaitTimeout(TimeoutError):
    pass


class WaitCancelled(RuntimeError):
    pass


class GpuEvent:
    def __init__(self, device=None):
        self._cuda = torch.cuda.is_available()
        self._ev = torch.cuda.Event() if self._cuda else None
        self._signalled = 0      # value the next/last record carries
        self._cancel = threading.Event()
        self._host_done = True

    def record(self, stream=None) -> int:
        self._signalled += 1
        if self._cuda:
            self._ev.record(stream or torch.cuda.current_stream())
        return self._signalled

    def query(self) -> bool:
        return self._ev.query() if self._cuda else self._host_done

    def cancel(self) -> None:
        self._cancel.set()

    def cpu_wait(self, timeout_s: float = 5.0) -> None:
        """Spin briefly, then yield, then sleep; raises WaitTimeout / WaitCancelled."""
        deadline = time.monotonic() + timeout_s
        spins = 0
        while not self.query():
            if self._cancel.is_set():
                raise WaitCancelled("event wait cancelled")
            if time.monotonic() >= deadline:
                raise WaitTimeout(f"event not signalled within {timeout_s}s")
            spins += 1
            if spins < 200:
                continue
            time.sleep(0 if spins < 2000 else 0.0002)

    def stream_wait(self, stream) -> None:
        if self._cuda:
            stream.wait_event(self._ev)


class GpuFence:
    """Make ``waiter`` stream wait for everything submitted so far on ``signaller``."""

    def __init__(self):
        self.event = GpuEvent()

    def signal(self, signaller=None) -> int:
        return self.event.record(signaller)

    def wait(self, waiter) -> None:
        self.event.stream_wait(waiter)

    def cpu_wait(self, timeout_s: float = 5.0) -> None:
        self.event.cpu_wait(timeout_s)


class StreamManager:
    def __init__(self, device=None, names=(STREAM_DEFAULT, STREAM_COMPUTE, STREAM_COPY)):
        self._cuda = torch.cuda.is_available()
        self._events: Dict[int, "torch.cuda.Event"] = {}
        self.waits_inserted = 0
        self.streams: Dict[str, Optional[torch.cuda.Stream]] = {}
        for n in names:
            if not self._cuda:
                self.streams[n] = None
            elif n == STREAM_DEFAULT:
                self.streams[n] = torch.cuda.current_stream(device)
            else:
                self.streams[n] = torch.cuda.Stream(device)

    def get(self, name: str):
        return self.streams[name]

    def submit(self, name: str, fn, reads=(), writes=(), temporaries=()):
        """Run ``fn`` on stream ``name`` after the operations still in flight on OTHER streams
        that it depends on: ``reads`` / ``writes`` are the tensors (or (address, end) ranges) it
        touches, and the process-wide hazard tracker (runtime.graph.HAZARDS) names the RAW / WAW /
        WAR predecessors whose completion events the stream then waits for. Work on one stream
        needs no event. With RMLX_DEBUG_SERIALIZE=1 the tracker reports every in-flight operation
        as a dependency, which serialises the schedule (crates/rmlx-metal/src/command.rs:130-311,
        the ``tracked_hazards`` switch of device.rs:23-32). Returns (op id, fn's result)."""
        from .graph import HAZARDS

        def ranges(items):
            out = []
            for t in items:
                if isinstance(t, torch.Tensor):
                    a = t.data_ptr()
                    out.append((a, a + max(1, t.numel() * t.element_size())))
                else:
                    out.append((int(t[0]), int(t[1])))
            return out

        deps = HAZARDS.submit(name, ranges(reads), ranges(writes), ranges(temporaries))
        op_id = HAZARDS.last_id()
        stream = self.streams[name]
        for dep, _kind in deps:
            ev = self._events.get(dep)
            if ev is not None and self._cuda:
                stream.wait_event(ev)
        self.waits_inserted += len(deps)
        if self._cuda:
            with torch.cuda.stream(stream):
                result = fn()
            ev = torch.cuda.Event()
            ev.record(stream)
            self._events[op_id] = ev
            # tensors the operation returns are its writes too (they did not exist before it ran)
            outs = [result] if isinstance(result, torch.Tensor) else \
                [r for r in result if isinstance(r, torch.Tensor)] if isinstance(result, (list, tuple)) else []
            HAZARDS.add_writes(op_id, ranges(outs))
        else:
            result = fn()
            HAZARDS.retire(op_id)      # host execution is synchronous
        return op_id, result

    def reap(self) -> int:
        """Retire the submitted operations whose events have completed; returns how many remain."""
        from .graph import HAZARDS
        for op_id in [k for k, ev in self._events.items() if ev.query()]:
            HAZARDS.retire(op_id)
            del self._events[op_id]
        return len(self._events)

    def order(self, before: str, after: str) -> GpuFence:
        """Everything queued on ``before`` happens before later work on ``after``."""
        f = GpuFence()
        f.signal(self.streams[before])
        if self._cuda:
            f.wait(self.streams[after])
        return f

    def compute_to_copy(self) -> GpuFence:
        return self.order(STREAM_COMPUTE, STREAM_COPY)

    def copy_to_compute(self) -> GpuFence:
        return self.order(STREAM_COPY, STREAM_COMPUTE)

    def synchronize(self, timeout_s: float = 30.0) -> None:
        for n, s in self.streams.items():
            ev = GpuEvent()
            ev.record(s)
            ev.cpu_wait(timeout_s)


class GpuErrorStore:
    """Collects what kernels report through their status words.

    Kernels of this package never trap: a bounded wait that gives up, or a failed argument check,
    writes a code into a device word and returns. Components register those words here (a one-element
    int32 tensor, or a callable returning the code); ``collect()`` reads them all, records every
    non-zero code with the source's name, clears the words and returns the new records. The
    counterpart of the reference's per-queue ``GpuErrorStore`` fed by command-buffer completion
    handlers (crates/rmlx-metal/src/command.rs:325-399)."""

    CODES = {1: "pipeline wait timed out", 2: "peer wait timed out", 3: "bad argument"}

    def __init__(self, max_records: int = 256):
        self._sources = {}
        self._records = []
        self.max_records = max_records

    def register(self, name: str, source) -> None:
        """``source``: an int32 tensor of one element (device or host), or ``() -> int``."""
        self._sources[name] = source

    def unregister(self, name: str) -> None:
        self._sources.pop(name, None)

    def collect(self):
        """Read and clear every registered word. Returns the list of new (name, code, meaning)."""
        new = []
        for name, src in self._sources.items():
            if callable(src):
                code = int(src())
            else:
                code = int(src.item())
                if code:
                    src.zero_()
            if code:
                new.append((name, code, self.CODES.get(code, "unknown status")))
        self._records = (self._records + new)[-self.max_records:]
        return new

    def records(self):
        return list(self._records)

    def has_errors(self) -> bool:
        return bool(self._records)

    def clear(self) -> None:
        self._records = []

    def raise_if_any(self) -> None:
        new = self.collect()
        if new:
            raise RuntimeError("; ".join(f"{n}: {m} (status {c})" for n, c, m in new))


# Process-wide store: components that own a status word register it here when they create it.
ERRORS = GpuErrorStore()
