"""CUDA-graph capture cache and a host-side hazard tracker.

``GraphCache`` keeps one captured graph per key (batch bucket, shapes) with hit/miss counters and
an LRU bound: the replayable equivalent of the reference's ExecGraph + IcbCache
(crates/rmlx-metal/src/exec_graph.rs:110-401, crates/rmlx-metal/src/icb.rs:320-420; note that the
reference's "ICB replay" re-encodes recorded dispatches on the CPU every time, icb.rs:106-168,
whereas a CUDA graph replays with no per-kernel host work).

``HazardTracker`` is the analogue of ``BarrierTracker`` (crates/rmlx-metal/src/command.rs:130-311):
given the address ranges an operation reads and writes and the stream it runs on, it reports the
RAW / WAW / WAR dependencies on operations still in flight on other streams, i.e. where an event
wait is required. ``serialize=True`` turns every dependency check into "always wait", the switch
used to bisect suspected races (the reference's ``tracked_hazards`` feature)."""
from __future__ import annotations

import gc
from collections import OrderedDict
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Callable, Hashable, List, Optional, Tuple

import torch


@contextmanager
def _no_cyclic_gc():
    """No automatic garbage collection while a stream is recording: a collection that happens to
    run inside the recording may finalise an object whose destructor makes a CUDA call that is not
    allowed during stream capture (another engine's graph being destroyed, a mapped region being
    released), which invalidates the recording. Garbage is collected first, outside it."""
    was_enabled = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        yield
    finally:
        if was_enabled:
            gc.enable()


class GraphCache:
    """``native=True``: graphs are recorded, kept and replayed by the native store
    (csrc/runtime/graph_exec.cu through ``runtime.native_graph.NativeGraphStore``) instead of
    ``torch.cuda.CUDAGraph``. A natively recorded function must not allocate; the warm-up run is
    watched, and a function whose warm-up asked torch's allocator for memory is captured through
    torch instead (``native_refused`` counts those)."""

    def __init__(self, max_entries: int = 64, native: bool = False):
        self.max_entries = max_entries
        self._g: "OrderedDict[Hashable, object]" = OrderedDict()
        self.hits = 0
        self.misses = 0
        self.captures = 0
        self.native = native
        self.native_captures = 0
        self.native_refused = 0
        self.capture_failures = 0      # recordings that were invalidated and tried again
        self.eager_fallbacks = 0       # keys that run launch by launch because recording kept failing
        self._store = None

    def __len__(self) -> int:
        return len(self._g)

    def get_or_capture(self, key: Hashable, fn: Callable[[], None], warmup: int = 1,
                       restore: Optional[Callable[[], None]] = None, device=None):
        """Returns a replayable object for ``fn`` (a CUDA graph; on CPU, ``fn`` itself).
        ``restore`` is called after the warm-up runs and after the capture: it puts back whatever
        state ``fn`` advances (a decode step moves its own positions), so that capturing leaves no
        trace."""
        g = self._g.get(key)
        if g is not None:
            self._g.move_to_end(key)
            self.hits += 1
            return g
        self.misses += 1
        g = self._capture(fn, warmup, restore, device, key)
        self._g[key] = g
        if len(self._g) > self.max_entries:
            _, old = self._g.popitem(last=False)
            if isinstance(old, _NativeReplay):
                old.drop()
        return g

    def _capture(self, fn, warmup, restore=None, device=None, key=None):
        self.captures += 1
        if not torch.cuda.is_available():
            return _HostReplay(fn)
        from ..utils.metrics import PERF
        PERF.add("graph_captures")
        s = torch.cuda.Stream(device=device)
        s.wait_stream(torch.cuda.current_stream(device))
        allocs0 = torch.cuda.memory_stats(device).get("allocation.all.allocated", 0)
        with torch.cuda.stream(s):
            for _ in range(max(warmup, 1) if self.native else warmup):
                fn()
        allocated = torch.cuda.memory_stats(device).get("allocation.all.allocated", 0) - allocs0
        torch.cuda.current_stream(device).wait_stream(s)
        torch.cuda.synchronize(device)
        if restore is not None:
            restore()
        if self.native:
            if allocated == 0:
                g = self._capture_native(fn, restore, device, key)
                if g is not None:
                    return g
            else:
                self.native_refused += 1
        # A recording can still be invalidated from outside (another thread's call): try once more
        # on another stream, then run launch by launch rather than fail.
        for _ in range(2):
            g = torch.cuda.CUDAGraph()
            try:
                with _no_cyclic_gc(), torch.cuda.graph(g, stream=s):
                    fn()
            except Exception as e:                       # noqa: BLE001
                if "captur" not in str(e).lower():
                    raise
                self.capture_failures += 1
                del g
                torch.cuda.synchronize(device)
                if restore is not None:
                    restore()
                s = torch.cuda.Stream(device=device)
                continue
            if restore is not None:
                restore()
            torch.cuda.synchronize(device)
            return g
        self.eager_fallbacks += 1
        return _HostReplay(fn)

    def _capture_native(self, fn, restore, device, key):
        from .. import _lib
        from .native_graph import NativeGraphStore
        if self._store is None:
            # the store's own bound is one above this cache's: eviction is decided here
            self._store = NativeGraphStore(self.max_entries + 1)
        try:
            with _no_cyclic_gc():
                self._store.capture(key, fn)
        except _lib.NativeError as e:
            if "captur" not in str(e).lower():
                raise
            self.capture_failures += 1
            torch.cuda.synchronize(device)
            if restore is not None:
                restore()
            return None
        if restore is not None:
            restore()
        torch.cuda.synchronize(device)
        self.native_captures += 1
        return _NativeReplay(self._store, key)

    def invalidate(self, key: Optional[Hashable] = None) -> None:
        dropped = list(self._g.values()) if key is None else [self._g.get(key)]
        for g in dropped:
            if isinstance(g, _NativeReplay):
                g.drop()
        if key is None:
            self._g.clear()
        else:
            self._g.pop(key, None)


class _NativeReplay:
    """Replays a graph of the native store on the current stream."""

    def __init__(self, store, key):
        self._store, self._key = store, key

    def replay(self):
        self._store.launch(self._key)

    def drop(self):
        self._store.invalidate(self._key)


class _HostReplay:
    def __init__(self, fn):
        self._fn = fn

    def replay(self):
        self._fn()


def bucket_for(batch: int, buckets=(1, 2, 4, 8, 16, 32, 64)) -> int:
    """Smallest capture bucket that holds ``batch`` rows."""
    for b in buckets:
        if batch <= b:
            return b
    raise ValueError(f"batch {batch} exceeds the largest bucket {buckets[-1]}")


@dataclass
class _Op:
    op_id: int
    stream: str
    reads: List[Tuple[int, int]]
    writes: List[Tuple[int, int]]


def _overlap(a: Tuple[int, int], b: Tuple[int, int]) -> bool:
    return a[0] < b[1] and b[0] < a[1]


class HazardTracker:
    def __init__(self, serialize: bool = False):
        self.serialize = serialize
        self._inflight: List[_Op] = []
        self._next = 0

    def submit(self, stream: str, reads=(), writes=(), temporaries=()) -> List[Tuple[int, str]]:
        """Register an op; returns [(op_id, kind)] it must wait for, kind in RAW / WAW / WAR.
        ``temporaries`` are ranges private to the op (exempt from tracking)."""
        tmp = list(temporaries)
        rd = [r for r in reads if not any(_overlap(r, t) for t in tmp)]
        wr = [w for w in writes if not any(_overlap(w, t) for t in tmp)]
        deps: List[Tuple[int, str]] = []
        for o in self._inflight:
            if o.stream == stream and not self.serialize:
                continue               # same stream: ordered by the stream itself
            if self.serialize:
                deps.append((o.op_id, "SERIAL"))
                continue
            if any(_overlap(r, w) for r in rd for w in o.writes):
                deps.append((o.op_id, "RAW"))
            elif any(_overlap(w, w2) for w in wr for w2 in o.writes):
                deps.append((o.op_id, "WAW"))
            elif any(_overlap(w, r) for w in wr for r in o.reads):
                deps.append((o.op_id, "WAR"))
        op = _Op(self._next, stream, rd, wr)
        self._next += 1
        self._inflight.append(op)
        return deps

    def add_writes(self, op_id: int, writes) -> None:
        """Ranges an in-flight operation turned out to write (its freshly allocated results)."""
        for o in self._inflight:
            if o.op_id == op_id:
                o.writes.extend(writes)

    def last_id(self) -> int:
        """Id of the operation submitted last."""
        return self._next - 1

    def retire(self, op_id: int) -> None:
        self._inflight = [o for o in self._inflight if o.op_id != op_id]

    def retire_stream(self, stream: str) -> None:
        self._inflight = [o for o in self._inflight if o.stream != stream]

    def retire_all(self) -> None:
        """Everything submitted so far has completed (a device synchronisation)."""
        self._inflight = []

    def in_flight(self) -> int:
        return len(self._inflight)


# Process-wide tracker: the multi-stream schedules (runtime.streams.StreamManager.submit) register
# their operations here; RMLX_DEBUG_SERIALIZE=1 makes every dependency check answer "wait".
import os as _os
HAZARDS = HazardTracker(serialize=_os.environ.get("RMLX_DEBUG_SERIALIZE", "0") == "1")
