"""Python face of the native execution runtime (csrc/runtime/graph_exec.cu): a keyed store of
instantiated CUDA graphs and events whose host waits have a deadline and a cancel flag.

``NativeGraphStore`` records what one thread submits to a stream between ``begin`` and ``end``,
keeps the instantiated graph under a key (LRU-bounded) and replays it with one call; it is the
native backend of ``runtime.graph.GraphCache`` (``native=True``). What is recorded must not
allocate: a graph replays the addresses it was recorded with, so buffers have to outlive it.
``NativeEvent`` / ``CancelFlag`` are the counterparts of GpuEvent's ``cpu_wait`` with deadline and
cancellation (crates/rmlx-metal/src/event.rs:15-117).
"""
from __future__ import annotations

import ctypes
from typing import Callable, Dict, Hashable, Optional

import torch

from .. import _lib

_lib.register_cuda_sigs({
    "rmlx_graphs_create": ("i", "p"),
    "rmlx_graphs_destroy": ("p", None),
    "rmlx_graphs_stream": ("p", "p"),
    "rmlx_graphs_has": ("pQ", "i"),
    "rmlx_graphs_begin": ("pp", "i"),
    "rmlx_graphs_end": ("pQp", "i"),
    "rmlx_graphs_abort": ("pp", "i"),
    "rmlx_graphs_launch": ("pQp", "i"),
    "rmlx_graphs_invalidate": ("pQi", "i"),
    "rmlx_graphs_stats": ("pp", None),
    "rmlx_event_create": ("i", "p"),
    "rmlx_event_destroy": ("p", None),
    "rmlx_event_record": ("pp", "i"),
    "rmlx_event_stream_wait": ("pp", "i"),
    "rmlx_event_wait_host": ("pqp", "i"),
    "rmlx_event_elapsed_ms": ("pp", "f"),
})


def _key64(key: Hashable) -> int:
    return hash(key) & 0xFFFFFFFFFFFFFFFF


class NativeGraphStore:
    def __init__(self, max_entries: int = 64):
        self._lib = _lib.cuda()
        self._h = self._lib.rmlx_graphs_create(int(max_entries))
        self._stream = None
        if not self._h:
            raise _lib.NativeError("graph store could not be created")

    def has(self, key: Hashable) -> bool:
        return bool(self._lib.rmlx_graphs_has(self._h, _key64(key)))

    @property
    def stream(self) -> torch.cuda.Stream:
        """The store's own recording stream (not one of torch's pooled streams)."""
        if self._stream is None:
            ptr = self._lib.rmlx_graphs_stream(self._h)
            if not ptr:
                raise _lib.NativeError("the recording stream could not be created")
            self._stream = torch.cuda.ExternalStream(ptr)
        return self._stream

    def capture(self, key: Hashable, fn: Callable[[], None], stream: Optional[torch.cuda.Stream] = None) -> int:
        """Record ``fn`` (which must submit to the current stream only and must not allocate) on
        ``stream`` (default: the store's own) and store the graph under ``key``. Work queued on
        the caller's current stream is waited for first. Returns the number of graph nodes."""
        stream = stream or self.stream
        stream.wait_stream(torch.cuda.current_stream())
        sp = stream.cuda_stream
        with torch.cuda.stream(stream):
            rc = self._lib.rmlx_graphs_begin(self._h, sp)
            if rc:
                raise _lib.NativeError(f"graph capture could not start (code {rc})")
            try:
                fn()
            except BaseException:
                self._lib.rmlx_graphs_abort(self._h, sp)
                raise
            nodes = self._lib.rmlx_graphs_end(self._h, _key64(key), sp)
        if nodes < 0:
            raise _lib.NativeError(f"graph capture failed (code {nodes})")
        return int(nodes)

    def launch(self, key: Hashable, stream: Optional[torch.cuda.Stream] = None) -> None:
        sp = _lib.stream_ptr(stream) if torch.cuda.is_available() else None     # no GPU: only the lookup runs
        rc = self._lib.rmlx_graphs_launch(self._h, _key64(key), sp)
        if rc == -3:
            raise KeyError(key)
        _lib.check(rc, "graph launch")

    def invalidate(self, key: Optional[Hashable] = None) -> int:
        return int(self._lib.rmlx_graphs_invalidate(self._h, 0 if key is None else _key64(key), int(key is None)))

    def stats(self) -> Dict[str, int]:
        out = (ctypes.c_uint64 * 7)()
        self._lib.rmlx_graphs_stats(self._h, out)
        names = ("entries", "hits", "misses", "captures", "evictions", "launches", "last_nodes")
        return {n: int(v) for n, v in zip(names, out)}

    def close(self) -> None:
        if self._h:
            self._stream = None
            self._lib.rmlx_graphs_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CancelFlag:
    """A flag another thread sets to end a host wait early."""

    def __init__(self):
        self._v = ctypes.c_int(0)

    def set(self) -> None:
        self._v.value = 1

    def clear(self) -> None:
        self._v.value = 0

    @property
    def ptr(self):
        return ctypes.byref(self._v)


class NativeEvent:
    DONE, TIMEOUT, CANCELLED = 0, 1, 2

    def __init__(self, timing: bool = False):
        self._lib = _lib.cuda()
        self._h = self._lib.rmlx_event_create(int(timing))
        if not self._h:
            raise _lib.NativeError("event could not be created")

    def record(self, stream: Optional[torch.cuda.Stream] = None) -> "NativeEvent":
        _lib.check(self._lib.rmlx_event_record(self._h, _lib.stream_ptr(stream)), "event record")
        return self

    def stream_wait(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        """``stream`` waits on the device for the work recorded before this event."""
        _lib.check(self._lib.rmlx_event_stream_wait(self._h, _lib.stream_ptr(stream)), "stream wait")

    def wait(self, timeout_s: Optional[float] = None, cancel: Optional[CancelFlag] = None) -> int:
        """Host wait. Returns DONE, TIMEOUT (the deadline passed) or CANCELLED."""
        us = -1 if timeout_s is None else int(timeout_s * 1e6)
        rc = self._lib.rmlx_event_wait_host(self._h, us, cancel.ptr if cancel is not None else None)
        if rc < 0:
            raise _lib.NativeError("the event reports a device error")
        return int(rc)

    def elapsed_ms(self, later: "NativeEvent") -> float:
        return float(self._lib.rmlx_event_elapsed_ms(self._h, later._h))

    def close(self) -> None:
        if self._h:
            self._lib.rmlx_event_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
