"""Cooperative shutdown flag shared between threads (crates/rmlx-core/src/shutdown.rs:7-52)."""
from __future__ import annotations

import threading


class ShutdownHandle:
    def __init__(self, ev: threading.Event):
        self._ev = ev

    def is_shutdown(self) -> bool:
        return self._ev.is_set()

    def wait(self, timeout: float) -> bool:
        return self._ev.wait(timeout)


class ShutdownSignal:
    def __init__(self):
        self._ev = threading.Event()

    def handle(self) -> ShutdownHandle:
        return ShutdownHandle(self._ev)

    def trigger(self) -> None:
        self._ev.set()

    def is_triggered(self) -> bool:
        return self._ev.is_set()
