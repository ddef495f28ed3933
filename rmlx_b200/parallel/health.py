"""Peer liveness among host processes: ``HeartbeatSender`` publishes a counter per rank in a
key-value store (``torch.distributed`` TCPStore, or any object with ``set`` / ``get``);
``HealthMonitor`` tracks last-seen times and missed beats and reports peers that exceeded the
timeout or the miss budget. Parameters as in crates/rmlx-distributed/src/health.rs:8-130 (interval
1 s, timeout 5 s, 3 misses). The reference implements these but never wires them into its init
(crates/rmlx-distributed/src/init.rs:522-538); ``Watchdog`` here is the wiring: a thread that
sends, checks, and calls ``on_failure`` so that the step loop can stop launching before the next
collective. Detection is entirely on the host; nothing on a GPU is made to fault or hang."""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional


@dataclass
class HeartbeatConfig:
    interval_s: float = 1.0
    timeout_s: float = 5.0
    max_missed: int = 3


class DictStore:
    """In-process stand-in for a TCPStore (tests, single process)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, k: str, v) -> None:
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        with self._lock:
            return self._d.get(k, b"")


class HeartbeatSender:
    def __init__(self, store, rank: int):
        self.store, self.rank, self.count = store, rank, 0

    def beat(self) -> int:
        self.count += 1
        self.store.set(f"hb/{self.rank}", str(self.count))
        return self.count


class HealthMonitor:
    def __init__(self, store, rank: int, world: int, cfg: Optional[HeartbeatConfig] = None,
                 clock: Callable[[], float] = time.monotonic):
        self.store, self.rank, self.world = store, rank, world
        self.cfg = cfg or HeartbeatConfig()
        self.clock = clock
        now = clock()
        self.last_count = {r: 0 for r in range(world) if r != rank}
        self.last_seen = {r: now for r in self.last_count}
        self.missed = {r: 0 for r in self.last_count}

    def poll(self) -> None:
        """Read every peer's counter once; a counter that did not move is one missed beat."""
        now = self.clock()
        for r in self.last_count:
            try:
                raw = self.store.get(f"hb/{r}")
                c = int(raw.decode() or 0) if raw else 0
            except Exception:
                c = self.last_count[r]
            if c > self.last_count[r]:
                self.last_count[r], self.last_seen[r], self.missed[r] = c, now, 0
            else:
                self.missed[r] += 1

    def failed_peers(self) -> List[int]:
        now = self.clock()
        return [r for r in self.last_count
                if self.missed[r] >= self.cfg.max_missed or now - self.last_seen[r] > self.cfg.timeout_s]

    def healthy(self) -> bool:
        return not self.failed_peers()


class Watchdog:
    """Background sender + monitor. ``ok()`` is what a step loop checks before each launch."""

    def __init__(self, store, rank: int, world: int, cfg: Optional[HeartbeatConfig] = None,
                 on_failure: Optional[Callable[[List[int]], None]] = None):
        self.cfg = cfg or HeartbeatConfig()
        self.sender = HeartbeatSender(store, rank)
        self.monitor = HealthMonitor(store, rank, world, self.cfg)
        self.on_failure = on_failure
        self._stop = threading.Event()
        self._failed: List[int] = []
        self._t: Optional[threading.Thread] = None

    def start(self) -> None:
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self) -> None:
        while not self._stop.wait(self.cfg.interval_s):
            self.sender.beat()
            self.monitor.poll()
            bad = self.monitor.failed_peers()
            if bad and not self._failed:
                self._failed = bad
                if self.on_failure:
                    self.on_failure(bad)

    def ok(self) -> bool:
        return not self._failed

    def failed(self) -> List[int]:
        return list(self._failed)

    def stop(self) -> None:
        self._stop.set()
        if self._t:
            self._t.join(timeout=2 * self.cfg.interval_s + 1)


class ProgressTracker:
    """Bulk polling of pending asynchronous operations with an error budget.

    An operation is anything with a non-blocking ``poll() -> bool`` (done or not) that may raise,
    e.g. ``runtime.streams.GpuEvent.query`` wrapped in a lambda, or a status-word check of a fused
    kernel. Completed operations leave the pending set; an exception counts as a poll error, and
    ``max_consecutive_errors`` (5) errors in a row with no success in between raise the health
    warning flag, which a step loop or the ``Watchdog`` callback can act on. Follows
    crates/rmlx-distributed/src/progress_tracker.rs:19,38-275 (consecutive-error threshold, bulk
    poll / wait helpers) with GPU events in place of RDMA completion queues."""

    def __init__(self, max_consecutive_errors: int = 5, clock: Callable[[], float] = time.monotonic):
        self.max_consecutive_errors = max_consecutive_errors
        self._clock = clock
        self._pending: Dict[int, Callable[[], bool]] = {}
        self._names: Dict[int, str] = {}
        self._next = 0
        self._lock = threading.Lock()
        self.consecutive_errors = 0
        self.total_errors = 0
        self.completed = 0
        self.health_warning = False
        self.last_error: Optional[str] = None

    def track(self, poll: Callable[[], bool], name: str = "") -> int:
        """Register a pending operation; returns its id."""
        with self._lock:
            oid = self._next
            self._next += 1
            self._pending[oid] = poll
            self._names[oid] = name or f"op{oid}"
            return oid

    def num_pending(self) -> int:
        return len(self._pending)

    def poll(self) -> List[int]:
        """Poll every pending operation once. Returns the ids that completed in this pass."""
        with self._lock:
            items = list(self._pending.items())
        done: List[int] = []
        for oid, fn in items:
            try:
                finished = bool(fn())
            except Exception as e:                      # noqa: BLE001 - any failure of a poll counts
                self.total_errors += 1
                self.consecutive_errors += 1
                self.last_error = f"{self._names.get(oid, oid)}: {e}"
                if self.consecutive_errors >= self.max_consecutive_errors:
                    self.health_warning = True
                continue
            self.consecutive_errors = 0
            if finished:
                done.append(oid)
        with self._lock:
            for oid in done:
                self._pending.pop(oid, None)
                self._names.pop(oid, None)
        self.completed += len(done)
        return done

    def wait_all(self, timeout_s: float = 5.0, interval_s: float = 0.0005) -> bool:
        """Poll until nothing is pending, the timeout passes, or the health warning is raised."""
        deadline = self._clock() + timeout_s
        while self._pending:
            self.poll()
            if not self._pending:
                break
            if self.health_warning or self._clock() >= deadline:
                return False
            time.sleep(interval_s)
        return True

    def reset_health(self) -> None:
        self.consecutive_errors = 0
        self.health_warning = False
        self.last_error = None
