"""Lock-protected runtime counters with ``snapshot()``: kernel launches and time, allocation
traffic, cache hits; MoE routing metrics; transport counters. Counterparts:
crates/rmlx-core/src/metrics.rs:6-100 (``RuntimeMetrics``), crates/rmlx-distributed/src/metrics.rs:6-130
(``MoeMetrics``), crates/rmlx-rdma/src/rdma_metrics.rs:6-95, crates/rmlx-distributed/src/perf_counters.rs:8-220.
``to_prometheus`` renders a snapshot in the Prometheus text format (the reference documents
compatibility but ships no exporter)."""
from __future__ import annotations

import threading
from typing import Dict, List


class Counters:
    def __init__(self, names: List[str]):
        self._v: Dict[str, float] = {n: 0 for n in names}
        self._lock = threading.Lock()

    def add(self, name: str, amount: float = 1) -> None:
        with self._lock:
            self._v[name] = self._v.get(name, 0) + amount

    def set_max(self, name: str, value: float) -> None:
        with self._lock:
            self._v[name] = max(self._v.get(name, 0), value)

    def get(self, name: str) -> float:
        with self._lock:
            return self._v.get(name, 0)

    def snapshot(self) -> Dict[str, float]:
        with self._lock:
            return dict(self._v)

    def reset(self) -> None:
        with self._lock:
            for k in self._v:
                self._v[k] = 0


class RuntimeMetrics(Counters):
    def __init__(self):
        super().__init__(["kernel_dispatches", "kernel_time_us", "graph_launches", "graph_captures",
                          "alloc_bytes", "free_bytes", "cache_hits", "cache_misses"])

    def record_kernel(self, time_us: float = 0.0, n: int = 1) -> None:
        self.add("kernel_dispatches", n)
        self.add("kernel_time_us", time_us)


class MoeMetrics(Counters):
    def __init__(self, num_experts: int = 0):
        super().__init__(["dispatch_local", "dispatch_fused", "dispatch_nccl", "overflow_tokens",
                          "zone_switches", "tokens_routed"])
        self.per_expert = [0] * num_experts

    def record_counts(self, counts) -> None:
        with self._lock:
            for e, c in enumerate(counts):
                if e < len(self.per_expert):
                    self.per_expert[e] += int(c)
            self._v["tokens_routed"] += int(sum(int(c) for c in counts))


class TransportMetrics(Counters):
    def __init__(self):
        super().__init__(["bytes_sent", "bytes_received", "collectives", "errors", "timeouts",
                          "host_copies", "device_syncs", "fallbacks"])


class PerfCounters(Counters):
    """Process-wide counters of the things that cost a serving loop time outside the kernels: bytes
    copied between host and device, host-side synchronisations, graph captures and replays, and
    falls back to a library path. The counterpart of the reference's global zero-copy KPI counters
    (crates/rmlx-distributed/src/perf_counters.rs:8-220: CPU copies, registrations, GPU syncs,
    bytes moved, fallbacks)."""

    def __init__(self):
        super().__init__(["h2d_bytes", "d2h_bytes", "peer_bytes", "host_syncs", "graph_captures",
                          "graph_replays", "library_fallbacks", "status_errors"])

    def record_d2h(self, tensor) -> None:
        self.add("d2h_bytes", tensor.numel() * tensor.element_size())
        self.add("host_syncs")

    def record_h2d(self, tensor) -> None:
        self.add("h2d_bytes", tensor.numel() * tensor.element_size())


GLOBAL = RuntimeMetrics()
PERF = PerfCounters()


def to_prometheus(prefix: str, snapshot: Dict[str, float]) -> str:
    return "".join(f"# TYPE {prefix}_{k} counter\n{prefix}_{k} {v}\n" for k, v in sorted(snapshot.items()))
