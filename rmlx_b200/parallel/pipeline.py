"""Per-layer compute / transfer overlap: layer N's compute runs while layer N-1's transfer (a
collective, an expert exchange, a device-to-host copy) is still in flight on a second stream. Stages
are chained with events; nothing blocks the host until ``finish``.

Counterpart of ``LayerPipeline`` (crates/rmlx-distributed/src/pipeline.rs:19-640): stages
Compute -> Transfer -> Complete per layer, ``measure_overlap`` and ``PipelineStats``. This is an
overlap schedule inside one rank, not pipeline parallelism across ranks.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, List

import torch


class Stage(Enum):
    IDLE = "idle"
    COMPUTE = "compute"
    TRANSFER = "transfer"
    COMPLETE = "complete"


@dataclass
class PipelineConfig:
    num_layers: int = 1
    sync_timeout_s: float = 30.0

    def validate(self) -> "PipelineConfig":
        if self.num_layers < 1 or self.sync_timeout_s <= 0:
            raise ValueError("bad pipeline configuration")
        return self


@dataclass
class PipelineStats:
    layers_run: int = 0
    compute_s: float = 0.0
    transfer_s: float = 0.0
    wall_s: float = 0.0
    stages: List[Stage] = field(default_factory=list)

    @property
    def overlap_ratio(self) -> float:
        """1 - wall / (compute + transfer): 0 = fully serial, -> 0.5 when both halves hide each other."""
        serial = self.compute_s + self.transfer_s
        return 0.0 if serial <= 0 else max(0.0, 1.0 - self.wall_s / serial)


class LayerPipeline:
    def __init__(self, config: PipelineConfig, device=None):
        self.cfg = config.validate()
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.device = device
        self.compute_stream = torch.cuda.current_stream(device) if self.cuda else None
        self.transfer_stream = torch.cuda.Stream(device) if self.cuda else None
        self.stats = PipelineStats(stages=[Stage.IDLE] * config.num_layers)
        self._pending: List = []

    def run(self, compute: Callable[[int], object], transfer: Callable[[int, object], object]) -> List[object]:
        """``compute(layer)`` on the compute stream; ``transfer(layer, result)`` on the transfer
        stream as soon as that layer's compute is done, while the next layer computes. Returns the
        transfer results (valid after ``finish``)."""
        outs: List[object] = []
        t0 = time.perf_counter()
        for l in range(self.cfg.num_layers):
            self.stats.stages[l] = Stage.COMPUTE
            c0 = time.perf_counter()
            y = compute(l)
            self.stats.compute_s += time.perf_counter() - c0
            self.stats.stages[l] = Stage.TRANSFER
            x0 = time.perf_counter()
            if self.cuda:
                done = torch.cuda.Event()
                done.record(self.compute_stream)
                self.transfer_stream.wait_event(done)
                with torch.cuda.stream(self.transfer_stream):
                    outs.append(transfer(l, y))
                fin = torch.cuda.Event()
                fin.record(self.transfer_stream)
                self._pending.append((l, fin))
            else:
                outs.append(transfer(l, y))
                self.stats.stages[l] = Stage.COMPLETE
            self.stats.transfer_s += time.perf_counter() - x0
            self.stats.layers_run += 1
        self.finish()
        self.stats.wall_s += time.perf_counter() - t0
        return outs

    def poll(self) -> int:
        """Mark finished transfers; returns how many are still in flight."""
        still = []
        for l, ev in self._pending:
            if ev.query():
                self.stats.stages[l] = Stage.COMPLETE
            else:
                still.append((l, ev))
        self._pending = still
        return len(still)

    def finish(self) -> None:
        deadline = time.monotonic() + self.cfg.sync_timeout_s
        while self.poll():
            if time.monotonic() > deadline:
                raise TimeoutError("pipeline transfers did not complete in time")
            time.sleep(0)
        if self.cuda:
            self.compute_stream.wait_stream(self.transfer_stream)

    def measure_overlap(self, compute, transfer) -> float:
        """Run once serially (transfer right after each compute, host-synchronised) and once
        pipelined; returns pipelined wall time / serial wall time (< 1 means overlap happened)."""
        def sync():
            if self.cuda:
                torch.cuda.synchronize(self.device)
        sync()
        t0 = time.perf_counter()
        for l in range(self.cfg.num_layers):
            y = compute(l)
            sync()
            transfer(l, y)
            sync()
        serial = time.perf_counter() - t0
        t0 = time.perf_counter()
        self.run(compute, transfer)
        sync()
        piped = time.perf_counter() - t0
        return piped / serial if serial > 0 else 1.0
