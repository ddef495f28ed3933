"""Idempotent warm-up: run the communication path and the kernels once before the first timed or
served request, and calibrate the MoE backend thresholds from what was measured.

Follows ``run_warmup(rdma_fn, jit_fn)`` with its calibration micro-benchmark
(crates/rmlx-distributed/src/warmup.rs:20-150): the two callables are the communication warm-up
(here: touch every peer through the collective the caller passes, which also faults in peer
mappings and brings NVLink up) and the kernel warm-up (here: run the step once so that modules are
loaded, function attributes set and lazily created buffers exist). A second call returns the first
call's result without running anything.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Optional

from .moe_policy import ThresholdCalibration


@dataclass
class WarmupResult:
    comm_s: float = 0.0
    kernels_s: float = 0.0
    calibration_s: float = 0.0
    calibration: Optional[ThresholdCalibration] = None
    timings_us: Dict[str, float] = field(default_factory=dict)
    ran: bool = False


@dataclass
class WarmupConfig:
    run_calibration: bool = True
    calibration_sizes: tuple = (4, 32, 128, 512)
    repeats: int = 3


class Warmup:
    def __init__(self, config: Optional[WarmupConfig] = None, clock: Callable[[], float] = time.perf_counter):
        self.config = config or WarmupConfig()
        self.clock = clock
        self._result: Optional[WarmupResult] = None

    @property
    def done(self) -> bool:
        return self._result is not None

    def run(self, comm_fn: Optional[Callable[[], None]] = None,
            kernel_fn: Optional[Callable[[], None]] = None,
            time_small: Optional[Callable[[int], float]] = None,
            time_large: Optional[Callable[[int], float]] = None) -> WarmupResult:
        """``time_small(n)`` / ``time_large(n)``: seconds for one MoE exchange of n tokens on the
        small-message path and on the large-message path; when both are given and calibration is
        on, the crossover token count becomes the policy's thresholds."""
        if self._result is not None:
            return WarmupResult(**{**self._result.__dict__, "ran": False})
        r = WarmupResult(ran=True)
        t0 = self.clock()
        if comm_fn is not None:
            comm_fn()
        r.comm_s = self.clock() - t0
        t0 = self.clock()
        if kernel_fn is not None:
            kernel_fn()
        r.kernels_s = self.clock() - t0
        if self.config.run_calibration and time_small is not None and time_large is not None:
            t0 = self.clock()
            r.calibration = self._calibrate(time_small, time_large, r.timings_us)
            r.calibration_s = self.clock() - t0
        self._result = r
        return r

    def _calibrate(self, time_small, time_large, timings) -> ThresholdCalibration:
        sizes = sorted(self.config.calibration_sizes)
        cross = None
        for n in sizes:
            ts = min(time_small(n) for _ in range(self.config.repeats))
            tl = min(time_large(n) for _ in range(self.config.repeats))
            timings[f"small_{n}"] = ts * 1e6
            timings[f"large_{n}"] = tl * 1e6
            if cross is None and tl < ts:
                cross = n
        base = ThresholdCalibration()
        if cross is None:                      # the small path won everywhere that was measured
            return ThresholdCalibration(sizes[-1], max(sizes[-1] * 2, base.large_n_min), base.switch_bytes)
        lo = max([s for s in sizes if s < cross], default=max(1, cross // 2))
        return ThresholdCalibration(small_n_max=lo, large_n_min=cross, switch_bytes=base.switch_bytes)
