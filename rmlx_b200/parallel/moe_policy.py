"""Which back-end carries a MoE dispatch, chosen from the token count with hysteresis and a
cool-down, plus the overflow guard.

``MoePolicy`` keeps the reference's 3-zone shape (crates/rmlx-distributed/src/moe_policy.rs:85-423):
small batches take the latency path, large ones the throughput path, the middle zone is decided by
a byte threshold; a switch needs the count to move past the boundary by the hysteresis margin, and
after a switch the choice is frozen for ``cooldown_s`` seconds or ``cooldown_calls`` calls. On this
hardware the zones map to: LOCAL (per-pair GEMV kernels with in-kernel all-reduce, decode),
FUSED (device-side all-to-all into peer slabs + grouped GEMM) and NCCL (library all-to-all, the
fallback). Environment overrides: RMLX_MOE_BACKEND, RMLX_MOE_CPU_N_MAX (kept as the small-zone
bound), RMLX_MOE_GPU_N_MIN, RMLX_MOE_GPU_SWITCH_BYTES.

``SparseGuard`` follows crates/rmlx-distributed/src/sparse_guard.rs:5-129: an EMA of the overflow
ratio over windows of 100 steps asks for more capacity above 5 %, for the dense fallback above
20 %, and resets once the ratio is back under control. With capacity-free routing nothing
overflows; the guard is used by the capacity-limited (reference-compatible) dispatch mode.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from enum import Enum
from typing import Callable, Mapping, Optional


class MoeBackend(Enum):
    LOCAL = "local"
    FUSED = "fused"
    NCCL = "nccl"


@dataclass
class ThresholdCalibration:
    """Measured crossover (tokens) between the small and the large path, from the warm-up run."""
    small_n_max: int = 64
    large_n_min: int = 320
    switch_bytes: int = 2 << 20


class MoePolicy:
    def __init__(self, calibration: Optional[ThresholdCalibration] = None, hysteresis: int = 16,
                 cooldown_s: float = 5.0, cooldown_calls: int = 1000,
                 env: Optional[Mapping[str, str]] = None, clock: Callable[[], float] = time.monotonic):
        env = os.environ if env is None else env
        c = calibration or ThresholdCalibration()
        self.small_n_max = int(env.get("RMLX_MOE_CPU_N_MAX", c.small_n_max))
        self.large_n_min = int(env.get("RMLX_MOE_GPU_N_MIN", c.large_n_min))
        self.switch_bytes = int(env.get("RMLX_MOE_GPU_SWITCH_BYTES", c.switch_bytes))
        self.hysteresis, self.cooldown_s, self.cooldown_calls = hysteresis, cooldown_s, cooldown_calls
        self.clock = clock
        forced = env.get("RMLX_MOE_BACKEND", "").lower()
        self._forced = MoeBackend(forced) if forced in ("local", "fused", "nccl") else None
        self._current: Optional[MoeBackend] = None
        self._switched_at = -1e30
        self._calls_since = 0
        self.zone_switches = 0

    def force_backend(self, b: Optional[MoeBackend]) -> None:
        self._forced = b

    def apply_calibration(self, c: ThresholdCalibration) -> None:
        self.small_n_max, self.large_n_min, self.switch_bytes = c.small_n_max, c.large_n_min, c.switch_bytes

    def _zone(self, n_tokens: int, nbytes: int, margin: int) -> MoeBackend:
        if n_tokens <= self.small_n_max - margin:
            return MoeBackend.LOCAL
        if n_tokens >= self.large_n_min + margin:
            return MoeBackend.FUSED
        if margin and self._current is not None:
            return self._current
        if n_tokens <= self.small_n_max:
            return MoeBackend.LOCAL
        if n_tokens >= self.large_n_min:
            return MoeBackend.FUSED
        return MoeBackend.FUSED if nbytes >= self.switch_bytes else MoeBackend.LOCAL

    def select(self, n_tokens: int, nbytes: int = 0) -> MoeBackend:
        if self._forced is not None:
            return self._forced
        self._calls_since += 1
        if self._current is None:
            self._current = self._zone(n_tokens, nbytes, 0)
            return self._current
        in_cooldown = (self.clock() - self._switched_at < self.cooldown_s and
                       self._calls_since < self.cooldown_calls)
        if in_cooldown:
            return self._current
        want = self._zone(n_tokens, nbytes, self.hysteresis)
        if want != self._current:
            self._current = want
            self._switched_at = self.clock()
            self._calls_since = 0
            self.zone_switches += 1
        return self._current


class GuardAction(Enum):
    NONE = 0
    INCREASE_CAPACITY = 1
    DENSE_FALLBACK = 2
    RESET = 3


class SparseGuard:
    def __init__(self, window: int = 100, increase_at: float = 0.05, dense_at: float = 0.20,
                 ema: float = 0.9):
        self.window, self.increase_at, self.dense_at, self.ema = window, increase_at, dense_at, ema
        self._overflow = self._total = self._steps = 0
        self.ratio_ema = 0.0
        self.state = GuardAction.NONE

    def record_step(self, overflow_tokens: int, total_tokens: int) -> GuardAction:
        self._overflow += overflow_tokens
        self._total += total_tokens
        self._steps += 1
        if self._steps < self.window:
            return GuardAction.NONE
        ratio = self._overflow / max(1, self._total)
        self.ratio_ema = self.ema * self.ratio_ema + (1 - self.ema) * ratio if self.ratio_ema else ratio
        self._overflow = self._total = self._steps = 0
        if self.ratio_ema > self.dense_at:
            self.state = GuardAction.DENSE_FALLBACK
        elif self.ratio_ema > self.increase_at:
            self.state = GuardAction.INCREASE_CAPACITY
        elif self.state != GuardAction.NONE:
            self.state = GuardAction.NONE
            return GuardAction.RESET
        return self.state
