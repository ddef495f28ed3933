"""NaN/Inf and entropy-drift monitor on logits with a Warn / Fallback verdict
(crates/rmlx-core/src/precision_guard.rs:5-174)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum

import torch


class GuardAction(Enum):
    OK = 0
    WARN = 1
    FALLBACK = 2


@dataclass
class PrecisionGuard:
    entropy_drift_warn: float = 0.5      # relative drift of the running entropy mean
    entropy_drift_fallback: float = 2.0
    ema: float = 0.9
    _mean: float = float("nan")
    nan_events: int = 0
    checks: int = 0

    def check(self, logits: torch.Tensor) -> GuardAction:
        self.checks += 1
        lf = logits.float()
        if not torch.isfinite(lf).all():
            self.nan_events += 1
            return GuardAction.FALLBACK
        p = torch.softmax(lf, -1)
        h = float(-(p * torch.log(p.clamp_min(1e-30))).sum(-1).mean())
        if math.isnan(self._mean):
            self._mean = h
            return GuardAction.OK
        drift = abs(h - self._mean) / max(self._mean, 1e-6)
        self._mean = self.ema * self._mean + (1 - self.ema) * h
        if drift > self.entropy_drift_fallback:
            return GuardAction.FALLBACK
        if drift > self.entropy_drift_warn:
            return GuardAction.WARN
        return GuardAction.OK
