"""Static plans and scratch for prompt processing.

``PrefillPlan`` lists, for a sequence length, the launches of one layer with their shapes and the
scratch each needs (the reference builds the same per-length ``PlanStep`` lists,
crates/rmlx-nn/src/prefill_plan.rs:16-300); ``PrefillPool`` keeps a few slots of pre-allocated
intermediates sized for the largest planned length so that chunks of a prompt do not allocate
(crates/rmlx-nn/src/prefill_pool.rs:33-160, crates/rmlx-nn/src/dynamic.rs:16-104).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..config import TransformerConfig
from .weights import ParallelLayout


@dataclass(frozen=True)
class PlanStep:
    name: str
    kernel: str
    m: int
    n: int
    k: int
    out_bytes: int

    @property
    def flops(self) -> float:
        return 2.0 * self.m * self.n * self.k


class PrefillPlan:
    def __init__(self, cfg: TransformerConfig, seq_len: int, layout: Optional[ParallelLayout] = None):
        layout = layout or ParallelLayout()
        hq, _, hkv, _ = layout.heads(cfg)
        d, hd, t = cfg.hidden_size, cfg.head_dim, seq_len
        self.cfg, self.seq_len = cfg, seq_len
        steps: List[PlanStep] = [
            PlanStep("attn_norm", "rms_norm", t, d, 1, t * d * 2),
            PlanStep("qkv", "gemm", t, (hq + 2 * hkv) * hd, d, t * (hq + 2 * hkv) * hd * 2),
            PlanStep("rope_kv", "rope_kv_write", t, (hq + 2 * hkv) * hd, 1, t * hq * hd * 2),
            PlanStep("attention", "flash_prefill", t, hq * hd, t // 2 + 1, t * hq * hd * 2),
            PlanStep("o_proj", "gemm+residual", t, d, hq * hd, t * d * 2),
            PlanStep("ffn_norm", "rms_norm", t, d, 1, t * d * 2),
        ]
        if cfg.ff_type.kind == "moe":
            m = cfg.ff_type.moe
            k, inter = m.num_experts_per_token, m.intermediate_dim // layout.world
            steps += [
                PlanStep("router", "gemm_f32+topk", t, m.num_experts, d, t * k * 8),
                PlanStep("scatter", "moe_scatter_rows", t * k, d, 1, t * k * d * 2),
                PlanStep("gate_up", "grouped_gemm+swiglu", t * k, 2 * inter, d, t * k * inter * 2),
                PlanStep("down", "grouped_gemm", t * k, d, inter, t * k * d * 2),
                PlanStep("combine", "moe_combine+residual", t, d, k, t * d * 2),
            ]
        else:
            inter = cfg.ff_type.intermediate_dim // layout.world
            steps += [
                PlanStep("gate_up", "gemm+swiglu", t, 2 * inter, d, t * inter * 2),
                PlanStep("down", "gemm+residual", t, d, inter, t * d * 2),
            ]
        self.steps: Tuple[PlanStep, ...] = tuple(steps)

    @property
    def scratch_bytes(self) -> int:
        """Peak of (a step's output + its input, i.e. the previous step's output)."""
        peak, prev = 0, 0
        for s in self.steps:
            peak = max(peak, prev + s.out_bytes)
            prev = s.out_bytes
        return peak

    @property
    def flops(self) -> float:
        return sum(s.flops for s in self.steps if "gemm" in s.kernel or s.kernel == "flash_prefill")


class PrefillPool:
    """``slots`` scratch buffers of ``bytes_per_slot`` each; ``acquire`` hands out a free one (or
    None when all are in use), ``release`` returns it."""

    def __init__(self, bytes_per_slot: int, slots: int = 4, device="cpu"):
        self.bytes_per_slot = int(bytes_per_slot)
        self._bufs = [torch.empty(self.bytes_per_slot, dtype=torch.uint8, device=device) for _ in range(slots)]
        self._free = list(range(slots))
        self._plans: Dict[int, PrefillPlan] = {}

    @classmethod
    def for_config(cls, cfg: TransformerConfig, max_seq_len: int, slots: int = 4, device="cpu",
                   layout: Optional[ParallelLayout] = None) -> "PrefillPool":
        pool = cls(PrefillPlan(cfg, max_seq_len, layout).scratch_bytes, slots, device)
        pool._cfg, pool._layout = cfg, layout
        return pool

    def plan(self, seq_len: int) -> PrefillPlan:
        p = self._plans.get(seq_len)
        if p is None:
            p = PrefillPlan(self._cfg, seq_len, self._layout)
            if p.scratch_bytes > self.bytes_per_slot:
                raise ValueError("sequence longer than the pool was sized for")
            self._plans[seq_len] = p
        return p

    def acquire(self) -> Optional[Tuple[int, torch.Tensor]]:
        if not self._free:
            return None
        i = self._free.pop()
        return i, self._bufs[i]

    def release(self, slot: int) -> None:
        if slot in self._free or not 0 <= slot < len(self._bufs):
            raise ValueError("slot is not in use")
        self._free.append(slot)

    @property
    def available(self) -> int:
        return len(self._free)


class DynamicExecContext:
    """``count`` intermediates of [max_seq_len, hidden] allocated once; a step of any length up to
    the maximum takes views of their first rows, so a varying sequence length never allocates
    (crates/rmlx-nn/src/dynamic.rs:16-104)."""

    def __init__(self, max_seq_len: int, hidden_dim: int, dtype=torch.bfloat16, num_intermediates: int = 4,
                 device="cpu"):
        if max_seq_len < 1 or hidden_dim < 1 or num_intermediates < 1:
            raise ValueError("DynamicExecContext: sizes must be positive")
        self._max, self._hidden, self.dtype = max_seq_len, hidden_dim, dtype
        self._bufs = [torch.zeros(max_seq_len, hidden_dim, dtype=dtype, device=device)
                      for _ in range(num_intermediates)]

    def max_seq_len(self) -> int:
        return self._max

    def hidden_dim(self) -> int:
        return self._hidden

    def num_intermediates(self) -> int:
        return len(self._bufs)

    def allocated_bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs)

    def get_intermediate(self, idx: int, actual_seq_len: int) -> torch.Tensor:
        """A view of the first ``actual_seq_len`` rows of intermediate ``idx`` (no copy)."""
        if not 0 <= idx < len(self._bufs):
            raise ValueError(f"DynamicExecContext: intermediate index {idx} >= count {len(self._bufs)}")
        if not 0 <= actual_seq_len <= self._max:
            raise ValueError(f"DynamicExecContext: actual_seq_len {actual_seq_len} > max_seq_len {self._max}")
        return self._bufs[idx][:actual_seq_len]
