"""Mixture-of-experts layers.

``ExpertGroup`` stacks expert weights (``[E, 2I, D]`` gate|up and ``[E, D, I]`` down) and runs
``grouped_forward``: all experts' tokens in one pass (crates/rmlx-nn/src/expert_group.rs:72-533).
``MoeLayer`` is gate -> top-k route -> experts -> weighted combine (+ optional shared expert),
with the strategies of crates/rmlx-nn/src/moe.rs:166-200 mapped as: PER_EXPERT (loop, the
oracle), GROUPED (rows sorted by expert, one grouped GEMM pair; tensor cores on CUDA), and
DECODE (per-pair GEMV kernels for a handful of tokens). Expert parallelism plugs in through an
``EpExchange``. Routing never leaves the device on CUDA (the reference reads it back to the host,
moe.rs:600-601). Also: aux-loss-free expert-bias update (moe.rs:372-410) and the GShard
load-balance loss (moe.rs:1954-2000).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import List, Optional, Tuple

import torch

from ..config import MoeConfig
from ..ops.weights import LinearWeight
from ..reference import ops as ref


class MoeStrategy(Enum):
    PER_EXPERT = "per_expert"
    GROUPED = "grouped"
    DECODE = "decode"


@dataclass
class MoeForwardMetrics:
    tokens: int = 0
    max_expert_load: int = 0
    empty_experts: int = 0


class ExpertGroup:
    def __init__(self, gate_up: LinearWeight, down: LinearWeight):
        assert gate_up.experts == down.experts and gate_up.experts > 0
        self.gate_up, self.down = gate_up, down
        self.num_experts = gate_up.experts
        self._dq = {}

    @staticmethod
    def from_experts(experts: List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]],
                     quant: Optional[str] = None, device="cpu", dtype=torch.bfloat16) -> "ExpertGroup":
        """experts: list of (gate [I, D], up [I, D], down [D, I]) fp32 tensors."""
        gu = torch.stack([torch.cat([g, u], 0) for g, u, _ in experts], 0)
        dn = torch.stack([d for _, _, d in experts], 0)
        return ExpertGroup(LinearWeight.from_dense(gu, quant, dtype, device),
                           LinearWeight.from_dense(dn, quant, dtype, device))

    def _dense(self, which: str, dtype):
        key = (which, dtype)
        if key not in self._dq:
            self._dq[key] = getattr(self, which).dequantized().to(dtype)
        return self._dq[key]

    def grouped_rows(self, x: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
        """x: rows sorted by expert, ``offsets`` [E+1]. Returns expert outputs in the same order."""
        if x.is_cuda and x.dtype == torch.bfloat16:
            try:
                from ..ops.grouped import grouped_expert_ffn
                return grouped_expert_ffn(x, offsets, self.gate_up, self.down)
            except ImportError:
                pass
        out = torch.empty(x.shape[0], self.down.n, dtype=x.dtype, device=x.device)
        gu, dn = self._dense("gate_up", x.dtype), self._dense("down", x.dtype)
        offs = offsets.tolist()
        for e in range(self.num_experts):
            lo, hi = offs[e], offs[e + 1]
            if hi > lo:       # empty experts are skipped
                out[lo:hi] = ref.swiglu(x[lo:hi] @ gu[e].t()) @ dn[e].t()
        return out

    def grouped_forward(self, batches: List[Tuple[int, torch.Tensor]]) -> List[Tuple[int, torch.Tensor]]:
        """The reference's call shape: ``[(expert_idx, input [b, D])] -> [(expert_idx, output)]``."""
        if not batches:
            return []
        order = sorted(range(len(batches)), key=lambda i: batches[i][0])
        counts = torch.zeros(self.num_experts, dtype=torch.int64)
        for e, xb in batches:
            counts[e] += xb.shape[0]
        offsets = torch.zeros(self.num_experts + 1, dtype=torch.int64)
        offsets[1:] = torch.cumsum(counts, 0)
        x = torch.cat([batches[i][1] for i in order], 0)
        y = self.grouped_rows(x, offsets.to(x.device))
        res: List[Optional[Tuple[int, torch.Tensor]]] = [None] * len(batches)
        pos = 0
        for i in order:
            n = batches[i][1].shape[0]
            res[i] = (batches[i][0], y[pos:pos + n])
            pos += n
        return res


class MoeLayer:
    def __init__(self, cfg: MoeConfig, router: torch.Tensor, experts: ExpertGroup,
                 strategy: MoeStrategy = MoeStrategy.GROUPED):
        self.cfg = cfg.validate()
        self.router = router                      # [E, D]
        self.experts = experts
        self.strategy = strategy
        self.expert_bias: Optional[torch.Tensor] = None
        self.shared: Optional[Tuple[LinearWeight, LinearWeight]] = None
        self.exchange = None
        self.policy = None                        # parallel.moe_policy.MoePolicy
        self.exchanges = {}                       # MoeBackend -> exchange (dispatch / combine)
        self.overlap: Optional[str] = None        # None | "sbo" | "tbo"
        self._pipeline = None
        self.metrics = MoeForwardMetrics()
        self.last_counts: Optional[torch.Tensor] = None

    # builders, as in crates/rmlx-nn/src/moe.rs:297-364
    def with_strategy(self, s: MoeStrategy) -> "MoeLayer":
        self.strategy = s
        return self

    def with_shared_expert(self, gate_up: LinearWeight, down: LinearWeight) -> "MoeLayer":
        self.shared = (gate_up, down)
        return self

    def with_exchange(self, exchange) -> "MoeLayer":
        self.exchange = exchange
        return self

    def with_policy(self, policy, exchanges) -> "MoeLayer":
        """Choose the exchange per call from the token count: ``exchanges`` maps a
        ``MoeBackend`` to an object with ``dispatch`` / ``combine`` (the device-side exchange for
        FUSED, the library all-to-all for NCCL); a backend without an entry falls back to the one
        set by ``with_exchange`` (crates/rmlx-distributed/src/moe_policy.rs:85-423)."""
        self.policy, self.exchanges = policy, dict(exchanges)
        return self

    def with_overlap(self, mode: Optional[str]) -> "MoeLayer":
        """``"sbo"``: the shared expert runs on a side stream beside the routed experts;
        ``"tbo"``: two token micro-batches alternate between two streams
        (crates/rmlx-nn/src/moe_pipeline.rs:45-500)."""
        if mode not in (None, "sbo", "tbo"):
            raise ValueError(f"unknown overlap mode {mode}")
        self.overlap = mode
        return self

    def forward_overlapped(self, x: torch.Tensor) -> torch.Tensor:
        """``forward`` under the schedule chosen by ``with_overlap`` (plain ``forward`` if none)."""
        if self.overlap is None:
            return self.forward(x)
        if self._pipeline is None:
            from .moe_pipeline import MoePipeline
            self._pipeline = MoePipeline(self)
        return self._pipeline.forward_sbo(x) if self.overlap == "sbo" else self._pipeline.forward_tbo(x)

    def _exchange_for(self, x: torch.Tensor):
        if self.policy is None:
            return self.exchange
        backend = self.policy.select(x.shape[0], x.numel() * x.element_size())
        self.metrics_backend = backend
        return self.exchanges.get(backend, self.exchange)

    def with_expert_bias(self, bias: torch.Tensor) -> "MoeLayer":
        self.expert_bias = bias
        return self

    def route(self, x: torch.Tensor):
        logits = x.float() @ self.router.float().t()
        if x.is_cuda:
            from ..ops import decode as D
            idx, wts, counts, offsets = D.topk_route(logits.contiguous(), self.cfg.num_experts_per_token,
                                                     self.expert_bias)
            return idx, wts, counts, logits
        idx, wts, counts = ref.topk_route(logits, self.cfg.num_experts_per_token, self.expert_bias)
        return idx, wts, counts, logits

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [T, D] -> [T, D] (no residual)."""
        t, k = x.shape[0], self.cfg.num_experts_per_token
        idx, wts, counts, _ = self.route(x)
        self.last_counts = counts
        self.metrics = MoeForwardMetrics(t, int(counts.max()), int((counts == 0).sum()))
        exchange = self._exchange_for(x)
        if exchange is not None:
            rows, layout = exchange.dispatch(x, idx)
            y = self.experts.grouped_rows(rows, layout.offsets)
            out = exchange.combine(y, wts, layout)
        elif self.strategy == MoeStrategy.PER_EXPERT:
            out = ref.moe_ffn(x, idx, wts, self.experts._dense("gate_up", x.dtype),
                              self.experts._dense("down", x.dtype))
        else:
            flat = idx.reshape(-1).long()
            order = torch.argsort(flat, stable=True)
            offsets = torch.zeros(self.cfg.num_experts + 1, dtype=torch.int64, device=x.device)
            offsets[1:] = torch.cumsum(torch.bincount(flat, minlength=self.cfg.num_experts), 0)
            y = self.experts.grouped_rows(x[order // k], offsets)
            out = torch.zeros(t, y.shape[-1], dtype=torch.float32, device=x.device)
            out.index_add_(0, order // k, y.float() * wts.reshape(-1)[order].float()[:, None])
        if self.shared is not None:
            gu, dn = self.shared
            a = ref.swiglu(x @ gu.dequantized().to(x.dtype).t())
            out = out + (a @ dn.dequantized().to(x.dtype).t()).float()
        return out.to(x.dtype)

    # training-side helpers
    def update_expert_bias(self, lr: float = 1e-3) -> torch.Tensor:
        if self.expert_bias is None:
            self.expert_bias = torch.zeros(self.cfg.num_experts, device=self.router.device)
        self.expert_bias = ref.expert_bias_update(self.expert_bias, self.last_counts.to(self.expert_bias.device), lr)
        return self.expert_bias

    def load_balance_loss(self, x: torch.Tensor) -> torch.Tensor:
        idx, _, _, logits = self.route(x)
        return ref.load_balance_loss(torch.softmax(logits.float(), -1), idx, self.cfg.num_experts)
