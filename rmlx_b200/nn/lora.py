"""LoRA adapters and a small trainer on top of PyTorch autograd.

``LoraConfig`` / ``LoraLayer`` / ``LoraModel`` / ``LoraTrainer`` with an MSE loss and an SGD
``train_step`` (crates/rmlx-core/src/lora.rs:9-450). The reference carries its own tape-based
reverse-mode autodiff and GPU gradient kernels for this (crates/rmlx-core/src/vjp.rs:5-362,
ops/vjp_gpu.rs, ops/sdpa_backward.rs); here differentiation is PyTorch's, and ``numerical_gradient``
is kept as the test oracle the reference uses for its VJPs."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, List

import torch


@dataclass
class LoraConfig:
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0

    @property
    def scaling(self) -> float:
        return self.alpha / self.rank


class LoraLayer:
    def __init__(self, base_weight: torch.Tensor, cfg: LoraConfig, seed: int = 0):
        """base_weight [out, in] stays frozen; A [rank, in] ~ N(0, 1/rank), B [out, rank] = 0."""
        g = torch.Generator().manual_seed(seed)
        self.base = base_weight.detach()
        self.cfg = cfg
        dev, dt = base_weight.device, torch.float32
        self.a = (torch.randn(cfg.rank, base_weight.shape[1], generator=g) / math.sqrt(cfg.rank)
                  ).to(dev, dt).requires_grad_(True)
        self.b = torch.zeros(base_weight.shape[0], cfg.rank, device=dev, dtype=dt, requires_grad=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = x @ self.base.to(x.dtype).t()
        return y + (x.float() @ self.a.t() @ self.b.t() * self.cfg.scaling).to(y.dtype)

    __call__ = forward

    def merged_weight(self) -> torch.Tensor:
        return (self.base.float() + self.cfg.scaling * self.b.detach() @ self.a.detach()).to(self.base.dtype)

    def parameters(self) -> List[torch.Tensor]:
        return [self.a, self.b]


class LoraModel:
    def __init__(self, layers: Dict[str, LoraLayer]):
        self.layers = layers

    def parameters(self) -> List[torch.Tensor]:
        return [p for l in self.layers.values() for p in l.parameters()]

    def num_trainable(self) -> int:
        return sum(p.numel() for p in self.parameters())


class LoraTrainer:
    def __init__(self, model: LoraModel, lr: float = 1e-2):
        self.model, self.lr = model, lr

    @staticmethod
    def mse_loss(pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return ((pred.float() - target.float()) ** 2).mean()

    def train_step(self, forward: Callable[[], torch.Tensor], target: torch.Tensor) -> float:
        params = self.model.parameters()
        for p in params:
            p.grad = None
        loss = self.mse_loss(forward(), target)
        loss.backward()
        with torch.no_grad():
            for p in params:
                if p.grad is not None:
                    p -= self.lr * p.grad
        return float(loss.detach())


def numerical_gradient(f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, eps: float = 1e-3
                       ) -> torch.Tensor:
    """Central differences of a scalar function, element by element (test oracle)."""
    g = torch.zeros_like(x, dtype=torch.float64)
    xf = x.detach().double().clone()
    flat, gf = xf.view(-1), g.view(-1)
    for i in range(flat.numel()):
        old = float(flat[i])
        flat[i] = old + eps
        hi = float(f(xf.to(x.dtype)))
        flat[i] = old - eps
        lo = float(f(xf.to(x.dtype)))
        flat[i] = old
        gf[i] = (hi - lo) / (2 * eps)
    return g.to(x.dtype)
