"""Mixtral: sliding-window attention plus a top-2 mixture of 8 experts per layer
(crates/rmlx-nn/src/models/mixtral.rs:21-330: ``mixtral_8x7b``, ``MixtralConfig`` with its
validation, ``MixtralModel`` with ``sliding_window_size`` / ``layer``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config import FeedForwardType, MoeConfig, TransformerConfig
from .transformer import TransformerModel
from .weights import from_state_dict, random_state_dict


def mixtral_8x7b() -> TransformerConfig:
    moe = MoeConfig(num_experts=8, num_experts_per_token=2, hidden_dim=4096, intermediate_dim=14336)
    return TransformerConfig(hidden_size=4096, num_heads=32, num_kv_heads=8, head_dim=128, num_layers=32,
                             vocab_size=32000, max_seq_len=32768, rope_theta=1e6, rms_norm_eps=1e-5,
                             ff_type=FeedForwardType.moe_(moe), sliding_window=4096,
                             name="mixtral-8x7b").validate()


def mixtral_tiny() -> TransformerConfig:
    moe = MoeConfig(num_experts=4, num_experts_per_token=2, hidden_dim=128, intermediate_dim=128)
    return TransformerConfig(hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, num_layers=2,
                             vocab_size=512, max_seq_len=128, rope_theta=1e6,
                             ff_type=FeedForwardType.moe_(moe), sliding_window=8, name="mixtral-tiny").validate()


@dataclass
class MixtralConfig:
    """The base transformer config plus what is Mixtral's own: the window and the expert counts
    (mixtral.rs:47-72). ``validate`` rejects a config whose pieces disagree."""
    base: TransformerConfig
    sliding_window_size: int
    num_experts: int
    num_experts_per_token: int

    def validate(self) -> "MixtralConfig":
        self.base.validate()
        moe = self.base.ff_type.moe
        if moe is None:
            raise ValueError("MixtralConfig: the feed-forward must be a mixture of experts")
        if self.sliding_window_size <= 0:
            raise ValueError("MixtralConfig: sliding_window_size must be positive")
        if not 0 < self.num_experts_per_token <= self.num_experts:
            raise ValueError("MixtralConfig: 0 < num_experts_per_token <= num_experts")
        if (moe.num_experts, moe.num_experts_per_token) != (self.num_experts, self.num_experts_per_token):
            raise ValueError("MixtralConfig: expert counts differ from the base config's")
        if (self.base.sliding_window or 0) != self.sliding_window_size:
            raise ValueError("MixtralConfig: window differs from the base config's")
        return self

    @classmethod
    def of(cls, base: TransformerConfig) -> "MixtralConfig":
        moe = base.ff_type.moe
        if moe is None:
            raise ValueError("MixtralConfig: the feed-forward must be a mixture of experts")
        return cls(base, base.sliding_window or 0, moe.num_experts, moe.num_experts_per_token).validate()


def mixtral_8x7b_full() -> MixtralConfig:
    return MixtralConfig.of(mixtral_8x7b())


class MixtralModel(TransformerModel):
    """``TransformerModel`` restricted to the Mixtral architecture. The window is applied inside
    the attention kernels (prompt and decode) and, in the serving engine, pages that have left the
    window go back to the pool."""

    def __init__(self, weights, **kw):
        self.mixtral = MixtralConfig.of(weights.cfg)
        super().__init__(weights, **kw)

    @classmethod
    def from_config(cls, cfg=None, seed: int = 0, device="cpu", dtype=torch.float32,
                    quant: Optional[str] = None) -> "MixtralModel":
        """``cfg``: a ``MixtralConfig`` or a ``TransformerConfig`` (default: the test-size preset)."""
        if isinstance(cfg, MixtralConfig):
            cfg = cfg.validate().base
        cfg = cfg or mixtral_tiny()
        MixtralConfig.of(cfg)
        return cls(from_state_dict(cfg, random_state_dict(cfg, seed), device=device, dtype=dtype, quant=quant))

    @classmethod
    def from_checkpoint(cls, model_dir: str, device="cpu", dtype=torch.bfloat16) -> "MixtralModel":
        from ..loader.safetensors_loader import load_model
        weights, _cfg = load_model(model_dir, device=device, dtype=dtype)
        return cls(weights)

    def num_layers(self) -> int:
        return self.cfg.num_layers

    def sliding_window_size(self) -> int:
        return self.mixtral.sliding_window_size

    def config(self) -> MixtralConfig:
        return self.mixtral

    def layer(self, idx: int):
        """Weights of block ``idx`` (None when out of range)."""
        return self.w.layers[idx] if 0 <= idx < len(self.w.layers) else None
