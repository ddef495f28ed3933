"""Qwen2: dense decoder with grouped-query attention and SwiGLU
(crates/rmlx-nn/src/models/qwen.rs:16-95: the ``qwen2_7b`` preset and ``Qwen2Model``, a
``TransformerModel`` that insists on the gated feed-forward)."""
from __future__ import annotations

from typing import Optional

import torch

from ..config import FeedForwardType, TransformerConfig
from .transformer import TransformerModel
from .weights import from_state_dict, random_state_dict


def qwen2_7b() -> TransformerConfig:
    return TransformerConfig(hidden_size=3584, num_heads=28, num_kv_heads=4, head_dim=128, num_layers=28,
                             vocab_size=152064, max_seq_len=32768, rope_theta=1e6, rms_norm_eps=1e-6,
                             ff_type=FeedForwardType.gated(18944), name="qwen2-7b").validate()


def qwen2_tiny() -> TransformerConfig:
    """Same architecture at test size."""
    return TransformerConfig(hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, num_layers=2,
                             vocab_size=512, max_seq_len=128, rope_theta=1e6,
                             ff_type=FeedForwardType.gated(256), name="qwen2-tiny").validate()


def _check(cfg: TransformerConfig) -> None:
    if cfg.ff_type.kind != "gated":
        raise ValueError("Qwen2Model: the feed-forward must be gated (SwiGLU)")
    if cfg.sliding_window:
        raise ValueError("Qwen2Model: no sliding window in this architecture")


class Qwen2Model(TransformerModel):
    """``TransformerModel`` restricted to the Qwen2 architecture, with the reference's accessors."""

    def __init__(self, weights, **kw):
        _check(weights.cfg)
        super().__init__(weights, **kw)

    @classmethod
    def from_config(cls, cfg: Optional[TransformerConfig] = None, seed: int = 0, device="cpu",
                    dtype=torch.float32, quant: Optional[str] = None) -> "Qwen2Model":
        """Random-initialised model of ``cfg`` (default: the test-size preset)."""
        cfg = cfg or qwen2_tiny()
        _check(cfg)
        return cls(from_state_dict(cfg, random_state_dict(cfg, seed), device=device, dtype=dtype, quant=quant))

    @classmethod
    def from_checkpoint(cls, model_dir: str, device="cpu", dtype=torch.bfloat16) -> "Qwen2Model":
        """An MLX-style / Hugging Face safetensors directory (config.json + shards)."""
        from ..loader.safetensors_loader import load_model
        weights, _cfg = load_model(model_dir, device=device, dtype=dtype)
        return cls(weights)

    def inner(self) -> TransformerModel:
        return self

    def num_layers(self) -> int:
        return self.cfg.num_layers

    def config(self) -> TransformerConfig:
        return self.cfg
