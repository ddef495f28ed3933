"""Mixtral presets (crates/rmlx-nn/src/models/mixtral.rs:21-330): sliding-window attention plus
8 experts, top-2, per layer."""
from __future__ import annotations

from ..config import FeedForwardType, MoeConfig, TransformerConfig
from .transformer import TransformerModel


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


MixtralModel = TransformerModel
