"""Qwen2 presets (crates/rmlx-nn/src/models/qwen.rs:16-95): dense decoder with GQA and SwiGLU."""
from __future__ import annotations

from ..config import FeedForwardType, TransformerConfig
from .transformer import TransformerModel


def qwen2_7b() -> TransformerConfig:
    return TransformerConfig(hidden_size=3584, num_heads=28, num_kv_heads=4, head_dim=128, num_layers=28,
                             vocab_size=152064, max_seq_len=32768, rope_theta=1e6, rms_norm_eps=1e-6,
                             ff_type=FeedForwardType.gated(18944), name="qwen2-7b").validate()


def qwen2_tiny() -> TransformerConfig:
    """Same architecture at test size."""
    return TransformerConfig(hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, num_layers=2,
                             vocab_size=512, max_seq_len=128, rope_theta=1e6,
                             ff_type=FeedForwardType.gated(256), name="qwen2-tiny").validate()


Qwen2Model = TransformerModel
