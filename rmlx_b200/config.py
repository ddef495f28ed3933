"""Typed configuration structs with ``validate()``.

Field names and defaults follow the reference's config structs so a user can carry settings over:
``TransformerConfig`` / ``FeedForwardType`` (crates/rmlx-nn/src/transformer.rs:38-109),
``MoeConfig`` (crates/rmlx-nn/src/moe.rs:114-132), ``AttentionConfig``
(crates/rmlx-nn/src/attention.rs:1790-1796), ``MlaConfig`` (crates/rmlx-nn/src/mla.rs:47-66),
``SchedulerConfig`` (crates/rmlx-nn/src/scheduler.rs:19-31), ``SamplerConfig``
(crates/rmlx-nn/src/sampler.rs:21-64), ``InitConfig`` (crates/rmlx-distributed/src/init.rs:38-95).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Optional


class ConfigError(ValueError):
    pass


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ConfigError(msg)


@dataclass
class MoeConfig:
    num_experts: int
    num_experts_per_token: int
    hidden_dim: int
    intermediate_dim: int
    capacity_factor: float = 1.0      # only used by the capacity-limited (reference-style) dispatch
    enable_fp8: bool = False          # FP8 (E4M3, per-token scale) dispatch payload
    num_shared_experts: int = 0       # DeepSeek-style always-on experts
    shared_intermediate_dim: int = 0
    norm_topk_prob: bool = True

    def validate(self) -> "MoeConfig":
        _require(1 <= self.num_experts <= 256, "num_experts must be in [1, 256]")
        _require(1 <= self.num_experts_per_token <= 8, "num_experts_per_token must be in [1, 8]")
        _require(self.num_experts_per_token <= self.num_experts, "top-k exceeds expert count")
        _require(self.hidden_dim > 0 and self.intermediate_dim > 0, "dims must be positive")
        _require(self.capacity_factor > 0, "capacity_factor must be positive")
        return self


@dataclass
class FeedForwardType:
    """kind: 'dense' (up -> act -> down), 'gated' (SwiGLU) or 'moe'."""
    kind: str = "gated"
    intermediate_dim: int = 0
    activation: str = "silu"
    moe: Optional[MoeConfig] = None

    @staticmethod
    def dense(intermediate_dim: int, activation: str = "gelu") -> "FeedForwardType":
        return FeedForwardType("dense", intermediate_dim, activation)

    @staticmethod
    def gated(intermediate_dim: int) -> "FeedForwardType":
        return FeedForwardType("gated", intermediate_dim, "silu")

    @staticmethod
    def moe_(cfg: MoeConfig) -> "FeedForwardType":
        return FeedForwardType("moe", cfg.intermediate_dim, "silu", cfg)

    def validate(self) -> "FeedForwardType":
        _require(self.kind in ("dense", "gated", "moe"), f"unknown ff kind {self.kind}")
        if self.kind == "moe":
            _require(self.moe is not None, "moe ff needs a MoeConfig")
            self.moe.validate()
        else:
            _require(self.intermediate_dim > 0, "intermediate_dim must be positive")
        return self


@dataclass
class MlaConfig:
    num_heads: int
    head_dim: int            # non-rope part of the q/k head
    v_head_dim: int
    hidden_size: int
    kv_lora_rank: int
    q_lora_rank: int         # 0 = no q compression
    rope_head_dim: int
    rope_theta: float = 10000.0
    max_seq_len: int = 4096

    def validate(self) -> "MlaConfig":
        _require(self.num_heads > 0 and self.head_dim > 0 and self.v_head_dim > 0, "bad head dims")
        _require(self.kv_lora_rank > 0 and self.rope_head_dim % 2 == 0, "bad latent dims")
        return self


@dataclass
class TransformerConfig:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    num_layers: int
    vocab_size: int
    max_seq_len: int = 4096
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    ff_type: FeedForwardType = field(default_factory=FeedForwardType)
    rope_traditional: bool = False
    sliding_window: int = 0          # 0 = full attention
    tie_embeddings: bool = False
    first_dense_layers: int = 0      # DeepSeek: leading layers use a dense FFN
    dense_intermediate_dim: int = 0  # FFN width of those layers
    mla: Optional[MlaConfig] = None
    name: str = "transformer"

    def validate(self) -> "TransformerConfig":
        _require(self.hidden_size > 0 and self.num_layers > 0 and self.vocab_size > 0, "bad sizes")
        _require(self.num_heads > 0 and self.num_kv_heads > 0, "head counts must be positive")
        _require(self.num_kv_heads <= self.num_heads, "num_kv_heads must be <= num_heads")
        _require(self.num_heads % self.num_kv_heads == 0, "num_heads must be a multiple of num_kv_heads")
        _require(self.head_dim % 2 == 0, "head_dim must be even for RoPE")
        self.ff_type.validate()
        if self.mla is not None:
            self.mla.validate()
        return self

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    def replace(self, **kw) -> "TransformerConfig":
        return dataclasses.replace(self, **kw)


@dataclass
class AttentionConfig:
    num_heads: int
    num_kv_heads: int
    head_dim: int
    max_seq_len: int = 4096
    rope_theta: float = 10000.0

    def validate(self) -> "AttentionConfig":
        _require(self.num_heads % self.num_kv_heads == 0, "heads must divide by kv heads")
        return self


@dataclass
class RotaryConfig:
    head_dim: int
    max_seq_len: int
    base_freq: float = 10000.0
    scale: float = 1.0
    traditional: bool = False


@dataclass
class QuantConfig:
    """MLX affine weight-only quantisation: w = scale * q + bias per group."""
    bits: int = 4
    group_size: int = 64

    def validate(self) -> "QuantConfig":
        _require(self.bits in (2, 3, 4, 6, 8), "bits must be one of 2,3,4,6,8")
        _require(self.group_size in (32, 64, 128), "group_size must be 32, 64 or 128")
        return self


@dataclass
class SchedulerConfig:
    max_batch_size: int = 64
    eos_token_id: int = -1
    block_size: int = 16
    max_prefill_chunk: int = 512

    def validate(self) -> "SchedulerConfig":
        _require(self.max_batch_size > 0 and self.block_size > 0, "bad scheduler sizes")
        _require(self.max_prefill_chunk > 0, "max_prefill_chunk must be positive")
        return self


@dataclass
class SamplerConfig:
    temperature: float = 0.0        # 0 = greedy
    top_k: int = 0                  # 0 = off
    top_p: float = 1.0              # 1 = off
    repetition_penalty: float = 1.0 # 1 = off
    seed: Optional[int] = None

    def validate(self) -> "SamplerConfig":
        _require(self.temperature >= 0, "temperature must be >= 0")
        _require(0 < self.top_p <= 1.0, "top_p must be in (0, 1]")
        _require(self.top_k >= 0, "top_k must be >= 0")
        _require(self.repetition_penalty > 0, "repetition_penalty must be > 0")
        return self


@dataclass
class InitConfig:
    """Process-group bring-up. Resolution order for rank/world: explicit fields, then RMLX_* env,
    then torchrun (RANK/WORLD_SIZE), then OMPI/PMI/SLURM env, else (0, 1)."""
    rank: Optional[int] = None
    world_size: Optional[int] = None
    backend: str = "auto"           # auto | nccl | gloo | loopback
    strict: bool = False            # fail instead of falling back to loopback
    master_addr: str = "127.0.0.1"
    master_port: int = 18520
    timeout_s: float = 120.0


# ------------------------------------------------------------------------------------------------
# Presets
# ------------------------------------------------------------------------------------------------
def tiny_dense_config() -> TransformerConfig:
    """The CPU plumbing config: hidden 256, 4 q / 2 kv heads, head_dim 64, SwiGLU 688, vocab 1024."""
    return TransformerConfig(hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, num_layers=2,
                             vocab_size=1024, max_seq_len=256, rope_theta=1e4, rms_norm_eps=1e-6,
                             ff_type=FeedForwardType.gated(688), name="tiny-dense").validate()


def moe_a22b_config(num_layers: int = 60, max_seq_len: int = 8192) -> TransformerConfig:
    """MoE-A22B-shaped decoder: hidden 4096, 64 q / 4 kv heads, head_dim 128, theta 1e6, 128 experts
    top-8 with expert SwiGLU width 1536, vocab 151936."""
    moe = MoeConfig(num_experts=128, num_experts_per_token=8, hidden_dim=4096, intermediate_dim=1536)
    return TransformerConfig(hidden_size=4096, num_heads=64, num_kv_heads=4, head_dim=128,
                             num_layers=num_layers, vocab_size=151936, max_seq_len=max_seq_len,
                             rope_theta=1e6, rms_norm_eps=1e-6, ff_type=FeedForwardType.moe_(moe),
                             name="moe-a22b").validate()
