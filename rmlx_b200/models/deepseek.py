"""DeepSeek-V3-style model: multi-head latent attention, a routed MoE with a shared expert, and
dense feed-forward in the first layers (crates/rmlx-nn/src/models/deepseek.rs:30-490). The preset
``deepseek_v3()`` is the published shape (hidden 7168, 128 heads, 61 layers, 256 experts top-8 of
width 2048, kv_lora 512, q_lora 1536, rope head 64, v head 128, one shared expert, first layer
dense). ``forward`` is the library-kernel path (PyTorch ops) with a contiguous latent cache; the
routed experts run through ``MoeLayer`` and therefore through this package's grouped kernels on
CUDA. ``new_paged_cache`` / ``prefill_paged`` / ``decode_paged`` keep the latents in pages and run
the decode attention in the absorbed form on the latent-attention kernel
(csrc/kernels/mla_decode.cu) for several sequences per step."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..config import MlaConfig, MoeConfig
from ..nn.mla import MlaAttention, MlaKvCache, MlaPagedCache, mla_decode_paged, random_mla_weights
from ..nn.moe import ExpertGroup, MoeLayer, MoeStrategy
from ..ops.weights import LinearWeight
from ..reference import ops as ref


@dataclass
class DeepSeekV3Config:
    hidden_size: int = 7168
    num_layers: int = 61
    vocab_size: int = 129280
    num_heads: int = 128
    head_dim: int = 128
    v_head_dim: int = 128
    kv_lora_rank: int = 512
    q_lora_rank: int = 1536
    rope_head_dim: int = 64
    rope_theta: float = 10000.0
    max_seq_len: int = 4096
    num_experts: int = 256
    num_experts_per_token: int = 8
    moe_intermediate: int = 2048
    capacity_factor: float = 1.25
    num_shared_experts: int = 1
    first_dense_layers: int = 1
    dense_intermediate: int = 18432
    rms_norm_eps: float = 1e-6

    def mla(self) -> MlaConfig:
        return MlaConfig(self.num_heads, self.head_dim, self.v_head_dim, self.hidden_size,
                         self.kv_lora_rank, self.q_lora_rank, self.rope_head_dim, self.rope_theta,
                         self.max_seq_len).validate()

    def moe(self) -> MoeConfig:
        return MoeConfig(self.num_experts, self.num_experts_per_token, self.hidden_size,
                         self.moe_intermediate, self.capacity_factor,
                         num_shared_experts=self.num_shared_experts,
                         shared_intermediate_dim=self.moe_intermediate).validate()


def deepseek_v3() -> DeepSeekV3Config:
    return DeepSeekV3Config()


def deepseek_tiny() -> DeepSeekV3Config:
    return DeepSeekV3Config(hidden_size=64, num_layers=3, vocab_size=256, num_heads=4, head_dim=16,
                            v_head_dim=24, kv_lora_rank=32, q_lora_rank=24, rope_head_dim=8,
                            max_seq_len=64, num_experts=8, num_experts_per_token=2, moe_intermediate=32,
                            first_dense_layers=1, dense_intermediate=96)


@dataclass
class DeepSeekBlock:
    norm1: torch.Tensor
    attn: MlaAttention
    norm2: torch.Tensor
    moe: Optional[MoeLayer] = None
    dense_gate_up: Optional[torch.Tensor] = None
    dense_down: Optional[torch.Tensor] = None


class DeepSeekV3Model:
    def __init__(self, cfg: DeepSeekV3Config, seed: int = 0, dtype=torch.float32, device="cpu", std=0.02):
        """Random-init model (weights N(0, std)); real checkpoints map onto the same fields."""
        self.cfg = cfg
        g = torch.Generator().manual_seed(seed)
        r = lambda *s: (torch.randn(*s, generator=g) * std).to(dtype).to(device)
        d = cfg.hidden_size
        self.embed = r(cfg.vocab_size, d)
        self.final_norm = torch.ones(d, dtype=dtype, device=device)
        self.lm_head = r(cfg.vocab_size, d)
        self.blocks: List[DeepSeekBlock] = []
        for i in range(cfg.num_layers):
            w = random_mla_weights(cfg.mla(), seed * 1000 + i, std, dtype)
            for f in w.__dataclass_fields__:
                v = getattr(w, f)
                if v is not None:
                    setattr(w, f, v.to(device))
            blk = DeepSeekBlock(torch.ones(d, dtype=dtype, device=device), MlaAttention(cfg.mla(), w, cfg.rms_norm_eps),
                                torch.ones(d, dtype=dtype, device=device))
            if i < cfg.first_dense_layers:
                blk.dense_gate_up, blk.dense_down = r(2 * cfg.dense_intermediate, d), r(d, cfg.dense_intermediate)
            else:
                m = cfg.moe()
                experts = ExpertGroup(LinearWeight.from_dense(r(m.num_experts, 2 * m.intermediate_dim, d).cpu(), None, dtype, device),
                                      LinearWeight.from_dense(r(m.num_experts, d, m.intermediate_dim).cpu(), None, dtype, device))
                layer = MoeLayer(m, r(m.num_experts, d) * 5, experts, MoeStrategy.GROUPED)
                si = m.shared_intermediate_dim * m.num_shared_experts
                if si:
                    layer.with_shared_expert(LinearWeight.from_dense(r(2 * si, d).cpu(), None, dtype, device),
                                             LinearWeight.from_dense(r(d, si).cpu(), None, dtype, device))
                blk.moe = layer
            self.blocks.append(blk)

    def new_cache(self, dtype=None) -> List[MlaKvCache]:
        return [MlaKvCache(self.cfg.mla(), dtype or self.embed.dtype, self.embed.device)
                for _ in self.blocks]

    @torch.no_grad()
    def forward(self, token_ids: torch.Tensor, cache: Optional[List[MlaKvCache]] = None) -> torch.Tensor:
        eps = self.cfg.rms_norm_eps
        h = self.embed[token_ids.long()]
        for i, b in enumerate(self.blocks):
            h = h + b.attn(ref.rms_norm(h, b.norm1, eps), None if cache is None else cache[i])
            xn = ref.rms_norm(h, b.norm2, eps)
            if b.moe is not None:
                h = h + b.moe.forward(xn)
            else:
                h = h + ref.swiglu(xn @ b.dense_gate_up.t()) @ b.dense_down.t()
        return (ref.rms_norm(h, self.final_norm, eps) @ self.lm_head.t()).float()

    # ------------------------------------------------------------------ paged latent cache
    def new_paged_cache(self, num_blocks: int, max_seqs: int = 8, dtype=None) -> List[MlaPagedCache]:
        return [MlaPagedCache(self.cfg.mla(), num_blocks, max_seqs, dtype=dtype or self.embed.dtype,
                              device=self.embed.device) for _ in self.blocks]

    def _ffn(self, b: DeepSeekBlock, h: torch.Tensor) -> torch.Tensor:
        xn = ref.rms_norm(h, b.norm2, self.cfg.rms_norm_eps)
        if b.moe is not None:
            return h + b.moe.forward(xn)
        return h + ref.swiglu(xn @ b.dense_gate_up.t()) @ b.dense_down.t()

    @torch.no_grad()
    def prefill_paged(self, token_ids: torch.Tensor, cache: List[MlaPagedCache], seq_id: int) -> torch.Tensor:
        """Run a prompt for ``seq_id`` (added to every layer's cache here), filling its latent
        pages. Returns the last token's logits [1, vocab]."""
        eps = self.cfg.rms_norm_eps
        h = self.embed[token_ids.long()]
        n = token_ids.numel()
        for i, b in enumerate(self.blocks):
            xn = ref.rms_norm(h, b.norm1, eps)
            cache[i].add_sequence(seq_id)
            cache[i].append(seq_id, *b.attn.compress(xn, torch.arange(n, device=h.device)))
            h = self._ffn(b, h + b.attn(xn, None))          # causal attention over the prompt itself
        return (ref.rms_norm(h[-1:], self.final_norm, eps) @ self.lm_head.t()).float()

    @torch.no_grad()
    def decode_paged(self, token_ids: torch.Tensor, cache: List[MlaPagedCache], seq_ids) -> torch.Tensor:
        """One token per sequence: token_ids [B] (row b continues sequence seq_ids[b]).
        Returns logits [B, vocab]."""
        eps = self.cfg.rms_norm_eps
        h = self.embed[token_ids.long()]
        for i, b in enumerate(self.blocks):
            h = h + mla_decode_paged(b.attn, ref.rms_norm(h, b.norm1, eps), cache[i], list(seq_ids))
            h = self._ffn(b, h)
        return (ref.rms_norm(h, self.final_norm, eps) @ self.lm_head.t()).float()
