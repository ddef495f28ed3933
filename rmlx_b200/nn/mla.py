"""Multi-head latent attention (DeepSeek): K/V are compressed to a latent ``c_kv`` of rank
``kv_lora_rank`` plus one decoupled RoPE key of ``rope_head_dim`` shared by all heads, and only
those are cached. Mirrors crates/rmlx-nn/src/mla.rs:47-730 (``MlaConfig``, ``MlaKvCache`` caching
``c_kv [seq, kv_lora_rank]`` and ``k_rope [seq, rope_head_dim]``, compress / expand / compute_q /
forward, compression-ratio helper at mla.rs:723)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from ..config import MlaConfig
from ..reference import ops as ref


class MlaKvCache:
    def __init__(self, cfg: MlaConfig, dtype=torch.bfloat16, device="cpu"):
        self.c_kv = torch.zeros(cfg.max_seq_len, cfg.kv_lora_rank, dtype=dtype, device=device)
        self.k_rope = torch.zeros(cfg.max_seq_len, cfg.rope_head_dim, dtype=dtype, device=device)
        self.seq_len = 0

    def append(self, c_kv: torch.Tensor, k_rope: torch.Tensor) -> None:
        n = c_kv.shape[0]
        self.c_kv[self.seq_len:self.seq_len + n] = c_kv.to(self.c_kv.dtype)
        self.k_rope[self.seq_len:self.seq_len + n] = k_rope.to(self.k_rope.dtype)
        self.seq_len += n

    def trim(self, n: int) -> None:
        self.seq_len = max(0, self.seq_len - n)


@dataclass
class MlaWeights:
    w_dkv: torch.Tensor          # [kv_lora_rank + rope_head_dim, hidden]   down-projection (+ rope key)
    kv_norm: torch.Tensor        # [kv_lora_rank]
    w_uk: torch.Tensor           # [heads * head_dim, kv_lora_rank]          latent -> keys
    w_uv: torch.Tensor           # [heads * v_head_dim, kv_lora_rank]        latent -> values
    w_q: Optional[torch.Tensor]  # [heads * (head_dim + rope_head_dim), hidden]  (q_lora_rank == 0)
    w_dq: Optional[torch.Tensor] = None    # [q_lora_rank, hidden]
    q_norm: Optional[torch.Tensor] = None  # [q_lora_rank]
    w_uq: Optional[torch.Tensor] = None    # [heads * (head_dim + rope_head_dim), q_lora_rank]
    w_o: Optional[torch.Tensor] = None     # [hidden, heads * v_head_dim]


def random_mla_weights(cfg: MlaConfig, seed: int = 0, std: float = 0.02, dtype=torch.float32) -> MlaWeights:
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) * std).to(dtype)
    h, qd = cfg.num_heads, cfg.head_dim + cfg.rope_head_dim
    w = MlaWeights(r(cfg.kv_lora_rank + cfg.rope_head_dim, cfg.hidden_size), torch.ones(cfg.kv_lora_rank, dtype=dtype),
                   r(h * cfg.head_dim, cfg.kv_lora_rank), r(h * cfg.v_head_dim, cfg.kv_lora_rank), None,
                   w_o=r(cfg.hidden_size, h * cfg.v_head_dim))
    if cfg.q_lora_rank:
        w.w_dq, w.q_norm, w.w_uq = r(cfg.q_lora_rank, cfg.hidden_size), torch.ones(cfg.q_lora_rank, dtype=dtype), r(h * qd, cfg.q_lora_rank)
    else:
        w.w_q = r(h * qd, cfg.hidden_size)
    return w


class MlaAttention:
    def __init__(self, cfg: MlaConfig, w: MlaWeights, eps: float = 1e-6):
        self.cfg, self.w, self.eps = cfg.validate(), w, eps
        self.cos, self.sin = ref.rope_tables(cfg.rope_head_dim, cfg.max_seq_len, cfg.rope_theta,
                                             device=w.w_dkv.device)
        self.scale = 1.0 / math.sqrt(cfg.head_dim + cfg.rope_head_dim)

    def compression_ratio(self, num_kv_heads: Optional[int] = None) -> float:
        """Bytes of a standard KV cache per token divided by bytes of the latent cache."""
        c = self.cfg
        std = 2 * (num_kv_heads or c.num_heads) * c.head_dim
        return std / (c.kv_lora_rank + c.rope_head_dim)

    def compress(self, x: torch.Tensor, pos: torch.Tensor):
        c = self.cfg
        ckr = x @ self.w.w_dkv.to(x.dtype).t()
        c_kv = ref.rms_norm(ckr[:, :c.kv_lora_rank], self.w.kv_norm, self.eps)
        k_rope = ref.apply_rope(ckr[:, None, c.kv_lora_rank:], pos, self.cos, self.sin).squeeze(1)
        return c_kv, k_rope

    def expand(self, c_kv: torch.Tensor):
        c = self.cfg
        k = (c_kv @ self.w.w_uk.to(c_kv.dtype).t()).view(-1, c.num_heads, c.head_dim)
        v = (c_kv @ self.w.w_uv.to(c_kv.dtype).t()).view(-1, c.num_heads, c.v_head_dim)
        return k, v

    def compute_q(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        c, w = self.cfg, self.w
        if w.w_dq is not None:
            q = ref.rms_norm(x @ w.w_dq.to(x.dtype).t(), w.q_norm, self.eps) @ w.w_uq.to(x.dtype).t()
        else:
            q = x @ w.w_q.to(x.dtype).t()
        q = q.view(-1, c.num_heads, c.head_dim + c.rope_head_dim)
        q_rope = ref.apply_rope(q[..., c.head_dim:], pos, self.cos, self.sin)
        return torch.cat([q[..., :c.head_dim], q_rope], -1)

    def forward(self, x: torch.Tensor, cache: Optional[MlaKvCache] = None) -> torch.Tensor:
        c = self.cfg
        t = x.shape[0]
        start = cache.seq_len if cache is not None else 0
        pos = torch.arange(start, start + t, device=x.device)
        c_kv, k_rope = self.compress(x, pos)
        if cache is not None:
            cache.append(c_kv, k_rope)
            c_all, kr_all = cache.c_kv[:cache.seq_len].to(x.dtype), cache.k_rope[:cache.seq_len].to(x.dtype)
        else:
            c_all, kr_all = c_kv, k_rope
        k_nope, v = self.expand(c_all)
        k = torch.cat([k_nope, kr_all[:, None, :].expand(-1, c.num_heads, -1)], -1)
        q = self.compute_q(x, pos)
        out = ref.sdpa(q, k, v, self.scale, start)              # v_head_dim may differ from head_dim
        return out.reshape(t, -1) @ self.w.w_o.to(x.dtype).t()

    __call__ = forward
