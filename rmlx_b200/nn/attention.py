"""Attention module and the non-paged KV cache family.

Caches (crates/rmlx-nn/src/attention.rs:27-245,970-1080,1592-1700,4417-4680):
  * ``LayerKvCache``      pre-allocated contiguous slabs ``[kv_heads, max_seq, head_dim]``, O(1)
                          append, ``trim``; ``seq_len`` doubles as the RoPE position offset
  * ``RotatingKvCache``   ring buffer of ``max_size`` tokens that pins the first ``keep`` tokens
                          (sliding-window models)
  * ``BatchKvCache``      one cache per sequence with ``filter`` / ``extend`` / ``offsets``
  * ``QuantizedKvCache``  K/V stored in 4- or 8-bit groups of 64 with bf16 scale and bias,
                          quantised on append (the reference keeps an fp32 shadow and re-quantises)
The paged cache lives in ``kv.paged``. ``Attention`` is MHA / GQA with a merged QKV weight,
RoPE, an optional sliding window, and the scaled-dot-product core (flash kernels on CUDA through
the paged path of the transformer model; the PyTorch core here serves slabs and the CPU).
Sliding-window masks: crates/rmlx-nn/src/sliding_window.rs:25-160.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence

import torch

from ..config import AttentionConfig
from ..ops.weights import LinearWeight
from ..reference import ops as ref
from .layers import Linear, RotaryEmbedding


class LayerKvCache:
    def __init__(self, kv_heads: int, head_dim: int, max_seq: int, dtype=torch.bfloat16, device="cpu"):
        self.k = torch.zeros(kv_heads, max_seq, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros(kv_heads, max_seq, head_dim, dtype=dtype, device=device)
        self.max_seq, self.seq_len = max_seq, 0

    @classmethod
    def preallocated(cls, kv_heads, head_dim, max_seq, dtype=torch.bfloat16, device="cpu"):
        return cls(kv_heads, head_dim, max_seq, dtype, device)

    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v: [n, kv_heads, head_dim]."""
        n = k.shape[0]
        if self.seq_len + n > self.max_seq:
            raise ValueError("KV cache overflow")
        self.k[:, self.seq_len:self.seq_len + n] = k.transpose(0, 1).to(self.k.dtype)
        self.v[:, self.seq_len:self.seq_len + n] = v.transpose(0, 1).to(self.v.dtype)
        self.seq_len += n

    def keys(self) -> torch.Tensor:      # [seq, kv_heads, head_dim]
        return self.k[:, :self.seq_len].transpose(0, 1)

    def values(self) -> torch.Tensor:
        return self.v[:, :self.seq_len].transpose(0, 1)

    def positions(self) -> torch.Tensor:
        return torch.arange(self.seq_len, device=self.k.device)

    def trim(self, n: int) -> None:
        self.seq_len = max(0, self.seq_len - n)


class RotatingKvCache:
    """Keeps the first ``keep`` tokens and the most recent ``max_size - keep``."""

    def __init__(self, kv_heads: int, head_dim: int, max_size: int, keep: int = 0,
                 dtype=torch.bfloat16, device="cpu"):
        assert 0 <= keep < max_size
        self.k = torch.zeros(max_size, kv_heads, head_dim, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.pos = torch.zeros(max_size, dtype=torch.int64, device=device)
        self.max_size, self.keep, self.seq_len = max_size, keep, 0   # seq_len = tokens ever seen

    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:
        for i in range(k.shape[0]):
            t = self.seq_len
            slot = t if t < self.max_size else self.keep + (t - self.keep) % (self.max_size - self.keep)
            self.k[slot], self.v[slot], self.pos[slot] = k[i].to(self.k.dtype), v[i].to(self.v.dtype), t
            self.seq_len += 1

    def _order(self) -> torch.Tensor:
        n = min(self.seq_len, self.max_size)
        return torch.argsort(self.pos[:n])

    def keys(self) -> torch.Tensor:
        return self.k[:min(self.seq_len, self.max_size)][self._order()]

    def values(self) -> torch.Tensor:
        return self.v[:min(self.seq_len, self.max_size)][self._order()]

    def positions(self) -> torch.Tensor:
        return self.pos[:min(self.seq_len, self.max_size)][self._order()]


class BatchKvCache:
    def __init__(self, make_cache):
        self._make = make_cache
        self.caches: List[LayerKvCache] = []

    def extend(self, n: int = 1) -> None:
        self.caches.extend(self._make() for _ in range(n))

    def filter(self, keep: Sequence[int]) -> None:
        self.caches = [self.caches[i] for i in keep]

    def offsets(self) -> List[int]:
        return [c.seq_len for c in self.caches]

    def __getitem__(self, i):
        return self.caches[i]

    def __len__(self):
        return len(self.caches)


class QuantizedKvCache:
    def __init__(self, kv_heads: int, head_dim: int, max_seq: int, bits: int = 8, group: int = 64,
                 device="cpu"):
        assert bits in (4, 8) and head_dim % group == 0
        self.bits, self.group, self.max_seq, self.seq_len = bits, group, max_seq, 0
        g = head_dim // group
        shp = (max_seq, kv_heads, head_dim)
        self.qk = torch.zeros(shp, dtype=torch.uint8, device=device)
        self.qv = torch.zeros(shp, dtype=torch.uint8, device=device)
        self.sk = torch.zeros(max_seq, kv_heads, g, 2, dtype=torch.bfloat16, device=device)
        self.sv = torch.zeros_like(self.sk)

    def _quant(self, x: torch.Tensor):
        n, h, d = x.shape
        xf = x.float().view(n, h, d // self.group, self.group)
        lo, hi = xf.amin(-1, keepdim=True), xf.amax(-1, keepdim=True)
        levels = (1 << self.bits) - 1
        scale = ((hi - lo) / levels).clamp_min(1e-8).to(torch.bfloat16).float()
        bias = lo.to(torch.bfloat16).float()
        q = torch.clamp(torch.round((xf - bias) / scale), 0, levels).to(torch.uint8).view(n, h, d)
        return q, torch.cat([scale, bias], -1).to(torch.bfloat16)

    def _dequant(self, q, sb):
        n, h, d = q.shape
        qf = q.float().view(n, h, d // self.group, self.group)
        return (qf * sb[..., 0:1].float() + sb[..., 1:2].float()).view(n, h, d)

    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:
        n = k.shape[0]
        sl = slice(self.seq_len, self.seq_len + n)
        self.qk[sl], self.sk[sl] = self._quant(k)
        self.qv[sl], self.sv[sl] = self._quant(v)
        self.seq_len += n

    def keys(self) -> torch.Tensor:
        return self._dequant(self.qk[:self.seq_len], self.sk[:self.seq_len])

    def values(self) -> torch.Tensor:
        return self._dequant(self.qv[:self.seq_len], self.sv[:self.seq_len])

    def positions(self) -> torch.Tensor:
        return torch.arange(self.seq_len, device=self.qk.device)

    def trim(self, n: int) -> None:
        self.seq_len = max(0, self.seq_len - n)

    def nbytes_per_token(self) -> float:
        h, d = self.qk.shape[1:]
        return 2 * (h * d * self.bits / 8 + h * (d // self.group) * 4)


def sliding_window_mask(q_len: int, kv_len: int, window: int, offset: int = 0, device=None) -> torch.Tensor:
    """Additive mask [q_len, kv_len]: query i (absolute position offset+i) sees keys j with
    pos-window < j <= pos."""
    qi = torch.arange(q_len, device=device)[:, None] + offset
    kj = torch.arange(kv_len, device=device)[None, :]
    ok = (kj <= qi) & (kj > qi - window)
    return torch.where(ok, 0.0, float("-inf"))


class Attention:
    def __init__(self, cfg: AttentionConfig, wqkv: LinearWeight, wo: LinearWeight,
                 window: int = 0, traditional_rope: bool = False, device=None):
        self.cfg = cfg.validate()
        self.qkv, self.o = Linear(wqkv), Linear(wo)
        self.window = window
        self.rope = RotaryEmbedding(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta,
                                    traditional=traditional_rope, device=device)
        self.scale = 1.0 / math.sqrt(cfg.head_dim)

    def forward(self, x: torch.Tensor, cache=None) -> torch.Tensor:
        """x [T, hidden] for one sequence; appends to ``cache`` (any cache class above)."""
        c = self.cfg
        hq, hkv, hd = c.num_heads, c.num_kv_heads, c.head_dim
        t = x.shape[0]
        start = cache.seq_len if cache is not None else 0
        pos = torch.arange(start, start + t, device=x.device)
        qkv = self.qkv(x)
        q = self.rope(qkv[:, :hq * hd].reshape(t, hq, hd), pos)
        k = self.rope(qkv[:, hq * hd:(hq + hkv) * hd].reshape(t, hkv, hd), pos)
        v = qkv[:, (hq + hkv) * hd:].reshape(t, hkv, hd)
        if cache is None:
            out = ref.sdpa(q, k, v, self.scale, 0, self.window)
        else:
            cache.append(k, v)
            kk, vv, kpos = cache.keys(), cache.values(), cache.positions()
            # general positions (rotating caches are not contiguous): build the mask explicitly
            qpos = pos[:, None]
            ok = kpos[None, :] <= qpos
            if self.window > 0:
                ok &= kpos[None, :] > qpos - self.window
            mask = torch.where(ok, 0.0, float("-inf"))
            out = ref.sdpa(q, kk.to(q.dtype), vv.to(q.dtype), self.scale, None, 0, mask)
        return self.o(out.reshape(t, hq * hd))

    __call__ = forward


@dataclass
class SlidingWindowAttentionConfig:
    """An attention config plus the window (crates/rmlx-nn/src/sliding_window.rs:25-36)."""
    base: AttentionConfig
    window_size: int

    def validate(self) -> "SlidingWindowAttentionConfig":
        self.base.validate()
        if self.window_size <= 0:
            raise ValueError("SlidingWindowAttention: window_size must be positive")
        return self


class SlidingWindowAttention(Attention):
    """Mistral-style attention: query i sees the keys of positions i - window + 1 .. i
    (crates/rmlx-nn/src/sliding_window.rs:37-160). With a ``RotatingKvCache`` of the window's size
    the cache never grows beyond it. On the device the same window is applied inside the flash
    kernels (``TransformerConfig.sliding_window``); this class is the layer-level form."""

    def __init__(self, config: SlidingWindowAttentionConfig, wqkv: LinearWeight, wo: LinearWeight,
                 traditional_rope: bool = False, device=None):
        self.sw_config = config.validate()
        super().__init__(config.base, wqkv, wo, window=config.window_size,
                         traditional_rope=traditional_rope, device=device)

    @classmethod
    def from_projections(cls, config: SlidingWindowAttentionConfig, wq: torch.Tensor, wk: torch.Tensor,
                         wv: torch.Tensor, wo: torch.Tensor, device=None) -> "SlidingWindowAttention":
        """Separate q / k / v / o projection matrices ([out, in]) stacked into the merged form."""
        wqkv = LinearWeight.from_dense(torch.cat([wq, wk, wv], 0), None, device=device)
        return cls(config, wqkv, LinearWeight.from_dense(wo, None, device=device), device=device)

    def window_size(self) -> int:
        return self.sw_config.window_size

    def base_config(self) -> AttentionConfig:
        return self.sw_config.base

    def build_sliding_window_mask(self, q_len: int, kv_len: int, offset: int = 0, device=None) -> torch.Tensor:
        return sliding_window_mask(q_len, kv_len, self.window, offset, device)

    def new_cache(self, chunk: int = 1, device="cpu", dtype=torch.float32) -> "RotatingKvCache":
        """A ring that holds what the layer needs when it is fed at most ``chunk`` tokens per call:
        window + chunk - 1 positions (the first query of a chunk still needs the window before it
        after the chunk's own keys have been appended)."""
        c = self.cfg
        return RotatingKvCache(c.num_kv_heads, c.head_dim, self.window + max(1, chunk) - 1, dtype=dtype,
                               device=device)
