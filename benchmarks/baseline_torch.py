"""The same MoE decoder written with library calls only: bf16 ``F.linear`` / ``torch.bmm`` (cuBLAS),
``scaled_dot_product_attention``, ``torch.topk`` and ``torch.distributed.all_reduce`` (NCCL), launched
eagerly. No kernel, engine or weight container of this package is used: this is the
"NCCL + cuBLAS PyTorch build of the same model on the same box" that the fused path is measured
against (the reference runs its baseline and Split-CB arms in one binary the same way,
crates/rmlx-nn/benches/distributed_bench.rs:45-54).

Tensor-parallel layout: query heads, the expert intermediate dimension and the vocabulary are split
over the ranks; a rank keeps the KV head(s) its query heads use; two all-reduces per layer.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F


class TorchMoeDecoder:
    def __init__(self, *, layers: int, hidden: int, heads: int, kv_heads: int, head_dim: int,
                 experts: int, top_k: int, inter: int, vocab: int, max_len: int, batch: int,
                 rank: int, world: int, device, theta: float = 1e6, eps: float = 1e-6,
                 std: float = 0.02, seed: int = 0):
        self.L, self.D, self.hd = layers, hidden, head_dim
        self.rank, self.world, self.dev, self.eps = rank, world, device, eps
        self.hq = heads // world
        self.hkv = max(1, kv_heads // world)
        self.E, self.k, self.I = experts, top_k, inter // world
        self.V = vocab // world if world > 1 else vocab
        self.vocab_base = rank * self.V if world > 1 else 0
        self.B, self.max_len = batch, max_len
        g = torch.Generator(device=device).manual_seed(seed * 7919 + rank)
        bf = dict(dtype=torch.bfloat16, device=device)

        def rnd(*shape):
            t = torch.empty(*shape, **bf)
            flat = t.view(-1, shape[-1])
            step = max(1, (1 << 28) // shape[-1])
            for r in range(0, flat.shape[0], step):
                flat[r:r + step].normal_(0.0, std, generator=g)
            return t

        self.embed = rnd(vocab, hidden)
        self.layers = []
        for _ in range(layers):
            self.layers.append(dict(
                n1=torch.ones(hidden, **bf), n2=torch.ones(hidden, **bf),
                wqkv=rnd((self.hq + 2 * self.hkv) * head_dim, hidden),
                wo=rnd(hidden, self.hq * head_dim),
                router=rnd(experts, hidden),
                gu=rnd(experts, 2 * self.I, hidden),
                dn=rnd(experts, hidden, self.I),
                k=torch.zeros(batch, self.hkv, max_len, head_dim, **bf),
                v=torch.zeros(batch, self.hkv, max_len, head_dim, **bf)))
        self.norm_f = torch.ones(hidden, **bf)
        self.lm_head = rnd(self.V, hidden)
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
        t = torch.arange(max_len, device=device).float()
        fr = torch.outer(t, inv)
        self.cos, self.sin = fr.cos(), fr.sin()
        self.scale = 1.0 / math.sqrt(head_dim)

    def nbytes(self) -> int:
        n = self.embed.numel() + self.lm_head.numel()
        for l in self.layers:
            n += sum(l[k].numel() for k in ("wqkv", "wo", "router", "gu", "dn"))
        return 2 * n

    def fill_context(self, ctx: int) -> None:
        for l in self.layers:
            l["k"][:, :, :ctx].normal_(0, 1)
            l["v"][:, :, :ctx].normal_(0, 1)

    def _rms(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * w

    def _rope(self, x, pos):
        # x [B, H, D]; rotate halves (non-interleaved layout)
        c, s = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        x1, x2 = x[..., :self.hd // 2].float(), x[..., self.hd // 2:].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(x.dtype)

    @torch.no_grad()
    def step(self, tokens: torch.Tensor, pos: int) -> torch.Tensor:
        """One decode step for ``tokens`` [B] at position ``pos`` (same for all rows). Returns the
        next tokens [B] (greedy)."""
        B, hq, hkv, hd = self.B, self.hq, self.hkv, self.hd
        h = self.embed[tokens]
        posv = torch.full((B,), pos, device=self.dev, dtype=torch.long)
        for l in self.layers:
            x = self._rms(h, l["n1"])
            qkv = F.linear(x, l["wqkv"])
            q = qkv[:, :hq * hd].view(B, hq, hd)
            k = qkv[:, hq * hd:(hq + hkv) * hd].view(B, hkv, hd)
            v = qkv[:, (hq + hkv) * hd:].view(B, hkv, hd)
            q, k = self._rope(q, posv), self._rope(k, posv)
            l["k"][:, :, pos] = k
            l["v"][:, :, pos] = v
            o = F.scaled_dot_product_attention(q[:, :, None, :], l["k"][:, :, :pos + 1],
                                               l["v"][:, :, :pos + 1], scale=self.scale,
                                               enable_gqa=True)
            a = F.linear(o.reshape(B, hq * hd), l["wo"])
            if self.world > 1:
                dist.all_reduce(a)
            h = h + a
            x = self._rms(h, l["n2"])
            probs = torch.softmax(F.linear(x, l["router"]).float(), -1)
            w, idx = torch.topk(probs, self.k, dim=-1)
            w = (w / w.sum(-1, keepdim=True)).to(h.dtype)
            gu = torch.matmul(l["gu"][idx], x[:, None, :, None]).squeeze(-1)      # [B, k, 2I]
            act = F.silu(gu[..., :self.I]) * gu[..., self.I:]
            dn = torch.matmul(l["dn"][idx], act[..., None]).squeeze(-1)           # [B, k, D]
            y = (dn * w[..., None]).sum(1)
            if self.world > 1:
                dist.all_reduce(y)
            h = h + y
        logits = F.linear(self._rms(h, self.norm_f), self.lm_head).float()
        val, idx = logits.max(-1)
        if self.world > 1:
            vals = torch.empty(self.world, B, device=self.dev)
            idxs = torch.empty(self.world, B, device=self.dev, dtype=torch.long)
            dist.all_gather_into_tensor(vals, val)
            dist.all_gather_into_tensor(idxs, idx + self.vocab_base)
            best = vals.argmax(0)
            idx = idxs.gather(0, best[None]).squeeze(0)
        return idx


def time_decode(model: TorchMoeDecoder, ctx: int, steps: int, warmup: int, windows: int = 1):
    """Device-timed decode steps (CUDA events); returns the list of per-window ms per step."""
    B = model.B
    tok = torch.ones(B, device=model.dev, dtype=torch.long)
    pos = ctx
    for _ in range(warmup):
        tok = model.step(tok, pos)
        pos += 1
    out = []
    for _ in range(windows):
        if model.world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            tok = model.step(tok, pos)
            pos += 1
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / steps)
    return out
