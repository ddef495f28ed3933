"""Plain PyTorch restatements of every hot op, used as the numerics oracle (fp32 on CPU) and as the
building blocks of the library-kernel baseline model. Nothing here launches a kernel of this
package.

Semantics follow the reference's kernels: RMSNorm (crates/rmlx-core/src/ops/rms_norm.rs), RoPE in
split-half or traditional layout with ``inv_freq[k] = base^(-2k/head_dim)``
(crates/rmlx-core/src/ops/rope.rs:15-60), GQA head mapping ``kv = h * kv_heads / heads``
(crates/rmlx-core/src/ops/sdpa.rs:832), SwiGLU, MLX affine quantisation ``w = s*q + b`` with
little-endian nibble packing (crates/rmlx-core/src/ops/quantized.rs:1-11,63-177), and the router:
softmax over all experts, k rounds of arg-max with the first index winning ties, weights
renormalised to sum 1 (crates/rmlx-core/src/ops/topk_route.rs:242-343).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


# ------------------------------------------------------------------------------------------------
# Norms / activations
# ------------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * w.float()
    return y.to(x.dtype)


def layer_norm(x, w, b, eps: float = 1e-5):
    return torch.nn.functional.layer_norm(x.float(), x.shape[-1:], None if w is None else w.float(),
                                          None if b is None else b.float(), eps).to(x.dtype)


def silu(x):
    return x * torch.sigmoid(x)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """gate_up[..., :I] is the gate, [..., I:] the up projection."""
    i = gate_up.shape[-1] // 2
    g, u = gate_up[..., :i].float(), gate_up[..., i:].float()
    return (silu(g) * u).to(gate_up.dtype)


# ------------------------------------------------------------------------------------------------
# RoPE
# ------------------------------------------------------------------------------------------------
def rope_tables(head_dim: int, max_pos: int, base: float = 10000.0, scale: float = 1.0,
                device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [max_pos, head_dim/2] in fp32 (computed in fp64)."""
    k = torch.arange(head_dim // 2, dtype=torch.float64, device=device)
    inv_freq = base ** (-2.0 * k / head_dim)
    pos = torch.arange(max_pos, dtype=torch.float64, device=device) * scale
    ang = pos[:, None] * inv_freq[None, :]
    return ang.cos().float(), ang.sin().float()


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
               traditional: bool = False, inverse: bool = False) -> torch.Tensor:
    """x: [T, H, D]; positions: [T] (long)."""
    c = cos[positions][:, None, :].float()
    s = sin[positions][:, None, :].float()
    if inverse:
        s = -s
    xf = x.float()
    if traditional:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack((a * c - b * s, b * c + a * s), dim=-1).flatten(-2)
    else:
        h = x.shape[-1] // 2
        a, b = xf[..., :h], xf[..., h:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return out.to(x.dtype)


# ------------------------------------------------------------------------------------------------
# Attention
# ------------------------------------------------------------------------------------------------
def sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, causal_offset: Optional[int],
         window: int = 0, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q: [Tq, Hq, D]; k, v: [Tk, Hkv, D]. Query i sits at absolute position causal_offset + i and
    sees keys j <= that position (and within ``window`` of it when window > 0). causal_offset None
    means no causal mask."""
    tq, hq, d = q.shape
    tk, hkv, _ = k.shape
    g = hq // hkv
    qf = q.float().view(tq, hkv, g, d).permute(1, 2, 0, 3)          # [Hkv, G, Tq, D]
    kf = k.float().permute(1, 0, 2)[:, None]                         # [Hkv, 1, Tk, D]
    vf = v.float().permute(1, 0, 2)[:, None]
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale               # [Hkv, G, Tq, Tk]
    if causal_offset is not None:
        qi = torch.arange(tq, device=q.device)[:, None] + causal_offset
        kj = torch.arange(tk, device=q.device)[None, :]
        allowed = kj <= qi
        if window > 0:
            allowed &= kj > qi - window
        s = s.masked_fill(~allowed, float("-inf"))
    if mask is not None:
        s = s + mask.float()
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf.expand(-1, g, -1, -1))                    # [Hkv, G, Tq, D]
    return o.permute(2, 0, 1, 3).reshape(tq, hq, v.shape[-1]).to(q.dtype)


def gather_paged(cache: torch.Tensor, block_table_row: torch.Tensor, length: int) -> torch.Tensor:
    """cache: [blocks, Hkv, page, D] -> contiguous [length, Hkv, D] for one sequence."""
    page = cache.shape[2]
    nblk = (length + page - 1) // page
    blocks = cache[block_table_row[:nblk].long()]                    # [nblk, Hkv, page, D]
    return blocks.permute(0, 2, 1, 3).reshape(nblk * page, cache.shape[1], cache.shape[3])[:length]


# ------------------------------------------------------------------------------------------------
# MLX affine quantisation (weight-only)
# ------------------------------------------------------------------------------------------------
def quantize_affine(w: torch.Tensor, bits: int = 4, group_size: int = 64
                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """w: [N, K] -> (packed int32 [N, K*bits/32], scales [N, K/group], biases [N, K/group]).
    Per group: scale = (max - min) / (2^bits - 1), bias = min; element i of a word sits at bit
    i*bits (little-endian)."""
    assert 32 % bits == 0, "packing here covers power-of-two widths"
    n, k = w.shape
    assert k % group_size == 0
    wf = w.float().view(n, k // group_size, group_size)
    lo, hi = wf.amin(-1, keepdim=True), wf.amax(-1, keepdim=True)
    levels = (1 << bits) - 1
    scale = ((hi - lo) / levels).clamp_min(1e-8)
    scale = scale.to(torch.bfloat16).float()       # what the kernels will see
    bias = lo.to(torch.bfloat16).float()
    q = torch.clamp(torch.round((wf - bias) / scale), 0, levels).to(torch.int64).view(n, k)
    per = 32 // bits
    q = q.view(n, k // per, per)
    shifts = (torch.arange(per, dtype=torch.int64) * bits).to(w.device)
    packed = (q << shifts).sum(-1)
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
    return packed, scale.squeeze(-1).to(torch.bfloat16), bias.squeeze(-1).to(torch.bfloat16)


def dequantize_affine(packed: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                      bits: int = 4, group_size: int = 64) -> torch.Tensor:
    """Inverse of quantize_affine: fp32 [.., N, K]."""
    per = 32 // bits
    shifts = (torch.arange(per, dtype=torch.int64) * bits).to(packed.device)
    words = packed.to(torch.int64) & 0xFFFFFFFF
    q = ((words[..., None] >> shifts) & ((1 << bits) - 1)).flatten(-2).float()
    shp = q.shape
    q = q.view(*shp[:-1], shp[-1] // group_size, group_size)
    w = q * scales.float()[..., None] + biases.float()[..., None]
    return w.view(shp)


# ------------------------------------------------------------------------------------------------
# MoE routing / combine
# ------------------------------------------------------------------------------------------------
def topk_route(logits: torch.Tensor, k: int, expert_bias: Optional[torch.Tensor] = None
               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """logits [T, E] -> (indices [T, k] int32, weights [T, k] fp32 summing to 1, counts [E] int32)."""
    lf = logits.float()
    if expert_bias is not None:
        lf = lf + expert_bias.float()
    p = torch.softmax(lf, dim=-1)
    work = p.clone()
    idx, wts = [], []
    for _ in range(k):
        m = work.max(dim=-1, keepdim=True).values
        first = (work == m).float().argmax(dim=-1)                   # lowest index among ties
        idx.append(first)
        wts.append(p.gather(1, first[:, None]).squeeze(1))
        work.scatter_(1, first[:, None], -1.0)
    idx = torch.stack(idx, 1)
    wts = torch.stack(wts, 1)
    wts = wts / wts.sum(-1, keepdim=True)
    counts = torch.bincount(idx.flatten(), minlength=logits.shape[-1]).to(torch.int32)
    return idx.to(torch.int32), wts, counts


def prefix_offsets(counts: torch.Tensor) -> torch.Tensor:
    out = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=counts.device)
    out[1:] = torch.cumsum(counts.to(torch.int64), 0).to(torch.int32)
    return out


def moe_ffn(x: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, w_gate_up: torch.Tensor,
            w_down: torch.Tensor) -> torch.Tensor:
    """x [T, D]; w_gate_up [E, 2I, D]; w_down [E, D, I] (already dequantised). Returns
    sum_k w[t,k] * down_e(silu(gate_e x) * up_e x) in fp32."""
    t, d = x.shape
    out = torch.zeros(t, w_down.shape[1], dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in idx.unique().tolist():
        tok, slot = (idx == e).nonzero(as_tuple=True)
        h = xf[tok] @ w_gate_up[e].float().t()
        a = swiglu(h)
        y = a @ w_down[e].float().t()
        out.index_add_(0, tok, y * wts[tok, slot][:, None].float())
    return out


def load_balance_loss(router_probs: torch.Tensor, idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """GShard auxiliary loss: E * sum_e f_e * P_e (crates/rmlx-nn/src/moe.rs:1954-2000)."""
    t = router_probs.shape[0]
    f = torch.bincount(idx.flatten().long(), minlength=num_experts).float() / max(1, idx.numel())
    p = router_probs.float().mean(0)
    return num_experts * (f * p).sum()


def expert_bias_update(bias: torch.Tensor, counts: torch.Tensor, lr: float) -> torch.Tensor:
    """Aux-loss-free balancing: bias[e] += lr * (mean_count - count[e]) (moe.rs:372-410)."""
    c = counts.float()
    return bias + lr * (c.mean() - c)
