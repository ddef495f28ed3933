"""Native prompt processing: the forward over many tokens of one sequence built from this package's
kernels only — RMSNorm, tcgen05 GEMMs (bf16 or Q4 dequantised in the main loop), RoPE + paged KV
write, paged causal flash attention, and for MoE layers top-k routing, row scatter, two grouped
tensor-core GEMMs with SwiGLU, and the weighted combine.

Counterpart of ``TransformerModel::forward_prefill_graph`` (crates/rmlx-nn/src/transformer.rs:
4416-4620), which encodes the 9 dispatches of a prefill layer into shared command buffers; here the
launches go to one stream and the sum over tensor-parallel ranks is injected by the caller.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib
from ..kv.paged import PagedKvCache
from ..ops import decode as D
from ..ops.attention import flash_prefill_paged
from ..ops.gemm import GemmStatus, gemm_bf16
from ..ops.grouped import moe_prefill_ffn
from ..ops.quantized import qmm
from ..ops.weights import LinearWeight, W_BF16


def _mm(x: torch.Tensor, w: LinearWeight, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    if w.kind == W_BF16:
        return gemm_bf16(x, w.w, residual=residual)
    return qmm(x, w, residual=residual)


class NativePrefill:
    """Callable ``(token_ids, cache, seq_id) -> last-token logits [1, vocab_local]`` (fp32)."""

    def __init__(self, model, chunk: int = 8192):
        self.m = model
        self.chunk = chunk
        cfg = model.cfg
        if cfg.head_dim not in (64, 128):
            raise ImportError("native prefill covers head_dim 64 and 128")
        if model.w.embed.dtype != torch.bfloat16:
            raise ImportError("native prefill needs bf16 activations")
        for lw in model.w.layers:
            if lw.experts_gate_up is not None and lw.expert_base != 0:
                raise ImportError("expert-parallel shards go through the exchange path")

    @torch.no_grad()
    def __call__(self, token_ids: torch.Tensor, cache: PagedKvCache, seq_id: int) -> torch.Tensor:
        logits = None
        for s in range(0, token_ids.numel(), self.chunk):
            logits = self._chunk(token_ids[s:s + self.chunk], cache, seq_id)
        return logits

    def _chunk(self, token_ids, cache, seq_id):
        m = self.m
        cfg, w = m.cfg, m.w
        t = token_ids.numel()
        hd, hq, hkv = cfg.head_dim, m.hq, m.hkv
        pos0 = cache.seq_len(seq_id)
        cache.reserve(seq_id, t)
        row = cache.block_table[cache.slot_of[seq_id]]
        pos = torch.arange(pos0, pos0 + t, dtype=torch.int32, device=m.device)
        seq = torch.zeros(t, dtype=torch.int32, device=m.device)
        h = D.embedding(w.embed, token_ids.to(torch.int32))
        q = torch.empty(t, hq, hd, dtype=torch.bfloat16, device=m.device)
        for li, lw in enumerate(w.layers):
            xn = D.rms_norm(h, lw.norm1, cfg.rms_norm_eps)
            qkv = _mm(xn, lw.wqkv)
            D.rope_kv_write(qkv, q, cache.k[li], cache.v[li], row.view(1, -1), pos, m.cos, m.sin,
                            hq, hkv, token_seq=seq, traditional=cfg.rope_traditional)
            attn = flash_prefill_paged(q, cache.k[li], cache.v[li], row, pos0, m.scale,
                                       cfg.sliding_window or 0)
            if m.layout.world > 1:
                h = h + m._sum(_mm(attn.view(t, hq * hd), lw.wo))
            else:
                h = _mm(attn.view(t, hq * hd), lw.wo, residual=h)
            xn = D.rms_norm(h, lw.norm2, cfg.rms_norm_eps)
            if lw.router is not None:
                moe = cfg.ff_type.moe
                logits = xn.float() @ lw.router.float().t()
                idx, wts, _, offsets = D.topk_route(logits, moe.num_experts_per_token, lw.expert_bias)
                single = m.layout.world == 1 and lw.shared_gate_up is None
                y = moe_prefill_ffn(xn, idx, wts, offsets, lw.experts_gate_up, lw.experts_down,
                                    residual=h if single else None)
                if lw.shared_gate_up is not None:
                    y = y + _mm(D.silu_mul(_mm(xn, lw.shared_gate_up)), lw.shared_down)
                h = y if single else h + m._sum(y)
            else:
                act = D.silu_mul(_mm(xn, lw.w_gate_up))
                if m.layout.world > 1:
                    h = h + m._sum(_mm(act, lw.w_down))
                else:
                    h = _mm(act, lw.w_down, residual=h)
        cache.commit(seq_id, t)
        GemmStatus.check(m.device)
        last = h[t - 1:t].contiguous()
        logits = D.rms_gemv(last, w.lm_head, w.final_norm, cfg.rms_norm_eps,
                            out=torch.empty(1, w.lm_head.n, dtype=torch.float32, device=m.device))
        if m.allgather_logits is not None and m.layout.world > 1 and w.lm_head.n != cfg.vocab_size:
            logits = m.allgather_logits(logits)
        return logits


def enable_native_prefill(model, chunk: int = 8192) -> bool:
    """Attach the native path to ``model.prefill``; False (and the library-kernel path stays) when the
    model's shapes are outside what the kernels cover."""
    try:
        model._native_prefill = NativePrefill(model, chunk)
        return True
    except ImportError:
        return False
