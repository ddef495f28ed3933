"""Decoder-only transformer: the library-kernel (PyTorch ops) forward used as oracle and baseline,
and the native forward built from this package's kernels.

API surface follows ``TransformerModel`` of crates/rmlx-nn/src/transformer.rs:4136-4402:
``forward`` (token ids -> logits, with an optional KV cache), ``forward_prefill`` and a cached
decode object (``CachedDecode``, crates/rmlx-nn/src/transformer.rs:3613-4050) that pre-resolves
every buffer and launch once. Where the reference batches ~5 layers per command buffer and syncs
once per token (crates/rmlx-metal/src/exec_graph.rs:198-311), the decode step here is one CUDA
graph over all layers, replayed per token with no host work in between; positions, lengths and
block tables are device buffers so the captured graph stays valid as the cache grows.

Tensor parallelism follows ``forward_with_group`` (crates/rmlx-nn/src/transformer.rs:4697-4857): two
sums of ``[tokens, hidden]`` per layer, after the attention output projection and after the
feed-forward block.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import torch

from ..kv.paged import PagedKvCache
from ..reference import ops as ref
from .weights import LayerWeights, ModelWeights


class TransformerModel:
    """Holds one rank's weights and runs them.

    ``allreduce`` is a callable ``t -> t`` summing a tensor over the tensor-parallel ranks (None on
    a single rank); ``allgather_logits`` concatenates vocabulary shards. They are injected so the
    same model runs over gloo on CPU, NCCL, or this package's peer-memory collectives.
    """

    def __init__(self, weights: ModelWeights, allreduce: Optional[Callable] = None,
                 allgather_logits: Optional[Callable] = None):
        self.w = weights
        self.cfg = weights.cfg
        self.layout = weights.layout
        self.allreduce = allreduce
        self.allgather_logits = allgather_logits
        self.device = weights.embed.device
        cfg = self.cfg
        self.hq, _, self.hkv, _ = self.layout.heads(cfg)
        self.cos, self.sin = ref.rope_tables(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta,
                                             device=self.device)
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self._deq_cache = {}

    # ------------------------------------------------------------------ helpers
    def new_cache(self, num_blocks: int, max_seqs: int = 64, max_blocks_per_seq: Optional[int] = None,
                  dtype=None, kv_quant: Optional[str] = None) -> PagedKvCache:
        """``kv_quant="q8"``: the cache is kept in the 8-bit affine format (half the bytes)."""
        cfg = self.cfg
        mb = max_blocks_per_seq or (cfg.max_seq_len + 15) // 16
        return PagedKvCache(num_blocks, cfg.num_layers, self.hkv, cfg.head_dim,
                            dtype=dtype or self.w.embed.dtype, device=self.device,
                            max_seqs=max_seqs, max_blocks_per_seq=mb, kv_quant=kv_quant)

    def _deq(self, lw, name: str, dtype):
        """Dense [.., N, K] view of a (possibly quantised) weight in the compute dtype, cached."""
        key = (id(lw), name, dtype)
        t = self._deq_cache.get(key)
        if t is None:
            t = getattr(lw, name).dequantized().to(dtype)
            self._deq_cache[key] = t
        return t

    def _sum(self, t: torch.Tensor) -> torch.Tensor:
        return self.allreduce(t) if (self.allreduce is not None and self.layout.world > 1) else t

    # ------------------------------------------------------------------ library-kernel forward
    @torch.no_grad()
    def forward(self, token_ids: torch.Tensor, cache: Optional[PagedKvCache] = None,
                seq_ids: Optional[Sequence[int]] = None, last_only: bool = False) -> torch.Tensor:
        """Library-kernel forward over one or more sequences.

        ``token_ids``: 1-D tensor of the new tokens of every sequence, concatenated in ``seq_ids``
        order with equal counts per sequence (prefill: n tokens of one sequence; decode: one token
        of each of B sequences). Without a cache, a single sequence is processed from position 0.
        Returns logits ``[tokens, vocab]`` (or one row per sequence with ``last_only``).
        """
        cfg, w = self.cfg, self.w
        dt = w.embed.dtype
        t_total = token_ids.numel()
        own_cache = cache is None
        if own_cache:
            cache = self.new_cache((t_total + 15) // 16 + 1, max_seqs=1)
            seq_ids = [0]
            cache.add_sequence(0)
        seq_ids = list(seq_ids)
        n = t_total // len(seq_ids)
        assert n * len(seq_ids) == t_total
        starts = []
        for s in seq_ids:
            starts.append(cache.seq_len(s))
            cache.reserve(s, n)
        pos = torch.cat([torch.arange(st, st + n, device=self.device) for st in starts])
        h = w.embed[token_ids.long()]
        for li, lw in enumerate(w.layers):
            h = self._layer_forward(li, lw, h, pos, cache, seq_ids, starts, n, dt)
        for s in seq_ids:
            cache.commit(s, n)
        if last_only:
            h = h.view(len(seq_ids), n, -1)[:, -1]
        xn = ref.rms_norm(h, w.final_norm, cfg.rms_norm_eps)
        logits = (xn @ self._deq(w, "lm_head", dt).t()).float()
        if self.allgather_logits is not None and self.layout.world > 1 and w.lm_head.n != cfg.vocab_size:
            logits = self.allgather_logits(logits)
        return logits

    def _layer_forward(self, li, lw: LayerWeights, h, pos, cache, seq_ids, starts, n, dt):
        cfg = self.cfg
        hd, hq, hkv = cfg.head_dim, self.hq, self.hkv
        xn = ref.rms_norm(h, lw.norm1, cfg.rms_norm_eps)
        qkv = xn @ self._deq(lw, "wqkv", dt).t()
        q = qkv[:, :hq * hd].view(-1, hq, hd)
        k = qkv[:, hq * hd:(hq + hkv) * hd].view(-1, hkv, hd)
        v = qkv[:, (hq + hkv) * hd:].view(-1, hkv, hd)
        q = ref.apply_rope(q, pos, self.cos, self.sin, cfg.rope_traditional)
        k = ref.apply_rope(k, pos, self.cos, self.sin, cfg.rope_traditional)
        outs = []
        for si, s in enumerate(seq_ids):
            sl = slice(si * n, (si + 1) * n)
            cache.append(li, s, k[sl], v[sl], starts[si])
            kk = cache.get_keys(li, s, starts[si] + n)
            vv = cache.get_values(li, s, starts[si] + n)
            outs.append(ref.sdpa(q[sl], kk, vv, self.scale, starts[si], cfg.sliding_window))
        attn = torch.cat(outs, 0).reshape(-1, hq * hd)
        h = h + self._sum(attn @ self._deq(lw, "wo", dt).t())
        xn = ref.rms_norm(h, lw.norm2, cfg.rms_norm_eps)
        if lw.router is not None:
            m = cfg.ff_type.moe
            logits = xn.float() @ lw.router.float().t()
            idx, wts, _ = ref.topk_route(logits, m.num_experts_per_token, lw.expert_bias)
            local = idx - lw.expert_base
            e_local = lw.experts_gate_up.experts
            mask = (local >= 0) & (local < e_local)
            lidx = torch.where(mask, local, torch.zeros_like(local))
            lwts = torch.where(mask, wts, torch.zeros_like(wts))
            y = ref.moe_ffn(xn, lidx, lwts, self._deq(lw, "experts_gate_up", dt),
                            self._deq(lw, "experts_down", dt))
            if lw.shared_gate_up is not None:
                a = ref.swiglu(xn @ self._deq(lw, "shared_gate_up", dt).t())
                y = y + (a @ self._deq(lw, "shared_down", dt).t()).float()
            y = y.to(dt)
        else:
            a = ref.swiglu(xn @ self._deq(lw, "w_gate_up", dt).t())
            y = a @ self._deq(lw, "w_down", dt).t()
        return h + self._sum(y)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, token_ids: torch.Tensor, cache: PagedKvCache, seq_id: int,
                all_logits: bool = False) -> torch.Tensor:
        """Run a prompt (or a chunk of one) for ``seq_id``, filling its KV pages. Returns the
        logits of the last token, ``[1, vocab]``, or with ``all_logits`` those of every position,
        ``[T, vocab]``. On CUDA this takes the native tensor-core path when it is available for
        the model's weights, else the library-kernel forward."""
        if token_ids.is_cuda:
            if not hasattr(self, "_native_prefill"):
                # first prompt on a GPU: attach the tensor-core path when the model's shapes and
                # layout are covered (single rank, head_dim 64 / 128, bf16 activations)
                self._native_prefill = None
                if self.layout.world == 1:
                    from .prefill import enable_native_prefill
                    enable_native_prefill(self)
            if self._native_prefill is not None:
                return self._native_prefill(token_ids, cache, seq_id, all_logits=all_logits)
        return self.forward(token_ids, cache, [seq_id], last_only=not all_logits)

    # ------------------------------------------------------------------ greedy generation (oracle)
    @torch.no_grad()
    def generate_greedy(self, prompt: torch.Tensor, steps: int, cache: Optional[PagedKvCache] = None
                        ) -> List[int]:
        cache = cache or self.new_cache((prompt.numel() + steps + 15) // 16 + 1, max_seqs=1)
        cache.add_sequence(0)
        logits = self.forward(prompt, cache, [0], last_only=True)
        out = []
        tok = int(logits[0].argmax())
        for _ in range(steps):
            out.append(tok)
            logits = self.forward(torch.tensor([tok], device=self.device), cache, [0], last_only=True)
            tok = int(logits[0].argmax())
        return out
