"""Native many-token forward: prompt processing and large-batch decode built from this package's
kernels only — RMSNorm, tcgen05 GEMMs (bf16 or Q4 dequantised in the main loop), RoPE + paged KV
write, paged flash attention (causal prefill kernel or split-KV decode kernel), and for MoE layers
top-k routing, row scatter, two grouped tensor-core GEMMs with SwiGLU, and the weighted combine.

``NativePrefill`` is the counterpart of ``TransformerModel::forward_prefill_graph``
(crates/rmlx-nn/src/transformer.rs:4416-4620), which encodes the 9 dispatches of a prefill layer
into shared command buffers. ``BatchedDecode`` serves decode batches beyond what the mat-vec
kernels take (more than 4 rows): one token of each of B sequences per step, every shape static, so
the whole step is captured in a CUDA graph (the reference's batched decode goes through the same
GEMM kernels with M = batch, crates/rmlx-nn/src/transformer.rs:4250-4402).

With tensor parallelism the row-parallel projections use the GEMM whose all-reduce runs inside the
kernel (``parallel.tp_gemm``) when a ``gemm_comm`` is attached to the model; the MoE block's partial
sums go through the injected ``allreduce``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import _lib
from ..kv.paged import PagedKvCache
from ..ops import decode as D
from ..runtime.graph import GraphCache, bucket_for
from ..ops.attention import flash_prefill_paged
from ..ops.gemm import GemmStatus, gemm_bf16
from ..ops.grouped import moe_prefill_ffn
from ..ops.quantized import qmm, xgemm
from ..ops.weights import LinearWeight, W_BF16, W_Q4


def _mm(x: torch.Tensor, w: LinearWeight, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    if w.kind == W_BF16:
        return gemm_bf16(x, w.w, residual=residual)
    return qmm(x, w, residual=residual)


def _gate_up_act(x: torch.Tensor, w: LinearWeight) -> torch.Tensor:
    """silu(x W_gate^T) * (x W_up^T) for W = [gate; up]: SwiGLU runs in the GEMM epilogue when the
    shape allows, else GEMM then the element-wise kernel."""
    q4_ok = w.kind == W_BF16 or (w.kind == W_Q4 and not w.scales_f16 and
                                 bool(_lib.cuda().rmlx_qgemm_supported(w.k)))
    if w.n % 256 == 0 and w.k % 8 == 0 and q4_ok:
        return xgemm(x, w, swiglu=True)
    return D.silu_mul(_mm(x, w))


def _router_logits(xn: torch.Tensor, router: torch.Tensor) -> torch.Tensor:
    """fp32 router logits from bf16 operands on this package's tensor-core GEMM, the accumulator
    stored unrounded (a bf16 result would create ties between experts)."""
    if xn.dtype == torch.bfloat16 and router.dtype == torch.bfloat16 and xn.shape[1] % 8 == 0:
        from ..ops.gemm import gemm_bf16_f32
        return gemm_bf16_f32(xn.contiguous(), router)
    return xn.float() @ router.float().t()


def _check_model(model) -> None:
    cfg = model.cfg
    if cfg.head_dim not in (64, 128):
        raise ImportError("the native forward covers head_dim 64 and 128")
    if model.w.embed.dtype != torch.bfloat16:
        raise ImportError("the native forward needs bf16 activations")


class _Layers:
    """The per-layer body shared by prefill and batched decode; ``attend`` does RoPE, the KV write
    and attention for the caller's token layout."""

    def __init__(self, model):
        _check_model(model)
        self.m = model
        self.comm = getattr(model, "gemm_comm", None)

    def _row_parallel(self, x: torch.Tensor, w: LinearWeight, h: torch.Tensor) -> torch.Tensor:
        m = self.m
        if m.layout.world == 1:
            return _mm(x, w, residual=h)
        if self.comm is not None:
            return self.comm.gemm_allreduce(x, w, residual=h.contiguous())
        return h + m._sum(_mm(x, w))

    def run(self, h: torch.Tensor, attend) -> torch.Tensor:
        m = self.m
        cfg, w = m.cfg, m.w
        t = h.shape[0]
        hd, hq = cfg.head_dim, m.hq
        for li, lw in enumerate(w.layers):
            xn = D.rms_norm(h, lw.norm1, cfg.rms_norm_eps)
            qkv = _mm(xn, lw.wqkv)
            attn = attend(li, qkv)
            h = self._row_parallel(attn.view(t, hq * hd), lw.wo, h)
            xn = D.rms_norm(h, lw.norm2, cfg.rms_norm_eps)
            if lw.router is not None:
                moe = cfg.ff_type.moe
                logits = _router_logits(xn, lw.router)
                idx, wts, _, offsets = D.topk_route(logits, moe.num_experts_per_token, lw.expert_bias)
                single = m.layout.world == 1 and lw.shared_gate_up is None
                y = moe_prefill_ffn(xn, idx, wts, offsets, lw.experts_gate_up, lw.experts_down,
                                    residual=h if single else None, expert_base=lw.expert_base)
                if lw.shared_gate_up is not None:
                    y = y + _mm(_gate_up_act(xn, lw.shared_gate_up), lw.shared_down)
                h = y if single else h + m._sum(y)
            else:
                act = _gate_up_act(xn, lw.w_gate_up)
                h = self._row_parallel(act, lw.w_down, h)
        return h

    def logits(self, rows: torch.Tensor) -> torch.Tensor:
        """Final norm + LM head for a few rows [R, D] -> fp32 [R, vocab] (gathered over TP ranks)."""
        m = self.m
        cfg, w = m.cfg, m.w
        r = rows.shape[0]
        if r <= 4:
            out = D.rms_gemv(rows.contiguous(), w.lm_head, w.final_norm, cfg.rms_norm_eps,
                             out=torch.empty(r, w.lm_head.n, dtype=torch.float32, device=m.device))
        else:
            xn = D.rms_norm(rows.contiguous(), w.final_norm, cfg.rms_norm_eps)
            if w.lm_head.kind == W_BF16 and w.lm_head.k % 8 == 0:
                from ..ops.gemm import gemm_bf16_f32       # accumulator stored unrounded
                out = gemm_bf16_f32(xn, w.lm_head.w)
            else:
                out = _mm(xn, w.lm_head).float()
        if m.allgather_logits is not None and m.layout.world > 1 and w.lm_head.n != cfg.vocab_size:
            out = m.allgather_logits(out)
        return out


class NativePrefill:
    """Callable ``(token_ids, cache, seq_id) -> last-token logits [1, vocab]`` (fp32); with
    ``all_logits=True`` the logits of every position of the call, ``[T, vocab]`` (what speculative
    verification needs: crates/rmlx-nn/src/sampler.rs verify helpers read one row per proposal)."""

    def __init__(self, model, chunk: int = 8192):
        self.m = model
        self.chunk = chunk
        self.layers = _Layers(model)

    @torch.no_grad()
    def __call__(self, token_ids: torch.Tensor, cache: PagedKvCache, seq_id: int,
                 all_logits: bool = False) -> torch.Tensor:
        parts = []
        for s in range(0, token_ids.numel(), self.chunk):
            parts.append(self._chunk(token_ids[s:s + self.chunk], cache, seq_id, all_logits))
        return torch.cat(parts, 0) if all_logits else parts[-1]

    def _chunk(self, token_ids, cache, seq_id, all_logits=False):
        m = self.m
        cfg = m.cfg
        t = token_ids.numel()
        hd, hq, hkv = cfg.head_dim, m.hq, m.hkv
        pos0 = cache.seq_len(seq_id)
        cache.reserve(seq_id, t)
        row = cache.block_table[cache.slot_of[seq_id]]
        pos = torch.arange(pos0, pos0 + t, dtype=torch.int32, device=m.device)
        seq = torch.zeros(t, dtype=torch.int32, device=m.device)
        q = torch.empty(t, hq, hd, dtype=torch.bfloat16, device=m.device)

        npages = (pos0 + t + cache.block_size - 1) // cache.block_size
        ident = torch.arange(npages, dtype=torch.int32, device=m.device) if cache.quantized else None

        def attend(li, qkv):
            D.rope_kv_write(qkv, q, cache.k[li], cache.v[li], row.view(1, -1), pos, m.cos, m.sin,
                            hq, hkv, token_seq=seq, traditional=cfg.rope_traditional, **cache.sb(li))
            if cache.quantized:
                # prompt attention over an 8-bit cache: the sequence's pages are expanded once per
                # layer into contiguous bf16 pages (amortised over the chunk's tokens)
                kk = D.kv_dequant_pages(cache.k[li], cache.k_sb[li], row, npages)
                vv = D.kv_dequant_pages(cache.v[li], cache.v_sb[li], row, npages)
                return flash_prefill_paged(q, kk, vv, ident, pos0, m.scale, cfg.sliding_window or 0)
            return flash_prefill_paged(q, cache.k[li], cache.v[li], row, pos0, m.scale,
                                       cfg.sliding_window or 0)

        h = self.layers.run(D.embedding(m.w.embed, token_ids.to(torch.int32)), attend)
        cache.commit(seq_id, t)
        GemmStatus.check(m.device)
        return self.layers.logits(h if all_logits else h[t - 1:t])


class BatchedDecode:
    """One decode step for up to ``max_batch`` sequences through the tensor-core kernels; shapes are
    static (idle rows point at the reserved page 0), so the step is one CUDA graph."""

    def __init__(self, model, cache: PagedKvCache, max_batch: int, use_graph: bool = True,
                 splits: Optional[int] = None):
        self.m, self.cache, self.B = model, cache, max_batch
        self.layers = _Layers(model)
        cfg, dev = model.cfg, model.device
        b = max_batch
        self.tokens = torch.zeros(b, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(b, dtype=torch.int32, device=dev)
        self.seq_lens = torch.zeros(b, dtype=torch.int32, device=dev)
        self.rows = torch.arange(b, dtype=torch.int32, device=dev)
        self.live = torch.zeros(b, dtype=torch.int32, device=dev)
        self.table = torch.zeros(b, cache.max_blocks_per_seq, dtype=torch.int32, device=dev)
        self.q = torch.empty(b, model.hq, cfg.head_dim, dtype=torch.bfloat16, device=dev)
        self.next_tokens = torch.zeros(b, dtype=torch.int32, device=dev)
        # one captured graph per batch bucket: a step runs the smallest bucket that holds the
        # bound rows (crates/rmlx-metal/src/icb.rs:357, a replay cache keyed by shape)
        self.buckets = tuple(x for x in (1, 2, 4, 8, 16, 32, 64) if x < b) + (b,)
        self.graphs = GraphCache(max_entries=len(self.buckets))
        self._splits_arg = splits
        self._fd = {}
        self.splits, self.fd = self._fd_plan(b)
        self.argmax_scratch = D.ArgmaxScratch(b, dev)
        self.seq_ids: List[int] = []
        self.launches_per_step = 0           # launches of this package's kernels in one step
        self.use_graph = use_graph and model.layout.world == 1 and not _lib.debug_serialize()
        self._logits = {}
        self._last_bucket = b

    def _fd_plan(self, nb: int):
        if nb not in self._fd:
            m, cfg = self.m, self.m.cfg
            sp = self._splits_arg or D.default_splits(
                nb, m.hkv, _lib.cuda().rmlx_flash_decode_gtiles(m.hq, m.hkv),
                self.cache.max_blocks_per_seq * 16)
            self._fd[nb] = (sp, D.FlashDecodeScratch(nb, m.hq, m.hkv, cfg.head_dim, sp, m.device))
        return self._fd[nb]

    def bucket(self) -> int:
        return bucket_for(max(1, len(self.seq_ids)), self.buckets)

    def bind(self, seq_ids: Sequence[int], last_tokens: Sequence[int]) -> None:
        assert len(seq_ids) <= self.B
        self.seq_ids = list(seq_ids)
        n = len(seq_ids)
        lens = [self.cache.seq_len(s) for s in seq_ids]
        # idle rows attend to one (zero) key on the reserved page 0 and never advance
        self.tokens.zero_(); self.positions.zero_(); self.seq_lens.fill_(1); self.live.zero_()
        self.tokens[:n] = torch.tensor(list(last_tokens), dtype=torch.int32)
        self.positions[:n] = torch.tensor(lens, dtype=torch.int32)
        self.seq_lens[:n] = torch.tensor([l + 1 for l in lens], dtype=torch.int32)
        self.live[:n] = 1
        self._saved_tokens = self.tokens.clone()
        self.refresh_tables()

    def refresh_tables(self) -> None:
        self.table.zero_()
        for i, s in enumerate(self.seq_ids):
            self.table[i].copy_(self.cache.block_table[self.cache.slot_of[s]])

    def reserve(self, steps: int) -> None:
        for s in self.seq_ids:
            self.cache.reserve(s, steps)
        self.refresh_tables()

    def _body(self, nb: Optional[int] = None) -> None:
        m, cfg, cache = self.m, self.m.cfg, self.cache
        nb = self.B if nb is None else nb
        splits, fd = self._fd_plan(nb)
        tokens, positions, seq_lens = self.tokens[:nb], self.positions[:nb], self.seq_lens[:nb]
        table, q, rows, live = self.table[:nb], self.q[:nb], self.rows[:nb], self.live[:nb]

        def attend(li, qkv):
            D.rope_kv_write(qkv, q, cache.k[li], cache.v[li], table, positions, m.cos,
                            m.sin, m.hq, m.hkv, token_seq=rows, traditional=cfg.rope_traditional,
                            **cache.sb(li))
            return D.flash_decode_paged(q, cache.k[li], cache.v[li], table, seq_lens,
                                        m.scale, splits, fd, cfg.sliding_window or 0, **cache.sb(li))

        h = self.layers.run(D.embedding(m.w.embed, tokens), attend)
        self._logits[nb] = self.layers.logits(h)
        D.argmax(self._logits[nb], self.next_tokens[:nb], self.argmax_scratch)
        # feed the tokens back and advance the bound rows (idle rows stay at length 0 on page 0)
        tokens.copy_(self.next_tokens[:nb] * live)
        positions.add_(live)
        seq_lens.add_(live)

    @property
    def logits(self) -> Optional[torch.Tensor]:
        """Logits of the last step: [bucket rows, vocab] (rows beyond the bound sequences are idle)."""
        return self._logits.get(self._last_bucket)

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """Run one step for every bound sequence; returns the next-token ids (device, int32)."""
        nb = self._last_bucket = self.bucket()
        if not self.use_graph:
            n0 = _lib.launch_count()
            self._body(nb)
            self.launches_per_step = _lib.launch_count() - n0
        else:
            def body():
                n0 = _lib.launch_count()
                self._body(nb)
                self.launches_per_step = _lib.launch_count() - n0
            # one warm-up run outside capture (lazy initialisations), state rewound after each
            self.graphs.get_or_capture(("batched", nb), body, warmup=1, restore=self._rewind,
                                       device=self.m.device).replay()
        for s in self.seq_ids:
            self.cache.commit(s, 1)
        return self.next_tokens

    def set_next_tokens(self, tokens: Sequence[int]) -> None:
        """Replace the tokens the last step fed back (its arg-max) with ones chosen by the caller,
        e.g. sampled from ``logits``; positions and lengths were already advanced by the step."""
        n = len(self.seq_ids)
        assert len(tokens) == n
        self.tokens[:n] = torch.tensor([int(t) for t in tokens], dtype=torch.int32)
        self._saved_tokens = self.tokens.clone()

    def _rewind(self) -> None:
        """Undo the state advance of a warm-up step (the KV slot it wrote is rewritten by the real one)."""
        n = len(self.seq_ids)
        lens = [self.cache.seq_len(s) for s in self.seq_ids]
        self.positions.zero_(); self.seq_lens.fill_(1)
        self.positions[:n] = torch.tensor(lens, dtype=torch.int32)
        self.seq_lens[:n] = torch.tensor([l + 1 for l in lens], dtype=torch.int32)
        self.tokens.copy_(self._saved_tokens)

    @torch.no_grad()
    def generate(self, steps: int) -> torch.Tensor:
        self.reserve(steps + 1)
        self._saved_tokens = self.tokens.clone()
        out = torch.zeros(len(self.seq_ids), steps, dtype=torch.int64)
        for i in range(steps):
            nxt = self.step()
            out[:, i] = nxt[:len(self.seq_ids)].cpu().long()
            self._saved_tokens = self.tokens.clone()
        GemmStatus.check(self.m.device)
        return out


def plan_chunk(model, scratch_limit_bytes: int = 4 << 30, longest: int = 8192) -> int:
    """Largest prompt chunk (a multiple of 128, at most ``longest``) whose per-layer intermediates
    stay within ``scratch_limit_bytes`` according to the layer's static plan
    (``models.prefill_plan.PrefillPlan``: every launch of a layer with its output size)."""
    from .prefill_plan import PrefillPlan
    chunk = longest
    while chunk > 128 and PrefillPlan(model.cfg, chunk, model.layout).scratch_bytes > scratch_limit_bytes:
        chunk -= 128
    return chunk


def enable_native_prefill(model, chunk: Optional[int] = None, scratch_limit_bytes: int = 4 << 30) -> bool:
    """Attach the native path to ``model.prefill``; False (and the library-kernel path stays) when the
    model's shapes are outside what the kernels cover. ``chunk`` None: the longest chunk whose
    intermediates fit ``scratch_limit_bytes`` (``plan_chunk``)."""
    try:
        if chunk is None:
            chunk = plan_chunk(model, scratch_limit_bytes)
        model._native_prefill = NativePrefill(model, chunk)
        return True
    except ImportError:
        return False
