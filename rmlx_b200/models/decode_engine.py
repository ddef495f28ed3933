"""Cached decode: every buffer, pointer and launch of a decode step is resolved once, the step is
captured in a CUDA graph, and each new token is one graph replay.

This is the B200 form of the reference's ``CachedDecode`` + fused 7-dispatch layer
(crates/rmlx-nn/src/transformer.rs:2306-2555,3613-4050) and of its ExecGraph / command-batcher
machinery (crates/rmlx-metal/src/exec_graph.rs:110-401). Per layer the captured step holds:

  1. RMSNorm + QKV projection  }  one kernel (rms_qkv_rope): the rotation and the page append
  2. RoPE(Q,K) + paged KV append }  happen in the projection's epilogue
  3. paged split-KV flash decode         (flash_decode_paged, merges its splits in-kernel)
  4. O projection + residual             (rms_gemv)             [tensor parallel: + all-reduce]
  5. MoE: RMSNorm + router + top-k       (moe_router)
  6.      expert gate/up + SwiGLU        (moe_gate_up)
  7.      expert down + weighted combine + residual (moe_down)  [tensor parallel: + all-reduce]
     or, for dense layers, gate/up + SwiGLU and down + residual.

and after the last layer: final RMSNorm + LM head, arg-max, and the advance kernel that feeds the
sampled token back as the next input. Consecutive kernels are chained with programmatic dependent
launch so each one's prologue overlaps its predecessor's tail.
"""
from __future__ import annotations

import os

from typing import List, Optional, Sequence

import torch

from .. import _lib
from ..kv.paged import PagedKvCache
from ..runtime.graph import GraphCache, bucket_for
from ..ops import decode as D
from .transformer import TransformerModel


class CachedDecode:
    def __init__(self, model: TransformerModel, cache: PagedKvCache, max_batch: int = 1,
                 use_graph: bool = True, pdl: bool = True, splits: Optional[int] = None,
                 comm=None, greedy: bool = True, step_kernel: Optional[bool] = None):
        if model.device.type != "cuda":
            raise _lib.NativeError("CachedDecode runs this package's CUDA kernels; on CPU use "
                                   "TransformerModel.forward")
        self.model, self.cache, self.B = model, cache, max_batch
        self.cfg = cfg = model.cfg
        self.comm = comm
        self.pdl = pdl
        self.use_graph = use_graph
        self.greedy = greedy
        # RoPE and the KV append run in the QKV projection's epilogue unless switched off
        self.fuse_rope = os.environ.get("RMLX_FUSE_ROPE", "1") != "0" and not cache.quantized
        # Which projections stream their weights depends on the shard size (measured on the
        # 60-layer model, 4-bit weights, tokens/s): one GPU 216.8 with only the expert projections
        # streaming against 207.6 with all of them; two GPUs 250 against 246; four GPUs 278.7
        # against 291.2. An explicit RMLX_DECODE_STREAM_OPS wins over this choice.
        if "RMLX_DECODE_STREAM_OPS" not in os.environ:
            D.set_stream(D.stream_enabled(), ops="all" if model.layout.world >= 4 else None)
        dev = model.device
        B, D_ = max_batch, cfg.hidden_size
        hq, hkv, hd = model.hq, model.hkv, cfg.head_dim
        i32 = dict(dtype=torch.int32, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.tokens = torch.zeros(B, **i32)
        self.positions = torch.zeros(B, **i32)
        self.seq_lens = torch.zeros(B, **i32)
        self.active = torch.zeros(B, **i32)
        self.next_tokens = torch.zeros(B, **i32)
        self.block_table = torch.zeros(B, cache.max_blocks_per_seq, **i32)
        self.h = torch.zeros(B, D_, **bf)
        self.h2 = torch.zeros(B, D_, **bf)
        self.qkv = torch.zeros(B, (hq + 2 * hkv) * hd, **bf)
        self.q = torch.zeros(B, hq, hd, **bf)
        self.attn = torch.zeros(B, hq, hd, **bf)
        self.vocab_local = model.w.lm_head.n
        self.logits = torch.zeros(B, cfg.vocab_size, dtype=torch.float32, device=dev)
        lib = _lib.cuda()
        gt = lib.rmlx_flash_decode_gtiles(hq, hkv)
        # One captured graph per batch bucket (1, 2, 4, ... max_batch): a step runs the smallest
        # bucket that holds the bound rows, so a serving engine sized for 8 rows does not pay for
        # 8 when one sequence is left. Split counts and attention scratch are planned per bucket.
        self.buckets = tuple(b for b in (1, 2, 4, 8, 16, 32, 64) if b < B) + (B,)
        # The steps are recorded and replayed by the native graph store (csrc/runtime/graph_exec.cu)
        # on one GPU; tensor-parallel engines keep torch's graphs unless RMLX_NATIVE_GRAPHS=1
        # (RMLX_NATIVE_GRAPHS=0 switches the native store off everywhere).
        native = os.environ.get("RMLX_NATIVE_GRAPHS", "1" if model.layout.world == 1 else "0") == "1"
        self.graphs = GraphCache(max_entries=len(self.buckets), native=native)
        self._splits_arg = splits
        self._fd = {}
        self.splits = splits or D.default_splits(B, hkv, gt, cfg.max_seq_len)
        self.fd_scratch = self._fd_plan(B)[1]
        for nb in self.buckets:       # planned up front: a step that allocates nothing can be recorded natively
            self._fd_plan(nb)
        moe = cfg.ff_type.moe
        if moe is not None:
            k = moe.num_experts_per_token
            i_local = max(l.experts_gate_up.n // 2 for l in model.w.layers if l.experts_gate_up is not None)
            self.idx = torch.zeros(B, k, **i32)
            self.wts = torch.zeros(B, k, dtype=torch.float32, device=dev)
            self.act = torch.zeros(B * k, i_local, **bf)
            self.router_scratch = D.RouterScratch(B, moe.num_experts, dev)
        dense_i = [l.w_gate_up.n // 2 for l in model.w.layers if l.w_gate_up is not None]
        if dense_i:
            self.dense_act = torch.zeros(B, max(dense_i), **bf)
        self.argmax_scratch = D.ArgmaxScratch(B, dev)
        self.seq_ids: List[int] = []
        self._launches_per_step = 0
        self.serialize = os.environ.get("RMLX_DEBUG_SERIALIZE", "0") == "1"
        # batch 1 on one GPU: the whole step is one persistent kernel when the model fits it
        self.step_kernel = None
        from .step_kernel import DecodeStepKernel
        if step_kernel is not False and not cache.quantized and \
                DecodeStepKernel.supported(model, max_batch, comm, force=bool(step_kernel)):
            sk = DecodeStepKernel(self)
            if sk.ok:
                self.step_kernel = sk
        if step_kernel and self.step_kernel is None:
            raise _lib.NativeError("the persistent step kernel does not take this model / batch")

    def _fd_plan(self, nb: int):
        """(splits, scratch) of the attention kernel for a step of ``nb`` rows."""
        if nb not in self._fd:
            m, cfg = self.model, self.cfg
            gt = _lib.cuda().rmlx_flash_decode_gtiles(m.hq, m.hkv)
            sp = self._splits_arg or D.default_splits(nb, m.hkv, gt, cfg.max_seq_len)
            self._fd[nb] = (sp, D.FlashDecodeScratch(nb, m.hq, m.hkv, cfg.head_dim, sp, m.device,
                                                     max_len=cfg.max_seq_len))
        return self._fd[nb]

    def bucket(self) -> int:
        """Rows the next step runs: the smallest bucket that holds the bound sequences."""
        return bucket_for(max(1, len(self.seq_ids)), self.buckets)

    # ------------------------------------------------------------------ binding
    def bind(self, seq_ids: Sequence[int], last_tokens: Sequence[int]) -> None:
        """Attach up to ``max_batch`` cached sequences to the batch rows and load their state."""
        assert len(seq_ids) <= self.B
        self.seq_ids = list(seq_ids)
        n = len(seq_ids)
        lens = [self.cache.seq_len(s) for s in seq_ids]
        self.tokens.zero_(); self.positions.zero_(); self.seq_lens.zero_(); self.active.zero_()
        self.tokens[:n] = torch.tensor(list(last_tokens), dtype=torch.int32)
        self.positions[:n] = torch.tensor(lens, dtype=torch.int32)
        self.seq_lens[:n] = torch.tensor([l + 1 for l in lens], dtype=torch.int32)
        self.active[:n] = 1
        # inactive rows still run (shape-stable graph): give them a harmless one-token context
        if n < self.B:
            self.seq_lens[n:] = 1
        self.refresh_tables()

    def refresh_tables(self) -> None:
        for b, s in enumerate(self.seq_ids):
            self.block_table[b].copy_(self.cache.block_table[self.cache.slot_of[s]])
        # Idle rows still run and append their key/value at position 0 of whatever page their row
        # names: it must be the reserved page 0, never a page left over from an earlier binding
        # (such a page may belong to a live sequence by now).
        self.block_table[len(self.seq_ids):].zero_()

    def reserve(self, steps: int) -> None:
        """Allocate KV blocks for the next ``steps`` tokens of every bound sequence."""
        for s in self.seq_ids:
            self.cache.reserve(s, steps)
        self.refresh_tables()

    # ------------------------------------------------------------------ the step
    def _run_step(self, nb: Optional[int] = None) -> None:
        m, cfg, w = self.model, self.cfg, self.model.w
        eps, pdl = cfg.rms_norm_eps, self.pdl
        tp = self.comm is not None and m.layout.world > 1
        n0 = _lib.launch_count()
        nb = self.B if nb is None else nb
        if self.step_kernel is not None:
            self.step_kernel.launch()
            self._finish_step(pdl=False, n0=n0, nb=nb)
            return
        splits, fd_scratch = self._fd_plan(nb)
        tokens, positions, seq_lens = self.tokens[:nb], self.positions[:nb], self.seq_lens[:nb]
        block_table, q, attn = self.block_table[:nb], self.q[:nb], self.attn[:nb]
        D.embedding(w.embed, tokens, out=self.h[:nb], pdl=False)
        h, h2 = self.h[:nb], self.h2[:nb]
        # several rows on 4-bit weights: the projection runs on the tensor-core mat-vec (eight rows
        # per pass) and RoPE + the KV append follow as their own small kernel
        fuse_rope = self.fuse_rope and not (nb >= 2 and w.layers[0].wqkv.kind == 1)
        for li, lw in enumerate(w.layers):
            if fuse_rope:
                D.rms_qkv_rope(h, lw.wqkv, lw.norm1, eps, q, self.cache.k[li], self.cache.v[li],
                               block_table, positions, m.cos, m.sin, m.hq, m.hkv,
                               traditional=cfg.rope_traditional, pdl=pdl)
            else:
                D.rms_gemv(h, lw.wqkv, lw.norm1, eps, out=self.qkv[:nb], pdl=pdl)
                D.rope_kv_write(self.qkv[:nb], q, self.cache.k[li], self.cache.v[li], block_table,
                                positions, m.cos, m.sin, m.hq, m.hkv,
                                traditional=cfg.rope_traditional, pdl=pdl, **self.cache.sb(li))
            D.flash_decode_paged(q, self.cache.k[li], self.cache.v[li], block_table,
                                 seq_lens, m.scale, splits, fd_scratch,
                                 cfg.sliding_window, out=attn, pdl=pdl, **self.cache.sb(li))
            a2 = attn.view(nb, -1)
            if tp:
                self.comm.gemv_allreduce(a2, lw.wo, residual=h, out=h2, pdl=pdl)
            else:
                D.rms_gemv(a2, lw.wo, None, eps, residual=h, out=h2, pdl=pdl)
            if lw.router is not None:
                moe = cfg.ff_type.moe
                k = moe.num_experts_per_token
                idx, wts, act = self.idx[:nb], self.wts[:nb], self.act[:nb * k]
                D.moe_router(h2, lw.router, lw.norm2, eps, k, lw.expert_bias,
                             self.router_scratch, idx, wts, pdl=pdl)
                D.moe_gate_up(h2, lw.experts_gate_up, lw.norm2, eps, idx, out=act,
                              expert_base=lw.expert_base, pdl=pdl)
                if tp:
                    self.comm.moe_down_allreduce(act, lw.experts_down, idx, wts,
                                                 residual=h2, out=h, expert_base=lw.expert_base,
                                                 pdl=pdl)
                else:
                    D.moe_down(act, lw.experts_down, idx, wts, residual=h2, out=h,
                               expert_base=lw.expert_base, pdl=pdl)
            else:
                act = self.dense_act[:nb, :lw.w_gate_up.n // 2]
                D.rms_gate_up_swiglu(h2, lw.w_gate_up, lw.norm2, eps, out=act, pdl=pdl)
                if tp:
                    self.comm.gemv_allreduce(act, lw.w_down, residual=h2, out=h, pdl=pdl)
                else:
                    D.rms_gemv(act, lw.w_down, None, eps, residual=h2, out=h, pdl=pdl)
        sharded_vocab = tp and self.vocab_local != cfg.vocab_size
        # vocabulary-parallel LM head: this rank's logits occupy the first vocab_local columns
        logits = self.logits[:nb, :self.vocab_local] if sharded_vocab else self.logits[:nb]
        D.rms_gemv(h, w.lm_head, w.final_norm, eps, out=logits, pdl=pdl)
        self._finish_step(pdl=pdl, n0=n0, logits=logits, sharded_vocab=sharded_vocab, nb=nb)

    def _finish_step(self, pdl: bool, n0: int, logits=None, sharded_vocab: bool = False,
                     nb: Optional[int] = None) -> None:
        """Greedy sampling and the advance kernel that feeds the token back."""
        w = self.model.w
        nb = self.B if nb is None else nb
        if logits is None:
            logits = self.logits[:nb]
        if self.greedy:
            nxt = self.next_tokens[:nb]
            if sharded_vocab:
                self.comm.argmax(logits, w.vocab_base, nxt, pdl=pdl)
            else:
                D.argmax(logits, out=nxt, scratch=self.argmax_scratch, pdl=pdl)
            rc = _lib.cuda().rmlx_decode_advance(nxt.data_ptr(), self.tokens.data_ptr(),
                                                 self.positions.data_ptr(), self.seq_lens.data_ptr(),
                                                 self.active.data_ptr(), nb, int(pdl),
                                                 _lib.stream_ptr())
            _lib.check(rc, "decode_advance")
        self._launches_per_step = _lib.launch_count() - n0

    def capture(self, nb: Optional[int] = None):
        """The captured step of bucket ``nb`` (default: the bucket of the bound rows), captured on
        first use: one eager warm-up run (sets kernel attributes), then the capture; the state
        the runs advance is put back after each."""
        nb = self.bucket() if nb is None else nb
        state = (self.tokens, self.positions, self.seq_lens)
        saved = [t.clone() for t in state]

        def restore():
            for t, sv in zip(state, saved):
                t.copy_(sv)

        return self.graphs.get_or_capture(("decode", nb), lambda: self._run_step(nb), warmup=1,
                                          restore=restore, device=self.model.device)

    def step(self) -> torch.Tensor:
        """Run one decode step for every bound row. Returns the device tensor of sampled tokens
        (greedy) — reading it is the caller's only synchronisation. KV blocks for the step must
        have been reserved. ``RMLX_DEBUG_SERIALIZE=1`` runs the step launch by launch instead
        (each launch followed by a device synchronisation and a read of the status words)."""
        if self.use_graph and not self.serialize:
            self.capture().replay()
        else:
            self._run_step(self.bucket())
        for s in self.seq_ids:
            self.cache.commit(s, 1)
        return self.next_tokens

    def set_next_tokens(self, tokens: Sequence[int]) -> None:
        """Replace the tokens the last step fed back (its arg-max) with ones chosen by the caller,
        e.g. sampled from ``logits``; positions and lengths were already advanced by the step."""
        n = len(self.seq_ids)
        assert len(tokens) == n
        self.tokens[:n] = torch.tensor([int(t) for t in tokens], dtype=torch.int32)

    @property
    def launches_per_step(self) -> int:
        return self._launches_per_step

    # ------------------------------------------------------------------ convenience
    @torch.no_grad()
    def generate(self, steps: int) -> torch.Tensor:
        """Greedy-generate ``steps`` tokens for the bound sequences: [n_seqs, steps] on the host."""
        self.reserve(steps + 1)
        out = torch.zeros(len(self.seq_ids), steps, dtype=torch.int64)
        for i in range(steps):
            nxt = self.step()
            out[:, i] = nxt[:len(self.seq_ids)].cpu().long()
        return out
