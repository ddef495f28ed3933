"""A small serving loop that wires the pieces the reference ships as separate, unwired libraries
(scheduler, sampler, prefix cache, paged KV cache; crates/rmlx-nn/src/scheduler.rs:109-131,
crates/rmlx-nn/src/prefix_cache.rs:9-17): requests are admitted by the continuous-batching
scheduler, prompts run in chunks through ``TransformerModel.prefill``, decode steps run batched,
on CUDA through the graph-captured ``CachedDecode``, on CPU through the library-kernel forward.
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional

import torch

from ..config import SamplerConfig, SchedulerConfig
from ..models.transformer import TransformerModel
from .prefix_cache import PrefixCache
from .sampler import Sampler
from .scheduler import GenerationRequest, Scheduler


class ServingEngine:
    def __init__(self, model: TransformerModel, num_blocks: int,
                 scheduler_cfg: Optional[SchedulerConfig] = None,
                 sampler_cfg: Optional[SamplerConfig] = None, comm=None,
                 use_prefix_cache: bool = False):
        self.model = model
        scfg = scheduler_cfg or SchedulerConfig()
        self.cache = model.new_cache(num_blocks, max_seqs=scfg.max_batch_size)
        self.sched = Scheduler(scfg, manage_blocks=False, on_admit=self.cache.add_sequence,
                               on_evict=self._on_evict)
        self.sampler = Sampler(sampler_cfg)
        self.greedy = self.sampler.cfg.temperature == 0.0 and self.sampler.cfg.repetition_penalty == 1.0
        self.outputs: Dict[int, List[int]] = {}
        self.last_token: Dict[int, int] = {}
        self._ids = itertools.count()
        self._finished: Dict[int, int] = {}
        self.prefix = PrefixCache(self.cache.block_size) if use_prefix_cache else None
        self._engine = None
        self._bound: List[int] = []
        if model.device.type == "cuda":
            # prompts through the tensor-core path; decode through the mat-vec engine for small
            # batches and through the tensor-core path (batch = GEMM rows) for larger ones
            from .. import _lib
            from ..models.decode_engine import CachedDecode
            from ..models.prefill import BatchedDecode, enable_native_prefill
            enable_native_prefill(model)
            if scfg.max_batch_size <= int(_lib.cuda().rmlx_gemv_max_batch()):
                self._engine = CachedDecode(model, self.cache, max_batch=scfg.max_batch_size, comm=comm,
                                            greedy=True)
            else:
                try:
                    self._engine = BatchedDecode(model, self.cache, max_batch=scfg.max_batch_size)
                except ImportError:
                    self._engine = None          # shapes outside the kernels: library-kernel forward

    def _on_evict(self, seq_id: int) -> None:
        self.cache.free_sequence(seq_id)
        self._bound = []

    # ------------------------------------------------------------------ public API
    def submit(self, prompt_tokens: List[int], max_output_len: int) -> int:
        sid = next(self._ids)
        self.sched.add_request(GenerationRequest(sid, list(prompt_tokens), max_output_len))
        self.outputs[sid] = []
        return sid

    def step(self) -> Dict[int, int]:
        """One scheduler step. Returns the tokens produced in it (seq_id -> token)."""
        plan = self.sched.schedule(self.cache.manager, self._finished)
        self._finished = {}
        produced: Dict[int, int] = {}
        dev = self.model.device
        for meta in plan.prefill_seqs:
            lo, hi = plan.prefill_chunk_range
            chunk = torch.tensor(self.sched.prompt_chunk(meta.seq_id, (lo, hi)), device=dev)
            logits = self.model.prefill(chunk, self.cache, meta.seq_id)
            if hi >= meta.prompt_len:      # prompt complete: its last logits give the first token
                tok = self.sampler.sample_token(logits[0].float().cpu(), self.outputs[meta.seq_id])
                produced[meta.seq_id] = tok
        ids = [m.seq_id for m in plan.decode_seqs]
        if ids:
            toks = self._decode(ids)
            for sid, tok in zip(ids, toks):
                produced[sid] = tok
        for sid, tok in produced.items():
            self.outputs[sid].append(tok)
            self.last_token[sid] = tok
            self.sched.update_sequence(sid, self.cache.manager, tok)
            self._finished[sid] = tok
        return produced

    def run_until_done(self, max_steps: int = 100000) -> Dict[int, List[int]]:
        for _ in range(max_steps):
            if not self.sched.has_work():
                break
            self.step()
        return self.outputs

    # ------------------------------------------------------------------ decode back-ends
    def _decode(self, ids: List[int]) -> List[int]:
        dev = self.model.device
        if self._engine is not None and self.greedy:
            if ids != self._bound:
                self._engine.bind(ids, [self.last_token[s] for s in ids])
                self._bound = list(ids)
            self._engine.reserve(1)
            nxt = self._engine.step()
            return [int(t) for t in nxt[:len(ids)].cpu()]
        toks = torch.tensor([self.last_token[s] for s in ids], device=dev)
        logits = self.model.forward(toks, self.cache, ids, last_only=True)
        return [self.sampler.sample_token(logits[i].float().cpu(), self.outputs[s])
                for i, s in enumerate(ids)]
