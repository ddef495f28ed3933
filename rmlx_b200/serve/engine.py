"""A small serving loop that wires the pieces the reference ships as separate, unwired libraries
(scheduler, sampler, prefix cache, paged KV cache; crates/rmlx-nn/src/scheduler.rs:109-131,
crates/rmlx-nn/src/prefix_cache.rs:9-17): requests are admitted by the continuous-batching
scheduler, prompts run in chunks through ``TransformerModel.prefill``, decode steps run batched,
on CUDA through the graph-captured ``CachedDecode``, on CPU through the library-kernel forward.
"""
from __future__ import annotations

import itertools
import os
from typing import Dict, List, Optional

import torch

from ..config import SamplerConfig, SchedulerConfig
from ..models.transformer import TransformerModel
from ..parallel.warmup import Warmup, WarmupResult
from ..utils.metrics import PERF
from ..utils.precision_guard import GuardAction, PrecisionGuard
from .prefix_cache import PrefixCache
from .sampler import Sampler
from .scheduler import GenerationRequest, Scheduler


class ServingEngine:
    def __init__(self, model: TransformerModel, num_blocks: int,
                 scheduler_cfg: Optional[SchedulerConfig] = None,
                 sampler_cfg: Optional[SamplerConfig] = None, comm=None,
                 use_prefix_cache: bool = False, sample_on_device: bool = False,
                 kv_quant: Optional[str] = None, precision_guard: Optional[PrecisionGuard] = None,
                 guard_every: int = 16):
        """``sample_on_device``: run the sampler's tensor ops where the logits are (only the chosen
        token ids come back) instead of on a host copy of the logits. ``kv_quant="q8"``: the KV
        cache is kept in the 8-bit format (half the bytes per cached token). ``precision_guard``:
        every ``guard_every``-th decode step (and every completed prompt) hands its logits to the
        guard; its verdicts are counted in ``guard_warnings`` / ``guard_fallbacks`` and the steps
        they came from listed in ``guard_events``."""
        self.model = model
        scfg = scheduler_cfg or SchedulerConfig()
        self.cache = model.new_cache(num_blocks, max_seqs=scfg.max_batch_size, kv_quant=kv_quant)
        # scheduler, block manager and prefix cache come from the native host library unless it
        # is switched off (the cache above made the same choice for its block manager)
        from . import native
        self.native = native.enabled()
        sched_cls = native.NativeScheduler if self.native else Scheduler
        self.sched = sched_cls(scfg, manage_blocks=False, on_admit=self._on_admit,
                               on_evict=self._on_evict, tables_in_meta=False)
        # host-side sampling (logits read back to the CPU) runs in the native library as well
        self.sampler = (native.NativeSampler if self.native else Sampler)(sampler_cfg)
        self.sample_on_device = sample_on_device
        self.greedy = self.sampler.cfg.temperature == 0.0 and self.sampler.cfg.repetition_penalty == 1.0
        self.outputs: Dict[int, List[int]] = {}
        self.last_token: Dict[int, int] = {}
        self._ids = itertools.count()
        self._finished: Dict[int, int] = {}
        prefix_cls = native.NativePrefixCache if self.native else PrefixCache
        self.prefix = prefix_cls(self.cache.block_size) if use_prefix_cache else None
        self._prompts: Dict[int, List[int]] = {}
        self.prefill_tokens = 0               # prompt tokens actually run (cached prefixes excluded)
        self.released_pages = 0               # sliding-window models: pages returned to the pool
        self._engine = None
        self._bound: List[int] = []
        self.guard = precision_guard
        self.guard_every = max(1, guard_every)
        self.guard_warnings = 0
        self.guard_fallbacks = 0
        self.guard_events: List[tuple] = []   # (decode step, GuardAction) of every verdict but OK
        self._decode_steps = 0
        self._comm = comm
        self._warmup = Warmup()
        if model.device.type == "cuda":
            # prompts through the tensor-core path; decode through the mat-vec engine for small
            # batches and through the tensor-core path (batch = GEMM rows) for larger ones
            from .. import _lib
            from ..models.decode_engine import CachedDecode
            from ..models.prefill import BatchedDecode, enable_native_prefill
            enable_native_prefill(model)
            # measured on the 60-layer MoE model (4-bit weights): the mat-vec engine takes 377 us
            # per layer at 8 rows against 434 for the tensor-core path, which wins from 16 rows on
            matvec_max = int(os.environ.get("RMLX_MATVEC_MAX_BATCH", "8"))
            if scfg.max_batch_size <= matvec_max:
                self._engine = CachedDecode(model, self.cache, max_batch=scfg.max_batch_size, comm=comm,
                                            greedy=True)
            else:
                try:
                    self._engine = BatchedDecode(model, self.cache, max_batch=scfg.max_batch_size)
                except ImportError:
                    self._engine = None          # shapes outside the kernels: library-kernel forward

    def _on_admit(self, seq_id: int) -> int:
        """New sequence; with a prefix cache, start it from the cached pages of the longest
        block-aligned prefix of its prompt. Returns how many prompt tokens that covers."""
        self.cache.add_sequence(seq_id)
        if self.prefix is None:
            return 0
        prompt = self._prompts[seq_id]
        bs = self.cache.block_size
        _, blocks = self.prefix.lookup(prompt)
        blocks = blocks[:(len(prompt) - 1) // bs]        # the last prompt token always runs
        if blocks:
            self.cache.adopt_prefix(seq_id, blocks, len(blocks) * bs)
        return len(blocks) * bs

    def _on_evict(self, seq_id: int) -> None:
        prompt = self._prompts.pop(seq_id, None)
        if self.prefix is not None and prompt is not None:
            # the finished sequence's full prompt pages stay behind for later requests; the cache
            # holds its own reference to each page it newly records
            table = self.cache.manager.block_table(seq_id)
            done = min(len(prompt), self.cache.seq_len(seq_id))
            for b in self.prefix.insert_blocks(prompt[:done], table):
                self.cache.manager.retain(b)
            for b in self.prefix.take_evicted():
                self.cache.manager.release(b)
        self.cache.free_sequence(seq_id)
        self._bound = []

    def reclaim(self, num_blocks: int) -> int:
        """Drop up to ``num_blocks`` least-recently-used prefix pages back to the free pool."""
        if self.prefix is None:
            return 0
        victims = self.prefix.evict(num_blocks)
        for b in victims:
            self.cache.manager.release(b)
        return len(victims)

    # ------------------------------------------------------------------ warm-up and logit monitor
    def warm_up(self, prompt_len: int = 8, new_tokens: int = 3) -> WarmupResult:
        """Run the communication path and every kernel once before the first real request: a
        barrier over the tensor-parallel group, then throw-away requests that fill each batch
        bucket of the decode engine in turn (prompt path, graph capture per bucket, sampler).
        Their pages, outputs and counters are dropped afterwards. A second call does nothing and
        returns the first call's timings (crates/rmlx-distributed/src/warmup.rs:20-150)."""
        def comm_fn():
            if self._comm is not None and hasattr(self._comm, "barrier"):
                self._comm.barrier()

        def kernel_fn():
            buckets = getattr(self._engine, "buckets", None) or (self.sched.cfg.max_batch_size,)
            guard, self.guard = self.guard, None          # throw-away logits stay out of the statistics
            try:
                for nb in buckets:
                    # prompts are admitted one per step: the first request must still be decoding
                    # when the last one joins, or the bucket's batch never forms
                    ids = [self.submit([1 + (i % 7)] * prompt_len, max(new_tokens, nb + 2)) for i in range(nb)]
                    self.run_until_done()
                    for sid in ids:
                        self.outputs.pop(sid, None)
                        self.last_token.pop(sid, None)
            finally:
                self.guard = guard
            if self.prefix is not None:                   # the throw-away prompts leave no cached pages
                self.reclaim(1 << 30)
            self.prefill_tokens = 0
            self.released_pages = 0
            self._decode_steps = 0

        return self._warmup.run(comm_fn=comm_fn, kernel_fn=kernel_fn)

    def _guard_check(self, logits: torch.Tensor) -> None:
        action = self.guard.check(logits)
        if action is GuardAction.OK:
            return
        if action is GuardAction.WARN:
            self.guard_warnings += 1
        else:
            self.guard_fallbacks += 1
        self.guard_events.append((self._decode_steps, action))

    # ------------------------------------------------------------------ public API
    def submit(self, prompt_tokens: List[int], max_output_len: int) -> int:
        sid = next(self._ids)
        self._prompts[sid] = [int(t) for t in prompt_tokens]
        self.sched.add_request(GenerationRequest(sid, list(prompt_tokens), max_output_len))
        self.outputs[sid] = []
        return sid

    def step(self) -> Dict[int, int]:
        """One scheduler step. Returns the tokens produced in it (seq_id -> token)."""
        waiting_len = self.sched.first_waiting_prompt_len() if self.prefix is not None else None
        if waiting_len is not None:
            # cached prefix pages give way to a request that would otherwise wait for blocks
            first = min(waiting_len, self.sched.cfg.max_prefill_chunk)
            short = -(-first // self.cache.block_size) - self.cache.manager.num_free_blocks()
            if short > 0:
                self.reclaim(short)
        plan = self.sched.schedule(self.cache.manager, self._finished)
        self._finished = {}
        produced: Dict[int, int] = {}
        dev = self.model.device
        for meta in plan.prefill_seqs:
            lo, hi = plan.prefill_chunk_range
            chunk = torch.tensor(self.sched.prompt_chunk(meta.seq_id, (lo, hi)), device=dev)
            logits = self.model.prefill(chunk, self.cache, meta.seq_id)
            self.prefill_tokens += hi - lo
            if hi >= meta.prompt_len:      # prompt complete: its last logits give the first token
                if self.guard is not None:
                    self._guard_check(logits[:1])
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
    def _release_outside_window(self, ids: List[int]) -> None:
        """Sliding-window models: pages that lie entirely before the window go back to the pool
        (checked when a sequence crosses a page boundary). Prefix-cached pages keep their own
        reference, so only this sequence's hold on them is dropped."""
        window = self.model.cfg.sliding_window or 0
        if window <= 0:
            return
        bs = self.cache.block_size
        for s in ids:
            if self.cache.seq_len(s) % bs == 0 and self.cache.seq_len(s) > window + bs:
                self.released_pages += self.cache.drop_front(s, window)

    def _decode(self, ids: List[int]) -> List[int]:
        dev = self.model.device
        self._release_outside_window(ids)
        self._decode_steps += 1
        guarded = self.guard is not None and self._decode_steps % self.guard_every == 0
        # the device engines compute full-vocabulary logits unless the LM head is sharded
        on_device = self._engine is not None and (self.greedy or self.model.layout.world == 1)
        if on_device:
            if ids != self._bound:
                self._engine.bind(ids, [self.last_token[s] for s in ids])
                self._bound = list(ids)
            self._engine.reserve(1)
            nxt = self._engine.step()
            if guarded:
                self._guard_check(self._engine.logits[:len(ids)])
            if self.greedy:
                PERF.record_d2h(nxt[:len(ids)])
                return [int(t) for t in nxt[:len(ids)].cpu()]
            # sampling: the step fed its arg-max back; replace it with the sampled tokens
            logits = self._engine.logits[:len(ids)]
            if not self.sample_on_device:
                PERF.record_d2h(logits)
                logits = logits.float().cpu()
            toks = self.sampler.sample_batch(logits, [self.outputs[s] for s in ids])
            self._engine.set_next_tokens(toks)
            return toks
        toks = torch.tensor([self.last_token[s] for s in ids], device=dev)
        logits = self.model.forward(toks, self.cache, ids, last_only=True)
        if guarded:
            self._guard_check(logits)
        if not self.sample_on_device:
            logits = logits.float().cpu()
        return self.sampler.sample_batch(logits, [self.outputs[s] for s in ids])
