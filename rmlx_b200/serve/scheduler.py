"""Continuous-batching scheduler: a waiting queue, an active set, KV-block admission control,
EOS / max-length eviction and chunked prefill interleaved with decode.

Same contract as the reference's ``Scheduler`` (crates/rmlx-nn/src/scheduler.rs:19-352): each call to
``schedule(block_manager, finished_tokens)`` evicts sequences that produced EOS or reached their
output budget, admits waiting requests while batch slots and KV blocks allow, and returns which
sequences prefill (at most one prompt chunk of ``max_prefill_chunk`` tokens per step) and which
decode. ``update_sequence`` records a generated token and grows the block table on a page boundary.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple

from ..config import SchedulerConfig
from ..kv.paged import BlockManager


@dataclass
class GenerationRequest:
    seq_id: int
    prompt_tokens: List[int]
    max_output_len: int


@dataclass
class SeqMeta:
    seq_id: int
    prompt_len: int
    current_len: int
    block_table: List[int]
    prefill_progress: int

    def is_chunked_prefill(self) -> bool:
        return 0 < self.prefill_progress < self.prompt_len


@dataclass
class SchedulerOutput:
    prefill_seqs: List[SeqMeta] = field(default_factory=list)
    decode_seqs: List[SeqMeta] = field(default_factory=list)
    evicted_seq_ids: List[int] = field(default_factory=list)
    prefill_chunk_range: Optional[Tuple[int, int]] = None


@dataclass
class _Active:
    prompt: List[int]
    max_output_len: int
    generated: int = 0
    prefill_progress: int = 0

    @property
    def prefilled(self) -> bool:
        return self.prefill_progress >= len(self.prompt)


class Scheduler:
    def __init__(self, config: SchedulerConfig, manage_blocks: bool = True, on_admit=None,
                 on_evict=None, tables_in_meta: bool = True):
        """``manage_blocks=False``: only check capacity; the caller's forward pass reserves and
        commits KV slots itself. ``on_admit`` / ``on_evict`` replace the default
        ``add_sequence`` / ``free_sequence`` calls on the block manager; ``on_admit`` may return the
        number of leading prompt tokens whose KV it found cached (prefill starts after them)."""
        self.cfg = config.validate()
        self.waiting: Deque[GenerationRequest] = deque()
        self.active: Dict[int, _Active] = {}
        self.manage_blocks = manage_blocks
        self.on_admit = on_admit
        self.on_evict = on_evict
        self.tables_in_meta = tables_in_meta      # False: SeqMeta.block_table stays empty (callers that
                                                  # read tables from the cache save the copies)

    # ------------------------------------------------------------------ queueing
    def add_request(self, req: GenerationRequest) -> None:
        if not req.prompt_tokens:
            raise ValueError("empty prompt")
        self.waiting.append(req)

    def num_waiting(self) -> int:
        return len(self.waiting)

    def num_active(self) -> int:
        return len(self.active)

    def has_work(self) -> bool:
        return bool(self.waiting or self.active)

    def first_waiting_prompt_len(self) -> Optional[int]:
        return len(self.waiting[0].prompt_tokens) if self.waiting else None

    # ------------------------------------------------------------------ one step
    def schedule(self, bm: BlockManager, finished_tokens: Optional[Dict[int, int]] = None
                 ) -> SchedulerOutput:
        """``finished_tokens``: seq_id -> token produced by the previous step."""
        out = SchedulerOutput()
        # 1. evict finished sequences
        for sid, tok in (finished_tokens or {}).items():
            a = self.active.get(sid)
            if a is None:
                continue
            if tok == self.cfg.eos_token_id or a.generated >= a.max_output_len:
                self._evict(sid, bm, out)
        # 2. admit while there is room
        while self.waiting and len(self.active) < self.cfg.max_batch_size:
            req = self.waiting[0]
            first = min(len(req.prompt_tokens), self.cfg.max_prefill_chunk)
            need = (first + bm.block_size - 1) // bm.block_size
            if need > bm.num_free_blocks():
                break
            self.waiting.popleft()
            cached = 0
            if self.on_admit is not None:
                cached = self.on_admit(req.seq_id) or 0     # prompt tokens whose KV is already cached
            else:
                bm.add_sequence(req.seq_id)
            a = _Active(list(req.prompt_tokens), req.max_output_len)
            # the last prompt token always runs: its logits give the first generated token
            a.prefill_progress = max(0, min(int(cached), len(a.prompt) - 1))
            self.active[req.seq_id] = a
        # 3. one prefill chunk (oldest unfinished prompt first), everyone else decodes
        prefilling = [sid for sid, a in self.active.items() if not a.prefilled]
        if prefilling:
            sid = prefilling[0]
            a = self.active[sid]
            lo = a.prefill_progress
            hi = min(len(a.prompt), lo + self.cfg.max_prefill_chunk)
            if bm.can_allocate(sid, hi - lo):
                if self.manage_blocks:
                    bm.reserve(sid, hi - lo)
                    bm.commit(sid, hi - lo)
                a.prefill_progress = hi
                out.prefill_seqs.append(self._meta(sid, bm))
                out.prefill_chunk_range = (lo, hi)
        for sid, a in self.active.items():
            if a.prefilled and not (out.prefill_seqs and out.prefill_seqs[0].seq_id == sid):
                if not bm.can_allocate(sid, 1):
                    continue        # stalls this step; blocks free up when others finish
                if self.manage_blocks:
                    bm.reserve(sid, 1)
                out.decode_seqs.append(self._meta(sid, bm))
        return out

    def update_sequence(self, seq_id: int, bm: BlockManager, token: int) -> None:
        """Record one generated token for ``seq_id`` (its KV slot was reserved by ``schedule``)."""
        a = self.active[seq_id]
        a.generated += 1
        if self.manage_blocks:
            bm.commit(seq_id, 1)

    def prompt_chunk(self, seq_id: int, rng: Tuple[int, int]) -> List[int]:
        return self.active[seq_id].prompt[rng[0]:rng[1]]

    # ------------------------------------------------------------------ internals
    def _meta(self, sid: int, bm: BlockManager) -> SeqMeta:
        a = self.active[sid]
        table = list(bm.block_table(sid)) if self.tables_in_meta else []
        return SeqMeta(sid, len(a.prompt), bm.seq_len(sid), table, a.prefill_progress)

    def _evict(self, sid: int, bm: BlockManager, out: SchedulerOutput) -> None:
        self.active.pop(sid, None)
        if self.on_evict is not None:
            self.on_evict(sid)
        else:
            bm.free_sequence(sid)
        out.evicted_seq_ids.append(sid)
