"""The serving core in the native host library (csrc/host/serving.cpp): prefix cache and
continuous-batching scheduler behind the interfaces of their Python namesakes
(``serve.prefix_cache.PrefixCache``, ``serve.scheduler.Scheduler``), which remain as the behavioural
oracle; the block manager of the same library is ``kv.native.NativeBlockManager`` (re-exported
here). The reference implements the three in Rust
(crates/rmlx-nn/src/paged_kv_cache.rs:36-631, prefix_cache.rs:27-330, scheduler.rs:19-352).

``RMLX_NATIVE_SERVING=0`` makes the serving engine and the paged cache use the Python classes.
"""
from __future__ import annotations

from array import array
from collections import deque
from ctypes import c_int, c_int64
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..config import SchedulerConfig
from ..kv.native import NativeBlockManager, _host, _ints, available, enabled  # noqa: F401 (re-exported)
from .scheduler import GenerationRequest, SchedulerOutput, SeqMeta


class NativePrefixCache:
    """``serve.prefix_cache.PrefixCache`` backed by the native library."""

    def __init__(self, block_size: int = 16, max_blocks: int = 0):
        self._lib = _host()
        self._h = self._lib.rmlx_pc_create(block_size, max_blocks)
        if not self._h:
            raise ValueError("bad prefix cache arguments")
        self.block_size, self.max_blocks = block_size, max_blocks

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rmlx_pc_destroy(h)

    def __len__(self) -> int:
        return self._lib.rmlx_pc_len(self._h)

    @property
    def hits(self) -> int:
        return self._lib.rmlx_pc_hits(self._h)

    @property
    def misses(self) -> int:
        return self._lib.rmlx_pc_misses(self._h)

    def insert(self, tokens: Sequence[int], blocks: Sequence[int]) -> int:
        return len(self.insert_blocks(tokens, blocks))

    def insert_blocks(self, tokens: Sequence[int], blocks: Sequence[int]) -> List[int]:
        out = (c_int * max(1, len(blocks)))()
        n = self._lib.rmlx_pc_insert(self._h, _ints(tokens), len(tokens), _ints(blocks), len(blocks),
                                     out, len(blocks))
        return list(out[:n])

    def lookup(self, tokens: Sequence[int]) -> Tuple[int, List[int]]:
        cap = len(tokens) // self.block_size
        out = (c_int * max(1, cap))()
        n = self._lib.rmlx_pc_lookup(self._h, _ints(tokens), len(tokens), out, cap)
        return n * self.block_size, list(out[:n])

    def evict(self, n: int) -> List[int]:
        n = max(0, min(int(n), len(self)))
        out = (c_int * max(1, n))()
        got = self._lib.rmlx_pc_evict(self._h, n, out, n)
        return list(out[:got])

    def take_evicted(self) -> List[int]:
        cap = 4096
        out = (c_int * cap)()
        victims: List[int] = []
        while True:
            got = self._lib.rmlx_pc_take_evicted(self._h, out, cap)
            victims += list(out[:got])
            if got < cap:
                return victims

    def clear(self) -> List[int]:
        return self.evict(len(self))


class NativeScheduler:
    """``serve.scheduler.Scheduler`` backed by the native library. It plans against a
    ``NativeBlockManager`` (the two live in the same library and talk directly)."""

    def __init__(self, config: SchedulerConfig, manage_blocks: bool = True, on_admit=None,
                 on_evict=None, tables_in_meta: bool = True):
        self.cfg = config.validate()
        self.tables_in_meta = tables_in_meta
        self._lib = _host()
        eos = -1 if self.cfg.eos_token_id is None else int(self.cfg.eos_token_id)
        self._h = self._lib.rmlx_sched_create(self.cfg.max_batch_size, eos, self.cfg.max_prefill_chunk,
                                              int(manage_blocks))
        if not self._h:
            raise ValueError("bad scheduler configuration")
        self.manage_blocks = manage_blocks
        self.on_admit, self.on_evict = on_admit, on_evict
        self._waiting: Deque[Tuple[int, int]] = deque()       # (seq_id, prompt length) mirror
        self._decode_buf = (c_int64 * self.cfg.max_batch_size)()
        self._meta_buf = (c_int * (4 * (self.cfg.max_batch_size + 1)))()
        self._tables = (c_int * (64 * self.cfg.max_batch_size))()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rmlx_sched_destroy(h)

    # ------------------------------------------------------------------ queueing
    def add_request(self, req: GenerationRequest) -> None:
        if not req.prompt_tokens:
            raise ValueError("empty prompt")
        rc = self._lib.rmlx_sched_add_request(self._h, req.seq_id, _ints(req.prompt_tokens),
                                              len(req.prompt_tokens), req.max_output_len)
        if rc != 0:
            raise ValueError("request rejected")
        self._waiting.append((req.seq_id, len(req.prompt_tokens)))

    def num_waiting(self) -> int:
        return self._lib.rmlx_sched_num_waiting(self._h)

    def num_active(self) -> int:
        return self._lib.rmlx_sched_num_active(self._h)

    def has_work(self) -> bool:
        return bool(self.num_waiting() or self.num_active())

    def first_waiting_prompt_len(self) -> Optional[int]:
        return self._waiting[0][1] if self._waiting else None

    # ------------------------------------------------------------------ one step
    def schedule(self, bm: NativeBlockManager, finished_tokens: Optional[Dict[int, int]] = None
                 ) -> SchedulerOutput:
        out = SchedulerOutput()
        lib = self._lib
        if finished_tokens:
            n = len(finished_tokens)
            seqs = array("q", finished_tokens.keys())
            toks = array("q", [-2 if t is None else int(t) for t in finished_tokens.values()])
            ended = (c_int64 * n)()
            k = lib.rmlx_sched_finish_many(self._h, (c_int64 * n).from_buffer(seqs),
                                           (c_int64 * n).from_buffer(toks), n, ended)
            for sid in ended[:k]:
                if self.on_evict is not None:
                    self.on_evict(sid)
                else:
                    bm.free_sequence(sid)
                out.evicted_seq_ids.append(sid)
        while True:
            sid = lib.rmlx_sched_admit_next(self._h, bm._h)
            if sid < 0:
                break
            self._waiting.popleft()
            if self.on_admit is not None:
                cached = self.on_admit(sid) or 0
                if cached:
                    lib.rmlx_sched_set_cached(self._h, sid, int(cached))
            else:
                bm.add_sequence(sid)
        prefill = (c_int64 * 3)()
        n_dec = lib.rmlx_sched_plan(self._h, bm._h, prefill, self._decode_buf, len(self._decode_buf))
        ids = ([int(prefill[0])] if prefill[0] >= 0 else []) + list(self._decode_buf[:n_dec])
        metas = self._describe(ids, bm)
        if prefill[0] >= 0:
            out.prefill_seqs.append(metas[0])
            out.prefill_chunk_range = (int(prefill[1]), int(prefill[2]))
            metas = metas[1:]
        out.decode_seqs.extend(metas)
        return out

    def _describe(self, ids: List[int], bm: NativeBlockManager) -> List[SeqMeta]:
        """``SeqMeta`` of every id from one call into the library."""
        n = len(ids)
        if not n:
            return []
        seqs = array("q", ids)
        want_tables = self.tables_in_meta
        while True:
            used = self._lib.rmlx_sched_describe(self._h, bm._h, (c_int64 * n).from_buffer(seqs), n,
                                                 self._meta_buf, self._tables if want_tables else None,
                                                 len(self._tables) if want_tables else 0)
            if used >= 0:
                break
            self._tables = (c_int * (2 * len(self._tables)))()     # longer sequences than seen so far
        m = self._meta_buf[:4 * n]
        if not want_tables:
            return [SeqMeta(sid, m[4 * i], m[4 * i + 2], [], m[4 * i + 1]) for i, sid in enumerate(ids)]
        t = self._tables[:used]
        out, pos = [], 0
        for i, sid in enumerate(ids):
            nt = m[4 * i + 3]
            out.append(SeqMeta(sid, m[4 * i], m[4 * i + 2], t[pos:pos + nt], m[4 * i + 1]))
            pos += nt
        return out

    def update_sequence(self, seq_id: int, bm: NativeBlockManager, token: int) -> None:
        if self._lib.rmlx_sched_update(self._h, bm._h, seq_id) != 0:
            raise KeyError(seq_id)

    def prompt_chunk(self, seq_id: int, rng: Tuple[int, int]) -> List[int]:
        lo, hi = rng
        buf = (c_int * max(1, hi - lo))()
        n = self._lib.rmlx_sched_prompt(self._h, seq_id, lo, hi, buf)
        if n < 0:
            raise KeyError(seq_id)
        return list(buf[:n])

    def _meta(self, sid: int, bm: NativeBlockManager) -> SeqMeta:
        info = (c_int * 3)()
        self._lib.rmlx_sched_info(self._h, sid, info)
        table = bm.block_table(sid) if bm.has_sequence(sid) else []
        return SeqMeta(sid, int(info[0]), bm.seq_len(sid), table, int(info[1]))


# ------------------------------------------------------------------------------------------------
# sampler
# ------------------------------------------------------------------------------------------------
import ctypes as _ct                                                    # noqa: E402
import os as _os                                                        # noqa: E402

import torch as _torch                                                  # noqa: E402

from .sampler import Sampler, SpecDecodeResult                          # noqa: E402

_FP = _ct.POINTER(_ct.c_float)
_sampler_bound = False


def _sampler_lib():
    global _sampler_bound
    lib = _host()
    if not _sampler_bound:
        ip = _ct.POINTER(_ct.c_int)
        sig = {
            "rmlx_sampler_create": (_ct.c_void_p, [_ct.c_float, _ct.c_int, _ct.c_float, _ct.c_float, _ct.c_uint64]),
            "rmlx_sampler_destroy": (None, [_ct.c_void_p]),
            "rmlx_sampler_probabilities": (_ct.c_int, [_ct.c_void_p, _ct.c_void_p, _ct.c_int, ip, _ct.c_int, _ct.c_void_p]),
            "rmlx_sampler_sample": (_ct.c_int, [_ct.c_void_p, _ct.c_void_p, _ct.c_int, _ct.c_int, ip, ip, ip]),
            "rmlx_sampler_uniform": (_ct.c_double, [_ct.c_void_p]),
            "rmlx_sampler_multinomial": (_ct.c_int, [_ct.c_void_p, _ct.c_void_p, _ct.c_int]),
            "rmlx_spec_greedy_verify": (_ct.c_int, [ip, _ct.c_int, _ct.c_void_p, _ct.c_int, _ct.c_int, ip]),
            "rmlx_spec_rejection_sample": (_ct.c_int, [_ct.c_void_p, ip, _ct.c_int, _ct.c_void_p, _ct.c_void_p,
                                                       _ct.c_int, _ct.c_int, ip]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _sampler_bound = True
    return lib


def _f32(t: "_torch.Tensor") -> "_torch.Tensor":
    return t.detach().to(_torch.float32).contiguous()


class NativeSampler(Sampler):
    """``serve.sampler.Sampler`` whose host-side work (logits or probabilities already on the CPU)
    runs in the native library (csrc/host/sampler.cpp): distribution shaping, the multinomial draw
    from the sampler's own seeded generator, and both speculative acceptance rules. Logits that
    live on a GPU keep the tensor-op path of the base class (only token ids leave the device).
    The distribution is the base class's to rounding; the random stream is its own, so a seed
    reproduces a run of this class, not the tokens of the other."""

    def __init__(self, config=None):
        super().__init__(config)
        self._lib = _sampler_lib()
        c = self.cfg
        seed = c.seed if c.seed is not None else int.from_bytes(_os.urandom(8), "little")
        self._h = self._lib.rmlx_sampler_create(c.temperature, c.top_k, c.top_p, c.repetition_penalty,
                                                seed & 0xFFFFFFFFFFFFFFFF)
        if not self._h:
            raise ValueError("bad sampler configuration")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rmlx_sampler_destroy(h)

    def probabilities(self, logits, history=()):
        if logits.is_cuda:
            return super().probabilities(logits, history)
        l = _f32(logits)
        out = _torch.empty_like(l)
        hist = _ints([int(t) for t in history])
        self._lib.rmlx_sampler_probabilities(self._h, l.data_ptr(), l.numel(), hist, len(history), out.data_ptr())
        return out

    def sample_token(self, logits, history=()):
        if logits.is_cuda:
            return super().sample_token(logits, history)
        return self.sample_batch(logits.reshape(1, -1), [list(history)])[0]

    def sample_batch(self, logits, histories=None):
        if logits.is_cuda:
            return super().sample_batch(logits, histories)
        l = _f32(logits)
        rows, vocab = l.shape
        out = (_ct.c_int * max(1, rows))()
        hist = off = None
        if histories is not None and self.cfg.repetition_penalty != 1.0:
            flat, offs = [], [0]
            for h in histories:
                flat += [int(t) for t in h]
                offs.append(len(flat))
            hist, off = _ints(flat), _ints(offs)
        self._lib.rmlx_sampler_sample(self._h, l.data_ptr(), rows, vocab, hist, off, out)
        return list(out[:rows])

    def greedy_verify(self, draft_tokens, target_logits):          # an instance method here: same call shape
        if target_logits.is_cuda:
            return Sampler.greedy_verify(draft_tokens, target_logits)
        l = _f32(target_logits)
        nxt = _ct.c_int(-1)
        draft = [int(t) for t in draft_tokens]
        n = self._lib.rmlx_spec_greedy_verify(_ints(draft), len(draft), l.data_ptr(), l.shape[0], l.shape[1],
                                              _ct.byref(nxt))
        return SpecDecodeResult(n, draft[:n], None if nxt.value < 0 else nxt.value)

    def rejection_sample(self, draft_tokens, draft_probs, target_probs):
        if draft_probs.is_cuda or target_probs.is_cuda:
            return super().rejection_sample(draft_tokens, draft_probs, target_probs)
        pd, pt = _f32(draft_probs), _f32(target_probs)
        nxt = _ct.c_int(-1)
        draft = [int(t) for t in draft_tokens]
        n = self._lib.rmlx_spec_rejection_sample(self._h, _ints(draft), len(draft), pd.data_ptr(), pt.data_ptr(),
                                                 pt.shape[0], pt.shape[1], _ct.byref(nxt))
        if n < 0:
            raise ValueError("rejection_sample: a draft token outside the vocabulary, or fewer target rows than draft tokens")
        return SpecDecodeResult(n, draft[:n], None if nxt.value < 0 else nxt.value)
