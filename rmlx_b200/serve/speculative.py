"""Draft-and-verify (speculative) generation for one sequence.

A small draft model proposes ``k`` tokens one at a time; the target model scores all of them (plus
the position after the last one) in a single forward over ``k + 1`` tokens; the longest accepted
prefix is kept together with one token from the target (the correction at the first mismatch, or
the bonus token after a fully accepted draft), and the KV pages both models wrote for rejected
positions are rolled back with ``PagedKvCache.trim``.

The reference ships only the verification helpers (``greedy_verify`` / ``rejection_sample`` /
``SpecDecodeResult`` in crates/rmlx-nn/src/sampler.rs:44-370 and ``PagedKvCache::trim``,
crates/rmlx-nn/src/paged_kv_cache.rs:557); this is the runner around them. With a greedy sampler
the output is exactly the target model's greedy continuation whatever the draft proposes; with
temperature > 0 acceptance follows the rejection-sampling rule, which preserves the target
distribution.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..config import SamplerConfig
from ..models.transformer import TransformerModel
from .sampler import Sampler


@dataclass
class SpecStats:
    rounds: int = 0               # target forwards after the prompt
    proposed: int = 0
    accepted: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0

    @property
    def tokens_per_round(self) -> float:
        return (self.accepted + self.rounds) / self.rounds if self.rounds else 0.0


class SpeculativeDecoder:
    def __init__(self, target: TransformerModel, draft: TransformerModel, k: int = 4,
                 sampler_cfg: Optional[SamplerConfig] = None, eos_token_id: Optional[int] = None):
        if k < 1:
            raise ValueError("k must be >= 1")
        if target.cfg.vocab_size != draft.cfg.vocab_size:
            raise ValueError("draft and target must share a vocabulary")
        self.target, self.draft, self.k = target, draft, k
        from . import native
        # host-side shaping, draws and acceptance rules run in the native library when it is there
        self.sampler = (native.NativeSampler if native.enabled() else Sampler)(sampler_cfg)
        self.greedy = self.sampler.cfg.temperature == 0.0
        self.eos = eos_token_id
        self.stats = SpecStats()

    # ------------------------------------------------------------------ helpers
    def _pick(self, logits: torch.Tensor, history: Sequence[int]):
        """(token, distribution or None) for one position of the draft."""
        if self.greedy:
            return self.sampler.sample_token(logits.cpu(), history), None
        probs = self.sampler.probabilities(logits.cpu(), history)
        return int(torch.multinomial(probs, 1, generator=self.sampler._generator(probs.device))), probs

    @torch.no_grad()
    def generate(self, prompt: Sequence[int], max_new_tokens: int) -> List[int]:
        tgt, drf, k = self.target, self.draft, self.k
        need = (len(prompt) + max_new_tokens + k + 1 + 15) // 16 + 2
        tc = tgt.new_cache(need, max_seqs=1)
        dc = drf.new_cache(need, max_seqs=1)
        tc.add_sequence(0)
        dc.add_sequence(0)
        ids = torch.tensor([int(t) for t in prompt], device=tgt.device)
        logits = tgt.prefill(ids, tc, 0)
        drf.prefill(ids.to(drf.device), dc, 0)
        out: List[int] = []
        pending = self.sampler.sample_token(logits[0].float().cpu(), out)   # first token: the target's
        out.append(pending)
        unfed = [pending]                  # tokens the draft has not seen yet
        while len(out) < max_new_tokens and pending != self.eos:
            # ---- draft: k proposals
            proposals: List[int] = []
            dprobs = []
            feed = unfed
            for _ in range(k):
                dl = drf.prefill(torch.tensor(feed, device=drf.device), dc, 0)
                tok, probs = self._pick(dl[0].float(), out + proposals)
                proposals.append(tok)
                dprobs.append(probs)
                feed = [tok]
            # the draft cache now holds everything up to proposals[k-2]; proposals[k-1] is unfed
            # ---- target: one forward over the pending token and the k proposals
            tl = tgt.prefill(torch.tensor([pending] + proposals, device=tgt.device), tc, 0,
                             all_logits=True).float().cpu()
            if self.greedy:
                res = self.sampler.greedy_verify(proposals, tl)
            else:
                tp = torch.stack([self.sampler.probabilities(tl[i], out + proposals[:i])
                                  for i in range(k + 1)])
                res = self.sampler.rejection_sample(proposals, torch.stack(dprobs), tp)
            a = res.num_accepted
            nxt = res.correction_token
            self.stats.rounds += 1
            self.stats.proposed += k
            self.stats.accepted += a
            # ---- roll back what was rejected: the target wrote pending + k proposals and keeps
            # pending + a of them; the draft wrote pending + (k - 1) proposals
            tc.trim(0, k - a)
            if a < k:
                dc.trim(0, (k - 1) - a)
                unfed = [nxt]
            else:
                unfed = [proposals[-1], nxt]
            out.extend(res.accepted_tokens)
            out.append(nxt)
            pending = nxt
            if self.eos is not None and self.eos in res.accepted_tokens:
                out = out[:out.index(self.eos) + 1]
                break
        return out[:max_new_tokens]
