"""Token sampling and speculative-decoding verification.

Order of operations and knobs follow the reference's ``Sampler`` (crates/rmlx-nn/src/sampler.rs:21-141):
repetition penalty -> temperature (0 = greedy) -> top-k (0 = off) -> top-p (1 = off) -> softmax ->
multinomial. ``greedy_verify`` and ``rejection_sample`` implement the two acceptance rules of
crates/rmlx-nn/src/sampler.rs:156-370 and return a ``SpecDecodeResult``; rollback of rejected draft
tokens is ``PagedKvCache.trim``.

Works on CPU or CUDA logits (greedy decode on the GPU uses the arg-max kernel inside the captured
step instead).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..config import SamplerConfig


@dataclass
class SpecDecodeResult:
    num_accepted: int
    accepted_tokens: List[int] = field(default_factory=list)
    correction_token: Optional[int] = None


class Sampler:
    def __init__(self, config: Optional[SamplerConfig] = None):
        self.cfg = (config or SamplerConfig()).validate()
        self._gen = None
        self._device_gens = {}
        if self.cfg.seed is not None:
            self._gen = torch.Generator().manual_seed(self.cfg.seed)

    # ------------------------------------------------------------------ distribution shaping
    def apply_repetition_penalty(self, logits: torch.Tensor, history: Sequence[int]) -> torch.Tensor:
        p = self.cfg.repetition_penalty
        if p == 1.0 or not history:
            return logits
        idx = torch.tensor(sorted(set(int(t) for t in history)), dtype=torch.long, device=logits.device)
        vals = logits[idx]
        logits = logits.clone()
        logits[idx] = torch.where(vals > 0, vals / p, vals * p)
        return logits

    def probabilities(self, logits: torch.Tensor, history: Sequence[int] = ()) -> torch.Tensor:
        """Final sampling distribution over the vocabulary for one position (fp32)."""
        cfg = self.cfg
        l = self.apply_repetition_penalty(logits.float(), history)
        if cfg.temperature == 0.0:
            out = torch.zeros_like(l)
            out[int(l.argmax())] = 1.0
            return out
        l = l / cfg.temperature
        if 0 < cfg.top_k < l.numel():
            kth = torch.topk(l, cfg.top_k).values[-1]
            l = torch.where(l < kth, torch.full_like(l, float("-inf")), l)
        probs = torch.softmax(l, dim=-1)
        if cfg.top_p < 1.0:
            sp, si = torch.sort(probs, descending=True)
            cum = torch.cumsum(sp, 0)
            keep = cum - sp < cfg.top_p            # always keeps the most likely token
            sp = torch.where(keep, sp, torch.zeros_like(sp))
            probs = torch.zeros_like(probs).scatter_(0, si, sp)
            probs = probs / probs.sum()
        return probs

    # ------------------------------------------------------------------ sampling
    def sample_token(self, logits: torch.Tensor, history: Sequence[int] = ()) -> int:
        if self.cfg.temperature == 0.0:
            return int(self.apply_repetition_penalty(logits.float(), history).argmax())
        probs = self.probabilities(logits, history).cpu()
        return int(torch.multinomial(probs, 1, generator=self._gen))

    # ------------------------------------------------------------------ whole batches at once
    def _generator(self, device: torch.device):
        """The seeded generator for ``device`` (one per device, derived from ``seed``), or None."""
        if self.cfg.seed is None:
            return None
        if device.type == "cpu":
            return self._gen
        g = self._device_gens.get(device)
        if g is None:
            g = torch.Generator(device=device).manual_seed(self.cfg.seed)
            self._device_gens[device] = g
        return g

    def probabilities_batch(self, logits: torch.Tensor,
                            histories: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """``probabilities`` for every row of ``logits`` [B, V] in one pass of tensor ops on the
        device the logits live on (no per-row Python loop, no copy of the logits to the host)."""
        cfg = self.cfg
        l = logits.float()
        if cfg.repetition_penalty != 1.0 and histories is not None and any(len(h) for h in histories):
            rows, cols = [], []
            for i, h in enumerate(histories):
                toks = sorted(set(int(t) for t in h))
                rows += [i] * len(toks)
                cols += toks
            r = torch.tensor(rows, dtype=torch.long, device=l.device)
            c = torch.tensor(cols, dtype=torch.long, device=l.device)
            vals = l[r, c]
            l = l.clone()
            l[r, c] = torch.where(vals > 0, vals / cfg.repetition_penalty, vals * cfg.repetition_penalty)
        if cfg.temperature == 0.0:
            return torch.zeros_like(l).scatter_(1, l.argmax(-1, keepdim=True), 1.0)
        l = l / cfg.temperature
        if 0 < cfg.top_k < l.shape[-1]:
            kth = torch.topk(l, cfg.top_k, dim=-1).values[:, -1:]
            l = torch.where(l < kth, torch.full_like(l, float("-inf")), l)
        probs = torch.softmax(l, dim=-1)
        if cfg.top_p < 1.0:
            sp, si = torch.sort(probs, dim=-1, descending=True)
            keep = torch.cumsum(sp, -1) - sp < cfg.top_p      # always keeps the most likely token
            sp = torch.where(keep, sp, torch.zeros_like(sp))
            probs = torch.zeros_like(probs).scatter_(1, si, sp)
            probs = probs / probs.sum(-1, keepdim=True)
        return probs

    def sample_batch(self, logits: torch.Tensor, histories: Optional[Sequence[Sequence[int]]] = None
                     ) -> List[int]:
        """One token per row of ``logits`` [B, V]; only the chosen ids leave the logits' device."""
        if self.cfg.temperature == 0.0:
            if self.cfg.repetition_penalty == 1.0 or histories is None:
                return logits.argmax(-1).tolist()
            return self.probabilities_batch(logits, histories).argmax(-1).tolist()
        probs = self.probabilities_batch(logits, histories)
        return torch.multinomial(probs, 1, generator=self._generator(probs.device))[:, 0].tolist()

    # ------------------------------------------------------------------ speculative decoding
    @staticmethod
    def greedy_verify(draft_tokens: Sequence[int], target_logits: torch.Tensor) -> SpecDecodeResult:
        """target_logits[i] are the target model's logits at the position of draft_tokens[i]
        (one extra row, if present, gives the bonus token after a fully accepted draft)."""
        accepted: List[int] = []
        for i, t in enumerate(draft_tokens):
            best = int(target_logits[i].argmax())
            if best != int(t):
                return SpecDecodeResult(len(accepted), accepted, best)
            accepted.append(int(t))
        bonus = None
        if target_logits.shape[0] > len(draft_tokens):
            bonus = int(target_logits[len(draft_tokens)].argmax())
        return SpecDecodeResult(len(accepted), accepted, bonus)

    def rejection_sample(self, draft_tokens: Sequence[int], draft_probs: torch.Tensor,
                         target_probs: torch.Tensor) -> SpecDecodeResult:
        """Accept draft token x with probability min(1, p_target(x) / p_draft(x)); on the first
        rejection sample the correction from normalise(max(0, p_target - p_draft))."""
        accepted: List[int] = []
        for i, t in enumerate(draft_tokens):
            t = int(t)
            pt, pd = float(target_probs[i, t]), float(draft_probs[i, t])
            u = float(torch.rand((), generator=self._gen))
            if pd <= 0.0 or u < min(1.0, pt / pd):
                accepted.append(t)
                continue
            resid = (target_probs[i].float() - draft_probs[i].float()).clamp_min(0).cpu()
            if float(resid.sum()) <= 0:
                resid = target_probs[i].float().cpu()
            tok = int(torch.multinomial(resid / resid.sum(), 1, generator=self._gen))
            return SpecDecodeResult(len(accepted), accepted, tok)
        bonus = None
        if target_probs.shape[0] > len(draft_tokens):
            bonus = int(torch.multinomial(target_probs[len(draft_tokens)].float().cpu(), 1,
                                          generator=self._gen))
        return SpecDecodeResult(len(accepted), accepted, bonus)
